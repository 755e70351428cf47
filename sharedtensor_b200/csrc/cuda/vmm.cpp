#include "vmm.hpp"

#include <cuda.h>
#include <cuda_runtime_api.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <mutex>

namespace st {

namespace {

struct Api {
  bool ok = false;
  decltype(&cuMemCreate) MemCreate = nullptr;
  decltype(&cuMemRelease) MemRelease = nullptr;
  decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
  decltype(&cuMemAddressFree) MemAddressFree = nullptr;
  decltype(&cuMemMap) MemMap = nullptr;
  decltype(&cuMemUnmap) MemUnmap = nullptr;
  decltype(&cuMemSetAccess) MemSetAccess = nullptr;
  decltype(&cuMemGetAllocationGranularity) MemGetAllocationGranularity = nullptr;
  decltype(&cuMemExportToShareableHandle) MemExportToShareableHandle = nullptr;
  decltype(&cuMemImportFromShareableHandle) MemImportFromShareableHandle = nullptr;
  decltype(&cuGetErrorString) GetErrorString = nullptr;
  decltype(&cuStreamWriteValue32) StreamWriteValue32 = nullptr;  // optional
};

template <class F>
bool load(const char* name, F* out) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qr;
  if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess || !fn) {
    cudaGetLastError();
    return false;
  }
  *out = reinterpret_cast<F>(fn);
  return true;
}

Api& api() {
  static Api a;
  static std::once_flag once;
  std::call_once(once, [] {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
      cudaGetLastError();
      return;
    }
    bool ok = true;
    ok &= load("cuMemCreate", &a.MemCreate);
    ok &= load("cuMemRelease", &a.MemRelease);
    ok &= load("cuMemAddressReserve", &a.MemAddressReserve);
    ok &= load("cuMemAddressFree", &a.MemAddressFree);
    ok &= load("cuMemMap", &a.MemMap);
    ok &= load("cuMemUnmap", &a.MemUnmap);
    ok &= load("cuMemSetAccess", &a.MemSetAccess);
    ok &= load("cuMemGetAllocationGranularity", &a.MemGetAllocationGranularity);
    ok &= load("cuMemExportToShareableHandle", &a.MemExportToShareableHandle);
    ok &= load("cuMemImportFromShareableHandle", &a.MemImportFromShareableHandle);
    ok &= load("cuGetErrorString", &a.GetErrorString);
    load("cuStreamWriteValue32", &a.StreamWriteValue32);
    a.ok = ok;
  });
  return a;
}

std::string cu_err(const char* what, CUresult r) {
  const char* s = nullptr;
  if (api().GetErrorString) api().GetErrorString(r, &s);
  return std::string(what) + ": " + (s ? s : "unknown driver error") + " (" + std::to_string(int(r)) + ")";
}

CUmemAllocationProp props_for(int device) {
  CUmemAllocationProp p;
  std::memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

bool map_rw(CUmemGenericAllocationHandle h, size_t bytes, int device, void** out, std::string* err) {
  Api& a = api();
  CUdeviceptr va = 0;
  CUresult r = a.MemAddressReserve(&va, bytes, 0, 0, 0);
  if (r != CUDA_SUCCESS) {
    if (err) *err = cu_err("cuMemAddressReserve", r);
    return false;
  }
  r = a.MemMap(va, bytes, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    if (err) *err = cu_err("cuMemMap", r);
    a.MemAddressFree(va, bytes);
    return false;
  }
  CUmemAccessDesc acc;
  std::memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = a.MemSetAccess(va, bytes, &acc, 1);
  if (r != CUDA_SUCCESS) {
    if (err) *err = cu_err("cuMemSetAccess", r);
    a.MemUnmap(va, bytes);
    a.MemAddressFree(va, bytes);
    return false;
  }
  *out = reinterpret_cast<void*>(va);
  return true;
}

}  // namespace

bool vmm_available() { return api().ok; }

bool stream_write_u32(void* stream, uint32_t* dev_ptr, uint32_t value) {
  Api& a = api();
  if (!a.StreamWriteValue32) return false;
  return a.StreamWriteValue32(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(dev_ptr), value, 0) == CUDA_SUCCESS;
}

size_t vmm_granularity(int device) {
  if (!api().ok) return 2u << 20;
  CUmemAllocationProp p = props_for(device);
  size_t g = 0;
  if (api().MemGetAllocationGranularity(&g, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || g == 0) g = 2u << 20;
  return g;
}

// Zero-fills fresh memory and returns once that is done.  Not cudaMemset: that runs on the legacy default stream,
// behind whatever the application has queued there, while the first users of the memory (the comm stream, a peer)
// are not ordered against that stream at all.
static void zero_now(void* ptr, size_t bytes) {
  cudaStream_t s = nullptr;
  if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) {
    cudaGetLastError();
    cudaMemset(ptr, 0, bytes);
    cudaDeviceSynchronize();
    return;
  }
  cudaMemsetAsync(ptr, 0, bytes, s);
  cudaStreamSynchronize(s);
  cudaStreamDestroy(s);
}

VmmBlock vmm_alloc(int device, size_t bytes, bool shareable, std::string* err) {
  VmmBlock b;
  b.device = device;
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(device);
  cudaFree(nullptr);  // make sure the primary context exists
  if (shareable && api().ok) {
    size_t g = vmm_granularity(device);
    size_t rounded = (bytes + g - 1) / g * g;
    CUmemAllocationProp p = props_for(device);
    CUmemGenericAllocationHandle h = 0;
    CUresult r = api().MemCreate(&h, rounded, &p, 0);
    if (r == CUDA_SUCCESS) {
      void* ptr = nullptr;
      if (map_rw(h, rounded, device, &ptr, err)) {
        b.ptr = ptr;
        b.bytes = rounded;
        b.handle = h;
        zero_now(ptr, rounded);
        if (prev >= 0) cudaSetDevice(prev);
        return b;
      }
      api().MemRelease(h);
    } else if (err) {
      *err = cu_err("cuMemCreate", r);
    }
    // fall through to the plain allocation
  }
  void* ptr = nullptr;
  cudaError_t e = cudaMalloc(&ptr, bytes);
  if (e != cudaSuccess) {
    if (err) *err = std::string("cudaMalloc: ") + cudaGetErrorString(e);
    if (prev >= 0) cudaSetDevice(prev);
    return b;
  }
  zero_now(ptr, bytes);
  b.ptr = ptr;
  b.bytes = bytes;
  b.plain = true;
  if (prev >= 0) cudaSetDevice(prev);
  return b;
}

int vmm_export_fd(const VmmBlock& b, std::string* err) {
  if (b.plain || !b.handle) {
    if (err) *err = "block is not shareable";
    return -1;
  }
  int fd = -1;
  CUresult r = api().MemExportToShareableHandle(&fd, b.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    if (err) *err = cu_err("cuMemExportToShareableHandle", r);
    return -1;
  }
  return fd;
}

VmmBlock vmm_import_fd(int fd, size_t bytes, int device, std::string* err) {
  VmmBlock b;
  b.device = device;
  b.imported = true;
  if (!api().ok) {
    if (err) *err = "CUDA virtual memory management API not available";
    return b;
  }
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(device);
  cudaFree(nullptr);
  CUmemGenericAllocationHandle h = 0;
  CUresult r = api().MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                  CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) {
    if (err) *err = cu_err("cuMemImportFromShareableHandle", r);
    if (prev >= 0) cudaSetDevice(prev);
    return b;
  }
  void* ptr = nullptr;
  if (!map_rw(h, bytes, device, &ptr, err)) {
    api().MemRelease(h);
    if (prev >= 0) cudaSetDevice(prev);
    return b;
  }
  b.ptr = ptr;
  b.bytes = bytes;
  b.handle = h;
  if (prev >= 0) cudaSetDevice(prev);
  return b;
}

void vmm_free(VmmBlock* b) {
  if (!b->ptr) return;
  if (b->plain) {
    cudaFree(b->ptr);
  } else {
    CUdeviceptr va = reinterpret_cast<CUdeviceptr>(b->ptr);
    api().MemUnmap(va, b->bytes);
    api().MemAddressFree(va, b->bytes);
    api().MemRelease(b->handle);
  }
  *b = VmmBlock();
}

// ---------------------------------------------------------------------------------------------
// AF_UNIX helpers (abstract namespace: no file system entry, vanishes with the process)
// ---------------------------------------------------------------------------------------------
static socklen_t abstract_addr(const std::string& name, sockaddr_un* a) {
  std::memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  size_t len = name.size();
  if (len > sizeof(a->sun_path) - 2) len = sizeof(a->sun_path) - 2;
  a->sun_path[0] = '\0';
  std::memcpy(a->sun_path + 1, name.data(), len);
  return socklen_t(offsetof(sockaddr_un, sun_path) + 1 + len);
}

int unix_listen_abstract(const std::string& name, std::string* err) {
  int fd = ::socket(AF_UNIX, SOCK_STREAM, 0);
  if (fd < 0) {
    if (err) *err = std::string("socket(AF_UNIX): ") + std::strerror(errno);
    return -1;
  }
  sockaddr_un a;
  socklen_t len = abstract_addr(name, &a);
  if (::bind(fd, reinterpret_cast<sockaddr*>(&a), len) < 0 || ::listen(fd, 16) < 0) {
    if (err) *err = std::string("bind/listen @") + name + ": " + std::strerror(errno);
    ::close(fd);
    return -1;
  }
  return fd;
}

int unix_connect_abstract(const std::string& name, int timeout_ms) {
  sockaddr_un a;
  socklen_t len = abstract_addr(name, &a);
  int waited = 0;
  while (true) {
    int fd = ::socket(AF_UNIX, SOCK_STREAM, 0);
    if (fd < 0) return -1;
    if (::connect(fd, reinterpret_cast<sockaddr*>(&a), len) == 0) return fd;
    ::close(fd);
    if (waited >= timeout_ms) return -1;
    ::usleep(10 * 1000);
    waited += 10;
  }
}

bool unix_send_fd(int sock, int fd_to_send, const void* msg, size_t msg_len) {
  struct msghdr mh;
  std::memset(&mh, 0, sizeof(mh));
  struct iovec iov;
  char dummy = 'F';
  iov.iov_base = msg_len ? const_cast<void*>(msg) : static_cast<void*>(&dummy);
  iov.iov_len = msg_len ? msg_len : 1;
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  char ctrl[CMSG_SPACE(sizeof(int))];
  std::memset(ctrl, 0, sizeof(ctrl));
  if (fd_to_send >= 0) {
    mh.msg_control = ctrl;
    mh.msg_controllen = sizeof(ctrl);
    struct cmsghdr* c = CMSG_FIRSTHDR(&mh);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(c), &fd_to_send, sizeof(int));
  }
  ssize_t r;
  do {
    r = ::sendmsg(sock, &mh, MSG_NOSIGNAL);
  } while (r < 0 && errno == EINTR);
  return r == ssize_t(iov.iov_len);
}

bool unix_recv_fd(int sock, int* fd_out, void* msg, size_t msg_len, int timeout_ms) {
  if (fd_out) *fd_out = -1;
  struct pollfd pfd = {sock, POLLIN, 0};
  int pr;
  do {
    pr = ::poll(&pfd, 1, timeout_ms);
  } while (pr < 0 && errno == EINTR);
  if (pr <= 0) return false;
  struct msghdr mh;
  std::memset(&mh, 0, sizeof(mh));
  struct iovec iov;
  char dummy;
  iov.iov_base = msg_len ? msg : static_cast<void*>(&dummy);
  iov.iov_len = msg_len ? msg_len : 1;
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  char ctrl[CMSG_SPACE(sizeof(int))];
  mh.msg_control = ctrl;
  mh.msg_controllen = sizeof(ctrl);
  ssize_t r;
  do {
    r = ::recvmsg(sock, &mh, MSG_WAITALL);
  } while (r < 0 && errno == EINTR);
  if (r != ssize_t(iov.iov_len)) return false;
  for (struct cmsghdr* c = CMSG_FIRSTHDR(&mh); c; c = CMSG_NXTHDR(&mh, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS && fd_out) std::memcpy(fd_out, CMSG_DATA(c), sizeof(int));
  }
  return true;
}

}  // namespace st
