// Peer-shareable device memory: CUDA virtual-memory-management allocations that can be exported as a
// POSIX file descriptor, sent to another process over an AF_UNIX socket (SCM_RIGHTS) and mapped there.
// This is the transport under the GPU edges: ring slots, flags and credit words of an edge live in such
// allocations and the neighbour stores into them over NVLink.  The reference's transport is a TCP
// socket per edge (src/sharedtensor.c:244-332); it stays available for cross-host edges.
//
// The driver API is reached through cudaGetDriverEntryPoint, so the module loads on machines without
// a driver (the build machine has no GPU).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

namespace st {

struct VmmBlock {
  void* ptr = nullptr;        // mapped address in this process
  size_t bytes = 0;           // mapped size (granularity-rounded)
  uint64_t handle = 0;        // CUmemGenericAllocationHandle
  int device = -1;            // device that owns the physical memory
  bool imported = false;
  bool plain = false;         // cudaMalloc fallback (not shareable)
};

// Allocates `bytes` of zero-filled device memory on `device`, mapped read/write for `device`.
// shareable=false or an unavailable driver API falls back to cudaMalloc (plain=true).
VmmBlock vmm_alloc(int device, size_t bytes, bool shareable, std::string* err);
// Exports the block as a file descriptor (caller closes it).  -1 on failure.
int vmm_export_fd(const VmmBlock& b, std::string* err);
// Maps a block exported by another process (or this one) for access from `device`.
VmmBlock vmm_import_fd(int fd, size_t bytes, int device, std::string* err);
void vmm_free(VmmBlock* b);
bool vmm_available();
// Writes one word of device memory in stream order without occupying an SM (cuStreamWriteValue32).  False if the
// driver does not offer it; the caller then uses a one-thread kernel.
bool stream_write_u32(void* stream, uint32_t* dev_ptr, uint32_t value);
size_t vmm_granularity(int device);

// fd passing
int unix_listen_abstract(const std::string& name, std::string* err);  // returns listening fd
int unix_connect_abstract(const std::string& name, int timeout_ms);   // returns fd or -1
bool unix_send_fd(int sock, int fd_to_send, const void* msg, size_t msg_len);
bool unix_recv_fd(int sock, int* fd_out, void* msg, size_t msg_len, int timeout_ms);

}  // namespace st
