// Python bindings of the CUDA side: the GPU replica/engine, the peer-memory helpers and the raw kernel
// launchers (the latter for kernel-level tests and benchmarks).  Pointers and streams cross as integers.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cuda_runtime_api.h>

#include "../core/codec.hpp"
#include "engine.hpp"
#include "round.h"
#include "vmm.hpp"

namespace py = pybind11;
using namespace st;

template <class T>
static T* ptr(uintptr_t p) {
  return reinterpret_cast<T*>(p);
}
static void* strm(uintptr_t s) { return reinterpret_cast<void*>(s); }
static void ck(int e, const char* what) {
  if (e != 0) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(cudaError_t(e)));
}

void bind_gpu_node(py::module_& m);

PYBIND11_MODULE(_cuda, m) {
  m.doc() = "sharedtensor_b200 sm_100a kernels, peer-memory transport and GPU engine";
  m.attr("TILE") = kTile;
  m.attr("MAX_LINKS") = kMaxLinks;
  m.attr("MAX_RINGS") = kMaxRings;
  m.attr("STATUS_WORDS") = int(kStWords);
  m.attr("TRACE_ENTRIES") = int(kTraceEntries);
  m.attr("TRACE_WORDS") = int(kTraceWords);
  m.def("status_names", [] {
    return std::vector<std::string>{"rounds", "tiles_processed", "frames_sent", "frames_recv", "blocked_no_credit", "errors",
                                    "last_work_count", "residual_max0", "residual_max1", "residual_max2", "pending_tiles",
                                    "wait_timeouts"};
  });
  m.def("vmm_available", &vmm_available);
  m.def("memcpy_d2d", [](uintptr_t dst, uintptr_t src, size_t bytes) {
    ck(int(cudaMemcpy(ptr<void>(dst), ptr<void>(src), bytes, cudaMemcpyDeviceToDevice)), "cudaMemcpy");
  });

  // ---- raw kernels ----
  m.def("snapshot_f32", [](uintptr_t v, uintptr_t out, int64_t n, uintptr_t s) {
    ck(launch_snapshot_f32(ptr<float>(v), ptr<float>(out), n, strm(s)), "snapshot_f32");
  });
  m.def("snapshot_bf16", [](uintptr_t v, uintptr_t out, int64_t n, uintptr_t s) {
    ck(launch_snapshot_bf16(ptr<float>(v), ptr<void>(out), n, strm(s)), "snapshot_bf16");
  });
  m.def("add", [](uintptr_t v, uintptr_t d, int64_t n, bool atomic, uintptr_t s) {
    ck(launch_add(ptr<float>(v), ptr<float>(d), n, atomic, strm(s)), "add");
  });
  m.def("sub_add", [](uintptr_t v, uintptr_t a, uintptr_t b, int64_t n, bool atomic, uintptr_t s) {
    ck(launch_sub_add(ptr<float>(v), ptr<float>(a), ptr<float>(b), n, atomic, strm(s)), "sub_add");
  });
  m.def("add_scaled_bf16", [](uintptr_t v, uintptr_t g, float alpha, int64_t n, bool atomic, uintptr_t s) {
    ck(launch_add_scaled_bf16(ptr<float>(v), ptr<void>(g), alpha, n, atomic, strm(s)), "add_scaled_bf16");
  });
  m.def("round_smem_bytes", &round_smem_bytes);
  m.def("table_scales_scratch_doubles", &table_scales_scratch_doubles);
  m.def("table_scales", [](uintptr_t x, uintptr_t offsets, int n_seg, int64_t n_total, uintptr_t scratch, uintptr_t out_sumsq,
                           uintptr_t out_exp, uintptr_t s) {
    ck(launch_table_scales(ptr<float>(x), ptr<int64_t>(offsets), n_seg, n_total, ptr<double>(scratch), ptr<double>(out_sumsq),
                           ptr<int8_t>(out_exp), strm(s)),
       "table_scales");
  });
  m.def("sample_sqerr", [](uintptr_t a, int64_t stride, uintptr_t b, int64_t count, uintptr_t out, uintptr_t s) {
    ck(launch_sample_sqerr(ptr<float>(a), stride, ptr<float>(b), count, ptr<double>(out), strm(s)), "sample_sqerr");
  });
  m.def("probe_converged", [](uintptr_t a, int64_t stride, uintptr_t b, int64_t count, double threshold, uintptr_t scratch, uintptr_t stamp,
                              uintptr_t last_err, uintptr_t s) {
    ck(launch_probe_converged(ptr<float>(a), stride, ptr<float>(b), count, threshold, ptr<double>(scratch), ptr<uint64_t>(stamp),
                              ptr<double>(last_err), strm(s)),
       "probe_converged");
  });
  m.def("stamp", [](uintptr_t out, uintptr_t s) { ck(launch_stamp(ptr<uint64_t>(out), strm(s)), "stamp"); });
  m.def("delay", [](uint64_t ns, uintptr_t s) { ck(launch_delay(ns, strm(s)), "delay"); });
  m.def("tensor_maxabs", [](uintptr_t v, uintptr_t k, int64_t n, uintptr_t out2, uintptr_t s) {
    ck(launch_tensor_maxabs(ptr<float>(v), ptr<float>(k), n, ptr<uint32_t>(out2), strm(s)), "tensor_maxabs");
  });
  m.def("tensor_encode", [](uintptr_t v, uintptr_t k, int64_t n, float scale, uintptr_t words, uintptr_t s) {
    ck(launch_tensor_encode(ptr<float>(v), ptr<float>(k), n, scale, ptr<uint32_t>(words), strm(s)), "tensor_encode");
  });
  m.def("tensor_decode", [](uintptr_t words, float scale, int64_t n, uintptr_t v, uintptr_t k, uintptr_t s) {
    ck(launch_tensor_decode(ptr<uint32_t>(words), scale, n, ptr<float>(v), k ? ptr<float>(k) : nullptr, 0, strm(s)), "tensor_decode");
  });

  // ---- GPU replica ----
  py::class_<GpuConfig>(m, "GpuConfig")
      .def(py::init<>())
      .def_readwrite("block", &GpuConfig::block)
      .def_readwrite("ring_slots", &GpuConfig::ring_slots)
      .def_readwrite("min_exp", &GpuConfig::min_exp)
      .def_readwrite("rel_bits", &GpuConfig::rel_bits)
      .def_readwrite("comm_ctas", &GpuConfig::comm_ctas)
      .def_readwrite("shareable", &GpuConfig::shareable)
      .def_readwrite("rounds_in_flight", &GpuConfig::rounds_in_flight)
      .def_readwrite("idle_sleep_us", &GpuConfig::idle_sleep_us)
      .def_readwrite("round_interval_us", &GpuConfig::round_interval_us)
      .def_readwrite("bits", &GpuConfig::bits)
      .def_readwrite("sweeps", &GpuConfig::sweeps)
      .def_readwrite("poll_deadline_us", &GpuConfig::poll_deadline_us)
      .def_readwrite("shape", &GpuConfig::shape)
      .def_readwrite("yield_to_updates", &GpuConfig::yield_to_updates)
      .def_readwrite("comm_high_priority", &GpuConfig::comm_high_priority)
      .def_readwrite("chunk_tiles", &GpuConfig::chunk_tiles)
      .def_readwrite("window_tiles", &GpuConfig::window_tiles);

  py::class_<GpuReplica>(m, "GpuReplica")
      .def(py::init<int, int64_t, const GpuConfig&>())
      .def("size", &GpuReplica::size)
      .def("padded", &GpuReplica::padded)
      .def("tiles", &GpuReplica::tiles)
      .def("values_ptr", [](GpuReplica& r) { return reinterpret_cast<uintptr_t>(r.values()); })
      .def("mirror_ptr", [](GpuReplica& r, int link) { return reinterpret_cast<uintptr_t>(r.mirror(link)); })
      .def("comm_stream", [](GpuReplica& r) { return reinterpret_cast<uintptr_t>(r.comm_stream()); })
      .def("edge_layout",
           [](GpuReplica& r) {
             EdgeBlockLayout l = r.edge_layout();
             py::dict d;
             d["off_payload"] = l.off_payload;
             d["off_flags"] = l.off_flags;
             d["off_credit"] = l.off_credit;
             d["bytes"] = l.bytes;
             return d;
           })
      .def("add_link", &GpuReplica::add_link)
      .def("remove_link", &GpuReplica::remove_link)
      .def("alloc_edge_block", &GpuReplica::alloc_edge_block)
      .def("free_edge_block", &GpuReplica::free_edge_block)
      .def("edge_block_ptr", [](GpuReplica& r, int id) { return reinterpret_cast<uintptr_t>(r.edge_block(id).ptr); })
      .def("edge_block_is_vmm", [](GpuReplica& r, int id) { return !r.edge_block(id).plain; })
      .def("attach_peer", [](GpuReplica& r, int link, int block, uintptr_t remote) { return r.attach_peer(link, block, ptr<void>(remote)); })
      .def("detach_peer", &GpuReplica::detach_peer)
      .def("unsend_unacknowledged", &GpuReplica::unsend_unacknowledged)
      .def("n_links", &GpuReplica::n_links)
      .def("n_peers", &GpuReplica::n_peers)
      .def("load_values", [](GpuReplica& r, uintptr_t src, uintptr_t s) { r.load_values(ptr<float>(src), strm(s)); })
      .def("add", [](GpuReplica& r, uintptr_t d, uintptr_t s) { r.add(ptr<float>(d), strm(s)); })
      .def("sub_add", [](GpuReplica& r, uintptr_t a, uintptr_t b, uintptr_t s) { r.sub_add(ptr<float>(a), ptr<float>(b), strm(s)); })
      .def("add_scaled_bf16", [](GpuReplica& r, uintptr_t g, float alpha, uintptr_t s) { r.add_scaled_bf16(ptr<void>(g), alpha, strm(s)); })
      .def("snapshot", [](GpuReplica& r, uintptr_t out, uintptr_t s) { r.snapshot(ptr<float>(out), strm(s)); })
      .def("snapshot_bf16", [](GpuReplica& r, uintptr_t out, uintptr_t s) { r.snapshot_bf16(ptr<void>(out), strm(s)); })
      .def("copy_mirror_from_values", &GpuReplica::copy_mirror_from_values)
      .def("round", &GpuReplica::round, py::arg("do_rx") = true, py::arg("do_tx") = true, py::arg("sweeps") = 1)
      .def("set_test_stall_tile", &GpuReplica::set_test_stall_tile)
      .def("check_guards", [](GpuReplica& r) { py::gil_scoped_release rel; return r.check_guards(); })
      .def("bits", &GpuReplica::bits)
      .def("debug_crumbs", &GpuReplica::debug_crumbs)
      .def("sync", [](GpuReplica& r) { py::gil_scoped_release rel; r.sync(); })
      .def("start_engine", &GpuReplica::start_engine)
      .def("stop_engine", [](GpuReplica& r) { py::gil_scoped_release rel; r.stop_engine(); })
      .def("engine_running", &GpuReplica::engine_running)
      .def("status", [](GpuReplica& r) { py::gil_scoped_release rel; return r.status(); })
      .def("launches", &GpuReplica::launches)
      .def("last_error", &GpuReplica::last_error);

  bind_gpu_node(m);
}
