// Python bindings of the host-side core: codec, tree join helpers, CPU replica node.
// Tensors cross this boundary as raw addresses (tensor.data_ptr()) plus element counts; the Python
// veneer checks dtype, contiguity and size before calling in.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "codec.hpp"
#include "node.hpp"
#include "tree.hpp"

namespace py = pybind11;
using namespace st;

template <class T>
static T* ptr(uintptr_t p) {
  return reinterpret_cast<T*>(p);
}

static py::dict edge_stats_dict(const EdgeStats& e) {
  py::dict d;
  static const char* names[] = {"free", "connected", "dead"};
  d["state"] = names[e.state];
  d["peer"] = e.peer;
  d["frames_sent"] = e.frames_sent;
  d["frames_recv"] = e.frames_recv;
  d["noop_sent"] = e.noop_sent;
  d["noop_recv"] = e.noop_recv;
  d["bytes_sent"] = e.bytes_sent;
  d["bytes_recv"] = e.bytes_recv;
  d["last_scale_sent"] = e.last_scale_sent;
  d["last_scale_recv"] = e.last_scale_recv;
  d["residual_rms"] = e.residual_rms;
  d["dropped_by_injection"] = e.dropped_by_injection;
  return d;
}

void bind_core(py::module_& m) {
  m.attr("SLOT_UP") = kSlotUp;
  m.attr("SLOT_LEFT") = kSlotLeft;
  m.attr("SLOT_RIGHT") = kSlotRight;

  // ---- codec ----
  m.def("sign_bytes", &sign_bytes);
  m.def("block_words", &block_words);
  m.def("block_scales", &block_scales);
  m.def("ref_scale_of", [](uintptr_t r, size_t n) { return ref_scale_of(ptr<float>(r), n); });
  m.def("encode_residual_ref",
        [](uintptr_t r, size_t n, uintptr_t bits) { return encode_residual_ref(ptr<float>(r), n, ptr<uint8_t>(bits)); });
  m.def(
      "encode_tensor",
      [](uintptr_t v, uintptr_t k, size_t n, uintptr_t bits, float min_scale, int rule) {
        return encode_tensor(ptr<float>(v), ptr<float>(k), n, ptr<uint8_t>(bits), min_scale, rule);
      },
      py::arg("v"), py::arg("k"), py::arg("n"), py::arg("bits"), py::arg("min_scale"), py::arg("rule") = 1);
  m.def("decode_tensor_add", [](uintptr_t bits, float scale, size_t n, uintptr_t dst, uintptr_t dst2) {
    decode_tensor_add(ptr<uint8_t>(bits), scale, n, ptr<float>(dst), dst2 ? ptr<float>(dst2) : nullptr);
  });
  m.def("encode_tensor_fast", [](uintptr_t v, uintptr_t k, size_t n, uintptr_t bits, float min_abs, float min_rel) {
    return encode_tensor_fast(ptr<float>(v), ptr<float>(k), n, ptr<uint8_t>(bits), min_abs, min_rel);
  });
  m.def("decode_tensor_add_fast", [](uintptr_t bits, float scale, size_t n, uintptr_t dst, uintptr_t dst2) {
    decode_tensor_add_fast(ptr<uint8_t>(bits), scale, n, ptr<float>(dst), dst2 ? ptr<float>(dst2) : nullptr);
  });
  m.def("encode_block_fast", [](uintptr_t v, uintptr_t k, size_t n, int block, int min_exp, int rel_bits, uintptr_t words,
                                uintptr_t scales) {
    BlockGate g;
    g.min_exp = min_exp;
    g.rel_bits = rel_bits;
    return encode_block_fast(ptr<float>(v), ptr<float>(k), n, block, g, ptr<uint32_t>(words), ptr<uint8_t>(scales));
  });
  m.def("decode_block_add_fast", [](uintptr_t words, uintptr_t scales, size_t n, int block, uintptr_t dst, uintptr_t dst2) {
    decode_block_add_fast(ptr<uint32_t>(words), ptr<uint8_t>(scales), n, block, ptr<float>(dst),
                          dst2 ? ptr<float>(dst2) : nullptr);
  });
  m.def("encode_block", [](uintptr_t v, uintptr_t k, size_t n, int block, int min_exp, int rel_bits, uintptr_t words,
                           uintptr_t scales) {
    BlockGate g;
    g.min_exp = min_exp;
    g.rel_bits = rel_bits;
    return encode_block(ptr<float>(v), ptr<float>(k), n, block, g, ptr<uint32_t>(words), ptr<uint8_t>(scales));
  });
  m.def("decode_block_add", [](uintptr_t words, uintptr_t scales, size_t n, int block, uintptr_t dst, uintptr_t dst2) {
    decode_block_add(ptr<uint32_t>(words), ptr<uint8_t>(scales), n, block, ptr<float>(dst),
                     dst2 ? ptr<float>(dst2) : nullptr);
  });
  m.def("encode_block_int", [](uintptr_t v, uintptr_t k, size_t n, int block, int min_exp, int rel_bits, int bits, uintptr_t codes,
                               uintptr_t scales) {
    if (bits != 2 && bits != 4 && bits != 8) throw std::invalid_argument("integer frames have 2, 4 or 8 bits per element");
    BlockGate g;
    g.min_exp = min_exp;
    g.rel_bits = rel_bits;
    return encode_block_int(ptr<float>(v), ptr<float>(k), n, block, g, bits, ptr<uint8_t>(codes), ptr<uint8_t>(scales));
  });
  m.def("encode_block_int8_fast", [](uintptr_t v, uintptr_t k, size_t n, int block, int min_exp, int rel_bits, uintptr_t codes,
                                     uintptr_t scales) {
    BlockGate g;
    g.min_exp = min_exp;
    g.rel_bits = rel_bits;
    return encode_block_int8_fast(ptr<float>(v), ptr<float>(k), n, block, g, ptr<uint8_t>(codes), ptr<uint8_t>(scales));
  });
  m.def("decode_block_int_add", [](uintptr_t codes, uintptr_t scales, size_t n, int block, int bits, float sign, uintptr_t dst,
                                   uintptr_t dst2) {
    decode_block_int_add(ptr<uint8_t>(codes), ptr<uint8_t>(scales), n, block, bits, sign, ptr<float>(dst),
                         dst2 ? ptr<float>(dst2) : nullptr);
  });
  m.def("decode_block_int8_add_fast", [](uintptr_t codes, uintptr_t scales, size_t n, int block, float sign, uintptr_t dst,
                                         uintptr_t dst2) {
    decode_block_int8_add_fast(ptr<uint8_t>(codes), ptr<uint8_t>(scales), n, block, sign, ptr<float>(dst),
                               dst2 ? ptr<float>(dst2) : nullptr);
  });
  m.def("block_int_steps", [](uintptr_t codes, uintptr_t scales, size_t n, int block, int bits, uintptr_t steps) {
    block_int_steps(ptr<uint8_t>(codes), ptr<uint8_t>(scales), n, block, bits, ptr<float>(steps));
  });
  m.def("block_sign_steps", [](uintptr_t words, uintptr_t scales, size_t n, int block, uintptr_t steps) {
    block_sign_steps(ptr<uint32_t>(words), ptr<uint8_t>(scales), n, block, ptr<float>(steps));
  });
  m.def("block_code_int", [](float xmax, uint32_t vmax_bits, int min_exp, int rel_bits, int bits) {
    BlockGate g;
    g.min_exp = min_exp;
    g.rel_bits = rel_bits;
    return block_code_int(xmax, vmax_bits, g, bits);
  });
  m.def("pack_tile_codes", [](uintptr_t codes, int bits, uintptr_t out) { pack_tile_codes(ptr<uint8_t>(codes), bits, ptr<uint32_t>(out)); });
  m.def("segment_sumsq", [](uintptr_t x, std::vector<int64_t> offsets) {
    std::vector<double> out(offsets.size() - 1);
    segment_sumsq(ptr<float>(x), offsets.data(), int(out.size()), out.data());
    return out;
  });

  // ---- tree join (exposed for protocol tests) ----
  m.def(
      "join_tree",
      [](const std::string& host, int port) {
        JoinResult r;
        {
          py::gil_scoped_release rel;
          r = join_tree(host, port, nullptr);
        }
        py::dict d;
        d["ok"] = r.ok;
        d["master"] = r.master;
        d["fd"] = r.fd;
        d["hops"] = r.hops;
        d["error"] = r.error;
        if (r.ok) d["listen_addr"] = addr_to_string(r.listen_addr);
        if (r.ok && !r.master) d["parent_addr"] = addr_to_string(r.parent_addr);
        return d;
      },
      "Walks the join protocol; returns the connected up socket's fd (caller owns it).");

  // ---- CPU node ----
  py::class_<NodeConfig>(m, "NodeConfig")
      .def(py::init<>())
      .def_readwrite("tcp_block", &NodeConfig::tcp_block)
      .def_readwrite("tcp_bits", &NodeConfig::tcp_bits)
      .def_readwrite("tcp_rule", &NodeConfig::tcp_rule)
      .def_readwrite("min_scale_abs", &NodeConfig::min_scale_abs)
      .def_readwrite("min_scale_rel", &NodeConfig::min_scale_rel)
      .def_readwrite("max_frames_per_s", &NodeConfig::max_frames_per_s)
      .def_readwrite("idle_keepalive_ms", &NodeConfig::idle_keepalive_ms)
      .def_readwrite("listen_backlog", &NodeConfig::listen_backlog)
      .def_readwrite("ready_mode", &NodeConfig::ready_mode)
      .def_readwrite("ready_bits", &NodeConfig::ready_bits)
      .def_readwrite("ready_timeout_ms", &NodeConfig::ready_timeout_ms)
      .def_readwrite("rejoin", &NodeConfig::rejoin)
      .def_readwrite("rejoin_backoff_ms", &NodeConfig::rejoin_backoff_ms)
      .def_property(
          "gate_min_exp", [](const NodeConfig& c) { return c.gate.min_exp; },
          [](NodeConfig& c, int v) { c.gate.min_exp = v; })
      .def_property(
          "gate_rel_bits", [](const NodeConfig& c) { return c.gate.rel_bits; },
          [](NodeConfig& c, int v) { c.gate.rel_bits = v; });

  py::class_<CpuNode>(m, "CpuNode")
      .def(py::init<int64_t, const NodeConfig&>())
      .def(
          "start",
          [](CpuNode& n, const std::string& host, int port, uintptr_t init) {
            py::gil_scoped_release rel;
            n.start(host, port, init ? ptr<float>(init) : nullptr);
          },
          py::arg("host"), py::arg("port"), py::arg("init") = 0)
      .def("wait_ready",
           [](CpuNode& n, int timeout_ms) {
             py::gil_scoped_release rel;
             return n.wait_ready(timeout_ms);
           })
      .def("add",
           [](CpuNode& n, uintptr_t d, int64_t count) {
             py::gil_scoped_release rel;
             n.add(ptr<float>(d), count);
           })
      .def("sub_add",
           [](CpuNode& n, uintptr_t a, uintptr_t b, int64_t count) {
             py::gil_scoped_release rel;
             n.sub_add(ptr<float>(a), ptr<float>(b), count);
           })
      .def("copy_to",
           [](CpuNode& n, uintptr_t out, int64_t count) {
             py::gil_scoped_release rel;
             n.copy_to(ptr<float>(out), count);
           })
      .def("import_values",
           [](CpuNode& n, uintptr_t v, int64_t count) {
             py::gil_scoped_release rel;
             n.import_values(ptr<float>(v), count);
           })
      .def("export_state",
           [](CpuNode& n) {
             std::vector<float> v;
             std::vector<float> mir[kNumSlots];
             n.export_state(&v, mir);
             py::dict d;
             d["values"] = py::bytes(reinterpret_cast<const char*>(v.data()), v.size() * 4);
             static const char* names[] = {"up", "left", "right"};
             for (int s = 0; s < kNumSlots; s++)
               if (!mir[s].empty())
                 d[names[s]] = py::bytes(reinterpret_cast<const char*>(mir[s].data()), mir[s].size() * 4);
             return d;
           })
      .def("flush",
           [](CpuNode& n, int timeout_ms, int quiet_ms) {
             py::gil_scoped_release rel;
             return n.flush(timeout_ms, quiet_ms);
           },
           py::arg("timeout_ms") = 10000, py::arg("quiet_ms") = 50)
      .def("close",
           [](CpuNode& n) {
             py::gil_scoped_release rel;
             n.close();
           })
      .def("size", &CpuNode::size)
      .def("is_master", &CpuNode::is_master)
      .def("inject_drop_frames", &CpuNode::inject_drop_frames)
      .def("inject_sever", &CpuNode::inject_sever)
      .def("stats", [](CpuNode& n) {
        NodeStats s = n.stats();
        py::dict d;
        d["master"] = s.master;
        d["ready"] = s.ready;
        d["closed"] = s.closed;
        d["n"] = s.n;
        d["listen_addr"] = s.listen_addr;
        d["adds"] = s.adds;
        d["copies"] = s.copies;
        d["redirects"] = s.redirects;
        d["rejoins"] = s.rejoins;
        d["edge_failures"] = s.edge_failures;
        py::list evs;
        for (const NodeEvent& ev : s.events) {
          py::dict e1;
          e1["ms"] = ev.ms;
          e1["kind"] = ev.kind;
          e1["detail"] = ev.detail;
          evs.append(e1);
        }
        d["events"] = evs;
        py::dict e;
        e["up"] = edge_stats_dict(s.edge[kSlotUp]);
        e["left"] = edge_stats_dict(s.edge[kSlotLeft]);
        e["right"] = edge_stats_dict(s.edge[kSlotRight]);
        d["edges"] = e;
        return d;
      });
}

PYBIND11_MODULE(_core, m) {
  m.doc() = "sharedtensor_b200 host-side core (codec, tree join, CPU replica node)";
  bind_core(m);
}
