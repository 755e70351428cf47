// Python bindings of the two kinds of GPU node (gpu_node.hpp: tree member, gpu_mesh_node.hpp: member of a fixed,
// fully connected group).
#include "gpu_mesh_node.hpp"
#include "gpu_node.hpp"

void bind_gpu_node(pybind11::module_& m) {
  namespace py = pybind11;
  using namespace st;
  py::class_<GpuNodeOptions>(m, "GpuNodeOptions")
      .def(py::init<>())
      .def_readwrite("rejoin", &GpuNodeOptions::rejoin)
      .def_readwrite("rejoin_backoff_ms", &GpuNodeOptions::rejoin_backoff_ms)
      .def_readwrite("upgrade_timeout_ms", &GpuNodeOptions::upgrade_timeout_ms)
      .def_readwrite("listen_backlog", &GpuNodeOptions::listen_backlog)
      .def_readwrite("start_engine", &GpuNodeOptions::start_engine);
  py::class_<GpuNode>(m, "GpuNode")
      .def(py::init<int, int64_t, const GpuConfig&, const GpuNodeOptions&>())
      .def("replica", &GpuNode::replica, py::return_value_policy::reference_internal)
      .def(
          "start",
          [](GpuNode& n, const std::string& host, int port, uintptr_t init, uintptr_t stream) {
            py::gil_scoped_release rel;
            n.start(host, port, reinterpret_cast<const float*>(init), reinterpret_cast<void*>(stream));
          },
          py::arg("host"), py::arg("port"), py::arg("init") = 0, py::arg("stream") = 0)
      .def("wait_ready",
           [](GpuNode& n, int ms) {
             py::gil_scoped_release rel;
             return n.wait_ready(ms);
           })
      .def("is_master", &GpuNode::is_master)
      .def("stats", &GpuNode::stats)
      .def("inject_sever", &GpuNode::inject_sever)
      .def("close", [](GpuNode& n) {
        py::gil_scoped_release rel;
        n.close();
      });
  py::class_<GpuMeshNode>(m, "GpuMeshNode")
      .def(py::init<int, int64_t, const GpuConfig&, int, int, bool>())
      .def("replica", &GpuMeshNode::replica, py::return_value_policy::reference_internal)
      .def(
          "start",
          [](GpuMeshNode& n, const std::string& host, int port, uintptr_t init, uintptr_t stream, int timeout_ms) {
            py::gil_scoped_release rel;
            n.start(host, port, reinterpret_cast<const float*>(init), reinterpret_cast<void*>(stream), timeout_ms);
          },
          py::arg("host"), py::arg("port"), py::arg("init") = 0, py::arg("stream") = 0, py::arg("timeout_ms") = 60000)
      .def("members_alive", &GpuMeshNode::members_alive)
      .def("dropped", &GpuMeshNode::dropped)
      .def("close", [](GpuMeshNode& n) {
        py::gil_scoped_release rel;
        n.close();
      });
}
