// GPU node: tree membership (TCP join, wire-compatible with the reference) plus the upgrade of
// same-host edges to peer-memory rings.  See gpu_node.cpp.
#pragma once
#include <pybind11/pybind11.h>

void bind_gpu_node(pybind11::module_& m);
