// Pieces shared by the pybind11 shims: the duck-typed tensor view that mirrors
// include/pyutils/pyutils.cuh:14-47 (class name "Tensor", contiguous, not on the CPU, ndim <= 4, data_ptr();
// no libtorch is linked) with the reference's RuntimeError texts, and the error-code translation.
#pragma once

#include <pybind11/pybind11.h>

#include <array>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/hk_attn.h"

namespace hk_shim {

namespace py = pybind11;

struct TensorView {
  uint64_t ptr = 0;
  std::array<int, 4> shape{1, 1, 1, 1};  // left-padded with 1s, like make_gl's (b, d, r, c)
  int device = 0;
  std::string dtype;
};

inline TensorView view_of(const py::object& obj) {
  if (py::hasattr(obj, "__class__") && obj.attr("__class__").attr("__name__").cast<std::string>() == "Tensor") {
    if (!obj.attr("is_contiguous")().cast<bool>()) throw std::runtime_error("Tensor must be contiguous");
    if (obj.attr("device").attr("type").cast<std::string>() == "cpu")
      throw std::runtime_error("Tensor must be on CUDA device");
    TensorView t;
    auto shape = obj.attr("shape").cast<py::tuple>();
    const size_t dims = shape.size();
    if (dims > 4) throw std::runtime_error("Expected Tensor.ndim <= 4");
    for (size_t i = 0; i < dims; ++i) t.shape[4 - dims + i] = shape[i].cast<int>();
    t.ptr = obj.attr("data_ptr")().cast<uint64_t>();
    py::object idx = obj.attr("device").attr("index");
    t.device = idx.is_none() ? -1 : idx.cast<int>();
    t.dtype = py::str(obj.attr("dtype")).cast<std::string>();
    return t;
  }
  throw std::runtime_error("Expected a torch.Tensor");
}

inline void require(bool cond, const std::string& msg) {
  if (!cond) throw std::runtime_error(msg);
}

inline void raise_for(int rc, const char* what) {
  if (rc == HK_OK) return;
  std::string msg = std::string(what) + ": " + hk_strerror(rc);
  if (rc == HK_ECUDA || rc == HK_EUNSUPPORTED) {
    const char* detail = hk_last_cuda_error();
    if (detail && detail[0]) msg += std::string(" (") + detail + ")";
  }
  throw std::runtime_error(msg);
}

}  // namespace hk_shim
