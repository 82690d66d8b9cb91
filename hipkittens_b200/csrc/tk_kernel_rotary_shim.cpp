// pybind11 shim for the reference's rotary module on top of the C ABI in hk_attn.h:
//   tk_kernel.dispatch_rotary(x, o, sin, cos)      (kernels/rotary/kernel.cpp:90-98; note the order: sin before cos)
// x, o [B, H, N, D] bf16, sin / cos [N, D/2] bf16 (kernels/rotary/test_python.py:17,36-45). Same duck-typed tensors and
// RuntimeError texts as the other shims; asynchronous on the null stream like the reference's dispatcher
// (kernel.cpp:83-88), with an optional `stream=` keyword.
#include <pybind11/pybind11.h>

#include "../../include/hk_attn.h"
#include "shim_common.h"

namespace py = pybind11;

namespace {

using namespace hk_shim;

void dispatch_rotary(py::object x_, py::object o_, py::object sin_, py::object cos_, py::object stream) {
  const TensorView x = view_of(x_), o = view_of(o_), sn = view_of(sin_), cs = view_of(cos_);
  require(x.dtype == "torch.bfloat16" && o.dtype == "torch.bfloat16" && sn.dtype == "torch.bfloat16" &&
              cs.dtype == "torch.bfloat16",
          "x, o, sin and cos must be torch.bfloat16");
  require(o.shape == x.shape, "o must have x's shape [B, H, N, D]");
  const int B = x.shape[0], H = x.shape[1], N = x.shape[2], D = x.shape[3];
  require(sn.shape == cs.shape && sn.shape[0] == 1 && sn.shape[1] == 1 && sn.shape[2] == N && 2 * sn.shape[3] <= D,
          "sin and cos must be [N, R/2] with R <= D");
  require(x.device == o.device && x.device == sn.device && x.device == cs.device,
          "all tensors must be on the same device");
  void* cu_stream = stream.is_none() ? nullptr : reinterpret_cast<void*>(stream.cast<uint64_t>());
  raise_for(hk_rotary(reinterpret_cast<const void*>(x.ptr), reinterpret_cast<void*>(o.ptr),
                      reinterpret_cast<const void*>(sn.ptr), reinterpret_cast<const void*>(cs.ptr), B, H, N, D,
                      2 * sn.shape[3], x.device, cu_stream),
            "dispatch_rotary");
}

}  // namespace

PYBIND11_MODULE(tk_kernel, m) {
  m.doc() = "tk_kernel python module (rotary, B200 build)";
  m.def("dispatch_rotary", &dispatch_rotary, py::arg("x"), py::arg("o"), py::arg("sin"), py::arg("cos"),
        py::arg("stream") = py::none());
}
