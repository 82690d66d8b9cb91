// pybind11 shim that keeps the reference's Python calling surface on top of the C ABI in hk_attn.h.
//
// Mirrors include/pyutils/pyutils.cuh:14-47 (from_object<gl>): arguments arrive as generic Python
// objects, are duck-typed as torch.Tensor (class name "Tensor", contiguous, not on the CPU, ndim <= 4,
// data_ptr()), and no libtorch is linked. The same RuntimeError messages are raised for the same
// conditions. Beyond the reference it also checks dtypes and that the five shapes agree, because the
// shapes are run-time arguments here rather than compile-time macros (kernels/attn/gqa/kernel.cpp:4-24).
//
// Build-time switches (one source, several modules, like the reference's one-.cpp-per-directory):
//   HK_MODULE_NAME      tk_kernel | tk_kernel_fwd          (kernel.cpp:583, attn_fwd_causal.cpp:632)
//   HK_ENTRY_NAME       "dispatch_micro" | "dispatch_fwd"
//   HK_DEFAULT_CAUSAL   0 | 1   causality was "which directory you built" in the reference
//   HK_SYNC_AFTER       0 | 1   dispatch_fwd blocks on the device (attn_fwd_causal.cpp:625-630)
#include <pybind11/pybind11.h>

#include <array>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/hk_attn.h"
#include "shim_common.h"

namespace py = pybind11;

#ifndef HK_MODULE_NAME
#define HK_MODULE_NAME tk_kernel
#endif
#ifndef HK_ENTRY_NAME
#define HK_ENTRY_NAME "dispatch_micro"
#endif
#ifndef HK_DEFAULT_CAUSAL
#define HK_DEFAULT_CAUSAL 0
#endif
#ifndef HK_SYNC_AFTER
#define HK_SYNC_AFTER 0
#endif

namespace {

using namespace hk_shim;

void dispatch(py::object q_, py::object k_, py::object v_, py::object o_, py::object l_, py::object causal,
              py::object softmax_scale, py::object stream) {
  const TensorView q = view_of(q_), k = view_of(k_), v = view_of(v_), o = view_of(o_), l = view_of(l_);
  require(q.dtype == "torch.bfloat16" && k.dtype == "torch.bfloat16" && v.dtype == "torch.bfloat16" &&
              o.dtype == "torch.bfloat16",
          "q, k, v and out must be torch.bfloat16");
  require(l.dtype == "torch.float32", "lse must be torch.float32");
  const int B = q.shape[0], N = q.shape[1], H = q.shape[2], D = q.shape[3];
  const int HKV = k.shape[2];
  require(k.shape == v.shape, "k and v shapes differ");
  require(k.shape[0] == B && k.shape[1] == N && k.shape[3] == D, "k/v must be [B, N, H_KV, D] matching q");
  require(o.shape == q.shape, "out must have q's shape [B, N, H, D]");
  require(l.shape[0] == B && l.shape[1] == H && l.shape[2] == 1 && l.shape[3] == N, "lse must be [B, H, 1, N]");
  require(q.device == k.device && q.device == v.device && q.device == o.device && q.device == l.device,
          "all tensors must be on the same device");
  const int is_causal = causal.is_none() ? HK_DEFAULT_CAUSAL : (causal.cast<bool>() ? 1 : 0);
  const float scale = softmax_scale.is_none() ? 0.f : softmax_scale.cast<float>();
  void* cu_stream = stream.is_none() ? nullptr : reinterpret_cast<void*>(stream.cast<uint64_t>());
  raise_for(hk_attn_fwd(reinterpret_cast<const void*>(q.ptr), reinterpret_cast<const void*>(k.ptr),
                        reinterpret_cast<const void*>(v.ptr), reinterpret_cast<void*>(o.ptr),
                        reinterpret_cast<float*>(l.ptr), B, N, H, HKV, D, is_causal, scale, q.device, cu_stream),
            HK_ENTRY_NAME);
#if HK_SYNC_AFTER
  raise_for(hk_last_device_status(q.device), HK_ENTRY_NAME);
#endif
}

void dispatch_paged_decode(py::object q_, py::object kp_, py::object vp_, py::object bt_, py::object cl_,
                           py::object o_, py::object l_, py::object ws_, py::object softmax_scale,
                           py::object stream) {
  const TensorView q = view_of(q_), kp = view_of(kp_), vp = view_of(vp_), bt = view_of(bt_), cl = view_of(cl_),
                   o = view_of(o_), l = view_of(l_), ws = view_of(ws_);
  require(q.dtype == "torch.bfloat16" && kp.dtype == "torch.bfloat16" && vp.dtype == "torch.bfloat16" &&
              o.dtype == "torch.bfloat16",
          "q, k_pages, v_pages and out must be torch.bfloat16");
  require(l.dtype == "torch.float32", "lse must be torch.float32");
  require(bt.dtype == "torch.int32" && cl.dtype == "torch.int32", "block_table and ctx_lens must be torch.int32");
  require(ws.dtype == "torch.uint8", "workspace must be a torch.uint8 tensor");
  const int S = q.shape[0], H = q.shape[2], D = q.shape[3];
  require(q.shape[1] == 1, "q must be [S, 1, H, D]");
  require(o.shape == q.shape, "out must have q's shape [S, 1, H, D]");
  require(kp.shape == vp.shape && kp.shape[3] == D, "k_pages/v_pages must be [P, page, H_KV, D]");
  require(bt.shape[2] == S && cl.shape[3] == S, "block_table must be [S, max_pages] and ctx_lens [S]");
  require(l.shape[0] == S && l.shape[1] == H && l.shape[2] == 1 && l.shape[3] == 1, "lse must be [S, H, 1, 1]");
  const size_t ws_bytes = size_t(ws.shape[0]) * ws.shape[1] * ws.shape[2] * ws.shape[3];
  const float scale = softmax_scale.is_none() ? 0.f : softmax_scale.cast<float>();
  void* cu_stream = stream.is_none() ? nullptr : reinterpret_cast<void*>(stream.cast<uint64_t>());
  raise_for(hk_attn_paged_decode(reinterpret_cast<const void*>(q.ptr), reinterpret_cast<const void*>(kp.ptr),
                                 reinterpret_cast<const void*>(vp.ptr), reinterpret_cast<const int32_t*>(bt.ptr),
                                 reinterpret_cast<const int32_t*>(cl.ptr), reinterpret_cast<void*>(o.ptr),
                                 reinterpret_cast<float*>(l.ptr), S, H, kp.shape[2], D, kp.shape[1], bt.shape[3],
                                 kp.shape[0], scale, reinterpret_cast<void*>(ws.ptr), ws_bytes, q.device,
                                 cu_stream),
            "dispatch_paged_decode");
}

}  // namespace

#define HK_STR2(x) #x
#define HK_STR(x) HK_STR2(x)

PYBIND11_MODULE(HK_MODULE_NAME, m) {
  m.doc() = HK_STR(HK_MODULE_NAME) " python module (B200 build)";
  m.def(HK_ENTRY_NAME, &dispatch, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"), py::arg("lse"),
        py::arg("causal") = py::none(), py::arg("softmax_scale") = py::none(), py::arg("stream") = py::none());
  m.def("dispatch_paged_decode", &dispatch_paged_decode, py::arg("q"), py::arg("k_pages"), py::arg("v_pages"),
        py::arg("block_table"), py::arg("ctx_lens"), py::arg("out"), py::arg("lse"), py::arg("workspace"),
        py::arg("softmax_scale") = py::none(), py::arg("stream") = py::none());
  m.def("paged_decode_workspace_bytes", [](int S, int H, int D, int max_pages, int page_size) {
    return hk_attn_paged_decode_workspace_bytes(S, H, D, max_pages, page_size);
  });
  m.def("device_status", [](int device) { return hk_last_device_status(device); });
  m.def("kernel_launch_count", []() { return hk_kernel_launch_count(); });
  m.attr("default_causal") = bool(HK_DEFAULT_CAUSAL);
}
