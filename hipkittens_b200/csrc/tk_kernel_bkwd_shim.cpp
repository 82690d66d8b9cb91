// pybind11 shim for the reference's two backward extension modules, on top of the C ABI in hk_attn.h:
//   tk_kernel_bkwd_prep   dispatch_prep(O, dO, delta), dispatch_dq_shuffle(dQ_in, dQ)
//                         (kernels/attn/gqa_backwards/attn_bkwd_prep.cpp:227-240)
//   tk_kernel_bkwd        dispatch_bwd_combined(Q, K, V, dO, dQ_in, dK, dV, L, delta)
//                         (kernels/attn/gqa_backwards/attn_bkwd_non_causal.cpp:3171-3185)
// Same argument order, same duck-typed tensors and RuntimeError texts, and like the reference's dispatchers
// every call blocks until the device is done (attn_bkwd_prep.cpp:188-195, attn_bkwd_non_causal.cpp:3164-3169).
// dQ_in keeps the reference's pre-shuffle [B,H,N,D] layout, so the three-call sequence of
// training/llama/llama/models/attentions/hipkittens.py:110-112 runs unchanged; it does not have to be
// zero-filled here because nothing is accumulated into it.
//
// Build-time switches: HK_BKWD_PREP (1 = tk_kernel_bkwd_prep, 0 = tk_kernel_bkwd), HK_DEFAULT_CAUSAL.
#include <pybind11/pybind11.h>

#include "../../include/hk_attn.h"
#include "shim_common.h"

namespace py = pybind11;

#ifndef HK_BKWD_PREP
#define HK_BKWD_PREP 0
#endif
#ifndef HK_DEFAULT_CAUSAL
#define HK_DEFAULT_CAUSAL 0
#endif

namespace {

using namespace hk_shim;

void* stream_of(const py::object& stream) {
  return stream.is_none() ? nullptr : reinterpret_cast<void*>(stream.cast<uint64_t>());
}

#if HK_BKWD_PREP

void dispatch_prep(py::object o_, py::object do_, py::object delta_, py::object stream) {
  const TensorView o = view_of(o_), d_o = view_of(do_), delta = view_of(delta_);
  require(o.dtype == "torch.bfloat16" && d_o.dtype == "torch.bfloat16", "O and dO must be torch.bfloat16");
  require(delta.dtype == "torch.float32", "delta must be torch.float32");
  require(o.shape == d_o.shape, "O and dO shapes differ");
  const int B = o.shape[0], N = o.shape[1], H = o.shape[2], D = o.shape[3];
  require(delta.shape[0] == B && delta.shape[1] == H && delta.shape[2] == 1 && delta.shape[3] == N,
          "delta must be [B, H, 1, N]");
  require(o.device == d_o.device && o.device == delta.device, "all tensors must be on the same device");
  raise_for(hk_attn_bwd_prep(reinterpret_cast<const void*>(o.ptr), reinterpret_cast<const void*>(d_o.ptr),
                             reinterpret_cast<float*>(delta.ptr), B, N, H, D, o.device, stream_of(stream)),
            "dispatch_prep");
  raise_for(hk_last_device_status(o.device), "dispatch_prep");
}

void dispatch_dq_shuffle(py::object in_, py::object out_, py::object stream) {
  const TensorView in = view_of(in_), out = view_of(out_);
  require(in.dtype == "torch.bfloat16" && out.dtype == "torch.bfloat16", "dQ tensors must be torch.bfloat16");
  const int B = in.shape[0], H = in.shape[1], N = in.shape[2], D = in.shape[3];
  require(out.shape[0] == B && out.shape[1] == N && out.shape[2] == H && out.shape[3] == D,
          "dQ_in must be [B, H, N, D] and dQ [B, N, H, D]");
  require(in.device == out.device, "all tensors must be on the same device");
  raise_for(hk_attn_dq_shuffle(reinterpret_cast<const void*>(in.ptr), reinterpret_cast<void*>(out.ptr), B, N, H, D,
                               in.device, stream_of(stream)),
            "dispatch_dq_shuffle");
  raise_for(hk_last_device_status(in.device), "dispatch_dq_shuffle");
}

#else

void dispatch_bwd_combined(py::object q_, py::object k_, py::object v_, py::object do_, py::object dq_,
                           py::object dk_, py::object dv_, py::object l_, py::object delta_, py::object causal,
                           py::object softmax_scale, py::object stream) {
  const TensorView q = view_of(q_), k = view_of(k_), v = view_of(v_), d_o = view_of(do_), dq = view_of(dq_),
                   dk = view_of(dk_), dv = view_of(dv_), l = view_of(l_), delta = view_of(delta_);
  for (const TensorView* t : {&q, &k, &v, &d_o, &dq, &dk, &dv})
    require(t->dtype == "torch.bfloat16", "Q, K, V, dO, dQ, dK and dV must be torch.bfloat16");
  require(l.dtype == "torch.float32" && delta.dtype == "torch.float32", "L and delta must be torch.float32");
  const int B = q.shape[0], N = q.shape[1], H = q.shape[2], D = q.shape[3];
  const int HKV = k.shape[2];
  require(k.shape == v.shape && k.shape[0] == B && k.shape[1] == N && k.shape[3] == D,
          "K/V must be [B, N, H_KV, D] matching Q");
  require(d_o.shape == q.shape, "dO must have Q's shape [B, N, H, D]");
  require(dk.shape == k.shape && dv.shape == v.shape, "dK/dV must have K's shape");
  require(dq.shape[0] == B && dq.shape[1] == H && dq.shape[2] == N && dq.shape[3] == D,
          "dQ_in must be [B, H, N, D] (the pre-shuffle layout)");
  for (const TensorView* t : {&l, &delta})
    require(t->shape[0] == B && t->shape[1] == H && t->shape[2] == 1 && t->shape[3] == N,
            "L and delta must be [B, H, 1, N]");
  for (const TensorView* t : {&k, &v, &d_o, &dq, &dk, &dv, &l, &delta})
    require(t->device == q.device, "all tensors must be on the same device");
  const int is_causal = causal.is_none() ? HK_DEFAULT_CAUSAL : (causal.cast<bool>() ? 1 : 0);
  const float scale = softmax_scale.is_none() ? 0.f : softmax_scale.cast<float>();
  raise_for(hk_attn_bwd(reinterpret_cast<const void*>(q.ptr), reinterpret_cast<const void*>(k.ptr),
                        reinterpret_cast<const void*>(v.ptr), reinterpret_cast<const void*>(d_o.ptr),
                        reinterpret_cast<const float*>(l.ptr), reinterpret_cast<const float*>(delta.ptr),
                        reinterpret_cast<void*>(dq.ptr), reinterpret_cast<void*>(dk.ptr),
                        reinterpret_cast<void*>(dv.ptr), B, N, H, HKV, D, is_causal, scale, HK_DQ_BHND, q.device,
                        stream_of(stream)),
            "dispatch_bwd_combined");
  raise_for(hk_last_device_status(q.device), "dispatch_bwd_combined");
}

#endif

}  // namespace

#if HK_BKWD_PREP
PYBIND11_MODULE(tk_kernel_bkwd_prep, m) {
  m.doc() = "tk_kernel_bkwd_prep python module (B200 build)";
  m.def("dispatch_prep", &dispatch_prep, py::arg("O"), py::arg("dO"), py::arg("delta"),
        py::arg("stream") = py::none());
  m.def("dispatch_dq_shuffle", &dispatch_dq_shuffle, py::arg("dQ_in"), py::arg("dQ"),
        py::arg("stream") = py::none());
}
#else
PYBIND11_MODULE(tk_kernel_bkwd, m) {
  m.doc() = "tk_kernel_bkwd python module (B200 build)";
  m.def("dispatch_bwd_combined", &dispatch_bwd_combined, py::arg("Q"), py::arg("K"), py::arg("V"), py::arg("dO"),
        py::arg("dQ_in"), py::arg("dK"), py::arg("dV"), py::arg("L"), py::arg("delta"),
        py::arg("causal") = py::none(), py::arg("softmax_scale") = py::none(), py::arg("stream") = py::none());
  m.attr("default_causal") = bool(HK_DEFAULT_CAUSAL);
}
#endif
