// Rotary position embedding as a pre-pass over q or k, the step directly before attention in the model
// (training/llama/llama/models/mha.py:217-220,236-239).
//
// Replaces the reference's tk_fused_rotary (kernels/rotary/kernel.cpp:44-74): for x [B, H, N, D] bf16 and
// cos, sin [N, R/2] bf16 (R = rotary dimension, R <= D),
//     o[..., i]       = x[..., i] * cos[n, i] - x[..., i + R/2] * sin[n, i]
//     o[..., i + R/2] = x[..., i + R/2] * cos[n, i] + x[..., i] * sin[n, i]        for i < R/2,
// and o[..., R:] = x[..., R:]. Like the reference kernel (and like the PyTorch expression in its harness,
// kernels/rotary/test_python.py:50-58, evaluated on bf16 tensors) every product and the sum are rounded to bf16
// separately (__hmul2 / __hsub2 / __hadd2 there; the explicitly rounded, never-fused intrinsics here), so the result is
// bit-identical to that expression.
//
// The same kernel serves x [B, N, H, D], the layout the attention kernels read (RotaryParams::n_div = H), so that q
// and k can be rotated where they lie, without the transposes the [B, H, N, D] form needs around it.
//
// Pure streaming: 16-byte loads and stores, one thread per 8 rotated pairs. HBM-bound: 2 x B*H*N*D*2 bytes per call;
// cos / sin (N * R bytes each) stay in L2.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hk {

struct RotaryParams {
  const __nv_bfloat16* x;    // [rows, D], rows = B*H*N with n fastest
  __nv_bfloat16* o;          // [rows, D]
  const __nv_bfloat16* cos;  // [N, R/2]
  const __nv_bfloat16* sin;  // [N, R/2]
  long long rows;
  int N, D, R;
  int n_div;   // the position of row r is (r / n_div) % N + pos0: 1 for [B,H,N,D], H for [B,N,H,D]
  int pos0;    // position of sequence index 0 (a chunk that continues a cached prefix starts at its offset)
};

__device__ __forceinline__ uint32_t rot_lo(uint32_t x1, uint32_t x2, uint32_t c, uint32_t s) {
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x1);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&x2);
  const __nv_bfloat162 cc = *reinterpret_cast<const __nv_bfloat162*>(&c);
  const __nv_bfloat162 ss = *reinterpret_cast<const __nv_bfloat162*>(&s);
  const __nv_bfloat162 r = __hsub2_rn(__hmul2_rn(a, cc), __hmul2_rn(b, ss));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t rot_hi(uint32_t x1, uint32_t x2, uint32_t c, uint32_t s) {
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x1);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&x2);
  const __nv_bfloat162 cc = *reinterpret_cast<const __nv_bfloat162*>(&c);
  const __nv_bfloat162 ss = *reinterpret_cast<const __nv_bfloat162*>(&s);
  const __nv_bfloat162 r = __hadd2_rn(__hmul2_rn(b, cc), __hmul2_rn(a, ss));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// Work unit = 8 rotated pairs (or 8 pass-through elements) of one row: `units_per_row` = R/16 pair units followed by
// (D - R)/8 copy units. grid = ceil(rows * units_per_row / 256), block = 256.
__global__ void __launch_bounds__(256) rotary_kernel(const RotaryParams p) {
  const int pair_units = p.R / 16;
  const int units_per_row = pair_units + (p.D - p.R) / 8;
  const long long gid = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  const long long row = gid / units_per_row;
  if (row >= p.rows) return;
  const int u = static_cast<int>(gid - row * units_per_row);
  const __nv_bfloat16* xr = p.x + row * p.D;
  __nv_bfloat16* orow = p.o + row * p.D;
  if (u < pair_units) {
    const int n = static_cast<int>((row / p.n_div) % p.N) + p.pos0;
    const int half = p.R / 2;
    const uint4 x1 = *reinterpret_cast<const uint4*>(xr + u * 8);
    const uint4 x2 = *reinterpret_cast<const uint4*>(xr + half + u * 8);
    const uint4 c = __ldg(reinterpret_cast<const uint4*>(p.cos + static_cast<size_t>(n) * half + u * 8));
    const uint4 s = __ldg(reinterpret_cast<const uint4*>(p.sin + static_cast<size_t>(n) * half + u * 8));
    uint4 lo, hi;
    lo.x = rot_lo(x1.x, x2.x, c.x, s.x);
    lo.y = rot_lo(x1.y, x2.y, c.y, s.y);
    lo.z = rot_lo(x1.z, x2.z, c.z, s.z);
    lo.w = rot_lo(x1.w, x2.w, c.w, s.w);
    hi.x = rot_hi(x1.x, x2.x, c.x, s.x);
    hi.y = rot_hi(x1.y, x2.y, c.y, s.y);
    hi.z = rot_hi(x1.z, x2.z, c.z, s.z);
    hi.w = rot_hi(x1.w, x2.w, c.w, s.w);
    *reinterpret_cast<uint4*>(orow + u * 8) = lo;
    *reinterpret_cast<uint4*>(orow + half + u * 8) = hi;
  } else {
    const int off = p.R + (u - pair_units) * 8;
    *reinterpret_cast<uint4*>(orow + off) = *reinterpret_cast<const uint4*>(xr + off);
  }
}

}  // namespace hk
