// Appends new K/V tokens to the paged KV cache that the decode kernel reads.
//
// The reference keeps a contiguous cache and writes new tokens with one slice assignment,
// kv_cache[batch, seqlen_offset : seqlen_offset + T] = kv (training/llama/llama/models/mha.py:16-42,
// `_update_kv_cache`). Here the cache is paged: token t of sequence s lands at position
// start_pos[s] + t, i.e. row (pos % 16) of page block_table[s, pos / 16]. Pure byte movement with 16-byte loads
// and stores, bound by HBM (2 x bytes moved) and, for a handful of tokens, by launch latency.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "paged_decode_sm100.cuh"
#include "rotary_sm100.cuh"

namespace hk {

struct AppendParams {
  const __nv_bfloat16* k_new;   // [S, T, H_KV, D]
  const __nv_bfloat16* v_new;
  __nv_bfloat16* k_pages;       // [P, 16, H_KV, D]
  __nv_bfloat16* v_pages;
  const int32_t* block_table;   // [S, max_pages]
  const int32_t* start_pos;     // [S] position of the first new token of each sequence
  int S, T, row_vec16;          // row_vec16 = H_KV * D * 2 / 16: 16-byte vectors per token row
  int max_pages, num_pages;
  int* status;
};

// grid = a few blocks per SM (grid-stride over the S * T tokens), block = 128 threads. A block keeps kAppendUnroll
// tokens in flight: their positions and page ids are looked up first, then all loads are issued before any store, so
// the dependent chain position -> page id -> destination of one token is covered by the copies of the others.
constexpr int kAppendUnroll = 4;

__global__ void __launch_bounds__(128) paged_kv_append_kernel(const AppendParams p) {
  const long long total = static_cast<long long>(p.S) * p.T;
  for (long long base = static_cast<long long>(blockIdx.x) * kAppendUnroll; base < total;
       base += static_cast<long long>(gridDim.x) * kAppendUnroll) {
    long long dst[kAppendUnroll];  // 16-byte vector index of the destination row, -1 = skip
#pragma unroll
    for (int u = 0; u < kAppendUnroll; ++u) {
      dst[u] = -1;
      const long long tok = base + u;
      if (tok >= total) continue;
      const int s = static_cast<int>(tok / p.T), t = static_cast<int>(tok - static_cast<long long>(s) * p.T);
      const int pos = p.start_pos[s] + t;
      const int page_slot = pos / kPageTokens;
      if (pos < 0 || page_slot >= p.max_pages) {
        if (threadIdx.x == 0) atomicCAS(p.status, 0, kStatusBadPage);
        continue;
      }
      const int id = p.block_table[size_t(s) * p.max_pages + page_slot];
      if (id < 0 || id >= p.num_pages) {  // never write through an id outside the pool
        if (threadIdx.x == 0) atomicCAS(p.status, 0, kStatusBadPage);
        continue;
      }
      dst[u] = (static_cast<long long>(id) * kPageTokens + pos % kPageTokens) * p.row_vec16;
    }
    for (int i = threadIdx.x; i < p.row_vec16; i += blockDim.x) {
      uint4 kv[kAppendUnroll], vv[kAppendUnroll];
#pragma unroll
      for (int u = 0; u < kAppendUnroll; ++u) {
        if (dst[u] < 0) continue;
        const long long src = (base + u) * p.row_vec16 + i;
        kv[u] = reinterpret_cast<const uint4*>(p.k_new)[src];
        vv[u] = reinterpret_cast<const uint4*>(p.v_new)[src];
      }
#pragma unroll
      for (int u = 0; u < kAppendUnroll; ++u) {
        if (dst[u] < 0) continue;
        reinterpret_cast<uint4*>(p.k_pages)[dst[u] + i] = kv[u];
        reinterpret_cast<uint4*>(p.v_pages)[dst[u] + i] = vv[u];
      }
    }
  }
}

// The same append with the rotary embedding of K applied on the way (the reference rotates q and k with a separate
// kernel before the cache update, training/llama/llama/models/mha.py:217-220 then 16-42; fused here, K is read once
// and written once, rotated, instead of being rewritten by a pre-pass first). Token t of sequence s has position
// start_pos[s] + t, which selects its row of cos / sin [cos_rows, R/2]; arithmetic is rotary_kernel's (every product
// and sum rounded to bf16), so the pages hold bit-for-bit what the pre-pass followed by the plain append would.
struct AppendRotaryParams {
  AppendParams a;
  const __nv_bfloat16* cos;   // [cos_rows, R/2]
  const __nv_bfloat16* sin;
  int cos_rows, H_KV, D, R;
};

__global__ void __launch_bounds__(128) paged_kv_append_rotary_kernel(const AppendRotaryParams q) {
  const AppendParams& p = q.a;
  const long long total = static_cast<long long>(p.S) * p.T;
  const int half = q.R / 2;
  const int pair_units = q.R / 16;                      // 8 rotated pairs each
  const int units_per_head = pair_units + (q.D - q.R) / 8;
  const int k_units = q.H_KV * units_per_head;
  for (long long tok = blockIdx.x; tok < total; tok += gridDim.x) {
    const int s = static_cast<int>(tok / p.T), t = static_cast<int>(tok - static_cast<long long>(s) * p.T);
    const int pos = p.start_pos[s] + t;
    const int page_slot = pos / kPageTokens;
    if (pos < 0 || page_slot >= p.max_pages || pos >= q.cos_rows) {
      if (threadIdx.x == 0) atomicCAS(p.status, 0, kStatusBadPage);  // outside the block table or the cos / sin table
      continue;
    }
    const int id = p.block_table[size_t(s) * p.max_pages + page_slot];
    if (id < 0 || id >= p.num_pages) {  // never write through an id outside the pool
      if (threadIdx.x == 0) atomicCAS(p.status, 0, kStatusBadPage);
      continue;
    }
    const long long dst = (static_cast<long long>(id) * kPageTokens + pos % kPageTokens) * p.row_vec16;
    const long long src = tok * p.row_vec16;
    // V: plain copy
    for (int i = threadIdx.x; i < p.row_vec16; i += blockDim.x)
      reinterpret_cast<uint4*>(p.v_pages)[dst + i] = reinterpret_cast<const uint4*>(p.v_new)[src + i];
    // K: rotated pairs, then the dimensions beyond the rotary dimension
    const __nv_bfloat16* krow = p.k_new + src * 8;
    __nv_bfloat16* kdst = p.k_pages + dst * 8;
    for (int i = threadIdx.x; i < k_units; i += blockDim.x) {
      const int head = i / units_per_head, u = i - head * units_per_head;
      const __nv_bfloat16* xr = krow + head * q.D;
      __nv_bfloat16* orow = kdst + head * q.D;
      if (u < pair_units) {
        const uint4 x1 = *reinterpret_cast<const uint4*>(xr + u * 8);
        const uint4 x2 = *reinterpret_cast<const uint4*>(xr + half + u * 8);
        const uint4 c = __ldg(reinterpret_cast<const uint4*>(q.cos + static_cast<size_t>(pos) * half + u * 8));
        const uint4 sn = __ldg(reinterpret_cast<const uint4*>(q.sin + static_cast<size_t>(pos) * half + u * 8));
        uint4 lo, hi;
        lo.x = rot_lo(x1.x, x2.x, c.x, sn.x);
        lo.y = rot_lo(x1.y, x2.y, c.y, sn.y);
        lo.z = rot_lo(x1.z, x2.z, c.z, sn.z);
        lo.w = rot_lo(x1.w, x2.w, c.w, sn.w);
        hi.x = rot_hi(x1.x, x2.x, c.x, sn.x);
        hi.y = rot_hi(x1.y, x2.y, c.y, sn.y);
        hi.z = rot_hi(x1.z, x2.z, c.z, sn.z);
        hi.w = rot_hi(x1.w, x2.w, c.w, sn.w);
        *reinterpret_cast<uint4*>(orow + u * 8) = lo;
        *reinterpret_cast<uint4*>(orow + half + u * 8) = hi;
      } else {
        const int off = q.R + (u - pair_units) * 8;
        *reinterpret_cast<uint4*>(orow + off) = *reinterpret_cast<const uint4*>(xr + off);
      }
    }
  }
}

}  // namespace hk
