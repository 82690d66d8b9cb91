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

}  // namespace hk
