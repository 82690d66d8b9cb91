// Appends new K/V tokens to the paged KV cache that the decode kernel reads.
//
// The reference keeps a contiguous cache and writes new tokens with one slice assignment,
// kv_cache[batch, seqlen_offset : seqlen_offset + T] = kv (training/llama/llama/models/mha.py:16-42,
// `_update_kv_cache`). Here the cache is paged: token t of sequence s lands at position
// start_pos[s] + t, i.e. row (pos % 16) of page block_table[s, pos / 16]. Pure byte movement:
// one 128-thread block moves the H_KV * D bf16 values of one token of K and of V with 16-byte
// loads and stores, so the kernel is bound by HBM (2 x bytes moved) and launch latency.
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

// grid = (T, S), block = 128
__global__ void __launch_bounds__(128) paged_kv_append_kernel(const AppendParams p) {
  const int t = blockIdx.x, s = blockIdx.y;
  const int pos = p.start_pos[s] + t;
  const int page_slot = pos / kPageTokens;
  if (pos < 0 || page_slot >= p.max_pages) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, kStatusBadPage);
    return;
  }
  const int id = p.block_table[size_t(s) * p.max_pages + page_slot];
  if (id < 0 || id >= p.num_pages) {  // never write through an id outside the pool
    if (threadIdx.x == 0) atomicCAS(p.status, 0, kStatusBadPage);
    return;
  }
  const size_t src = (size_t(s) * p.T + t) * p.row_vec16;
  const size_t dst = (size_t(id) * kPageTokens + pos % kPageTokens) * p.row_vec16;
  const uint4* ks = reinterpret_cast<const uint4*>(p.k_new) + src;
  const uint4* vs = reinterpret_cast<const uint4*>(p.v_new) + src;
  uint4* kd = reinterpret_cast<uint4*>(p.k_pages) + dst;
  uint4* vd = reinterpret_cast<uint4*>(p.v_pages) + dst;
  for (int i = threadIdx.x; i < p.row_vec16; i += blockDim.x) {
    kd[i] = ks[i];
    vd[i] = vs[i];
  }
}

}  // namespace hk
