// Paged-KV GQA decode for sm_100a: one query token per sequence, KV cache in 16-token pages that are
// reached through a block table. The reference has no such kernel; the math is the forward's
// (kernels/attn/gqa/kernel.cpp:569-573 for L) applied to one query row that sees its whole context.
//
// Split-K layout: a CTA owns a chunk of 512 or 1024 consecutive tokens of one (sequence, kv head) and all
// G = H / H_KV query heads of that kv head, so every K/V byte of the context is read exactly once.
// Inside the CTA each of the 4 warps streams its own pages (page w, w+4, ...) through a private
// cp.async ring of 16-byte copies; scores and the PV product run on mma.sync m16n8k16 (bf16, fp32
// accumulate) with the G heads in the 16-row M dimension, which is far more than an HBM-bound kernel
// needs and keeps the CUDA cores free for address generation and the exponentials.
// Sequences that fit one chunk are finished in place; longer ones leave per-chunk (O, m, l) partials
// in the workspace, which `paged_decode_combine_kernel` merges.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace hk {

constexpr int kPageTokens = 16;
constexpr int kDecodeD = 128;
constexpr int kChunkPagesMin = 32;                    // pages per CTA: 32 (512 tokens) or 64 (1024 tokens),
constexpr int kChunkPagesMax = 64;                    // chosen per launch by decode_pick_chunk_pages
constexpr int kDecodeWarps = 4;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kDecodeStages = 3;                      // pages in flight per warp
constexpr int kSlabBytes = kPageTokens * kDecodeD * 2;   // one page of one kv head: 4 KB
constexpr int kStageBytes = 2 * kSlabBytes;           // K slab + V slab
constexpr int kDecodeSmemBytes = kDecodeWarps * kDecodeStages * kStageBytes;  // 96 KB
constexpr int kMaxCombineSplits = 256;

enum : int { kStatusBadPage = 2, kStatusBadLen = 4 };  // 3 is the backward kernels' kStatusSmemAlign

struct DecodeParams {
  const __nv_bfloat16* q;        // [S,1,H,128]
  const __nv_bfloat16* k_pages;  // [P,16,H_KV,128]
  const __nv_bfloat16* v_pages;
  const int32_t* block_table;    // [S,max_pages]
  const int32_t* ctx_lens;       // [S]
  __nv_bfloat16* o;              // [S,1,H,128]
  float* lse;                    // [S,H,1,1]
  int S, H, H_KV, max_pages, num_pages;
  int chunk_pages;               // pages per CTA (kChunkPagesMin or kChunkPagesMax)
  float scale, scale_log2;
  void* workspace;
  int* status;
};

// The workspace is laid out for the smaller chunk size (the larger split count), whichever size a launch uses.
__host__ __device__ inline int decode_max_splits(int max_pages) {
  return (max_pages + kChunkPagesMin - 1) / kChunkPagesMin;
}
// 1024-token chunks halve the partial results and were measured 4-5 % faster on the 64-sequence workload
// (94.5 % vs 90.7 % of the copy bandwidth); 512-token chunks keep more CTAs in flight when the batch is
// small. Take the large chunk when it still gives every SM two rounds of two CTAs.
inline int decode_pick_chunk_pages(int S, int H_KV, int max_pages, int sm_count) {
  const long long ctas = 1ll * S * H_KV * ((max_pages + kChunkPagesMax - 1) / kChunkPagesMax);
  return ctas >= 4ll * sm_count ? kChunkPagesMax : kChunkPagesMin;
}
// Workspace: partial O as fp32 [S][H][splits][128], then (m, l) pairs as fp32 [S][H][splits][2].
// Shapes the two kernels can be launched for: the combine kernel holds one weight per split in shared memory
// (kMaxCombineSplits of them, counted for the smaller chunk size so that either chunk choice fits), and sequences
// and kv heads are grid dimensions y and z.
inline bool decode_shape_supported(int S, int H_KV, int max_pages) {
  return S > 0 && S <= 65535 && H_KV > 0 && H_KV <= 65535 && max_pages > 0 &&
         decode_max_splits(max_pages) <= kMaxCombineSplits;
}
inline size_t decode_workspace_bytes(int S, int H, int D, int max_pages, int page_size) {
  if (S <= 0 || S > 65535 || H <= 0 || D != kDecodeD || page_size != kPageTokens || max_pages <= 0) return 0;
  if (decode_max_splits(max_pages) > kMaxCombineSplits) return 0;
  const size_t splits = decode_max_splits(max_pages);
  const size_t o_bytes = size_t(S) * H * splits * kDecodeD * sizeof(float);
  const size_t ml_bytes = size_t(S) * H * splits * 2 * sizeof(float);
  return ((o_bytes + 255) & ~size_t(255)) + ((ml_bytes + 255) & ~size_t(255));
}

namespace dec {

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D = A(16x16, row) * B(16x8, col) + D, bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

}  // namespace dec

// grid = (max_splits, H_KV, S), block = 128 threads, dynamic smem = kDecodeSmemBytes.
template <int G>
__global__ void __launch_bounds__(kDecodeThreads, 2) paged_decode_split_kernel(const DecodeParams p) {
  using namespace dec;
  extern __shared__ __align__(128) uint8_t dsmem[];
  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  // A length beyond what the block-table row can address is clamped to the row's capacity and reported; nothing
  // past the row is read.
  int ctx = p.ctx_lens[seq];
  if (ctx > p.max_pages * kPageTokens) {
    ctx = p.max_pages * kPageTokens;
    if (threadIdx.x == 0) atomicCAS(p.status, 0, kStatusBadLen);
  }
  const int chunk_tokens = p.chunk_pages * kPageTokens;
  const int tok0 = split * chunk_tokens;
  if (tok0 >= ctx) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int total_pages = (ctx + kPageTokens - 1) / kPageTokens;
  const int page0 = split * p.chunk_pages;
  const int chunk_pages = min(p.chunk_pages, total_pages - page0);
  // this warp's pages: page0 + warp + 4*i
  const int my_pages = (chunk_pages - warp + kDecodeWarps - 1) / kDecodeWarps;
  const float c = p.scale_log2;

  // page ids of this warp, one per lane (at most kChunkPagesMax / 4 = 16 are used)
  int my_id = 0;
  if (lane < my_pages) {
    my_id = p.block_table[size_t(seq) * p.max_pages + page0 + warp + kDecodeWarps * lane];
    if (my_id < 0 || my_id >= p.num_pages) {
      atomicCAS(p.status, 0, kStatusBadPage);  // never dereference an id outside the pool
      my_id = 0;
    }
  }

  // Q fragments: row g = head kvh*G+g (rows >= G are zero), 8 k-steps of 16 columns
  uint32_t qa[8][2];
  {
    const __nv_bfloat16* qrow = p.q + (size_t(seq) * p.H + kvh * G + (g < G ? g : 0)) * kDecodeD;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t lo = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t);
      uint32_t hi = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t);
      qa[ks][0] = (g < G) ? lo : 0u;
      qa[ks][1] = (g < G) ? hi : 0u;
    }
  }

  const uint32_t ring = ptx::smem_u32(dsmem) + warp * (kDecodeStages * kStageBytes);
  const size_t row_elems = size_t(p.H_KV) * kDecodeD;  // elements between consecutive tokens of a page

  // 16-byte gather of one page of this kv head: lane copies chunks lane, lane+32, ... of the 256
  // chunks (16 tokens x 16 chunks) of K and of V; chunk index is XOR-swizzled with the token so that
  // ldmatrix reads are bank-conflict free.
  auto fetch = [&](int i) {
    if (i < my_pages) {
      const int id = __shfl_sync(0xffffffffu, my_id, i);
      const size_t base = (size_t(id) * kPageTokens) * row_elems + size_t(kvh) * kDecodeD;
      const uint32_t st = ring + (i % kDecodeStages) * kStageBytes;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int ch_lin = r * 32 + lane;
        const int tok = ch_lin >> 4, ch = ch_lin & 15;
        const size_t src = base + size_t(tok) * row_elems + ch * 8;
        const uint32_t dst = tok * 256 + ((ch ^ (tok & 7)) << 4);
        cp_async16(st + dst, p.k_pages + src);
        cp_async16(st + kSlabBytes + dst, p.v_pages + src);
      }
    }
    cp_async_commit();
  };

  float oacc[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) oacc[j][0] = oacc[j][1] = oacc[j][2] = oacc[j][3] = 0.f;
  float m = -INFINITY, l = 0.f;

#pragma unroll
  for (int i = 0; i < kDecodeStages - 1; ++i) fetch(i);

  for (int i = 0; i < my_pages; ++i) {
    fetch(i + kDecodeStages - 1);
    cp_async_wait<kDecodeStages - 1>();
    __syncwarp();
    const uint32_t sK = ring + (i % kDecodeStages) * kStageBytes;
    const uint32_t sV = sK + kSlabBytes;

    // ---- S[16 x 16 tokens] = Q K^T
    float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      const int mi = lane >> 3, r = lane & 7;
      const int tok = r + 8 * (mi >> 1);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const int ch = ks * 2 + (mi & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(sK + tok * 256 + ((ch ^ (tok & 7)) << 4), b0, b1, b2, b3);
        mma_16816(sc[0], qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
        mma_16816(sc[1], qa[ks][0], 0u, qa[ks][1], 0u, b2, b3);
      }
    }
    // ---- online softmax over this page (row g, tokens nt*8 + 2t + {0,1})
    const int tok_base = (page0 + warp + kDecodeWarps * i) * kPageTokens;
    float sv[4] = {sc[0][0], sc[0][1], sc[1][0], sc[1][1]};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int tok = tok_base + (e >> 1) * 8 + 2 * t + (e & 1);
      if (tok >= ctx) sv[e] = -INFINITY;
    }
    float pm = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
    pm = fmaxf(pm, __shfl_xor_sync(0xffffffffu, pm, 1));
    pm = fmaxf(pm, __shfl_xor_sync(0xffffffffu, pm, 2));
    const float m_new = fmaxf(m, pm);
    if (__any_sync(0xffffffffu, (m_new - m) * c > kRescaleThresholdLog2)) {
      const float alpha = ptx::ex2_approx((m - m_new) * c);  // m = -inf on the first page gives 0
      l *= alpha;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        oacc[j][0] *= alpha;
        oacc[j][1] *= alpha;
      }
      m = m_new;
    }
    const float mc = m * c;
    float pv[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      pv[e] = ptx::ex2_approx(fmaf(sv[e], c, -mc));
      l += pv[e];
    }
    const uint32_t pa0 = ptx::pack_bf16x2(pv[0], pv[1]);
    const uint32_t pa2 = ptx::pack_bf16x2(pv[2], pv[3]);
    // ---- O[16 x 128] += P[16 x 16 tokens] V[16 tokens x 128]
    {
      const int mi = lane >> 3, r = lane & 7;
      const int tok = r + 8 * (mi & 1);
#pragma unroll
      for (int jp = 0; jp < 8; ++jp) {
        const int ch = jp * 2 + (mi >> 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(sV + tok * 256 + ((ch ^ (tok & 7)) << 4), b0, b1, b2, b3);
        mma_16816(oacc[2 * jp], pa0, 0u, pa2, 0u, b0, b1);
        mma_16816(oacc[2 * jp + 1], pa0, 0u, pa2, 0u, b2, b3);
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);

  // ---- merge the 4 warps through shared memory (the ring is idle now)
  __syncthreads();
  float* sm_o = reinterpret_cast<float*>(dsmem);                    // [4][8][128]
  float* sm_m = sm_o + kDecodeWarps * 8 * kDecodeD;                 // [4][8]
  float* sm_l = sm_m + kDecodeWarps * 8;                            // [4][8]
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float2 v2 = make_float2(oacc[j][0], oacc[j][1]);
    *reinterpret_cast<float2*>(sm_o + (warp * 8 + g) * kDecodeD + j * 8 + 2 * t) = v2;
  }
  if (t == 0) {
    sm_m[warp * 8 + g] = m;
    sm_l[warp * 8 + g] = l;
  }
  __syncthreads();
  const int d = threadIdx.x;  // 128 threads <-> 128 output columns
  const int n_splits = (ctx + chunk_tokens - 1) / chunk_tokens;
  const int max_splits = decode_max_splits(p.max_pages);
  float* ws_o = reinterpret_cast<float*>(p.workspace);
  const size_t o_bytes = (size_t(p.S) * p.H * max_splits * kDecodeD * sizeof(float) + 255) & ~size_t(255);
  float* ws_ml = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.workspace) + o_bytes);
#pragma unroll
  for (int h = 0; h < G; ++h) {
    float M = sm_m[h];
#pragma unroll
    for (int w = 1; w < kDecodeWarps; ++w) M = fmaxf(M, sm_m[w * 8 + h]);
    float acc = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float wgt = ptx::ex2_approx((sm_m[w * 8 + h] - M) * c);
      acc += wgt * sm_o[(w * 8 + h) * kDecodeD + d];
      lsum += wgt * sm_l[w * 8 + h];
    }
    const int head = kvh * G + h;
    if (n_splits == 1) {
      p.o[(size_t(seq) * p.H + head) * kDecodeD + d] = __float2bfloat16(acc / lsum);
      if (d == 0) p.lse[size_t(seq) * p.H + head] = M * p.scale + __logf(lsum);
    } else {
      const size_t slot = (size_t(seq) * p.H + head) * max_splits + split;
      ws_o[slot * kDecodeD + d] = acc;
      if (d == 0) {
        ws_ml[slot * 2] = M;
        ws_ml[slot * 2 + 1] = lsum;
      }
    }
  }
  // programmatic dependent launch: this CTA's results are written, the combine grid may be set up
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// grid = (H, S), block = 128 threads (one per output column). Merges the per-chunk partials of
// sequences that span more than one chunk.
__global__ void __launch_bounds__(kDecodeD) paged_decode_combine_kernel(const DecodeParams p) {
  // launched with programmatic stream serialization: wait here until the split grid has completed and its
  // partials are visible (a no-op under an ordinary launch)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int head = blockIdx.x, seq = blockIdx.y;
  const int ctx = min(p.ctx_lens[seq], p.max_pages * kPageTokens);  // clamped as in the split kernel, which reports it
  const int d = threadIdx.x;
  if (ctx <= 0) {  // defined output for an empty context
    p.o[(size_t(seq) * p.H + head) * kDecodeD + d] = __float2bfloat16(0.f);
    if (d == 0) p.lse[size_t(seq) * p.H + head] = -INFINITY;
    return;
  }
  const int chunk_tokens = p.chunk_pages * kPageTokens;
  const int n_splits = (ctx + chunk_tokens - 1) / chunk_tokens;
  if (n_splits == 1) return;  // finished by the split kernel
  const int max_splits = decode_max_splits(p.max_pages);
  const float* ws_o = reinterpret_cast<const float*>(p.workspace);
  const size_t o_bytes = (size_t(p.S) * p.H * max_splits * kDecodeD * sizeof(float) + 255) & ~size_t(255);
  const float* ws_ml = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(p.workspace) + o_bytes);
  const size_t slot0 = (size_t(seq) * p.H + head) * max_splits;
  __shared__ float s_w[kMaxCombineSplits];
  __shared__ float s_M, s_L;
  if (threadIdx.x < 32) {
    float M = -INFINITY;
    for (int i = threadIdx.x; i < n_splits; i += 32) M = fmaxf(M, ws_ml[(slot0 + i) * 2]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    float L = 0.f;
    for (int i = threadIdx.x; i < n_splits; i += 32) {
      const float w = ptx::ex2_approx((ws_ml[(slot0 + i) * 2] - M) * p.scale_log2);
      s_w[i] = w;
      L += w * ws_ml[(slot0 + i) * 2 + 1];
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
    if (threadIdx.x == 0) {
      s_M = M;
      s_L = L;
    }
  }
  __syncthreads();
  float acc = 0.f;
#pragma unroll 4
  for (int i = 0; i < n_splits; ++i) acc += s_w[i] * __ldg(ws_o + (slot0 + i) * kDecodeD + d);
  p.o[(size_t(seq) * p.H + head) * kDecodeD + d] = __float2bfloat16(acc / s_L);
  if (d == 0) p.lse[size_t(seq) * p.H + head] = s_M * p.scale + __logf(s_L);
}

inline int prepare_decode_kernels(char* err, size_t err_len) {
  cudaError_t e;
#define HK_PREP(G)                                                                                      \
  e = cudaFuncSetAttribute(paged_decode_split_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                           kDecodeSmemBytes);                                                           \
  if (e != cudaSuccess) {                                                                               \
    snprintf(err, err_len, "decode kernel attribute: %s", cudaGetErrorString(e));                       \
    return -3;                                                                                          \
  }
  HK_PREP(1) HK_PREP(2) HK_PREP(3) HK_PREP(4) HK_PREP(5) HK_PREP(6) HK_PREP(7) HK_PREP(8)
#undef HK_PREP
  return 0;
}

inline cudaError_t launch_paged_decode(DecodeParams p, int sm_count, cudaStream_t stream, int* launched) {
  p.chunk_pages = decode_pick_chunk_pages(p.S, p.H_KV, p.max_pages, sm_count);
  const int splits = (p.max_pages + p.chunk_pages - 1) / p.chunk_pages;
  if (splits > kMaxCombineSplits) return cudaErrorInvalidValue;
  const dim3 grid(splits, p.H_KV, p.S);
  const int G = p.H / p.H_KV;
  switch (G) {
#define HK_CASE(g) \
  case g: paged_decode_split_kernel<g><<<grid, kDecodeThreads, kDecodeSmemBytes, stream>>>(p); break;
    HK_CASE(1) HK_CASE(2) HK_CASE(3) HK_CASE(4) HK_CASE(5) HK_CASE(6) HK_CASE(7) HK_CASE(8)
#undef HK_CASE
    default: return cudaErrorInvalidValue;
  }
  *launched += 1;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  // The combine grid is launched with programmatic stream serialization, so that its launch overlaps the tail
  // of the split grid; it blocks in griddepcontrol.wait until the split grid is complete.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.H, p.S);
  cfg.blockDim = dim3(kDecodeD);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, paged_decode_combine_kernel, p);
  *launched += 1;
  return e;
}

}  // namespace hk
