// bf16 grouped-query flash-attention forward for sm_100a (B200).
//
// Replaces the reference's attend_ker<D> (kernels/attn/gqa/kernel.cpp:102-574 and
// kernels/attn/gqa_causal/kernel.cpp:181-691): O = softmax(scale * Q K^T) V and
// L = logsumexp(scale * Q K^T), Q/O [B,N,H,D], K/V [B,N,H_KV,D], L [B,H,1,N].
//
// Design (one persistent CTA per SM, 384 threads):
//   warps 0-3   softmax warpgroup of slot 0   (one thread per query row, TMEM lane = row)
//   warps 4-7   softmax warpgroup of slot 1
//   warp  8     TMA producer: Q tiles once per work item, K/V tiles through a shared-memory ring
//   warp  9     UMMA issuer: S = Q K^T (both operands in shared memory) and O += P V (P read from
//               TMEM, V from shared memory, MN-major), accumulators in TMEM
//   warps 10-11 idle (they complete the producer warpgroup for the register re-allocation)
// A work item is a pair of 128-row query tiles ("slots") that share one KV head, so each K/V tile
// staged in shared memory feeds two S and two O accumulators. While the tensor pipe works on one
// slot the other slot's softmax runs, which is what hides the exponentials under the MMAs.
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D); bf16 P overwrites the
// first 64 columns of its own S.
//
// Numerics: Q stays unscaled bf16; p = exp2(s*c - m*c) with c = scale*log2(e) in fp32; the running
// max m is only refreshed when it grew by more than 8 in log2 units (the reference's lazy rescale,
// kernels/attn/gqa/kernel.cpp:68,268-281); P is rounded to bf16 (RNE) for the PV product while the
// row sum uses the fp32 values; L = m*scale + ln(l) (kernel.cpp:569-573 in the natural-log domain).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace hk {

constexpr int kBlockM = 128;        // query rows per slot
constexpr int kBlockN = 128;        // keys per KV tile
constexpr int kFwdThreads = 384;
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThresholdLog2 = 8.0f;
constexpr uint64_t kWaitLimitNs = 4000ull * 1000 * 1000;  // 4 s: far beyond any legitimate wait

// Device status codes written to FwdParams::status (0 = OK).
enum : int { kStatusOk = 0, kStatusTimeout = 1 };

struct FwdParams {
  __nv_bfloat16* o;     // [B,N,H,D]
  float* lse;           // [B,H,1,N]
  int B, N, H, H_KV;
  int n_items;          // number of work items (slot pairs)
  int pair_heads;       // 1: slots = two heads of one group at the same q block; 0: two q blocks of one head
  float scale;          // softmax scale
  float scale_log2;     // scale * log2(e)
  int* status;          // device word: first non-zero status wins
};

template <int D>
struct FwdSmem {
  static constexpr int kTileBytes = kBlockM * D * 2;            // one 128 x D bf16 tile
  static constexpr int kSubTileBytes = kBlockM * 128;           // 128 rows x 64 bf16 (128 B swizzled rows)
  static constexpr int kStages = (D == 128) ? 5 : 8;
  static constexpr int kDynBytes = (2 + kStages) * kTileBytes + 1024;  // + slack for 1024-B alignment
};

struct WorkItem {
  int b, kvh;
  int head[2];
  int qb[2];
  int n[2];  // KV tiles each slot consumes (0 = slot unused)
};

// Work-item order. Non-causal: (batch, kv head) outermost so one unit's K/V stay in L2 while all of
// its query tiles stream through. Causal: longest rows first (q block descending) so the tail of the
// launch is made of short items, with the slot pairs that share a K/V prefix adjacent.
template <bool CAUSAL>
__device__ __forceinline__ WorkItem decode_item(const FwdParams& p, int idx) {
  WorkItem w;
  const int G = p.H / p.H_KV;
  const int NQB = p.N / kBlockM;
  const int units = p.B * p.H_KV;
  int unit, qb0, qb1, h0, h1;
  if (p.pair_heads) {
    const int hp_n = G / 2;
    int qb, hp;
    if (CAUSAL) {
      const int per_qb = units * hp_n;
      qb = NQB - 1 - idx / per_qb;
      const int rem = idx % per_qb;
      unit = rem / hp_n;
      hp = rem % hp_n;
    } else {
      const int per_unit = hp_n * NQB;
      unit = idx / per_unit;
      const int rem = idx % per_unit;
      qb = rem / hp_n;
      hp = rem % hp_n;
    }
    qb0 = qb1 = qb;
    h0 = 2 * hp;
    h1 = h0 + 1;
  } else {
    const int NQP = (NQB + 1) / 2;
    int qp, hg;
    if (CAUSAL) {
      const int per_qp = units * G;
      qp = NQP - 1 - idx / per_qp;
      const int rem = idx % per_qp;
      unit = rem / G;
      hg = rem % G;
    } else {
      const int per_unit = G * NQP;
      unit = idx / per_unit;
      const int rem = idx % per_unit;
      qp = rem / G;
      hg = rem % G;
    }
    qb0 = 2 * qp;
    qb1 = 2 * qp + 1;
    h0 = h1 = hg;
  }
  w.b = unit / p.H_KV;
  w.kvh = unit % p.H_KV;
  w.head[0] = w.kvh * G + h0;
  w.head[1] = w.kvh * G + h1;
  w.qb[0] = qb0;
  w.qb[1] = qb1;
  w.n[0] = CAUSAL ? qb0 + 1 : NQB;
  w.n[1] = (qb1 < NQB) ? (CAUSAL ? qb1 + 1 : NQB) : 0;
  return w;
}

// Items are dealt to CTAs in a snake (boustrophedon) order so that, with a length-sorted causal list,
// every CTA receives the same mix of long and short items.
__device__ __forceinline__ int item_for_round(int round, int cta, int n_cta) {
  return round * n_cta + ((round & 1) ? (n_cta - 1 - cta) : cta);
}

template <int D, bool CAUSAL>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  using namespace ptx;
  using SM = FwdSmem<D>;
  constexpr int kStages = SM::kStages;
  constexpr int kTile = SM::kTileBytes;
  constexpr int kSub = SM::kSubTileBytes;
  constexpr int kChunks = D / 64;  // 64-column TMA boxes per tile row

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                 // 2 tiles
  uint8_t* sKV = smem + 2 * kTile;    // kStages tiles, K and V alternate through the ring

  __shared__ uint64_t q_full[2], q_empty[2], s_full[2], p_full[2], o_full[2];
  __shared__ uint64_t kv_full[kStages], kv_empty[kStages];
  __shared__ uint32_t tmem_base_slot;
  __shared__ uint32_t abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 4);  // one arrival per softmax warp
      mbar_init(&o_full[s], 1);
    }
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    fence_mbar_init();
  }
  if (warp == 8) {
    tmem_alloc(&tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;
  volatile uint32_t* abortp = &abort_flag;

  if (warp < 8) {
    // ------------------------------------------------------------------ softmax warpgroups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const int slot = warp >> 2;
    const int row = (warp & 3) * 32 + lane;                      // row inside the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_addr + slot * kBlockN;
    const uint32_t tO = tmem + lane_addr + 2 * kBlockN + slot * D;
    const float c = p.scale_log2;
    uint32_t s_cnt = 0, o_cnt = 0;
    bool ok = true;
    for (int round = 0; ok; ++round) {
      const int idx = item_for_round(round, blockIdx.x, gridDim.x);
      if (idx >= p.n_items) {
        // a snake round may leave this CTA without an item while lower-numbered CTAs still have one
        if (round * static_cast<int>(gridDim.x) >= p.n_items) break;
        continue;
      }
      const WorkItem w = decode_item<CAUSAL>(p, idx);
      const int nkv = w.n[slot];
      if (nkv == 0) continue;
      float m = 0.f, l = 0.f;
      for (int j = 0; j < nkv && ok; ++j) {
        ok = mbar_wait(&s_full[slot], s_cnt & 1, abortp, kWaitLimitNs);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ++s_cnt;
        tc_fence_after();
        uint32_t su[kBlockN];  // one row of S, fp32 bit patterns
#define HK_S(i) __uint_as_float(su[(i)])
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) tmem_ld32(tS + cc * 32, su + cc * 32);
        tmem_wait_ld();
        if (CAUSAL && j == nkv - 1) {
          // diagonal tile: key (j*128 + col) is visible to query (qb*128 + row) iff col <= row
#pragma unroll
          for (int i = 0; i < kBlockN; ++i) su[i] = (i > row) ? 0xff800000u : su[i];
        }
        float bm0 = fmaxf(HK_S(0), HK_S(1)), bm1 = fmaxf(HK_S(2), HK_S(3));
#pragma unroll
        for (int i = 4; i < kBlockN; i += 4) {
          bm0 = fmaxf(bm0, fmaxf(HK_S(i), HK_S(i + 1)));
          bm1 = fmaxf(bm1, fmaxf(HK_S(i + 2), HK_S(i + 3)));
        }
        const float bm = fmaxf(bm0, bm1);
        if (j == 0) {
          m = bm;
        } else {
          const float m_new = fmaxf(m, bm);
          const bool grow = (m_new - m) * c > kRescaleThresholdLog2;
          if (__any_sync(0xffffffffu, grow)) {
            // The previous PV of this slot has completed (the commit that released this S tile
            // was issued after it), so O is stable and nothing writes it until we publish P.
            const float alpha = ex2_approx((m - m_new) * c);
            l *= alpha;
            m = m_new;
#pragma unroll
            for (int cc = 0; cc < D / 32; ++cc) {
              uint32_t o[32];
              tmem_ld32(tO + cc * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(tO + cc * 32, o);
            }
          }
        }
        const float mc = m * c;
        float l0 = 0.f, l1 = 0.f;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = ex2_approx(fmaf(HK_S(cc * 32 + 2 * i), c, -mc));
            const float p1 = ex2_approx(fmaf(HK_S(cc * 32 + 2 * i + 1), c, -mc));
            l0 += p0;
            l1 += p1;
            pk[i] = pack_bf16x2(p0, p1);
          }
          tmem_st16(tS + cc * 16, pk);
        }
        l += l0 + l1;
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[slot]);
#undef HK_S
      }
      if (!ok) break;
      // ---- epilogue of this slot: O / l -> bf16, L = m*scale + ln(l)
      ok = mbar_wait(&o_full[slot], o_cnt & 1, abortp, kWaitLimitNs);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ++o_cnt;
      tc_fence_after();
      const float inv_l = 1.0f / l;
      const int qrow = w.qb[slot] * kBlockM + row;
      const int head = w.head[slot];
      __nv_bfloat16* orow = p.o + ((static_cast<size_t>(w.b) * p.N + qrow) * p.H + head) * D;
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t o[32];
        tmem_ld32(tO + cc * 32, o);
        tmem_wait_ld();
        uint4* dst = reinterpret_cast<uint4*>(orow + cc * 32);
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          uint4 val;
          val.x = pack_bf16x2(__uint_as_float(o[v4 * 8 + 0]) * inv_l, __uint_as_float(o[v4 * 8 + 1]) * inv_l);
          val.y = pack_bf16x2(__uint_as_float(o[v4 * 8 + 2]) * inv_l, __uint_as_float(o[v4 * 8 + 3]) * inv_l);
          val.z = pack_bf16x2(__uint_as_float(o[v4 * 8 + 4]) * inv_l, __uint_as_float(o[v4 * 8 + 5]) * inv_l);
          val.w = pack_bf16x2(__uint_as_float(o[v4 * 8 + 6]) * inv_l, __uint_as_float(o[v4 * 8 + 7]) * inv_l);
          dst[v4] = val;
        }
      }
      p.lse[(static_cast<size_t>(w.b) * p.H + head) * p.N + qrow] = m * p.scale + __logf(l);
      // order this slot's TMEM reads before the next item's PV (published through p_full)
      tc_fence_before();
    }
  } else {
    // ------------------------------------------------------------------ producer warpgroup
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
    if (warp == 8 && lane == 0) {
      // ---------------- TMA producer
      prefetch_tmap(&tmap_q);
      prefetch_tmap(&tmap_k);
      prefetch_tmap(&tmap_v);
      uint32_t q_cnt[2] = {0, 0};
      uint32_t kv_cnt = 0;  // tiles pushed into the ring so far
      bool ok = true;
      auto push_kv = [&](const CUtensorMap* tm, int b, int kvh, int tile) -> bool {
        const int st = kv_cnt % kStages;
        const uint32_t ph = (kv_cnt / kStages) & 1;
        if (!mbar_wait(&kv_empty[st], ph ^ 1, abortp, kWaitLimitNs)) return false;
        mbar_expect_tx(&kv_full[st], kTile);
        uint8_t* dst = sKV + st * kTile;
#pragma unroll
        for (int ch = 0; ch < kChunks; ++ch)
          tma_load_4d(dst + ch * kSub, tm, &kv_full[st], ch * 64, kvh, tile * kBlockN, b);
        ++kv_cnt;
        return true;
      };
      for (int round = 0; ok; ++round) {
        const int idx = item_for_round(round, blockIdx.x, gridDim.x);
        if (idx >= p.n_items) {
          if (round * static_cast<int>(gridDim.x) >= p.n_items) break;
          continue;
        }
        const WorkItem w = decode_item<CAUSAL>(p, idx);
        for (int s = 0; s < 2 && ok; ++s) {
          if (w.n[s] == 0) continue;
          ok = mbar_wait(&q_empty[s], (q_cnt[s] & 1) ^ 1, abortp, kWaitLimitNs);
          if (!ok) break;
          ++q_cnt[s];
          mbar_expect_tx(&q_full[s], kTile);
#pragma unroll
          for (int ch = 0; ch < kChunks; ++ch)
            tma_load_4d(sQ + s * kTile + ch * kSub, &tmap_q, &q_full[s], ch * 64, w.head[s], w.qb[s] * kBlockM,
                        w.b);
        }
        const int nmax = max(w.n[0], w.n[1]);
        if (ok) ok = push_kv(&tmap_k, w.b, w.kvh, 0);
        for (int j = 0; j < nmax && ok; ++j) {
          ok = push_kv(&tmap_v, w.b, w.kvh, j);
          if (ok && j + 1 < nmax) ok = push_kv(&tmap_k, w.b, w.kvh, j + 1);
        }
      }
    } else if (warp == 9 && lane == 0) {
      // ---------------- UMMA issuer
      constexpr uint32_t idesc_qk = make_idesc_bf16(kBlockM, kBlockN, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(kBlockM, D, true);
      const uint32_t sQ_u = smem_u32(sQ), sKV_u = smem_u32(sKV);
      uint32_t q_cnt[2] = {0, 0}, p_cnt[2] = {0, 0};
      uint32_t kv_cnt = 0;  // tiles consumed from the ring so far
      bool ok = true;
      // S[slot] = Q[slot] * K^T with K in ring stage `st`
      auto issue_qk = [&](int s, int st) {
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * kSub + (k % 4) * 32;
          umma_ss(tmem + s * kBlockN, make_smem_desc(sQ_u + s * kTile + off, 16, 1024),
                  make_smem_desc(sKV_u + st * kTile + off, 16, 1024), idesc_qk, k > 0);
        }
      };
      // O[slot] (+)= P[slot] * V with V in ring stage `st`; P is bf16 in TMEM (8 columns per 16 keys)
      auto issue_pv = [&](int s, int st, bool acc) {
#pragma unroll
        for (int k = 0; k < kBlockN / 16; ++k)
          umma_ts(tmem + 2 * kBlockN + s * D, tmem + s * kBlockN + k * 8,
                  make_smem_desc(sKV_u + st * kTile + k * 2048, kSub, 1024), idesc_pv, (acc || k > 0) ? 1u : 0u);
      };
      for (int round = 0; ok; ++round) {
        const int idx = item_for_round(round, blockIdx.x, gridDim.x);
        if (idx >= p.n_items) {
          if (round * static_cast<int>(gridDim.x) >= p.n_items) break;
          continue;
        }
        const WorkItem w = decode_item<CAUSAL>(p, idx);
        const int nmax = max(w.n[0], w.n[1]);
        // ---- first K tile: S = Q K0^T for both slots
        int st_k = kv_cnt % kStages;
        ok = mbar_wait(&kv_full[st_k], (kv_cnt / kStages) & 1, abortp, kWaitLimitNs);
        ++kv_cnt;
        for (int s = 0; s < 2 && ok; ++s) {
          if (w.n[s] == 0) continue;
          ok = mbar_wait(&q_full[s], q_cnt[s] & 1, abortp, kWaitLimitNs);
          if (!ok) break;
          ++q_cnt[s];
          tc_fence_after();
          issue_qk(s, st_k);
          umma_commit(&s_full[s]);
          if (w.n[s] == 1) umma_commit(&q_empty[s]);
        }
        if (!ok) break;
        umma_commit(&kv_empty[st_k]);
        for (int j = 0; j < nmax && ok; ++j) {
          const int st_v = kv_cnt % kStages;
          const uint32_t ph_v = (kv_cnt / kStages) & 1;
          ++kv_cnt;
          bool v_ready = false, k_ready = false;
          int st_kn = 0;
          uint32_t ph_kn = 0;
          const bool has_next = (j + 1 < nmax);
          if (has_next) {
            st_kn = kv_cnt % kStages;
            ph_kn = (kv_cnt / kStages) & 1;
            ++kv_cnt;
          }
          for (int s = 0; s < 2 && ok; ++s) {
            if (j >= w.n[s]) continue;
            ok = mbar_wait(&p_full[s], p_cnt[s] & 1, abortp, kWaitLimitNs);
            if (!ok) break;
            ++p_cnt[s];
            if (!v_ready) {
              ok = mbar_wait(&kv_full[st_v], ph_v, abortp, kWaitLimitNs);
              if (!ok) break;
              v_ready = true;
            }
            tc_fence_after();
            issue_pv(s, st_v, j > 0);
            if (j + 1 < w.n[s]) {
              if (!k_ready) {
                ok = mbar_wait(&kv_full[st_kn], ph_kn, abortp, kWaitLimitNs);
                if (!ok) break;
                k_ready = true;
                tc_fence_after();
              }
              issue_qk(s, st_kn);
              umma_commit(&s_full[s]);
              if (j + 2 == w.n[s]) umma_commit(&q_empty[s]);  // last QK of this slot: Q may be replaced
            } else {
              umma_commit(&o_full[s]);
            }
          }
          if (!ok) break;
          umma_commit(&kv_empty[st_v]);
          if (has_next) umma_commit(&kv_empty[st_kn]);
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (abort_flag != 0) {
    // Give copies and MMAs that are still in flight time to land before TMEM and shared memory go away.
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) {
    }
    if (tid == 0) atomicCAS(p.status, kStatusOk, kStatusTimeout);
    __syncthreads();
  }
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace hk
