// bf16 grouped-query flash-attention forward for sm_100a (B200).
//
// Replaces the reference's attend_ker<D> (kernels/attn/gqa/kernel.cpp:102-574 and
// kernels/attn/gqa_causal/kernel.cpp:181-691): O = softmax(scale * Q K^T) V and
// L = logsumexp(scale * Q K^T), Q/O [B,N,H,D], K/V [B,NK,H_KV,D] (or 16-token pages reached through a block
// table), L [B,H,1,N]; optional per-batch key lengths; causal masks aligned to the last query and the last kept key.
//
// Design (one persistent CTA per SM, 384 threads):
//   warps 0-3   softmax warpgroup of slot 0   (one thread per query row, TMEM lane = row)
//   warps 4-7   softmax warpgroup of slot 1
//   warp  8     TMA producer: Q tiles once per work item, K/V tiles through a shared-memory ring
//   warp  9     UMMA issuer: S = Q K^T (both operands in shared memory) and O += P V (P read from
//               TMEM, V from shared memory, MN-major), accumulators in TMEM
//   warp  10    D = 64 only: second UMMA issuer (warp 9 then issues the Q K^T products, warp 10 the P V ones)
//   warp  11    D = 128: store thread, sends each finished O tile from its shared-memory staging buffer to global
//               memory with TMA (the softmax warps write their rows there, swizzled, instead of storing 32 scattered
//               rows per instruction from registers). D = 64 non-causal: Q loader (O is stored from registers there)
//   (warp 10 at D = 128, and all but one lane of warps 9-11, are idle; they complete the producer warpgroup for
//   the register re-allocation)
// A work item is a pair of 128-row query tiles ("slots") that share one KV head, so each K/V tile
// staged in shared memory feeds two S and two O accumulators. While the tensor pipe works on one
// slot the other slot's softmax runs, which is what hides the exponentials under the MMAs.
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D); bf16 P overwrites the
// first 64 columns of its own S (D = 128) or has columns [384,448) / [448,512) of its own (D = 64).
//
// Numerics: Q stays unscaled bf16; p = exp2(s*c - m*c) with c = scale*log2(e) in fp32; the running
// max m is only refreshed when it grew by more than 8 in log2 units (the reference's lazy rescale,
// kernels/attn/gqa/kernel.cpp:68,268-281) - it is not even looked for after an item's first tile, unless a
// row sum overflows (see the softmax loop); P is rounded to bf16 (RNE) for the PV product while the
// row sum uses the fp32 values; L = m*scale + ln(l) (kernel.cpp:569-573 in the natural-log domain).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "sm100_ptx.cuh"

namespace hk {

constexpr int kBlockM = 128;        // query rows per slot
constexpr int kBlockN = 128;        // keys per KV tile
constexpr int kFwdThreads = 384;
constexpr int kFwdRegsAtLaunch = 168;   // 65536 / 384, rounded down to a multiple of 8; see setmaxnreg below
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThresholdLog2 = 8.0f;
// Of every kEmuMod column pairs of a score row, this many take their exponentials from a cubic polynomial on the
// FMA pipe (ptx::ex2_poly2, relative error 1e-4) instead of the MUFU: an exponential costs its warp's scheduler 8
// clocks at the MUFU, a polynomial pair about 13 against the 16 of two MUFU ones. A quarter of the pairs is the best
// share for both head dimensions (D = 64: +3 %, half of them -10 %; D = 128: +1 %, a third of them -3 %). It is taken
// at D = 64 only: it raises the error of L from 1e-5 to 1e-4 (of the 1e-3 allowed), which one per cent does not buy
// at D = 128. Which pairs matters as much as how many, through the instruction schedule the compiler arrives at: the
// non-causal D = 64 kernel is fastest with the first two of every eight pairs (+1.4 % over one of every four; the
// same quarter at other offsets or in runs of four is 0.5 to 3 % slower), the causal one with one of every four.
#ifndef HK_EMU_MOD
#define HK_EMU_MOD 4
#endif
// 1: non-causal D = 64 sends O through shared memory and TMA as well (two staging tiles per slot, the store issued
// by one of the slot's own threads); 0: 32-byte stores from registers, as causal D = 64 always does.
#ifndef HK_D64_STAGE_OUT
#define HK_D64_STAGE_OUT 1
#endif
#ifndef HK_EMU_CNT_D64
#define HK_EMU_CNT_D64 1
#endif
#ifndef HK_EMU_CNT_D128
#define HK_EMU_CNT_D128 0
#endif
#ifndef HK_EMU_MOD_D64_NONCAUSAL
#define HK_EMU_MOD_D64_NONCAUSAL 8
#endif
#ifndef HK_EMU_CNT_D64_NONCAUSAL
#define HK_EMU_CNT_D64_NONCAUSAL 2
#endif
constexpr uint64_t kWaitLimitCycles = 8000ull * 1000 * 1000;  // SM cycles, > 4 s: far beyond any legitimate wait

// Device status codes written to FwdParams::status (0 = OK).
enum : int { kStatusOk = 0, kStatusTimeout = 1, kStatusFwdBadPage = 2 };  // 2 = the decode kernels' kStatusBadPage

// Division of a non-negative int below 2^31 by a divisor fixed at launch: a multiply-high and a shift instead of the
// ~40 dependent instructions of a 32-bit division. The work-item decode below divides ten times per item, on the
// critical path of the MMA issuer and of the softmax warps between two items (1 600 clocks per item before).
// mul = ceil(2^(31+L) / d) with L = ceil(log2 d); n / d = umulhi(n, mul) >> (L - 1) for 0 <= n < 2^31 (d = 1: n).
struct FastDiv {
  uint32_t d = 1, mul = 0, shift = 0;
  FastDiv() = default;
  explicit FastDiv(int divisor) : d(static_cast<uint32_t>(divisor)) {
    if (d > 1) {
      uint32_t L = 0;
      while ((1ull << L) < d) ++L;
      mul = static_cast<uint32_t>(((1ull << (31 + L)) + d - 1) / d);
      shift = L - 1;
    }
  }
  // the same arithmetic on the host (the self-test of the C ABI checks it against the division it replaces)
  int div_host(int n) const {
    return d == 1 ? n : static_cast<int>(((static_cast<uint64_t>(static_cast<uint32_t>(n)) * mul) >> 32) >> shift);
  }
#ifdef __CUDACC__
  __device__ __forceinline__ int div(int n) const {
    return d == 1 ? n : static_cast<int>(__umulhi(static_cast<uint32_t>(n), mul) >> shift);
  }
  __device__ __forceinline__ void divmod(int n, int& q, int& r) const {
    q = div(n);
    r = n - q * static_cast<int>(d);
  }
#endif
};

struct FwdParams {
  __nv_bfloat16* o;     // [B,N,H,D]
  float* lse;           // [B,H,1,N]
  int B, N, H, H_KV;    // N = query rows per batch element
  int NK;               // keys per batch element (N for self-attention)
  int n_items;          // number of work items (slot pairs)
  int pair_heads;       // 1: slots = two heads of one group at the same q block; 0: two q blocks of one head
  int group_units;      // causal order: (batch, kv-head) units swept together, sized so their K/V fit in L2
  int group_items;      // work items of a full group (all items when there is one group)
  int rounds_per_group; // ceil(group_items / CTAs): a group is dealt in rounds of its own
  int total_rounds;     // rounds_per_group * number of groups
  // Item decode, prepared by set_item_decode(): an item index splits into (unit, q tile or q tile pair, head or head
  // pair inside the group) by these divisors
  int G, nqb, units;    // H / H_KV, query tiles per sequence, B * H_KV
  int inner;            // slot pairs per q position inside a unit: G / 2 (two heads per item) or G (two q tiles)
  int last_group;       // index of the last causal sweep group (it may hold fewer units)
  FastDiv fd_rounds, fd_group_items, fd_per_unit, fd_inner, fd_per_q, fd_per_q_last, fd_hkv;
  float scale;          // softmax scale
  float scale_log2;     // scale * log2(e)
  const int* kv_lens;   // optional device [B]: batch b attends to keys [0, kv_lens[b]) only; null = NK
  // Paged K/V (null block_table = contiguous): key j of batch element b is row j % 16 of page
  // block_table[b * max_pages + j / 16] of a pool [num_pages, 16, H_KV, D]; the K and V tensor maps then describe
  // the pools as [num_pages * 16 rows, H_KV, D] with a 16-row box, and NK = max_pages * 16.
  const int* block_table;
  int max_pages, num_pages;
  int* status;          // device word: first non-zero status wins
#ifdef HK_TRACE
  long long* trace;     // [3 roles][4096] clock stamps of CTA 0 (debug builds only)
#endif
};

template <int D, bool CAUSAL>
struct FwdSmem {
  static constexpr int kTileBytes = kBlockM * D * 2;            // one 128 x D bf16 tile
  static constexpr int kSubTileBytes = kBlockM * 128;           // 128 rows x 64 bf16 (128 B swizzled rows)
  static constexpr int kStages = (D == 128) ? 4 : 8;            // a fifth stage at D = 128 measured no faster
  // Staging from which O leaves through TMA. D = 128: one [128 x 128] tile (two 64-column halves) that the slots use
  // in turn. D = 64 non-causal: two [128 x 64] tiles per slot, used alternately. D = 64 causal: none (it stores from
  // registers, and shared memory it does not need is L1 cache it does).
  static constexpr int kOutStageBytes =
      (D == 128) ? kTileBytes : ((HK_D64_STAGE_OUT && !CAUSAL) ? 4 * kSubTileBytes : 0);
  static constexpr int kDynBytes = (2 + kStages) * kTileBytes + kOutStageBytes + 1024;  // + alignment slack
};

struct WorkItem {
  int b, kvh;
  int kv_len;  // keys this batch element attends to
  int off;     // causal: query row r sees keys [0, r + off], off = kv_len - N (the reference aligns the mask to the
               // last query and the last kept key, training/llama/llama/models/attentions/base.py:104-116)
  int head[2];
  int qb[2];
  int n[2];  // KV tiles each slot consumes (0 = slot unused)
};

// Work-item order. Non-causal: (batch, kv head) outermost so one unit's K/V stay in L2 while all of
// its query tiles stream through. Causal: units are swept in groups whose K/V fit in L2 together; inside
// a group the longest rows come first (q block descending), with the slot pairs that share a K/V prefix
// adjacent. (One sweep over all units at once keeps every unit's K/V live at the same time - 128 MB at
// N = 8192 - and was measured to re-read K/V from HBM 2.6 times over.)
template <bool CAUSAL>
__device__ __forceinline__ WorkItem decode_item(const FwdParams& p, int idx) {
  WorkItem w;
  const int G = p.G;
  const int NQB = p.nqb;  // the last block may be partial
  // an item is (unit, q position, pair inside the group); a q position is a q tile (two heads per item) or a pair
  // of q tiles (one head per item), of which there are nq per unit
  const int nq = p.pair_heads ? NQB : (NQB + 1) / 2;
  int unit, qx, hx;
  if (CAUSAL) {
    const int grp = min(p.fd_group_items.div(idx), p.last_group);
    const int within = idx - grp * p.group_items;
    int qd, rem;
    if (grp == p.last_group) p.fd_per_q_last.divmod(within, qd, rem);
    else p.fd_per_q.divmod(within, qd, rem);
    qx = nq - 1 - qd;
    int u;
    p.fd_inner.divmod(rem, u, hx);
    unit = grp * p.group_units + u;
  } else {
    int rem;
    p.fd_per_unit.divmod(idx, unit, rem);
    p.fd_inner.divmod(rem, qx, hx);
  }
  int qb0, qb1, h0, h1;
  if (p.pair_heads) {
    qb0 = qb1 = qx;
    h0 = 2 * hx;
    h1 = h0 + 1;
  } else {
    qb0 = 2 * qx;
    qb1 = 2 * qx + 1;
    h0 = h1 = hx;
  }
  p.fd_hkv.divmod(unit, w.b, w.kvh);
  w.head[0] = w.kvh * G + h0;
  w.head[1] = w.kvh * G + h1;
  w.qb[0] = qb0;
  w.qb[1] = qb1;
  // key-padding lengths: tiles beyond the batch element's own length are never loaded
  w.kv_len = p.kv_lens ? min(max(p.kv_lens[w.b], 1), p.NK) : p.NK;
  w.off = w.kv_len - p.N;
  const int n_kv = (w.kv_len + kBlockN - 1) / kBlockN;
  // causal: the last row of query block qb sees keys up to qb*128 + 127 + off; a block none of whose rows sees a
  // key gets no tiles (its rows are written as O = 0, L = -inf by the softmax warps)
  auto causal_tiles = [&](int qb) { return min(max((qb * kBlockM + kBlockM + w.off + kBlockN - 1) / kBlockN, 0), n_kv); };
  w.n[0] = CAUSAL ? causal_tiles(qb0) : n_kv;
  w.n[1] = (qb1 < NQB) ? (CAUSAL ? causal_tiles(qb1) : n_kv) : 0;
  return w;
}

// Items are dealt to CTAs in a snake (boustrophedon) order so that, with a length-sorted causal list,
// every CTA receives the same mix of long and short items. Every group of units is dealt in rounds of its own
// (the last round of a group may be partial) and consecutive groups start the snake from opposite ends: a round
// that straddled two groups would hand the longest items of the next group to the CTAs that also got the
// longer items of this one (2 % imbalance with 64 MB groups, 7 % with 32 MB groups of the N = 8192 shape).
// Returns the item index, or -1 when this CTA has no item in this round.
template <typename Params>
__device__ __forceinline__ int item_for_round(const Params& p, int round, int cta, int n_cta) {
  const int grp = p.fd_rounds.div(round);  // round / rounds_per_group
  const int r = round - grp * p.rounds_per_group;
  const int first = grp * p.group_items;
  const int in_grp = r * n_cta + (((r + grp) & 1) ? (n_cta - 1 - cta) : cta);
  return (in_grp < min(p.group_items, p.n_items - first)) ? first + in_grp : -1;
}

// Host side: fills the fields the item decode reads. Call after B, N, H, H_KV, pair_heads, group_units, group_items
// and rounds_per_group are set.
inline void set_item_decode(FwdParams& p) {
  p.G = p.H / p.H_KV;
  p.nqb = (p.N + kBlockM - 1) / kBlockM;
  p.units = p.B * p.H_KV;
  p.inner = p.pair_heads ? p.G / 2 : p.G;
  const int nq = p.pair_heads ? p.nqb : (p.nqb + 1) / 2;
  p.last_group = (p.units - 1) / p.group_units;
  p.fd_rounds = FastDiv(p.rounds_per_group);
  p.fd_group_items = FastDiv(p.group_units * p.inner * nq);
  p.fd_per_unit = FastDiv(p.inner * nq);
  p.fd_inner = FastDiv(p.inner);
  p.fd_per_q = FastDiv(p.group_units * p.inner);
  p.fd_per_q_last = FastDiv((p.units - p.last_group * p.group_units) * p.inner);
  p.fd_hkv = FastDiv(p.H_KV);
}

#ifdef HK_TRACE
// Phase stamps for tuning: CTA 0, one thread per role appends (event id, SM clock) pairs.
#define HK_STAMP(role, ev)                                                            \
  do {                                                                                \
    if (blockIdx.x == 0 && trace_on && trace_n < 2040) {                              \
      p.trace[(role) * 4096 + 2 * trace_n] = (ev);                                    \
      p.trace[(role) * 4096 + 2 * trace_n + 1] = clock64();                           \
      ++trace_n;                                                                      \
    }                                                                                 \
  } while (0)
#else
#define HK_STAMP(role, ev) do {} while (0)
#endif
#if defined(HK_TRACE) && HK_TRACE >= 2
#define HK_STAMP2(role, ev) HK_STAMP(role, ev)
#else
#define HK_STAMP2(role, ev) do {} while (0)
#endif

template <int D, bool CAUSAL>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                const FwdParams p) {
  using namespace ptx;
  using SM = FwdSmem<D, CAUSAL>;
  constexpr int kStages = SM::kStages;
  constexpr int kTile = SM::kTileBytes;
  constexpr int kSub = SM::kSubTileBytes;
  constexpr int kChunks = D / 64;  // 64-column TMA boxes per tile row
  // With D = 64 the two O accumulators need only 128 TMEM columns, which leaves room for P outside S
  // (columns [384,448) and [448,512)). S(j+1) = Q K(j+1)^T can then be issued as soon as the softmax has
  // read S(j), instead of after O += P(j) V(j), and a slot's softmax never waits for the tensor pipe.
  constexpr bool kSepP = (D == 64);
  // Registers after the re-balancing: 8 softmax warps and 4 others share the 168 x 384 the CTA was launched with.
  // 208 / 88 everywhere except the non-causal D = 64 kernel, which compiles to a 4 % faster schedule with 216 / 72
  // (200 / 104 and 224 / 56 are both slower there, and 216 / 72 is 2.5 % slower for causal D = 64: the effect is the
  // compiler's instruction schedule, not spills).
  constexpr int kSoftmaxRegs = (D == 64 && !CAUSAL) ? 216 : 208;
  constexpr int kOtherRegs = (D == 64 && !CAUSAL) ? 72 : 88;
  static_assert(8 * kSoftmaxRegs + 4 * kOtherRegs == 12 * kFwdRegsAtLaunch, "registers taken = registers released");
  constexpr int kEmuMod = (D == 64 && !CAUSAL) ? HK_EMU_MOD_D64_NONCAUSAL : HK_EMU_MOD;
  constexpr int kEmuCnt = (D == 64) ? (CAUSAL ? HK_EMU_CNT_D64 : HK_EMU_CNT_D64_NONCAUSAL) : HK_EMU_CNT_D128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                 // 2 tiles
  uint8_t* sKV = smem + 2 * kTile;    // kStages tiles, K and V alternate through the ring
  // D = 128: O leaves through TMA from one [128 x 128] staging tile (two 64-column halves) that the two slots use
  // in turn, sent by the store thread. D = 64: see kStage64 below.
  uint8_t* sOut = sKV + kStages * kTile;
  constexpr bool kTmaOut = (D == 128);
  // D = 64 non-causal: O leaves through two staging tiles per slot and TMA stores issued by one of the slot's own
  // threads (+0.7 to +3 %, the more the shorter the sequence). Causal D = 64 keeps the 32-byte stores from
  // registers: the staged form measured 3-4 % slower there.
  constexpr bool kStage64 = (D == 64) && !CAUSAL && (HK_D64_STAGE_OUT != 0);
  // D = 64, non-causal: the Q tiles are loaded by a thread of their own (warp 11, which has no stores to send
  // there). Measured +1.7 % there, but -7 % at D = 64 causal and -2 % at D = 128 with short items, where the
  // producer thread goes on loading Q itself.
  constexpr bool kQThread = (D == 64) && !CAUSAL;

  __shared__ uint64_t q_full[2], q_empty[2], s_full[2], p_full[2], o_full[2];
  __shared__ uint64_t s_free[2], p_free[2];  // D = 64 only: S has been read / P has been consumed
  __shared__ uint64_t kv_full[kStages], kv_empty[kStages];
  // O staging (D = 128): so_turn[slot] - the store thread gives the staging tile to the slot (its previous contents
  // have been read out); so_full[slot] - the slot's four warps have written their rows into it
  __shared__ uint64_t so_turn[2], so_full[2];
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
      mbar_init(&s_free[s], 4);
      mbar_init(&p_free[s], 1);
      mbar_init(&so_full[s], 4);
      mbar_init(&so_turn[s], 1);
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
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
    const int slot = warp >> 2;
    const int row = (warp & 3) * 32 + lane;                      // row inside the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_addr + slot * kBlockN;
    const uint32_t tO = tmem + lane_addr + 2 * kBlockN + slot * D;
    const uint32_t tP = kSepP ? tmem + lane_addr + 384 + slot * 64 : tS;  // bf16 P: 64 packed columns
    const float c = p.scale_log2;
    uint32_t s_cnt = 0, o_cnt = 0, pv_cnt = 0;
    // Staging buffer of this slot and the number of times it has been used before the current item. With one
    // buffer for both slots its uses are ordered: item by item, and inside an item the slot with fewer K/V tiles
    // (which finishes first) before the other; both slots and the store warp derive that order from the item.
    bool ok = true;
#ifdef HK_TRACE
    const bool trace_on = ((warp & 3) == 0) && lane == 0 && p.trace != nullptr;
    int trace_n = 0;
#endif
    for (int round = 0; ok; ++round) {
      if (round >= p.total_rounds) break;
      const int idx = item_for_round(p, round, blockIdx.x, gridDim.x);
      if (idx < 0) continue;  // a partial round leaves some CTAs without an item
      const WorkItem w = decode_item<CAUSAL>(p, idx);
      const int nkv = w.n[slot];
      // causal: the last key this thread's row sees, and the first tile the diagonal (or the end of the keys) runs
      // through - the last one, and the one before it when off is not a multiple of the tile. Key j*128 + i is
      // visible to query row r iff it is <= r + off and < kv_len; tile j needs masking iff its last key is beyond
      // what the block's FIRST row sees, (j+1)*128 - 1 > min(qb*128 + off, kv_len - 1) (CTA-uniform). Both are
      // fixed for the item, so the per-tile test is one comparison.
      const int row_last_key = min(w.qb[slot] * kBlockM + row + w.off, w.kv_len - 1);
      const int j_mask = (min(w.qb[slot] * kBlockM + w.off, w.kv_len - 1) + 1) >> 7;
      if (nkv == 0) {
        if (CAUSAL && w.qb[slot] * kBlockM < p.N) {
          // a query block that sees no key at all (more queries than keys): defined output, no products
          const int qrow = w.qb[slot] * kBlockM + row;
          if (qrow < p.N) {
            uint4* dst = reinterpret_cast<uint4*>(p.o + ((static_cast<size_t>(w.b) * p.N + qrow) * p.H + w.head[slot]) * D);
#pragma unroll
            for (int v4 = 0; v4 < D / 8; ++v4) dst[v4] = make_uint4(0u, 0u, 0u, 0u);
            p.lse[(static_cast<size_t>(w.b) * p.H + w.head[slot]) * p.N + qrow] = -INFINITY;
          }
        }
        continue;
      }
      float m = 0.f, l = 0.f;
      for (int j = 0; j < nkv && ok; ++j) {
        HK_STAMP2(slot, 0);
        ok = mbar_wait(&s_full[slot], s_cnt & 1, abortp, kWaitLimitCycles);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ++s_cnt;
        tc_fence_after();
        HK_STAMP(slot, 1);
        if constexpr (kSepP) {
          uint32_t su[kBlockN];  // one row of S, fp32 bit patterns
#define HK_S(i) __uint_as_float(su[(i)])
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) tmem_ld32(tS + cc * 32, su + cc * 32);
          tmem_wait_ld();
          HK_STAMP2(slot, 2);
          if (kSepP) {
            // S(j) is in registers: the issuer may overwrite it with the next S of this slot right away
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free[slot]);
          }
          if (CAUSAL && j >= j_mask) {
            const int lim = row_last_key - j * kBlockN;
#pragma unroll
            for (int i = 0; i < kBlockN; ++i) su[i] = (i > lim) ? 0xff800000u : su[i];
          }
          if (!CAUSAL && j == nkv - 1 && (w.kv_len & (kBlockN - 1)) != 0) {
            // partial last tile: keys at or beyond the length are padding (or, beyond N, zeros filled by TMA)
            const int rem = w.kv_len - j * kBlockN;
#pragma unroll
            for (int i = 0; i < kBlockN; ++i) su[i] = (i >= rem) ? 0xff800000u : su[i];
          }
          // the first tile fixes m; later tiles take their exponentials against the m the row has and are redone
          // with their maximum only if a row sum comes out huge or not finite
          auto row_max = [&]() {
            float bm0 = fmaxf(HK_S(0), HK_S(1)), bm1 = fmaxf(HK_S(2), HK_S(3));
            float bm2 = fmaxf(HK_S(4), HK_S(5)), bm3 = fmaxf(HK_S(6), HK_S(7));
#pragma unroll
            for (int i = 8; i < kBlockN; i += 8) {
              bm0 = max3(bm0, HK_S(i), HK_S(i + 1));
              bm1 = max3(bm1, HK_S(i + 2), HK_S(i + 3));
              bm2 = max3(bm2, HK_S(i + 4), HK_S(i + 5));
              bm3 = max3(bm3, HK_S(i + 6), HK_S(i + 7));
            }
            return fmaxf(fmaxf(bm0, bm2), fmaxf(bm1, bm3));
          };
          auto raise_max = [&](float bm) {
            if (j == 0) {
              m = bm;
              return;
            }
            const float m_new = fmaxf(m, bm);
            const bool grow = (m_new - m) * c > kRescaleThresholdLog2;
            if (__any_sync(0xffffffffu, grow)) {
              const float alpha = (m == -INFINITY) ? 0.f : ex2_approx((m - m_new) * c);
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
          };
          const uint64_t c2 = pack2(c, c);
          // exponentials of the whole row against m, P stored chunk by chunk; returns the row sum of the tile
          auto exps_and_store = [&]() -> float {
            const float nmc = (CAUSAL && m == -INFINITY) ? 0.f : -(m * c);
            const uint64_t nmc2 = pack2(nmc, nmc);
            uint64_t lacc0 = pack2(0.f, 0.f), lacc1 = pack2(0.f, 0.f);
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              uint32_t pk[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const uint64_t x2 = fma2(pack2(HK_S(cc * 32 + 2 * i), HK_S(cc * 32 + 2 * i + 1)), c2, nmc2);
                uint64_t p2;
                float p0, p1;
                if ((i % kEmuMod) < kEmuCnt) {
                  p2 = ex2_poly2(x2);
                  unpack2(p2, p0, p1);
                } else {
                  float x0, x1;
                  unpack2(x2, x0, x1);
                  p0 = ex2_approx(x0);
                  p1 = ex2_approx(x1);
                  p2 = pack2(p0, p1);
                }
                if (i & 1) lacc1 = add2(lacc1, p2); else lacc0 = add2(lacc0, p2);
                pk[i] = pack_bf16x2(p0, p1);
              }
              tmem_st16(tP + cc * 16, pk);
            }
            float a0, a1, b0, b1;
            unpack2(lacc0, a0, a1);
            unpack2(lacc1, b0, b1);
            return (a0 + a1) + (b0 + b1);
          };
          bool exact = j == 0 || (CAUSAL && w.off < 0 && __any_sync(0xffffffffu, m == -INFINITY));
          float bm_first = 0.f;
          if (exact) bm_first = row_max();
          if (kSepP && pv_cnt > 0) {
            // S(j) may be ready before O += P(j-1) V(j-1) has finished: wait for that product before
            // rescaling O or overwriting P
            ok = mbar_wait(&p_free[slot], (pv_cnt - 1) & 1, abortp, kWaitLimitCycles);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
          }
          ++pv_cnt;
          if (exact) raise_max(bm_first);
          HK_STAMP2(slot, 3);
          float l_tile = exps_and_store();
          if (!exact && __any_sync(0xffffffffu, !(l_tile < 1e30f))) {
            // a score far above m: the P just stored is not published yet, S is still in registers - do the tile
            // again the exact way
            raise_max(row_max());
            l_tile = exps_and_store();
          }
          l += l_tile;
#undef HK_S
        } else {
          // ---- D = 128. Any reference value m within ~100 powers of two of a row's true maximum gives the same O
          // and L: p = exp2(s*c - m*c) neither overflows nor loses the row's largest terms, P keeps its relative
          // precision in bf16, and L = m*scale + ln(l) does not care which m it was. So after the first tile of an
          // item the row maximum is not computed at all (it costs ~240 clocks of the chain S -> softmax -> P V that
          // bounds this kernel): the exponentials are taken against the m the row already has and P is held in
          // registers until the row sums are known. Only if one of them is huge or not finite is the tile redone
          // the exact way, with its maximum and the rescaling of O; S is still intact in TMEM then, because nothing
          // has been stored over it.
          uint32_t su[kBlockN];  // one row of S, fp32 bit patterns
#define HK_S(i) __uint_as_float(su[(i)])
          auto load_scores = [&]() {
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) tmem_ld32(tS + cc * 32, su + cc * 32);
            tmem_wait_ld();
            if (CAUSAL && j >= j_mask) {
              const int lim = row_last_key - j * kBlockN;
#pragma unroll
              for (int i = 0; i < kBlockN; ++i) su[i] = (i > lim) ? 0xff800000u : su[i];
            }
            if (!CAUSAL && j == nkv - 1 && (w.kv_len & (kBlockN - 1)) != 0) {
              // partial last tile: keys at or beyond the length are padding (or, beyond N, zeros filled by TMA)
              const int rem = w.kv_len - j * kBlockN;
#pragma unroll
              for (int i = 0; i < kBlockN; ++i) su[i] = (i >= rem) ? 0xff800000u : su[i];
            }
          };
          load_scores();
          HK_STAMP2(slot, 2);
          // the first tile fixes m; so does any tile of a row that has not seen a key yet (only possible with more
          // queries than kept keys, off < 0)
          bool exact = j == 0 || (CAUSAL && w.off < 0 && __any_sync(0xffffffffu, m == -INFINITY));
          uint32_t pk[kBlockN / 2];
          float l_tile;
          for (;;) {
            if (exact) {
              float bm0 = fmaxf(HK_S(0), HK_S(1)), bm1 = fmaxf(HK_S(2), HK_S(3));
              float bm2 = fmaxf(HK_S(4), HK_S(5)), bm3 = fmaxf(HK_S(6), HK_S(7));
#pragma unroll
              for (int i = 8; i < kBlockN; i += 8) {
                bm0 = max3(bm0, HK_S(i), HK_S(i + 1));
                bm1 = max3(bm1, HK_S(i + 2), HK_S(i + 3));
                bm2 = max3(bm2, HK_S(i + 4), HK_S(i + 5));
                bm3 = max3(bm3, HK_S(i + 6), HK_S(i + 7));
              }
              const float bm = fmaxf(fmaxf(bm0, bm2), fmaxf(bm1, bm3));
              if (j == 0) {
                m = bm;
              } else {
                const float m_new = fmaxf(m, bm);
                const bool grow = (m_new - m) * c > kRescaleThresholdLog2;
                if (__any_sync(0xffffffffu, grow)) {
                  // The previous PV of this slot has completed (the commit that released this S tile was issued
                  // after it), so O is stable and nothing writes it until we publish P.
                  const float alpha = (m == -INFINITY) ? 0.f : ex2_approx((m - m_new) * c);
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
            }
            // p = exp2(s*c - m*c), two columns per instruction where the hardware has packed fp32 forms
            HK_STAMP2(slot, 3);
            const uint64_t c2 = pack2(c, c);
            // a causal row that has seen no key yet has m = -inf: subtract nothing, its exponentials are exp2(-inf) = 0
            const float nmc = (CAUSAL && m == -INFINITY) ? 0.f : -(m * c);
            const uint64_t nmc2 = pack2(nmc, nmc);
            uint64_t lacc0 = pack2(0.f, 0.f), lacc1 = pack2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < kBlockN / 2; ++i) {
              const uint64_t x2 = fma2(pack2(HK_S(2 * i), HK_S(2 * i + 1)), c2, nmc2);
              uint64_t p2;
              float p0, p1;
              if ((i % kEmuMod) < kEmuCnt) {
                p2 = ex2_poly2(x2);
                unpack2(p2, p0, p1);
              } else {
                float x0, x1;
                unpack2(x2, x0, x1);
                p0 = ex2_approx(x0);
                p1 = ex2_approx(x1);
                p2 = pack2(p0, p1);
              }
              if (i & 1) lacc1 = add2(lacc1, p2); else lacc0 = add2(lacc0, p2);
              pk[i] = pack_bf16x2(p0, p1);
            }
            {
              float a0, a1, b0, b1;
              unpack2(lacc0, a0, a1);
              unpack2(lacc1, b0, b1);
              l_tile = (a0 + a1) + (b0 + b1);
            }
            // exp2 saturates to +inf, so a score too far above m shows in the row sum (as does a NaN)
            if (exact || !__any_sync(0xffffffffu, !(l_tile < 1e30f))) break;
            load_scores();
            exact = true;
          }
          l += l_tile;
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) tmem_st16(tP + cc * 16, pk + cc * 16);
#undef HK_S
        }
        HK_STAMP2(slot, 4);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[slot]);
        HK_STAMP(slot, 5);
      }
      if (!ok) break;
      // ---- epilogue of this slot: O / l -> bf16, L = m*scale + ln(l)
      ok = mbar_wait(&o_full[slot], o_cnt & 1, abortp, kWaitLimitCycles);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ++o_cnt;
      tc_fence_after();
      const float inv_l = (CAUSAL && l == 0.f) ? 0.f : 1.0f / l;  // l = 0: a row that sees no key gets O = 0, L = -inf
      const int qrow = w.qb[slot] * kBlockM + row;
      const int head = w.head[slot];
      const bool row_exists = qrow < p.N;  // rows of a partial last block beyond N are computed but not stored
      // O leaves through shared memory: a thread's row goes into the staging tile in the 128-byte-swizzled layout
      // (conflict-free 16-byte stores) and the store warp sends the tile to global memory as TMA boxes, which write
      // whole 128-byte lines and clip the rows beyond N. (Storing from registers, each thread its own row, touched
      // 32 separate lines per instruction and cost almost two tile periods per work item.)
      if constexpr (kStage64) {
        // D = 64: the slot's rows go into one of its two staging tiles, swizzled, and one of its threads sends the
        // tile off with a TMA store. Tile k & 1 of the slot was last used by its store k - 2; the issuing thread
        // waits for its previous store (k - 1) to have been read before it arrives on so_full, and every warp waits
        // on so_full, so that when epilogue k + 1 starts the tile it writes is known to be free. (32-byte stores
        // from registers, each thread its own row, kept the store unit busy for ~1 500 clocks per item and slot.)
        const bool issuer_thread = (warp & 3) == 0 && lane == 0;
        uint8_t* const so_tile = sOut + (slot * 2 + ((o_cnt - 1) & 1)) * kSub;
        uint8_t* const so_row = so_tile + row * 128;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t o[32];
          tmem_ld32(tO + cc * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 val;
            val.x = pack_bf16x2(__uint_as_float(o[u * 8 + 0]) * inv_l, __uint_as_float(o[u * 8 + 1]) * inv_l);
            val.y = pack_bf16x2(__uint_as_float(o[u * 8 + 2]) * inv_l, __uint_as_float(o[u * 8 + 3]) * inv_l);
            val.z = pack_bf16x2(__uint_as_float(o[u * 8 + 4]) * inv_l, __uint_as_float(o[u * 8 + 5]) * inv_l);
            val.w = pack_bf16x2(__uint_as_float(o[u * 8 + 6]) * inv_l, __uint_as_float(o[u * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(so_row + (((cc * 4 + u) ^ (row & 7)) << 4)) = val;
          }
        }
        fence_proxy_async();  // this thread's stores, visible to the TMA engine
        __syncwarp();
        if (lane == 0) {
          if (issuer_thread) bulk_wait_group_read0();  // the slot's previous store has left its tile
          mbar_arrive(&so_full[slot]);
        }
        ok = mbar_wait(&so_full[slot], (o_cnt - 1) & 1, abortp, kWaitLimitCycles);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (issuer_thread) {
          tma_store_4d(&tmap_o, so_tile, 0, head, w.qb[slot] * kBlockM, w.b);
          bulk_commit_group();
        }
      } else if constexpr (!kTmaOut) {
        // straight from registers, 32 bytes per store where the tensor allows it
        __nv_bfloat16* orow = p.o + ((static_cast<size_t>(w.b) * p.N + qrow) * p.H + head) * D;
        const bool wide = (reinterpret_cast<uintptr_t>(p.o) & 31) == 0;  // rows are multiples of 128 bytes apart
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t o[32];
          tmem_ld32(tO + cc * 32, o);
          tmem_wait_ld();
          uint32_t r[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            r[i] = pack_bf16x2(__uint_as_float(o[2 * i]) * inv_l, __uint_as_float(o[2 * i + 1]) * inv_l);
          if (row_exists) {
            if (wide) {
              st_global_v8(orow + cc * 32, r);
              st_global_v8(orow + cc * 32 + 16, r + 8);
            } else {
              uint4* dst = reinterpret_cast<uint4*>(orow + cc * 32);
#pragma unroll
              for (int v4 = 0; v4 < 4; ++v4) dst[v4] = make_uint4(r[v4 * 4], r[v4 * 4 + 1], r[v4 * 4 + 2], r[v4 * 4 + 3]);
            }
          }
        }
      } else {
        uint32_t o[32];
        tmem_ld32(tO, o);
        uint8_t* const so_row = sOut + row * 128;
        // the staging tile is this slot's once the store thread says so (the tile's previous contents are on their
        // way; the slots take turns in the order in which their tiles finish)
        ok = mbar_wait(&so_turn[slot], (o_cnt - 1) & 1, abortp, kWaitLimitCycles);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {  // 32 columns = 64 bytes = four 16-byte units of the row's 128-byte half
          tmem_wait_ld();
          uint4 val[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            val[u].x = pack_bf16x2(__uint_as_float(o[u * 8 + 0]) * inv_l, __uint_as_float(o[u * 8 + 1]) * inv_l);
            val[u].y = pack_bf16x2(__uint_as_float(o[u * 8 + 2]) * inv_l, __uint_as_float(o[u * 8 + 3]) * inv_l);
            val[u].z = pack_bf16x2(__uint_as_float(o[u * 8 + 4]) * inv_l, __uint_as_float(o[u * 8 + 5]) * inv_l);
            val[u].w = pack_bf16x2(__uint_as_float(o[u * 8 + 6]) * inv_l, __uint_as_float(o[u * 8 + 7]) * inv_l);
          }
          if (cc + 1 < D / 32) tmem_ld32(tO + (cc + 1) * 32, o);
#pragma unroll
          for (int u = 0; u < 4; ++u)
            *reinterpret_cast<uint4*>(so_row + (cc >> 1) * kSub + ((((cc & 1) * 4 + u) ^ (row & 7)) << 4)) = val[u];
        }
        fence_proxy_async();  // this thread's stores, visible to the TMA engine
        __syncwarp();
        if (lane == 0) mbar_arrive(&so_full[slot]);
      }
      if (row_exists)
        p.lse[(static_cast<size_t>(w.b) * p.H + head) * p.N + qrow] =
            (CAUSAL && l == 0.f) ? -INFINITY : m * p.scale + __logf(l);
      // order this slot's TMEM reads before the next item's PV (published through p_full)
      tc_fence_before();
    }
    if (kStage64 && (warp & 3) == 0 && lane == 0) bulk_wait_group0();  // the last tiles have left
  } else {
    // ------------------------------------------------------------------ producer warpgroup
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
    if (warp == 8) {
      // ---------------- TMA producer. Contiguous K/V: one thread (lane 0) walks the work list. Paged K/V: the whole
      // warp does, lane 0 doing the waits and lanes 0-7 each fetching one page of a K/V tile (one thread issuing the
      // 8 or 16 small boxes of a tile, after 8 dependent block-table reads, could not keep the ring full).
      auto produce = [&](auto paged_tag) {
        constexpr bool kPaged = decltype(paged_tag)::value;
        if (lane == 0) {
          if (!kQThread) prefetch_tmap(&tmap_q);
          prefetch_tmap(&tmap_k);
          prefetch_tmap(&tmap_v);
        }
        uint32_t q_cnt[2] = {0, 0};
        int ring_st = 0;        // next ring stage to fill
        uint32_t ring_par = 0;  // its phase parity
        bool ok = true;
        auto push_kv = [&](const CUtensorMap* tm, int b, int kvh, int tile, int kv_len) -> bool {
          const int st = ring_st;
          bool good = true;
          if (lane == 0) {
            good = mbar_wait(&kv_empty[st], ring_par ^ 1, abortp, kWaitLimitCycles);
            if (good) mbar_expect_tx(&kv_full[st], kTile);
          }
          if (kPaged) good = __shfl_sync(0xffffffffu, good, 0);
          if (!good) return false;
          uint8_t* dst = sKV + st * kTile;
          if (!kPaged) {
#pragma unroll
            for (int ch = 0; ch < kChunks; ++ch)
              tma_load_4d(dst + ch * kSub, tm, &kv_full[st], ch * 64, kvh, tile * kBlockN, b);
          } else if (lane < kBlockN / 16) {
            // the tile's 128 keys are 8 pages of 16, one lane and one 16-row box each. Pages beyond the context
            // repeat its last page, so that every row of the tile holds cache contents (those keys are masked; their
            // V rows meet p = 0). An id outside the pool is reported and replaced, never dereferenced.
            const int total_pages = (kv_len + 15) >> 4;
            int id = __ldg(p.block_table + static_cast<size_t>(b) * p.max_pages +
                           min(tile * (kBlockN / 16) + lane, total_pages - 1));
            if (id < 0 || id >= p.num_pages) {
              atomicCAS(p.status, kStatusOk, kStatusFwdBadPage);
              id = 0;
            }
#pragma unroll
            for (int ch = 0; ch < kChunks; ++ch)
              tma_load_4d(dst + ch * kSub + lane * (16 * 128), tm, &kv_full[st], ch * 64, kvh, id * 16, 0);
          }
          if (++ring_st == kStages) {
            ring_st = 0;
            ring_par ^= 1;
          }
          return true;
        };
        for (int round = 0; ok; ++round) {
          if (round >= p.total_rounds) break;
          const int idx = item_for_round(p, round, blockIdx.x, gridDim.x);
          if (idx < 0) continue;
          const WorkItem w = decode_item<CAUSAL>(p, idx);
          const int nmax = max(w.n[0], w.n[1]);
          // the first K tile is requested before the Q tiles: the stage it goes to is free two K/V tiles before the
          // previous item ends, the Q tiles only when that item's last Q K^T has been issued
          if (nmax > 0) ok = push_kv(&tmap_k, w.b, w.kvh, 0, w.kv_len);
          if (!kQThread && lane == 0 && ok) {
            for (int s = 0; s < 2 && ok; ++s) {
              if (w.n[s] == 0) continue;
              ok = mbar_wait(&q_empty[s], (q_cnt[s] & 1) ^ 1, abortp, kWaitLimitCycles);
              if (!ok) break;
              ++q_cnt[s];
              mbar_expect_tx(&q_full[s], kTile);
#pragma unroll
              for (int ch = 0; ch < kChunks; ++ch)
                tma_load_4d(sQ + s * kTile + ch * kSub, &tmap_q, &q_full[s], ch * 64, w.head[s], w.qb[s] * kBlockM,
                            w.b);
            }
          }
          if (kPaged) ok = __shfl_sync(0xffffffffu, ok, 0);
          for (int j = 0; j < nmax && ok; ++j) {
            ok = push_kv(&tmap_v, w.b, w.kvh, j, w.kv_len);
            if (ok && j + 1 < nmax) ok = push_kv(&tmap_k, w.b, w.kvh, j + 1, w.kv_len);
          }
        }
      };
      if (p.block_table != nullptr) produce(std::true_type{});
      else if (lane == 0) produce(std::false_type{});
    } else if (kSepP && (warp == 9 || warp == 10) && lane == 0) {
      // ---------------- D = 64: two UMMA issuers. P has TMEM columns of its own, so S(j+1) = Q K(j+1)^T and
      // O += P(j) V(j) of a slot do not order each other: warp 9 issues every Q K^T, warp 10 every P V, each with
      // its own three waits and three commits per KV tile. (One thread issuing both spends ~600 clocks per group of
      // MMAs on waits, fences and commits, 3 400 per KV tile for 1 456 clocks of MMA work.)
      constexpr uint32_t idesc_qk = make_idesc_bf16(kBlockM, kBlockN, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(kBlockM, D, true);
      constexpr uint32_t desc_hi = smem_desc_hi(1024);
      constexpr uint32_t tile16 = kTile >> 4;
      const uint32_t q_lo0 = smem_desc_lo(smem_u32(sQ), 16);
      const uint32_t k_lo0 = smem_desc_lo(smem_u32(sKV), 16);
      const uint32_t v_lo0 = smem_desc_lo(smem_u32(sKV), kSub);
      const bool is_qk = (warp == 9);
      uint32_t pos = is_qk ? 0u : 1u;   // ring position of this role's next tile: K tiles even, V tiles odd
      uint32_t q_par[2] = {0, 0}, cnt[2] = {0, 0};  // cnt: products issued so far per slot
      bool ok = true;
      for (int round = 0; ok; ++round) {
        if (round >= p.total_rounds) break;
        const int idx = item_for_round(p, round, blockIdx.x, gridDim.x);
        if (idx < 0) continue;
        const WorkItem w = decode_item<CAUSAL>(p, idx);
        const int nmax = max(w.n[0], w.n[1]);
        for (int j = 0; j < nmax && ok; ++j) {
          const int st = static_cast<int>(pos % kStages);
          const uint32_t par = (pos / kStages) & 1u;
          pos += 2;
          ok = mbar_wait(&kv_full[st], par, abortp, kWaitLimitCycles);
          for (int s = 0; s < 2 && ok; ++s) {
            if (j >= w.n[s]) continue;
            if (is_qk) {
              if (j == 0) {
                ok = mbar_wait(&q_full[s], q_par[s], abortp, kWaitLimitCycles);
                q_par[s] ^= 1;
                if (!ok) break;
              }
              // S of this slot is free once the softmax has read the previous one (nothing to wait for the first time)
              ok = mbar_wait(&s_free[s], (cnt[s] & 1) ^ 1, abortp, kWaitLimitCycles);
              if (!ok) break;
              ++cnt[s];
              tc_fence_after();
              const uint32_t a = q_lo0 + s * tile16, b = k_lo0 + st * tile16, d = tmem + s * kBlockN;
#pragma unroll
              for (int k = 0; k < D / 16; ++k)
                umma_ss_lohi(d, a + k * 2, b + k * 2, desc_hi, idesc_qk, k > 0 ? 1u : 0u);
              umma_commit(&s_full[s]);
              if (j + 1 == w.n[s]) umma_commit(&q_empty[s]);
            } else {
              ok = mbar_wait(&p_full[s], cnt[s] & 1, abortp, kWaitLimitCycles);
              if (!ok) break;
              ++cnt[s];
              tc_fence_after();
              const uint32_t b = v_lo0 + st * tile16, d = tmem + 2 * kBlockN + s * D, a = tmem + 384 + s * 64;
#pragma unroll
              for (int k = 0; k < kBlockN / 16; ++k)
                umma_ts_lohi(d, a + k * 8, b + k * 128, desc_hi, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
              umma_commit(&p_free[s]);
              if (j + 1 == w.n[s]) umma_commit(&o_full[s]);
            }
          }
          if (ok) umma_commit(&kv_empty[st]);
        }
      }
    } else if (!kSepP && warp == 9 && lane == 0) {
      // ---------------- UMMA issuer (D = 128)
      // One thread issues for both slots, strictly alternating slot 0 / slot 1. The alternation is what
      // keeps the two softmax warpgroups half a period apart, so that one slot's exponentials run under
      // the other slot's MMAs. (Two independent issuers, one per slot, were measured: the slots drift
      // into lock-step, both softmaxes and then both MMA chunks run at the same time, and throughput
      // drops by 30 %.)
      constexpr uint32_t idesc_qk = make_idesc_bf16(kBlockM, kBlockN, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(kBlockM, D, true);
      // Descriptor words: the high word is constant; the low word is (address >> 4) | (lbo >> 4) << 16 and
      // a K step only adds a constant to it (tiles are 1024-byte aligned, so nothing carries out).
      constexpr uint32_t desc_hi = smem_desc_hi(1024);
      constexpr uint32_t tile16 = kTile >> 4;
      const uint32_t q_lo0 = smem_desc_lo(smem_u32(sQ), 16);      // Q tile of slot 0 (K-major)
      const uint32_t k_lo0 = smem_desc_lo(smem_u32(sKV), 16);     // ring stage 0 as a K tile (K-major)
      const uint32_t v_lo0 = smem_desc_lo(smem_u32(sKV), kSub);   // ring stage 0 as a V tile (MN-major)
      uint32_t q_par[2] = {0, 0}, p_par[2] = {0, 0};  // phase parities of q_full / p_full per slot
      int ring_st = 0;                                // next ring stage to consume
      uint32_t ring_par = 0;                          // its phase parity
      bool ok = true;
#ifdef HK_TRACE
      const bool trace_on = p.trace != nullptr;
      int trace_n = 0;
#endif
      // S[slot] = Q[slot] * K^T with K in ring stage `st`
      auto issue_qk = [&](int s, int st) {
        const uint32_t a = q_lo0 + s * tile16, b = k_lo0 + st * tile16, d = tmem + s * kBlockN;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          constexpr uint32_t sub16 = kSub >> 4;
          const uint32_t off = (k / 4) * sub16 + (k % 4) * 2;  // 32 bytes per K step inside a 128-byte row
          umma_ss_lohi(d, a + off, b + off, desc_hi, idesc_qk, k > 0 ? 1u : 0u);
        }
      };
      // O[slot] (+)= P[slot] * V with V in ring stage `st`; P is bf16 in TMEM (8 columns per 16 keys)
      auto issue_pv = [&](int s, int st, bool acc) {
        const uint32_t b = v_lo0 + st * tile16, d = tmem + 2 * kBlockN + s * D;
        const uint32_t a = kSepP ? tmem + 384 + s * 64 : tmem + s * kBlockN;
#pragma unroll
        for (int k = 0; k < kBlockN / 16; ++k)
          umma_ts_lohi(d, a + k * 8, b + k * 128, desc_hi, idesc_pv, (acc || k > 0) ? 1u : 0u);
      };
      auto ring_next = [&]() {
        if (++ring_st == kStages) {
          ring_st = 0;
          ring_par ^= 1;
        }
      };
      // The pipe runs only a couple of MMAs behind this thread, so whatever the thread does between the
      // last MMA of one slot and the first MMA of the other is a bubble in the tensor pipe. Between slots
      // there is therefore only the S-ready commit and the wait for the other slot's P; ring bookkeeping,
      // the waits for the next K/V tiles and the ring releases all sit at the end of a trip, after slot 1's
      // Q K^T, where this thread has nothing to issue until slot 0's next P arrives.
      // The first valid round at or after `from` (rounds in which this CTA has no item are skipped), or total_rounds.
      auto next_round = [&](int from, int& idx) {
        for (int r = from; r < p.total_rounds; ++r) {
          idx = item_for_round(p, r, blockIdx.x, gridDim.x);
          if (idx >= 0) return r;
        }
        idx = -1;
        return p.total_rounds;
      };
      // At the end of an item this thread would wait for slot 1's last P before it could turn to the next item, and
      // slot 0's softmax warps, done with their epilogue, would wait some 2 500 clocks for their first S. So when
      // slot 0's last P V has been issued, the next item's first Q K^T of that slot follows it at once - if the next
      // Q tile and the next item's first K tile have already arrived (tested, never waited for: this thread must
      // not stall in front of the other slot's products). S of the slot is free by then: its softmax warps have
      // published the last P, which the P V just issued reads and the new product, behind it in the pipe, overwrites.
      // Slot 0 only: doing the same for slot 1 brings the two slots' first tiles too close together, their softmaxes
      // run at the same time, and every shape measured 1-2 % slower.
      bool pre_issued0 = false;
      auto try_early_qk0 = [&](int n_next) {
        if (n_next == 0 || !mbar_test_wait(&kv_full[ring_st], ring_par) || !mbar_test_wait(&q_full[0], q_par[0]))
          return;
        q_par[0] ^= 1;
        tc_fence_after();
        issue_qk(0, ring_st);
        umma_commit(&s_full[0]);
        if (n_next == 1) umma_commit(&q_empty[0]);
        pre_issued0 = true;
      };
      int idx = -1, nidx = -1;
      int round = next_round(0, idx), nround = 0;
      WorkItem w, wn;
      if (idx >= 0) w = decode_item<CAUSAL>(p, idx);
      for (; ok && round < p.total_rounds; round = nround, w = wn) {
        // the item after this one, for the early issue of its first products
        nround = next_round(round + 1, nidx);
        wn.n[0] = wn.n[1] = 0;
        if (nidx >= 0) wn = decode_item<CAUSAL>(p, nidx);
        const int n0 = w.n[0], n1 = w.n[1];
        const int nmax = max(n0, n1);
        if (nmax == 0) continue;  // causal with more queries than keys: neither block sees a key
        // ---- first K tile: S = Q K0^T for both slots (a slot whose product was issued at the end of the previous
        // item is skipped; the tile's arrival has been seen then, and this wait returns at once)
        ok = mbar_wait(&kv_full[ring_st], ring_par, abortp, kWaitLimitCycles);
        if (!ok) break;
        if (n0 > 0 && !pre_issued0) {
          ok = mbar_wait(&q_full[0], q_par[0], abortp, kWaitLimitCycles);
          if (!ok) break;
          q_par[0] ^= 1;
          tc_fence_after();
          issue_qk(0, ring_st);
          umma_commit(&s_full[0]);
          if (n0 == 1) umma_commit(&q_empty[0]);
        }
        if (n1 > 0) {
          ok = mbar_wait(&q_full[1], q_par[1], abortp, kWaitLimitCycles);
          if (!ok) break;
          q_par[1] ^= 1;
          tc_fence_after();
          issue_qk(1, ring_st);
          umma_commit(&s_full[1]);
          if (n1 == 1) umma_commit(&q_empty[1]);
        }
        pre_issued0 = false;
        umma_commit(&kv_empty[ring_st]);
        ring_next();
        {
          // stages of V(0) and K(1)
          int st_v = ring_st;
          ok = mbar_wait(&kv_full[st_v], ring_par, abortp, kWaitLimitCycles);
          ring_next();
          int st_k = ring_st;
          if (ok && nmax > 1) {
            ok = mbar_wait(&kv_full[st_k], ring_par, abortp, kWaitLimitCycles);
            ring_next();
          }
          for (int j = 0; j < nmax && ok; ++j) {
            int nst_v = 0, nst_k = 0;
            // ---- slot 0
            if (j < n0) {
              ok = mbar_wait(&p_full[0], p_par[0], abortp, kWaitLimitCycles);
              if (!ok) break;
              p_par[0] ^= 1;
              HK_STAMP(2, 12);
              tc_fence_after();
              issue_pv(0, st_v, j > 0);
              if (j + 1 < n0) {
                issue_qk(0, st_k);
                umma_commit(&s_full[0]);
                HK_STAMP(2, 14);
                if (j + 2 == n0) umma_commit(&q_empty[0]);  // last QK of this slot: Q may be replaced
              } else {
                umma_commit(&o_full[0]);
              }
            }
            // ring_st is the next item's first K tile once no tile of this item is left to be waited for
            if (j + 1 == nmax) try_early_qk0(wn.n[0]);
            // ---- slot 1
            if (j < n1) {
              ok = mbar_wait(&p_full[1], p_par[1], abortp, kWaitLimitCycles);
              if (!ok) break;
              p_par[1] ^= 1;
              HK_STAMP(2, 13);
              tc_fence_after();
              issue_pv(1, st_v, j > 0);
            }
            if (j < n1) {
              if (j + 1 < n1) {
                issue_qk(1, st_k);
                umma_commit(&s_full[1]);
                HK_STAMP(2, 15);
                if (j + 2 == n1) umma_commit(&q_empty[1]);
              } else {
                umma_commit(&o_full[1]);
              }
            }
            // V(j) and K(j+1) were last read by the MMAs above. Their stages are released here, and the next trip's
            // tiles V(j+1), K(j+2) awaited here, at the end of the trip, where this thread would only be waiting for
            // the next P of slot 0 anyway. (In the middle of the trip a wait for a tile that is a little late held
            // up slot 1's Q K^T by some 300 clocks per tile; releases deferred to the next trip shortened the
            // producer's lead by a third of a period.)
            umma_commit(&kv_empty[st_v]);
            if (j + 1 < nmax) {
              umma_commit(&kv_empty[st_k]);
              nst_v = ring_st;
              ok = mbar_wait(&kv_full[nst_v], ring_par, abortp, kWaitLimitCycles);
              ring_next();
              if (ok && j + 2 < nmax) {
                nst_k = ring_st;
                ok = mbar_wait(&kv_full[nst_k], ring_par, abortp, kWaitLimitCycles);
                ring_next();
              }
              if (!ok) break;
            }
            st_v = nst_v;
            st_k = nst_k;
          }
        }
      }
    } else if (kQThread && warp == 11 && lane == 0) {
      // ---------------- Q loader (D = 64, non-causal): a thread of its own, so that the K/V producer never waits behind a Q
      // tile that cannot be replaced yet and requests the next item's first K/V tiles as early as the ring allows
      prefetch_tmap(&tmap_q);
      uint32_t q_cnt0 = 0, q_cnt1 = 0;
      bool ok = true;
      for (int round = 0; ok; ++round) {
        if (round >= p.total_rounds) break;
        const int idx = item_for_round(p, round, blockIdx.x, gridDim.x);
        if (idx < 0) continue;
        const WorkItem w = decode_item<CAUSAL>(p, idx);
        if (w.n[0] > 0) {
          ok = mbar_wait(&q_empty[0], (q_cnt0 & 1) ^ 1, abortp, kWaitLimitCycles);
          if (!ok) break;
          ++q_cnt0;
          mbar_expect_tx(&q_full[0], kTile);
#pragma unroll
          for (int ch = 0; ch < kChunks; ++ch)
            tma_load_4d(sQ + ch * kSub, &tmap_q, &q_full[0], ch * 64, w.head[0], w.qb[0] * kBlockM, w.b);
        }
        if (w.n[1] > 0) {
          ok = mbar_wait(&q_empty[1], (q_cnt1 & 1) ^ 1, abortp, kWaitLimitCycles);
          if (!ok) break;
          ++q_cnt1;
          mbar_expect_tx(&q_full[1], kTile);
#pragma unroll
          for (int ch = 0; ch < kChunks; ++ch)
            tma_load_4d(sQ + kTile + ch * kSub, &tmap_q, &q_full[1], ch * 64, w.head[1], w.qb[1] * kBlockM, w.b);
        }
      }
    } else if (kTmaOut && warp == 11 && lane == 0) {
      // ---------------- store thread: gives the staging tile to one slot at a time and sends what the slot wrote
      // there to global memory. Order of the turns: item by item and, inside an item, the slot with fewer K/V tiles
      // (which finishes first) before the other.
      prefetch_tmap(&tmap_o);
      uint32_t full_cnt0 = 0, full_cnt1 = 0;  // tiles sent so far, per slot
      bool ok = true;
      for (int round = 0; ok; ++round) {
        if (round >= p.total_rounds) break;
        const int idx = item_for_round(p, round, blockIdx.x, gridDim.x);
        if (idx < 0) continue;
        const WorkItem w = decode_item<CAUSAL>(p, idx);
        const int first = (w.n[1] < w.n[0]) ? 1 : 0;
        for (int t = 0; t < 2 && ok; ++t) {
          const int s = t == 0 ? first : 1 - first;
          // selects, not indexing with s: the item stays in registers
          const int n_s = s ? w.n[1] : w.n[0], head_s = s ? w.head[1] : w.head[0], qb_s = s ? w.qb[1] : w.qb[0];
          if (n_s == 0) continue;
          mbar_arrive(&so_turn[s]);
          ok = mbar_wait_parked(&so_full[s], (s ? full_cnt1 : full_cnt0) & 1, abortp, kWaitLimitCycles);
          if (!ok) break;
          full_cnt0 += s ? 0u : 1u;
          full_cnt1 += s ? 1u : 0u;
#pragma unroll
          for (int ch = 0; ch < kChunks; ++ch)
            tma_store_4d(&tmap_o, sOut + ch * kSub, ch * 64, head_s, qb_s * kBlockM, w.b);
          bulk_commit_group();
          bulk_wait_group_read0();  // the tile may be overwritten
        }
      }
      bulk_wait_group0();  // the last boxes have reached global memory
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
