// bf16 grouped-query flash-attention backward for sm_100a (B200).
//
// Replaces the reference's three backward entry points: attend_prep_ker
// (kernels/attn/gqa_backwards/attn_bkwd_prep.cpp:164-186, delta = rowsum(dO * O)),
// attend_bwd_combined_ker (kernels/attn/gqa_backwards/attn_bkwd_non_causal.cpp:48-49 and
// kernels/attn/gqa_causal_backwards/attn_bkwd_causal.cpp:50; dQ, dK, dV) and attend_dq_shuffle_ker
// (attn_bkwd_prep.cpp:199-223, dQ [B,H,N,D] -> [B,N,H,D]).
//
// With P = exp(scale * Q K^T - L), dP = dO V^T and dS = P * (dP - delta):
//     dV = P^T dO        dK = scale * dS^T Q        dQ = scale * dS K
// The reference accumulates dQ with packed-bf16 atomic adds from the kernel that owns a K/V block. Here
// nothing is accumulated across thread blocks: two kernels each own their outputs outright, which makes
// every gradient bit-reproducible from run to run, at the price of computing S and dP twice.
//   attn_bwd_dkdv_kernel  one K/V block of 128 keys stays in shared memory; the query tiles of all heads
//                         of the group stream past it. Everything is computed transposed (S^T = K Q^T,
//                         dP^T = V dO^T) so that the key index is the TMEM lane: P^T and dS^T are then
//                         already in the A-operand position of dV += P^T dO and dK += dS^T Q.
//   attn_bwd_dq_kernel    one query tile of 128 rows stays in shared memory; the K/V tiles stream past it:
//                         S = Q K^T, dP = dO V^T, dQ += dS K.
// Both kernels are persistent (one CTA per SM, 640 threads by default): warps 0-15 do the element-wise work
// (four threads per TMEM lane, 32 columns each), then one warp each for the TMA producer, the two UMMA-issuing
// roles and, in the dK/dV kernel, the loader of the per-row statistics.
// TMEM is laid out so that a score-shaped accumulator is free for the next product as soon as the element-wise
// warps hold it in registers (its bf16 successor goes elsewhere: see the column maps in the kernels).
//
// Any sequence length works (the reference's kernels need a multiple of 256): TMA zero-fills the rows of a partial
// last tile, their statistics are read as zero, and their gradient rows are not stored.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "attn_fwd_sm100.cuh"
#include "sm100_ptx.cuh"

// This header may be included more than once: the part that does not depend on the thread layout is compiled
// once; the main kernels and their helpers are compiled into namespace hk::HK_BWD_NS with HK_BWD_PARTS threads per
// TMEM lane, so that a translation unit can hold two layouts (the 8-warp one serves the causal instantiations,
// where it measured 3 to 7 % faster; the 16-warp one the others).
#ifndef HK_ATTN_BWD_SHARED_PART
#define HK_ATTN_BWD_SHARED_PART
namespace hk {

enum : int { kStatusSmemAlign = 3 };  // dynamic shared memory did not start on a 1024-byte boundary

// Of every kBwdEmuMod column pairs of a score row, kBwdEmuCnt take their exponentials from the cubic polynomial on the
// FMA pipe (ptx::ex2_poly2, relative error 1e-4, far inside the bf16 rounding of P and dS) instead of the MUFU.
#ifndef HK_BWD_EMU_MOD
#define HK_BWD_EMU_MOD 4
#endif
#ifndef HK_BWD_EMU_CNT
#define HK_BWD_EMU_CNT 1
#endif
constexpr int kBwdEmuMod = HK_BWD_EMU_MOD;
constexpr int kBwdEmuCnt = HK_BWD_EMU_CNT;

struct BwdParams {
  const float* lse;     // [B,H,1,N] from the forward pass (natural log)
  const float* delta;   // [B,H,1,N] rowsum(dO * O)
  __nv_bfloat16* dq;    // written through the three strides below
  __nv_bfloat16* dk;    // [B,NK,H_KV,D]
  __nv_bfloat16* dv;    // [B,NK,H_KV,D]
  long long dq_stride_b, dq_stride_n, dq_stride_h;  // elements; [B,N,H,D] or [B,H,N,D]
  int B, N, H, H_KV;    // N = query rows per batch element
  int NK;               // keys per batch element (N for self-attention)
  int n_items;
  int group_units;      // causal order: (batch, kv-head) units swept together (L2 residency)
  int group_items;      // work items of a full group (all items when there is one group)
  int rounds_per_group; // ceil(group_items / CTAs): a group is dealt in rounds of its own (see item_for_round)
  int total_rounds;     // rounds_per_group * number of groups
  // Item decode by multiply-and-shift division (see FastDiv), set per kernel by set_bwd_decode()
  int G;                // H / H_KV
  int last_group;       // index of the last causal sweep group (it may hold fewer units)
  FastDiv fd_rounds;    // rounds_per_group
  FastDiv fd_hkv;       // H_KV
  FastDiv fd_unit;      // items per unit: key blocks (dK/dV kernel) or G * query tiles (dQ kernel)
  FastDiv fd_inner;     // dQ kernel: query tiles (non-causal order) or G (causal order)
  FastDiv fd_group;     // causal: items of a full group
  FastDiv fd_in_grp, fd_in_grp_last;  // causal: items per key block / query tile in a full group, in the last group
  int n_pairs;          // causal dK/dV kernel: pairs of key blocks (j, NBK - 1 - j) over all units
  FastDiv fd_pairs;     // pairs per unit, (NBK + 1) / 2
  float scale;
  float scale_log2;
  const int* kv_lens;   // optional device [B]: batch b attends to keys [0, kv_lens[b]) only; null = NK
  int* status;
#ifdef HK_TRACE
  long long* trace;     // [4 roles][4096] clock stamps of CTA 0 (debug builds only)
#endif
};

template <int D>
struct BwdSmem {
  static constexpr int kTileBytes = kBlockM * D * 2;
  static constexpr int kSubTileBytes = kBlockM * 128;
  static constexpr int kRingA = (D == 128) ? 3 : 6;  // dK/dV kernel: Q tiles (live for a whole iteration)
  static constexpr int kRingB = (D == 128) ? 2 : 4;  // dK/dV kernel: dO tiles
  // dQ kernel: a K tile lives from S(n) to dQ(n), more than an iteration, so its ring is the deep one; a V tile is
  // consumed by one early product, and its successor is not needed for another ~1500 clocks: one stage is enough
  // at D = 128, where shared memory holds 7 tiles.
  static constexpr int kRingK = (D == 128) ? 4 : 7;
  static constexpr int kRingV = (D == 128) ? 1 : 3;
  static constexpr int kTiles = 2 + kRingA + kRingB;
  static_assert(2 + kRingK + kRingV == kTiles, "both kernels use the same shared-memory footprint");
  static constexpr int kStatBytes = 2 * 2 * kBlockM * 4;  // two stages of (L, delta) for one query tile
  static constexpr int kBarBytes = 512;
  static constexpr int kDynBytes = kTiles * kTileBytes + kStatBytes + kBarBytes;
};
static_assert(BwdSmem<128>::kDynBytes <= 232448, "shared memory budget of one CTA");

// ------------------------------------------------------------------------------------ delta = rowsum(dO * O)
// D/8 lanes per (batch, position, head) row, 16 bytes of O and of dO per lane; memory-bound (reads O and dO
// once). grid = ceil(B*N*H / rows per block), block = 256.
template <int D>
__global__ void __launch_bounds__(256) attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o,
                                                            const __nv_bfloat16* __restrict__ d_o,
                                                            float* __restrict__ delta, int B, int N, int H) {
  constexpr int kLanesPerRow = D / 8;               // 16 or 8
  constexpr int kRowsPerWarp = 32 / kLanesPerRow;   // 2 or 4
  const int lane = threadIdx.x & 31;
  const int sub = lane % kLanesPerRow;
  const long long row = (static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5)) * kRowsPerWarp + lane / kLanesPerRow;
  const long long rows = static_cast<long long>(B) * N * H;
  float acc = 0.f;
  if (row < rows) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(o + row * D) + sub);
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(d_o + row * D) + sub);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
    const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&aw[i]);
      const __nv_bfloat162 y = *reinterpret_cast<const __nv_bfloat162*>(&bw[i]);
      acc = fmaf(__low2float(x), __low2float(y), acc);
      acc = fmaf(__high2float(x), __high2float(y), acc);
    }
  }
#pragma unroll
  for (int off = kLanesPerRow / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (row < rows && sub == 0) {
    const long long bn = row / H;
    const int h = static_cast<int>(row - bn * H);
    const long long b = bn / N;
    const int n = static_cast<int>(bn - b * N);
    delta[(b * H + h) * N + n] = acc;
  }
}

// ------------------------------------------------------------------------------------ dQ [B,H,N,D] -> [B,N,H,D]
// Pure byte movement, 16 bytes per thread. grid = ceil(B*N*H*D/8 / 256), block = 256.
__global__ void __launch_bounds__(256) attn_dq_shuffle_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                              int B, int N, int H, int vec_per_row) {
  const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  const long long total = static_cast<long long>(B) * N * H * vec_per_row;
  if (idx >= total) return;
  // idx enumerates the destination [B,N,H,vec]
  const int v = static_cast<int>(idx % vec_per_row);
  long long r = idx / vec_per_row;
  const int h = static_cast<int>(r % H);
  r /= H;
  const int n = static_cast<int>(r % N);
  const long long b = r / N;
  dst[idx] = src[((b * H + h) * N + n) * vec_per_row + v];
}

// Dynamic shared memory of both main kernels: tiles first (1024-byte aligned for the 128-byte swizzle),
// then the (L, delta) stages, then the mbarriers and two control words.
}  // namespace hk
#endif  // HK_ATTN_BWD_SHARED_PART

#ifndef HK_BWD_NS
#define HK_BWD_NS bwd_layout
#endif
namespace hk {
namespace HK_BWD_NS {


// Element-wise warps: kBwdParts threads share one TMEM lane (one score row), each owning 128 / kBwdParts columns.
// 4 parts = 16 element-wise warps (4 per scheduler) in a 640-thread CTA without register re-allocation; 2 parts =
// 8 warps in a 384-thread CTA that re-balances registers like the forward kernel. Sixteen warps measured 1 to 2 %
// faster on the non-causal shapes, eight 3 to 7 % faster on the causal ones (every barrier the issuers wait for
// collects half as many arrivals); 4 is the default when nothing is said.
#ifndef HK_BWD_PARTS
#define HK_BWD_PARTS 4
#endif
constexpr int kBwdParts = HK_BWD_PARTS;
static_assert(kBwdParts == 2 || kBwdParts == 4, "2 or 4 threads per TMEM lane");
constexpr int kBwdCW = 4 * kBwdParts;              // element-wise warps
constexpr int kBwdPC = 128 / kBwdParts;            // score columns per element-wise thread
constexpr int kBwdThreads = 32 * (kBwdCW + 4);     // + TMA producer, two UMMA issuers, statistics loader (idle in dQ)
// Register budget: all warps start with kBwdRegsAtLaunch; the element-wise warps then grow by exactly what the
// other four warps give up (setmaxnreg only moves registers inside the CTA's own allocation: asking for more than
// was released would block forever): 8 x (208 - 168) = 4 x (168 - 88). With 4 parts (640 threads) every thread keeps
// its 96 registers: the element-wise code fits, and no re-allocation is done.
constexpr int kBwdRegsAtLaunch = kBwdParts == 2 ? 168 : 96;
constexpr int kBwdRegsGrown = kBwdParts == 2 ? 208 : 96;
constexpr int kBwdRegsShrunk = kBwdParts == 2 ? 88 : 96;
static_assert(kBwdCW * (kBwdRegsGrown - kBwdRegsAtLaunch) == 4 * (kBwdRegsAtLaunch - kBwdRegsShrunk),
              "registers taken by the element-wise warps must equal the registers released by the other warps");

// kBwdPC fp32 columns of this thread's lane -> registers / kBwdPC/2 packed bf16 columns -> TMEM
__device__ __forceinline__ void bwd_ld_part(uint32_t taddr, uint32_t* r) {
#pragma unroll
  for (int c = 0; c < kBwdPC / 32; ++c) ptx::tmem_ld32(taddr + c * 32, r + c * 32);
}
__device__ __forceinline__ void bwd_st_packed(uint32_t taddr, const uint32_t* r) {
  if constexpr (kBwdPC == 64) ptx::tmem_st32(taddr, r);
  else ptx::tmem_st16(taddr, r);
}
__device__ __forceinline__ void bwd_grow_registers() {
  if constexpr (kBwdParts == 2) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    static_assert(kBwdParts != 2 || kBwdRegsGrown == 208, "keep the immediate above in step");
  }
}
__device__ __forceinline__ void bwd_shrink_registers() {
  if constexpr (kBwdParts == 2) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
    static_assert(kBwdParts != 2 || kBwdRegsShrunk == 88, "keep the immediate above in step");
  }
}

// ------------------------------------------------------------------------------------ shared helpers
// The two UMMA-issuing roles run either as one thread (lane 0 of their warp) or as a whole warp that keeps
// its control flow and descriptor arithmetic warp-uniform and elects one lane per group of tcgen05 instructions
// (measured 1.5 to 4 % faster on every backward shape tried; the same change to the forward kernel's single
// issuer measured equal at D = 128 and 8 % slower at D = 64, so the forward kernel keeps its one thread).
#ifndef HK_BWD_WARP_ISSUE
#define HK_BWD_WARP_ISSUE 1
#endif
constexpr bool kBwdWarpIssue = HK_BWD_WARP_ISSUE != 0;
__device__ __forceinline__ bool iss_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                         uint64_t limit_cycles) {
  bool ok = ptx::mbar_wait(bar, parity, abort_flag, limit_cycles);
  if (kBwdWarpIssue) ok = __all_sync(0xffffffffu, ok);
  return ok;
}
__device__ __forceinline__ bool iss_elect() { return !kBwdWarpIssue || ptx::elect_one(); }
// S-shaped product with both operands in shared memory, K-major, 128 B swizzle: d[128 x 128] = a * b^T
// over D. `a_lo` / `b_lo` are descriptor low words of the two 128 x D tiles.
template <int D>
__device__ __forceinline__ void bwd_issue_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo) {
  constexpr uint32_t idesc = ptx::make_idesc_bf16(kBlockM, kBlockN, false);
  constexpr uint32_t desc_hi = ptx::smem_desc_hi(1024);
  constexpr uint32_t sub16 = BwdSmem<D>::kSubTileBytes >> 4;
#pragma unroll
  for (int k = 0; k < D / 16; ++k) {
    const uint32_t off = (k / 4) * sub16 + (k % 4) * 2;  // 32 bytes per 16-element step inside a 128-byte row
    ptx::umma_ss_lohi(d_tmem, a_lo + off, b_lo + off, desc_hi, idesc, k > 0 ? 1u : 0u);
  }
}
// Gradient-shaped product: d[128 x D] (+)= a * b, a = bf16 [128 x 128] in TMEM (each of the kBwdParts thread
// groups of a row keeps its packed columns inside the kBwdPC columns it owns, starting at `a_tmem`),
// b = a 128 x D tile in shared memory read MN-major (its rows are the contraction index).
template <int D>
__device__ __forceinline__ void bwd_issue_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo_mn, bool acc) {
  constexpr uint32_t idesc = ptx::make_idesc_bf16(kBlockM, D, true);
  constexpr uint32_t desc_hi = ptx::smem_desc_hi(1024);
#pragma unroll
  for (int k = 0; k < kBlockN / 16; ++k)
    ptx::umma_ts_lohi(d_tmem, a_tmem + ((16 * k) / kBwdPC) * kBwdPC + ((16 * k) % kBwdPC) / 2, b_lo_mn + k * 128,
                      desc_hi, idesc, (acc || k > 0) ? 1u : 0u);
}

// Accumulator rows (this thread's TMEM lane, D / kBwdParts columns from `taddr`) -> bf16 -> global, scaled.
template <int D>
__device__ __forceinline__ void bwd_store_part_row(uint32_t taddr, __nv_bfloat16* dst, float mul, bool row_exists) {
  constexpr int kCols = D / kBwdParts;  // 64, 32 or 16
  constexpr int kChunk = kCols >= 32 ? 32 : 16;
#pragma unroll
  for (int cc = 0; cc < kCols / kChunk; ++cc) {
    uint32_t o[kChunk];
    if constexpr (kChunk == 32) ptx::tmem_ld32(taddr + cc * 32, o);
    else ptx::tmem_ld16(taddr, o);
    ptx::tmem_wait_ld();
    if (!row_exists) continue;  // the TMEM load above is warp-collective, the store is per row
    uint32_t r[kChunk / 2];
#pragma unroll
    for (int i = 0; i < kChunk / 2; ++i)
      r[i] = ptx::pack_bf16x2(__uint_as_float(o[2 * i]) * mul, __uint_as_float(o[2 * i + 1]) * mul);
    __nv_bfloat16* out = dst + cc * kChunk;
    // 32 bytes per store where the row allows it: each thread writes a row of its own, so every store instruction
    // touches 32 separate lines, and half as many instructions is half the time in the store unit
    if ((reinterpret_cast<uintptr_t>(out) & 31) == 0) {
#pragma unroll
      for (int v8 = 0; v8 < kChunk / 16; ++v8) ptx::st_global_v8(out + v8 * 16, r + v8 * 8);
    } else {
#pragma unroll
      for (int v4 = 0; v4 < kChunk / 8; ++v4)
        reinterpret_cast<uint4*>(out)[v4] = make_uint4(r[v4 * 4], r[v4 * 4 + 1], r[v4 * 4 + 2], r[v4 * 4 + 3]);
    }
  }
}

// ------------------------------------------------------------------------------------ dK, dV
struct DkdvItem {
  int b, kvh, j;   // batch, kv head, key block
  int kv_len;      // keys this batch element attends to
  int off;         // causal: query row r sees keys [0, r + off], off = kv_len - N (the reference aligns the mask to
                   // the last query and the last kept key, training/llama/llama/models/attentions/base.py:104-116)
  int i_min;       // first query tile this key block meets
  int cnt_i;       // query tiles per head this key block meets
  int n_iter;      // heads of the group x query tiles; 0 for a key block nobody sees (beyond kv_len, or causal
                   // with every query before it)
};

// Work order: one (batch, kv head) unit's key blocks are adjacent so that the CTAs running at the same
// time read the same Q / dO tiles from L2; an item index is unit * key blocks + key block.
//
// Causal: key block j meets G * (NBQ - j) query tiles, 64 times more for the first block than for the last at
// N = 8192, and a unit has fewer blocks than the GPU has SMs, so no dealing of single blocks to CTAs balances. The
// blocks are therefore dealt in pairs (j, NBK - 1 - j) of the same unit, which all cost the same: a CTA's round 2r
// is the first block of its r-th pair and round 2r + 1 the second (none for the middle block of an odd count).
template <bool CAUSAL>
__device__ __forceinline__ int dkdv_item_for_round(const BwdParams& p, int round, int cta, int n_cta) {
  if (!CAUSAL) return item_for_round(p, round, cta, n_cta);
  const int pair = (round >> 1) * n_cta + cta;
  if (pair >= p.n_pairs) return -1;
  int unit, jp;
  p.fd_pairs.divmod(pair, unit, jp);
  const int nbk = static_cast<int>(p.fd_unit.d);
  const int j = (round & 1) ? nbk - 1 - jp : jp;
  if ((round & 1) && j == jp) return -1;
  return unit * nbk + j;
}

template <bool CAUSAL>
__device__ __forceinline__ DkdvItem decode_dkdv_item(const BwdParams& p, int idx) {
  DkdvItem w;
  const int NBQ = (p.N + kBlockM - 1) / kBlockM;   // query tiles
  int unit;
  p.fd_unit.divmod(idx, unit, w.j);
  p.fd_hkv.divmod(unit, w.b, w.kvh);
  w.kv_len = p.kv_lens ? min(max(p.kv_lens[w.b], 1), p.NK) : p.NK;
  w.off = w.kv_len - p.N;
  // causal: key c is seen by query rows r >= c - off; the first key of the block, j*128, is the one seen by most
  w.i_min = CAUSAL ? max(w.j * kBlockN - w.off, 0) / kBlockM : 0;
  w.cnt_i = max(NBQ - w.i_min, 0);
  w.n_iter = (w.j * kBlockN >= w.kv_len) ? 0 : p.G * w.cnt_i;
  return w;
}

template <int D, bool CAUSAL>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                     const BwdParams p) {
  using namespace ptx;
  using SM = BwdSmem<D>;
  constexpr int kTile = SM::kTileBytes;
  constexpr int kSub = SM::kSubTileBytes;
  constexpr int kChunks = D / 64;
  constexpr int RA = SM::kRingA, RB = SM::kRingB;
  enum { KV_FULL = 0, KV_EMPTY, ST_FULL, DP_FULL, P_FULL, DS_FULL, ACC_FULL, S_FREE, QA_FULL = 8, QA_EMPTY = 14,
         RB_FULL = 20, RB_EMPTY = 24, STAT_FULL = 28, STAT_EMPTY = 30, DP_FREE = 32, Y_FREE = 33, CTRL = 34 };
  static_assert(RA <= 6 && RB <= 4, "barrier slots");

  extern __shared__ __align__(1024) uint8_t bwd_smem[];
  uint8_t* sK = bwd_smem;
  uint8_t* sV = bwd_smem + kTile;
  uint8_t* sQ = bwd_smem + 2 * kTile;          // RA stages
  uint8_t* sDO = sQ + RA * kTile;              // RB stages
  float* sStat = reinterpret_cast<float*>(bwd_smem + SM::kTiles * kTile);  // [2 stages][-L log2e 128 | -delta 128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(bwd_smem + SM::kTiles * kTile + SM::kStatBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + CTRL);
  uint32_t* abort_word = tmem_slot + 1;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if ((smem_u32(bwd_smem) & 1023u) != 0) {  // uniform over the CTA; nothing has been allocated yet
    if (tid == 0) atomicCAS(p.status, kStatusOk, kStatusSmemAlign);
    return;
  }
  if (tid == 0) {
    *abort_word = 0;
    mbar_init(bars + KV_FULL, 1);
    mbar_init(bars + KV_EMPTY, 1);  // K and V only feed issuer A's products
    mbar_init(bars + ST_FULL, 1);
    mbar_init(bars + DP_FULL, 1);
    mbar_init(bars + P_FULL, kBwdCW);    // one arrival per element-wise warp
    mbar_init(bars + DS_FULL, kBwdCW);
    mbar_init(bars + S_FREE, kBwdCW);
    mbar_init(bars + DP_FREE, kBwdCW);
    mbar_init(bars + Y_FREE, 1);
    mbar_init(bars + ACC_FULL, 1);
    for (int s = 0; s < RA; ++s) {
      mbar_init(bars + QA_FULL + s, 1);
      mbar_init(bars + QA_EMPTY + s, 1);
    }
    for (int s = 0; s < RB; ++s) {
      mbar_init(bars + RB_FULL + s, 1);
      mbar_init(bars + RB_EMPTY + s, 2);  // dO feeds dP^T (issuer A) and dV (issuer B)
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bars + STAT_FULL + s, 1);   // one arrival by the statistics loader warp
      mbar_init(bars + STAT_EMPTY + s, kBwdCW);
    }
    fence_mbar_init();
  }
  if (warp == kBwdCW) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  volatile uint32_t* abortp = abort_word;
  const int G = p.G;
  // TMEM columns: X [0,128) takes the two score-shaped products in turn, S^T(n) then dP^T(n), each free again as soon
  // as the element-wise warps hold it in registers; Y [128,256) holds the two bf16 operands, P^T in [128,192) and dS^T
  // in [192,256), free again when dV(n) and dK(n) have consumed them; dK [256,256+D); dV [256+D,256+2D). Nothing
  // fp32 aliases anything bf16, so no product has to wait behind another one's operands.
  // With D = 64 the accumulators leave 128 columns over: dP^T then gets a region of its own, [384,512), so that
  // S^T(n+1) only waits for S^T(n) to be read and dP^T(n+1) for dP^T(n), and both products are in flight long before
  // the element-wise warps need them (kSplitX).
  constexpr bool kSplitX = (D == 64);
  constexpr uint32_t cX = 0, cY = 128, cDK = 256, cDV = 256 + D;
  constexpr uint32_t cXdP = kSplitX ? 384 : cX;

  if (warp < kBwdCW) {
    // ------------------------------------------------------------------ element-wise warps
    bwd_grow_registers();
    const int part = warp >> 2;                        // which kBwdPC query columns of the tile
    const int row = (warp & 3) * 32 + lane;            // key row inside the block == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tX = tmem + lane_addr + cX + part * kBwdPC;
    const uint32_t tXdP = tmem + lane_addr + cXdP + part * kBwdPC;
    const uint32_t tPt = tmem + lane_addr + cY + part * (kBwdPC / 2);        // this thread's packed columns of P^T
    const uint32_t tDSt = tmem + lane_addr + cY + 64 + part * (kBwdPC / 2);  // ... and of dS^T
    const float c = p.scale_log2;
    uint32_t it = 0, acc_cnt = 0;
    bool ok = true;
#ifdef HK_TRACE
#ifndef HK_TRACE_WARP
#define HK_TRACE_WARP (kBwdCW - 1)
#endif
    const bool trace_on = (warp == 0 || warp == HK_TRACE_WARP) && lane == 0 && p.trace != nullptr;
    const int trole = warp == 0 ? 0 : 1;  // first and last element-wise warp: their distance is the skew between warps
    int trace_n = 0;
#endif
    for (int round = 0; ok; ++round) {
      if (round >= p.total_rounds) break;
      const int idx = dkdv_item_for_round<CAUSAL>(p, round, blockIdx.x, gridDim.x);
      if (idx < 0) continue;  // a partial round leaves some CTAs without an item
      const DkdvItem w = decode_dkdv_item<CAUSAL>(p, idx);
      const bool pad_row = w.j * kBlockN + row >= w.kv_len;  // this key is padding (or lies beyond NK)
      const bool pad_block = (w.j + 1) * kBlockN > w.kv_len;  // uniform over the CTA: only such a block has padded keys
      if (w.n_iter == 0) {
        // nobody sees this key block (padding, or causal with every query before it): its gradients are zero and no
        // product was issued for it
        if (w.j * kBlockN + row < p.NK) {
          const size_t off =
              ((static_cast<size_t>(w.b) * p.NK + w.j * kBlockN + row) * p.H_KV + w.kvh) * D + part * (D / kBwdParts);
#pragma unroll
          for (int v = 0; v < D / kBwdParts / 8; ++v) {
            reinterpret_cast<uint4*>(p.dk + off)[v] = make_uint4(0, 0, 0, 0);
            reinterpret_cast<uint4*>(p.dv + off)[v] = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      // i_rel: position of the pair's query tile among the cnt_i tiles of its head (n % cnt_i, without the division)
      for (int n = 0, i_rel = 0; n < w.n_iter && ok; ++n, ++it, i_rel = (i_rel + 1 == w.cnt_i) ? 0 : i_rel + 1) {
        HK_STAMP(trole, 0);
        // a query tile the diagonal runs through: its first row does not see the block's last key (with an offset
        // that is not a multiple of the tile these are two tiles per head, else the one at the block's own position)
        const int i_t = w.i_min + i_rel;
        const bool diag = CAUSAL && (i_t * kBlockM + w.off < w.j * kBlockN + kBlockN - 1);
        const float* sL = sStat + (it & 1) * 256 + part * kBwdPC;
        const float* sDl = sL + 128;
        // ---- S^T into registers; X is free for dP^T of this pair right away
        ok = mbar_wait(bars + ST_FULL, it & 1, abortp, kWaitLimitCycles) &&
             mbar_wait(bars + STAT_FULL + (it & 1), (it >> 1) & 1, abortp, kWaitLimitCycles);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        HK_STAMP(trole, 1);
        uint32_t su[kBwdPC];
        bwd_ld_part(tX, su);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + S_FREE);
        // ---- p = exp2(s * c - L * log2(e)), kept in fp32 for dS (two columns per packed fp32x2 instruction)
        {
          const uint64_t c2 = pack2(c, c);
#pragma unroll
          for (int q4 = 0; q4 < kBwdPC / 4; ++q4) {
            const float4 l4 = *reinterpret_cast<const float4*>(sL + q4 * 4);  // -L * log2(e) of four query columns
            const uint64_t xa = fma2(pack2(__uint_as_float(su[q4 * 4 + 0]), __uint_as_float(su[q4 * 4 + 1])), c2,
                                     pack2(l4.x, l4.y));
            const uint64_t xb = fma2(pack2(__uint_as_float(su[q4 * 4 + 2]), __uint_as_float(su[q4 * 4 + 3])), c2,
                                     pack2(l4.z, l4.w));
            float x0, x1, x2, x3;
            // all 16 compute warps take their exponentials at the same time, which makes this phase MUFU-bound
            // (16 results per clock and SM): a share of the column pairs goes through the FMA-pipe polynomial
            if ((2 * q4) % kBwdEmuMod < kBwdEmuCnt) unpack2(ex2_poly2(xa), x0, x1);
            else {
              unpack2(xa, x0, x1);
              x0 = ex2_approx(x0);
              x1 = ex2_approx(x1);
            }
            if ((2 * q4 + 1) % kBwdEmuMod < kBwdEmuCnt) unpack2(ex2_poly2(xb), x2, x3);
            else {
              unpack2(xb, x2, x3);
              x2 = ex2_approx(x2);
              x3 = ex2_approx(x3);
            }
            su[q4 * 4 + 0] = __float_as_uint(x0);
            su[q4 * 4 + 1] = __float_as_uint(x1);
            su[q4 * 4 + 2] = __float_as_uint(x2);
            su[q4 * 4 + 3] = __float_as_uint(x3);
          }
          if (diag) {
            // key j*128 + row is seen by query i_t*128 + col iff key <= query + off: earlier queries see nothing
            // (this also zeroes the infinities that rows without any key, whose L is -inf, produce above)
            const int lim = row + (w.j - i_t) * kBlockN - w.off;
#pragma unroll
            for (int col = 0; col < kBwdPC; ++col) su[col] = (part * kBwdPC + col) < lim ? 0u : su[col];
          }
          if (pad_block) {
            // a padded key is seen by nobody: P^T and dS^T rows are zero, so are its dK and dV rows
#pragma unroll
            for (int col = 0; col < kBwdPC; ++col) su[col] = pad_row ? 0u : su[col];
          }
        }
        HK_STAMP(trole, 2);
        // ---- dP^T into registers; X is free for S^T of the next pair
        ok = mbar_wait(bars + DP_FULL, it & 1, abortp, kWaitLimitCycles);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        HK_STAMP(trole, 3);
        uint32_t du[kBwdPC];
        bwd_ld_part(tXdP, du);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + DP_FREE);
        // ---- Y is free once dV and dK of the previous pair have consumed their operands (first pair ever: at once)
        ok = mbar_wait(bars + Y_FREE, (it & 1) ^ 1, abortp, kWaitLimitCycles);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        {
          uint32_t pk[kBwdPC / 2];
#pragma unroll
          for (int i = 0; i < kBwdPC / 2; ++i)
            pk[i] = pack_bf16x2(__uint_as_float(su[2 * i]), __uint_as_float(su[2 * i + 1]));
          bwd_st_packed(tPt, pk);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + P_FULL);
        HK_STAMP(trole, 4);
        // ---- dS^T = P^T * (dP^T - delta)
        {
          uint32_t pk[kBwdPC / 2];
#pragma unroll
          for (int q4 = 0; q4 < kBwdPC / 4; ++q4) {
            const float4 d4 = *reinterpret_cast<const float4*>(sDl + q4 * 4);  // -delta of four query columns
            const uint64_t ta = add2(pack2(__uint_as_float(du[q4 * 4 + 0]), __uint_as_float(du[q4 * 4 + 1])),
                                     pack2(d4.x, d4.y));
            const uint64_t tb = add2(pack2(__uint_as_float(du[q4 * 4 + 2]), __uint_as_float(du[q4 * 4 + 3])),
                                     pack2(d4.z, d4.w));
            float ds0, ds1, ds2, ds3;
            unpack2(mul2(pack2(__uint_as_float(su[q4 * 4 + 0]), __uint_as_float(su[q4 * 4 + 1])), ta), ds0, ds1);
            unpack2(mul2(pack2(__uint_as_float(su[q4 * 4 + 2]), __uint_as_float(su[q4 * 4 + 3])), tb), ds2, ds3);
            pk[q4 * 2] = pack_bf16x2(ds0, ds1);
            pk[q4 * 2 + 1] = pack_bf16x2(ds2, ds3);
          }
          bwd_st_packed(tDSt, pk);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bars + DS_FULL);
          mbar_arrive(bars + STAT_EMPTY + (it & 1));
        }
        HK_STAMP(trole, 5);
      }
      if (!ok) break;
      // ---- epilogue: dK = scale * acc, dV = acc
      ok = mbar_wait(bars + ACC_FULL, acc_cnt & 1, abortp, kWaitLimitCycles);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ++acc_cnt;
      tc_fence_after();
      const size_t off = ((static_cast<size_t>(w.b) * p.NK + w.j * kBlockN + row) * p.H_KV + w.kvh) * D + part * (D / kBwdParts);
      const bool row_exists = w.j * kBlockN + row < p.NK;  // keys of a partial last block beyond NK are computed, not stored
      bwd_store_part_row<D>(tmem + lane_addr + cDK + part * (D / kBwdParts), p.dk + off, p.scale, row_exists);
      bwd_store_part_row<D>(tmem + lane_addr + cDV + part * (D / kBwdParts), p.dv + off, 1.0f, row_exists);
      tc_fence_before();  // orders these reads before the next item's first dV product (published through P_FULL)
    }
  } else {
    bwd_shrink_registers();
    if (warp == kBwdCW && lane == 0) {
      // ---------------- TMA producer
      prefetch_tmap(&tmap_q);
      prefetch_tmap(&tmap_k);
      prefetch_tmap(&tmap_v);
      prefetch_tmap(&tmap_do);
      uint32_t item_cnt = 0;
      int qa = 0, rb = 0;
      uint32_t qa_par = 0, rb_par = 0;
      bool ok = true;
      for (int round = 0; ok; ++round) {
        if (round >= p.total_rounds) break;
        const int idx = dkdv_item_for_round<CAUSAL>(p, round, blockIdx.x, gridDim.x);
        if (idx < 0) continue;  // a partial round leaves some CTAs without an item
        const DkdvItem w = decode_dkdv_item<CAUSAL>(p, idx);
        if (w.n_iter == 0) continue;  // key block wholly beyond this batch element's length: nothing to do
        ok = mbar_wait(bars + KV_EMPTY, (item_cnt & 1) ^ 1, abortp, kWaitLimitCycles);
        if (!ok) break;
        ++item_cnt;
        mbar_expect_tx(bars + KV_FULL, 2 * kTile);
#pragma unroll
        for (int ch = 0; ch < kChunks; ++ch) {
          tma_load_4d(sK + ch * kSub, &tmap_k, bars + KV_FULL, ch * 64, w.kvh, w.j * kBlockN, w.b);
          tma_load_4d(sV + ch * kSub, &tmap_v, bars + KV_FULL, ch * 64, w.kvh, w.j * kBlockN, w.b);
        }
        for (int n = 0, g_rel = 0, i_rel = 0; n < w.n_iter && ok; ++n) {
          const int head = w.kvh * G + g_rel;  // n / cnt_i and n % cnt_i, counted instead of divided
          const int i = w.i_min + i_rel;
          if (++i_rel == w.cnt_i) {
            i_rel = 0;
            ++g_rel;
          }
          ok = mbar_wait(bars + QA_EMPTY + qa, qa_par ^ 1, abortp, kWaitLimitCycles);
          if (!ok) break;
          mbar_expect_tx(bars + QA_FULL + qa, kTile);
#pragma unroll
          for (int ch = 0; ch < kChunks; ++ch)
            tma_load_4d(sQ + qa * kTile + ch * kSub, &tmap_q, bars + QA_FULL + qa, ch * 64, head, i * kBlockM, w.b);
          if (++qa == RA) {
            qa = 0;
            qa_par ^= 1;
          }
          ok = mbar_wait(bars + RB_EMPTY + rb, rb_par ^ 1, abortp, kWaitLimitCycles);
          if (!ok) break;
          mbar_expect_tx(bars + RB_FULL + rb, kTile);
#pragma unroll
          for (int ch = 0; ch < kChunks; ++ch)
            tma_load_4d(sDO + rb * kTile + ch * kSub, &tmap_do, bars + RB_FULL + rb, ch * 64, head, i * kBlockM, w.b);
          if (++rb == RB) {
            rb = 0;
            rb_par ^= 1;
          }
        }
      }
    } else if (warp == kBwdCW + 1 && (kBwdWarpIssue || lane == 0)) {
      // ---------------- UMMA issuer A: the two score-shaped products, S^T = K Q^T and dP^T = V dO^T, which take
      // turns in X: each is issued as soon as the element-wise warps have read its predecessor.
      // Two threads issue because a thread that issues returns only a few MMAs ahead of the pipe: with one issuer
      // every commit and mbarrier wait between two products (~180 clocks) let the pipe run dry.
      constexpr uint32_t tile16 = kTile >> 4;
      const uint32_t k_lo = smem_desc_lo(smem_u32(sK), 16);
      const uint32_t v_lo = smem_desc_lo(smem_u32(sV), 16);
      const uint32_t q_lo0 = smem_desc_lo(smem_u32(sQ), 16);       // K-major view (B of S^T)
      const uint32_t do_lo0 = smem_desc_lo(smem_u32(sDO), 16);     // K-major view (B of dP^T)
      uint32_t item_cnt = 0, it = 0;
      int qa = 0, rb = 0;
      uint32_t qa_par = 0, rb_par = 0;
      bool ok = true;
#ifdef HK_TRACE
      const bool trace_on = p.trace != nullptr && lane == 0;
      int trace_n = 0;
#endif
      for (int round = 0; ok; ++round) {
        if (round >= p.total_rounds) break;
        const int idx = dkdv_item_for_round<CAUSAL>(p, round, blockIdx.x, gridDim.x);
        if (idx < 0) continue;  // a partial round leaves some CTAs without an item
        const DkdvItem w = decode_dkdv_item<CAUSAL>(p, idx);
        if (w.n_iter == 0) continue;  // key block wholly beyond this batch element's length: nothing to do
        ok = iss_wait(bars + KV_FULL, item_cnt & 1, abortp, kWaitLimitCycles);
        if (!ok) break;
        ++item_cnt;
        for (int n = 0; n < w.n_iter && ok; ++n, ++it) {
          // S^T(n): dP^T of the previous pair has been read out of X (first pair ever: passes at once); with a
          // region of its own, S^T(n) only waits for S^T(n-1) to be read
          ok = iss_wait(bars + (kSplitX ? S_FREE : DP_FREE), (it & 1) ^ 1, abortp, kWaitLimitCycles) &&
               iss_wait(bars + QA_FULL + qa, qa_par, abortp, kWaitLimitCycles);
          if (!ok) break;
          tc_fence_after();
          HK_STAMP(2, 12);
          if (iss_elect()) {
            bwd_issue_ss<D>(tmem + cX, k_lo, q_lo0 + qa * tile16);
            umma_commit(bars + ST_FULL);
          }
          HK_STAMP(2, 13);
          if (++qa == RA) {
            qa = 0;
            qa_par ^= 1;
          }
          // dP^T(n): S^T(n) has been read out of X (own region: dP^T(n-1) has been read)
          ok = iss_wait(bars + (kSplitX ? DP_FREE : S_FREE), kSplitX ? ((it & 1) ^ 1) : (it & 1), abortp,
                        kWaitLimitCycles) &&
               iss_wait(bars + RB_FULL + rb, rb_par, abortp, kWaitLimitCycles);
          if (!ok) break;
          tc_fence_after();
          if (iss_elect()) {
            bwd_issue_ss<D>(tmem + cXdP, v_lo, do_lo0 + rb * tile16);
            umma_commit(bars + DP_FULL);
            umma_commit(bars + RB_EMPTY + rb);  // first of two arrivals (issuer B: after dV of this stage)
          }
          HK_STAMP(2, 17);
          if (++rb == RB) {
            rb = 0;
            rb_par ^= 1;
          }
        }
        if (!ok) break;
        if (iss_elect()) umma_commit(bars + KV_EMPTY);
      }
    } else if (warp == kBwdCW + 2 && (kBwdWarpIssue || lane == 0)) {
      // ---------------- UMMA issuer B: the two gradient-shaped products, dV += P^T dO and dK += dS^T Q
      constexpr uint32_t tile16 = kTile >> 4;
      constexpr uint32_t idesc = make_idesc_bf16(kBlockM, D, true);
      constexpr uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t q_mn0 = smem_desc_lo(smem_u32(sQ), kSub);     // MN-major view (B of dK)
      const uint32_t do_mn0 = smem_desc_lo(smem_u32(sDO), kSub);   // MN-major view (B of dV)
      uint32_t it = 0;
      int qa = 0, rb = 0;
      uint32_t qa_par = 0, rb_par = 0;
      bool ok = true;
#ifdef HK_TRACE
      const bool trace_on = p.trace != nullptr && lane == 0;
      int trace_n = 0;
#endif
      for (int round = 0; ok; ++round) {
        if (round >= p.total_rounds) break;
        const int idx = dkdv_item_for_round<CAUSAL>(p, round, blockIdx.x, gridDim.x);
        if (idx < 0) continue;  // a partial round leaves some CTAs without an item
        const DkdvItem w = decode_dkdv_item<CAUSAL>(p, idx);
        if (w.n_iter == 0) continue;  // key block wholly beyond this batch element's length: nothing to do
        for (int n = 0; n < w.n_iter && ok; ++n, ++it) {
          ok = iss_wait(bars + P_FULL, it & 1, abortp, kWaitLimitCycles) &&
               iss_wait(bars + RB_FULL + rb, rb_par, abortp, kWaitLimitCycles);
          if (!ok) break;
          tc_fence_after();
          HK_STAMP(3, 10);
          if (iss_elect()) {
            const uint32_t b_lo = do_mn0 + rb * tile16;
#pragma unroll
            for (int k = 0; k < kBlockN / 16; ++k)
              umma_ts_lohi(tmem + cDV, tmem + cY + k * 8, b_lo + k * 128, desc_hi, idesc, (n > 0 || k > 0) ? 1u : 0u);
            umma_commit(bars + RB_EMPTY + rb);  // second of two arrivals
          }
          HK_STAMP(3, 11);
          if (++rb == RB) {
            rb = 0;
            rb_par ^= 1;
          }
          ok = iss_wait(bars + DS_FULL, it & 1, abortp, kWaitLimitCycles) &&
               iss_wait(bars + QA_FULL + qa, qa_par, abortp, kWaitLimitCycles);
          if (!ok) break;
          tc_fence_after();
          HK_STAMP(3, 14);
          if (iss_elect()) {
            const uint32_t b_lo = q_mn0 + qa * tile16;
#pragma unroll
            for (int k = 0; k < kBlockN / 16; ++k)
              umma_ts_lohi(tmem + cDK, tmem + cY + 64 + k * 8, b_lo + k * 128, desc_hi, idesc, (n > 0 || k > 0) ? 1u : 0u);
            // S^T of this stage (issuer A) completed before dS^T could be computed, so this one arrival frees Q
            umma_commit(bars + QA_EMPTY + qa);
            umma_commit(bars + Y_FREE);
          }
          HK_STAMP(3, 15);
          if (++qa == RA) {
            qa = 0;
            qa_par ^= 1;
          }
        }
        if (!ok) break;
        if (iss_elect()) umma_commit(bars + ACC_FULL);
      }
    } else if (warp == kBwdCW + 3) {
      // ---------------- statistics loader: L and delta of each query tile -> shared memory (indexed by column in
      // this kernel), zeros beyond N. Plain guarded loads, so any N and any alignment of the two arrays work; with
      // zeros there a padded query column gives p = 1, dP = 0, dS = 0 and meets zero-filled rows of dO and Q in the
      // products, so nothing has to be masked.
      // The values of a tile are fetched into registers one iteration before the stage that takes them is free, so the
      // global-memory latency never sits between STAT_EMPTY and STAT_FULL.
      uint32_t it = 0;
      bool ok = true;
      float lv[kBlockM / 32], dv_[kBlockM / 32];
      auto fetch = [&](const DkdvItem& w, int n) {
        const int head = w.kvh * G + n / w.cnt_i;
        const int i = w.i_min + n % w.cnt_i;
        const size_t base = (static_cast<size_t>(w.b) * p.H + head) * p.N;
#pragma unroll
        for (int t = 0; t < kBlockM / 32; ++t) {
          const int pos = i * kBlockM + t * 32 + lane;
          const bool in = pos < p.N;
          // stored ready for use: -L * log2(e) is the addend of the exponent, -delta the addend of dP
          lv[t] = in ? __ldg(p.lse + base + pos) * -1.4426950408889634f : 0.f;
          dv_[t] = in ? -__ldg(p.delta + base + pos) : 0.f;
        }
      };
      for (int round = 0; ok; ++round) {
        if (round >= p.total_rounds) break;
        const int idx = dkdv_item_for_round<CAUSAL>(p, round, blockIdx.x, gridDim.x);
        if (idx < 0) continue;  // a partial round leaves some CTAs without an item
        const DkdvItem w = decode_dkdv_item<CAUSAL>(p, idx);
        if (w.n_iter == 0) continue;  // key block wholly beyond this batch element's length: nothing to do
        fetch(w, 0);
        for (int n = 0; n < w.n_iter && ok; ++n, ++it) {
          const int ss = it & 1;
          ok = mbar_wait(bars + STAT_EMPTY + ss, ((it >> 1) & 1) ^ 1, abortp, kWaitLimitCycles);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
#pragma unroll
          for (int t = 0; t < kBlockM / 32; ++t) {
            sStat[ss * 256 + t * 32 + lane] = lv[t];
            sStat[ss * 256 + 128 + t * 32 + lane] = dv_[t];
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bars + STAT_FULL + ss);
          if (n + 1 < w.n_iter) fetch(w, n + 1);
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    // Give copies and MMAs that are still in flight time to land before TMEM and shared memory go away.
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) {
    }
    if (tid == 0) atomicCAS(p.status, kStatusOk, kStatusTimeout);
    __syncthreads();
  }
  if (warp == kBwdCW) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------ dQ
struct DqItem {
  int b, h, kvh, i;  // batch, query head, its kv head, query tile
  int kv_len;        // keys this batch element attends to
  int off;           // causal: query row r sees keys [0, r + off], off = kv_len - N
  int n_iter;        // key tiles this query tile meets (0: none of its rows sees a key; dQ = 0)
};

// Work order: the query tiles of one (batch, kv head) unit are adjacent so that concurrently running CTAs
// stream the same K / V tiles from L2. Causal: L2-sized groups of units, last query tile (the longest) first.
template <bool CAUSAL>
__device__ __forceinline__ DqItem decode_dq_item(const BwdParams& p, int idx) {
  DqItem w;
  const int NB = (p.N + kBlockM - 1) / kBlockM;  // the last tile may be partial
  const int G = p.G;
  int unit, g;
  if (CAUSAL) {
    const int grp = min(p.fd_group.div(idx), p.last_group);
    const int within = idx - grp * p.group_items;
    int qd, rem;
    if (grp == p.last_group) p.fd_in_grp_last.divmod(within, qd, rem);
    else p.fd_in_grp.divmod(within, qd, rem);
    w.i = NB - 1 - qd;
    int u;
    p.fd_inner.divmod(rem, u, g);
    unit = grp * p.group_units + u;
  } else {
    int rem;
    p.fd_unit.divmod(idx, unit, rem);
    p.fd_inner.divmod(rem, g, w.i);
  }
  p.fd_hkv.divmod(unit, w.b, w.kvh);
  w.h = w.kvh * G + g;
  w.kv_len = p.kv_lens ? min(max(p.kv_lens[w.b], 1), p.NK) : p.NK;
  w.off = w.kv_len - p.N;
  const int n_kv = (w.kv_len + kBlockN - 1) / kBlockN;
  // causal: the last row of the tile sees keys up to i*128 + 127 + off
  w.n_iter = CAUSAL ? min(max((w.i * kBlockM + kBlockM + w.off + kBlockN - 1) / kBlockN, 0), n_kv) : n_kv;
  return w;
}

template <int D, bool CAUSAL>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                   const BwdParams p) {
  using namespace ptx;
  using SM = BwdSmem<D>;
  constexpr int kTile = SM::kTileBytes;
  constexpr int kSub = SM::kSubTileBytes;
  constexpr int kChunks = D / 64;
  constexpr int RA = SM::kRingK, RB = SM::kRingV;
  enum { QDO_FULL = 0, QDO_EMPTY, S_FULL, S_FREE, DP_FULL, DP_FREE, DS_FULL, DS_FREE, KA_FULL = 8, KA_EMPTY = 15,
         VB_FULL = 22, VB_EMPTY = 25, DQ_FULL = 28, CTRL = 32 };
  static_assert(RA <= 7 && RB <= 3, "barrier slots");

  extern __shared__ __align__(1024) uint8_t bwd_smem[];
  uint8_t* sQ = bwd_smem;
  uint8_t* sDO = bwd_smem + kTile;
  uint8_t* sK = bwd_smem + 2 * kTile;   // RA stages
  uint8_t* sV = sK + RA * kTile;        // RB stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(bwd_smem + SM::kTiles * kTile + SM::kStatBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + CTRL);
  uint32_t* abort_word = tmem_slot + 1;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if ((smem_u32(bwd_smem) & 1023u) != 0) {
    if (tid == 0) atomicCAS(p.status, kStatusOk, kStatusSmemAlign);
    return;
  }
  if (tid == 0) {
    *abort_word = 0;
    mbar_init(bars + QDO_FULL, 1);
    mbar_init(bars + QDO_EMPTY, 2);  // Q released by issuer A, dO by issuer B
    mbar_init(bars + S_FULL, 1);
    mbar_init(bars + S_FREE, kBwdCW);     // one arrival per element-wise warp once its part is in registers
    mbar_init(bars + DP_FULL, 1);
    mbar_init(bars + DP_FREE, kBwdCW);
    mbar_init(bars + DS_FULL, kBwdCW);
    mbar_init(bars + DS_FREE, 1);
    mbar_init(bars + DQ_FULL, 1);
    for (int s = 0; s < RA; ++s) {
      mbar_init(bars + KA_FULL + s, 1);
      mbar_init(bars + KA_EMPTY + s, 1);
    }
    for (int s = 0; s < RB; ++s) {
      mbar_init(bars + VB_FULL + s, 1);
      mbar_init(bars + VB_EMPTY + s, 1);
    }
    fence_mbar_init();
  }
  if (warp == kBwdCW) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  volatile uint32_t* abortp = abort_word;
  // TMEM columns: S [0,128)  dP [128,256)  dQ [256,256+D)  dS (bf16, 64 packed columns) [384,448).
  // Nothing aliases: S and dP are free for the next tile as soon as they are in registers.
  constexpr uint32_t cS = 0, cDP = 128, cDQ = 256, cDS = 384;

  if (warp < kBwdCW) {
    // ------------------------------------------------------------------ element-wise warps
    bwd_grow_registers();
    const int part = warp >> 2;                        // which kBwdPC key columns of the tile
    const int row = (warp & 3) * 32 + lane;            // query row inside the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_addr + cS + part * kBwdPC;
    const uint32_t tP = tmem + lane_addr + cDP + part * kBwdPC;
    const uint32_t tDS = tmem + lane_addr + cDS + part * (kBwdPC / 2);
    const float c = p.scale_log2;
    uint32_t it = 0, dq_cnt = 0;
    bool ok = true;
#ifdef HK_TRACE
    const bool trace_on = (warp == 0) && lane == 0 && p.trace != nullptr;
    int trace_n = 0;
#endif
    for (int round = 0; ok; ++round) {
      if (round >= p.total_rounds) break;
      const int idx = item_for_round(p, round, blockIdx.x, gridDim.x);
      if (idx < 0) continue;  // a partial round leaves some CTAs without an item
      const DqItem w = decode_dq_item<CAUSAL>(p, idx);
      const size_t srow = (static_cast<size_t>(w.b) * p.H + w.h) * p.N + static_cast<size_t>(w.i) * kBlockM + row;
      const bool row_exists = w.i * kBlockM + row < p.N;  // rows of a partial last tile beyond N: zero statistics
      if (w.n_iter == 0) {
        // causal with more queries than kept keys: no row of this tile sees a key, dQ = 0 and no product is issued
        if (row_exists) {
          __nv_bfloat16* dst0 = p.dq + w.b * p.dq_stride_b + (static_cast<long long>(w.i) * kBlockM + row) * p.dq_stride_n +
                                w.h * p.dq_stride_h + part * (D / kBwdParts);
#pragma unroll
          for (int v = 0; v < D / kBwdParts / 8; ++v) reinterpret_cast<uint4*>(dst0)[v] = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const float nl = row_exists ? p.lse[srow] * -1.4426950408889634f : 0.f;
      const float dl = row_exists ? p.delta[srow] : 0.f;
      for (int n = 0; n < w.n_iter && ok; ++n, ++it) {
        // a key tile the diagonal (or the end of the kept keys) runs through: the tile's first row does not see
        // its last key
        const bool diag = CAUSAL && ((n + 1) * kBlockN - 1 > min(w.i * kBlockM + w.off, w.kv_len - 1));
        HK_STAMP(0, 0);
        ok = mbar_wait(bars + S_FULL, it & 1, abortp, kWaitLimitCycles);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        HK_STAMP(0, 1);
        uint32_t su[kBwdPC];
        bwd_ld_part(tS, su);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + S_FREE);  // issuer A may overwrite S with the next tile's
        {
          const uint64_t c2 = pack2(c, c), nl2 = pack2(nl, nl);
#pragma unroll
          for (int i = 0; i < kBwdPC / 2; ++i) {
            float x0, x1;
            const uint64_t x2 = fma2(pack2(__uint_as_float(su[2 * i]), __uint_as_float(su[2 * i + 1])), c2, nl2);
            // a share of the column pairs through the FMA-pipe polynomial, as in the dK/dV kernel
            if (i % kBwdEmuMod < kBwdEmuCnt) unpack2(ex2_poly2(x2), x0, x1);
            else {
              unpack2(x2, x0, x1);
              x0 = ex2_approx(x0);
              x1 = ex2_approx(x1);
            }
            su[2 * i] = __float_as_uint(x0);
            su[2 * i + 1] = __float_as_uint(x1);
          }
          if (diag) {
            // key n*128 + col is seen by query i*128 + row iff it is <= query + off and < kv_len (this also zeroes
            // the infinities of a row without any key, whose L is -inf)
            const int lim = min(w.i * kBlockM + row + w.off, w.kv_len - 1) - n * kBlockN;
#pragma unroll
            for (int col = 0; col < kBwdPC; ++col) su[col] = (part * kBwdPC + col) > lim ? 0u : su[col];
          }
          if (!CAUSAL && n == w.n_iter - 1 && (w.kv_len & (kBlockN - 1)) != 0) {
            // partial last tile: keys at or beyond the length are padding
            const int rem = w.kv_len - n * kBlockN;
#pragma unroll
            for (int col = 0; col < kBwdPC; ++col) su[col] = (part * kBwdPC + col) >= rem ? 0u : su[col];
          }
        }
        HK_STAMP(0, 2);
        ok = mbar_wait(bars + DP_FULL, it & 1, abortp, kWaitLimitCycles);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        HK_STAMP(0, 3);
        uint32_t pk[kBwdPC / 2];
        {
          uint32_t du[kBwdPC];
          bwd_ld_part(tP, du);
          tmem_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bars + DP_FREE);  // issuer B may overwrite dP with the next tile's
          const uint64_t ndl2 = pack2(-dl, -dl);
#pragma unroll
          for (int i = 0; i < kBwdPC / 2; ++i) {
            float ds0, ds1;
            unpack2(mul2(pack2(__uint_as_float(su[2 * i]), __uint_as_float(su[2 * i + 1])),
                         add2(pack2(__uint_as_float(du[2 * i]), __uint_as_float(du[2 * i + 1])), ndl2)),
                    ds0, ds1);
            pk[i] = pack_bf16x2(ds0, ds1);
          }
        }
        // dS of the previous tile has been consumed by its dQ product (first tile ever: passes at once)
        ok = mbar_wait(bars + DS_FREE, (it & 1) ^ 1, abortp, kWaitLimitCycles);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        bwd_st_packed(tDS, pk);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + DS_FULL);
        HK_STAMP(0, 4);
      }
      if (!ok) break;
      // ---- epilogue: dQ = scale * acc
      ok = mbar_wait(bars + DQ_FULL, dq_cnt & 1, abortp, kWaitLimitCycles);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ++dq_cnt;
      tc_fence_after();
      __nv_bfloat16* dst = p.dq + w.b * p.dq_stride_b + (static_cast<long long>(w.i) * kBlockM + row) * p.dq_stride_n +
                           w.h * p.dq_stride_h + part * (D / kBwdParts);
      bwd_store_part_row<D>(tmem + lane_addr + cDQ + part * (D / kBwdParts), dst, p.scale, row_exists);
      tc_fence_before();  // orders these reads before the next item's first dQ product (published through DS_FULL)
    }
  } else {
    bwd_shrink_registers();
    if (warp == kBwdCW && lane == 0) {
      // ---------------- TMA producer
      prefetch_tmap(&tmap_q);
      prefetch_tmap(&tmap_k);
      prefetch_tmap(&tmap_v);
      prefetch_tmap(&tmap_do);
      uint32_t item_cnt = 0;
      int ka = 0, vb = 0;
      uint32_t ka_par = 0, vb_par = 0;
      bool ok = true;
      for (int round = 0; ok; ++round) {
        if (round >= p.total_rounds) break;
        const int idx = item_for_round(p, round, blockIdx.x, gridDim.x);
        if (idx < 0) continue;  // a partial round leaves some CTAs without an item
        const DqItem w = decode_dq_item<CAUSAL>(p, idx);
        if (w.n_iter == 0) continue;  // no row of this tile sees a key: nothing is loaded or issued
        ok = mbar_wait(bars + QDO_EMPTY, (item_cnt & 1) ^ 1, abortp, kWaitLimitCycles);
        if (!ok) break;
        ++item_cnt;
        mbar_expect_tx(bars + QDO_FULL, 2 * kTile);
#pragma unroll
        for (int ch = 0; ch < kChunks; ++ch) {
          tma_load_4d(sQ + ch * kSub, &tmap_q, bars + QDO_FULL, ch * 64, w.h, w.i * kBlockM, w.b);
          tma_load_4d(sDO + ch * kSub, &tmap_do, bars + QDO_FULL, ch * 64, w.h, w.i * kBlockM, w.b);
        }
        for (int n = 0; n < w.n_iter && ok; ++n) {
          ok = mbar_wait(bars + KA_EMPTY + ka, ka_par ^ 1, abortp, kWaitLimitCycles);
          if (!ok) break;
          mbar_expect_tx(bars + KA_FULL + ka, kTile);
#pragma unroll
          for (int ch = 0; ch < kChunks; ++ch)
            tma_load_4d(sK + ka * kTile + ch * kSub, &tmap_k, bars + KA_FULL + ka, ch * 64, w.kvh, n * kBlockN, w.b);
          if (++ka == RA) {
            ka = 0;
            ka_par ^= 1;
          }
          ok = mbar_wait(bars + VB_EMPTY + vb, vb_par ^ 1, abortp, kWaitLimitCycles);
          if (!ok) break;
          mbar_expect_tx(bars + VB_FULL + vb, kTile);
#pragma unroll
          for (int ch = 0; ch < kChunks; ++ch)
            tma_load_4d(sV + vb * kTile + ch * kSub, &tmap_v, bars + VB_FULL + vb, ch * 64, w.kvh, n * kBlockN, w.b);
          if (++vb == RB) {
            vb = 0;
            vb_par ^= 1;
          }
        }
      }
    } else if (warp == kBwdCW + 1 && (kBwdWarpIssue || lane == 0)) {
      // ---------------- UMMA issuer A: S = Q K^T, as soon as the previous S has been read
      // Two issuing threads, as in the dK/dV kernel: this one runs ahead with the S products, issuer B follows
      // with dP (as soon as the previous dP has been read) and dQ += dS K.
      constexpr uint32_t tile16 = kTile >> 4;
      const uint32_t q_lo = smem_desc_lo(smem_u32(sQ), 16);
      const uint32_t k_lo0 = smem_desc_lo(smem_u32(sK), 16);      // K-major view (B of S)
      uint32_t item_cnt = 0, sf_cnt = 0;
      int ks = 0;
      uint32_t ks_par = 0;
      bool ok = true;
#ifdef HK_TRACE
      const bool trace_on = p.trace != nullptr && lane == 0;
      int trace_n = 0;
#endif
      for (int round = 0; ok; ++round) {
        if (round >= p.total_rounds) break;
        const int idx = item_for_round(p, round, blockIdx.x, gridDim.x);
        if (idx < 0) continue;  // a partial round leaves some CTAs without an item
        const DqItem w = decode_dq_item<CAUSAL>(p, idx);
        if (w.n_iter == 0) continue;  // no row of this tile sees a key: nothing is loaded or issued
        ok = iss_wait(bars + QDO_FULL, item_cnt & 1, abortp, kWaitLimitCycles);
        if (!ok) break;
        ++item_cnt;
        for (int n = 0; n < w.n_iter && ok; ++n, ++sf_cnt) {
          ok = iss_wait(bars + S_FREE, (sf_cnt & 1) ^ 1, abortp, kWaitLimitCycles) &&
               iss_wait(bars + KA_FULL + ks, ks_par, abortp, kWaitLimitCycles);
          if (!ok) break;
          tc_fence_after();
          HK_STAMP(2, 12);
          if (iss_elect()) {
            bwd_issue_ss<D>(tmem + cS, q_lo, k_lo0 + ks * tile16);
            umma_commit(bars + S_FULL);
          }
          HK_STAMP(2, 13);
          if (++ks == RA) {
            ks = 0;
            ks_par ^= 1;
          }
        }
        if (!ok) break;
        if (iss_elect()) umma_commit(bars + QDO_EMPTY);  // Q has fed its last product (issuer B arrives for dO)
      }
    } else if (warp == kBwdCW + 2 && (kBwdWarpIssue || lane == 0)) {
      // ---------------- UMMA issuer B: dP = dO V^T, dQ += dS K
      constexpr uint32_t tile16 = kTile >> 4;
      const uint32_t do_lo = smem_desc_lo(smem_u32(sDO), 16);
      const uint32_t k_mn0 = smem_desc_lo(smem_u32(sK), kSub);    // MN-major view (B of dQ)
      const uint32_t v_lo0 = smem_desc_lo(smem_u32(sV), 16);
      uint32_t item_cnt = 0, it = 0, dpf_cnt = 0;
      int kq = 0, vb = 0;
      uint32_t kq_par = 0, vb_par = 0;
      bool ok = true;
#ifdef HK_TRACE
      const bool trace_on = p.trace != nullptr && lane == 0;
      int trace_n = 0;
#endif
      auto issue_dp = [&]() -> bool {
        // the previous dP has been read (first dP ever: passes at once)
        if (!iss_wait(bars + DP_FREE, (dpf_cnt & 1) ^ 1, abortp, kWaitLimitCycles)) return false;
        if (!iss_wait(bars + VB_FULL + vb, vb_par, abortp, kWaitLimitCycles)) return false;
        ++dpf_cnt;
        tc_fence_after();
        if (iss_elect()) {
          bwd_issue_ss<D>(tmem + cDP, do_lo, v_lo0 + vb * tile16);
          umma_commit(bars + DP_FULL);
          umma_commit(bars + VB_EMPTY + vb);
        }
        if (++vb == RB) {
          vb = 0;
          vb_par ^= 1;
        }
        return true;
      };
      for (int round = 0; ok; ++round) {
        if (round >= p.total_rounds) break;
        const int idx = item_for_round(p, round, blockIdx.x, gridDim.x);
        if (idx < 0) continue;  // a partial round leaves some CTAs without an item
        const DqItem w = decode_dq_item<CAUSAL>(p, idx);
        if (w.n_iter == 0) continue;  // no row of this tile sees a key: nothing is loaded or issued
        ok = iss_wait(bars + QDO_FULL, item_cnt & 1, abortp, kWaitLimitCycles);
        if (!ok) break;
        ++item_cnt;
        ok = issue_dp();
        if (!ok) break;
        if (w.n_iter == 1 && iss_elect()) umma_commit(bars + QDO_EMPTY);  // dO has fed its last product
        for (int n = 0; n < w.n_iter && ok; ++n, ++it) {
          if (n + 1 < w.n_iter) {
            ok = issue_dp();
            if (!ok) break;
            if (n + 2 == w.n_iter && iss_elect()) umma_commit(bars + QDO_EMPTY);
            HK_STAMP(3, 12);
          }
          ok = iss_wait(bars + DS_FULL, it & 1, abortp, kWaitLimitCycles) &&
               iss_wait(bars + KA_FULL + kq, kq_par, abortp, kWaitLimitCycles);
          if (!ok) break;
          tc_fence_after();
          HK_STAMP(3, 10);
          if (iss_elect()) {
            constexpr uint32_t idesc = make_idesc_bf16(kBlockM, D, true);
            constexpr uint32_t desc_hi = smem_desc_hi(1024);
            const uint32_t b_lo = k_mn0 + kq * tile16;
#pragma unroll
            for (int k = 0; k < kBlockN / 16; ++k)
              umma_ts_lohi(tmem + cDQ, tmem + cDS + k * 8, b_lo + k * 128, desc_hi, idesc, (n > 0 || k > 0) ? 1u : 0u);
            // S of this tile (issuer A) completed before dS could be computed, so this one arrival frees the K tile
            umma_commit(bars + KA_EMPTY + kq);
            umma_commit(bars + DS_FREE);
          }
          HK_STAMP(3, 11);
          if (++kq == RA) {
            kq = 0;
            kq_par ^= 1;
          }
        }
        if (!ok) break;
        if (iss_elect()) umma_commit(bars + DQ_FULL);
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) {
    }
    if (tid == 0) atomicCAS(p.status, kStatusOk, kStatusTimeout);
    __syncthreads();
  }
  if (warp == kBwdCW) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace HK_BWD_NS
}  // namespace hk
#undef HK_BWD_NS
#undef HK_BWD_PARTS
