// Host side of libhk_attn: argument validation, TMA descriptors, launches. C ABI in include/hk_attn.h.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/hk_attn.h"
// The backward kernels are compiled in two thread layouts (see the header): 16 element-wise warps for the
// non-causal instantiations, 8 for the causal ones.
#define HK_BWD_NS bwd16
#define HK_BWD_PARTS 4
#include "attn_bwd_sm100.cuh"
#define HK_BWD_NS bwd8
#define HK_BWD_PARTS 2
#include "attn_bwd_sm100.cuh"
#include "attn_fwd_sm100.cuh"
#include "paged_decode_sm100.cuh"
#include "paged_kv_append_sm100.cuh"
#include "rotary_sm100.cuh"

namespace {

constexpr int kMaxDevices = 64;

thread_local char g_cuda_err[256] = "";
std::atomic<unsigned long long> g_launches{0};

int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, cudaGetErrorString(e));
  return HK_ECUDA;
}
#define HK_CUDA(call)                                   \
  do {                                                  \
    cudaError_t e__ = (call);                           \
    if (e__ != cudaSuccess) return cuda_fail(e__, #call); \
  } while (0)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Per-device state: SM count, the device status word, one-time kernel attribute set-up.
struct DeviceState {
  std::mutex mu;
  bool ready = false;     // set once init_device succeeded; a failed attempt is retried by the next call
  int sm_count = 0;
  int cc_major = 0;
  int* status = nullptr;  // device word
};
DeviceState g_dev[kMaxDevices];

template <int D, bool CAUSAL>
int prepare_fwd_kernel() {
  auto* fn = hk::attn_fwd_kernel<D, CAUSAL>;
  HK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, hk::FwdSmem<D, CAUSAL>::kDynBytes));
  cudaFuncAttributes attr;
  HK_CUDA(cudaFuncGetAttributes(&attr, fn));
  // The kernel re-balances registers between warpgroups (208 per softmax thread, 88 per producer thread);
  // that only adds up if it was compiled to exactly kFwdRegsAtLaunch registers per thread at launch.
  // Refuse to launch otherwise: a register pool that is too small would block the re-allocation forever.
  if (attr.numRegs != hk::kFwdRegsAtLaunch) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "attn_fwd_kernel<%d,%d> compiled to %d registers, expected %d", D,
             int(CAUSAL), attr.numRegs, hk::kFwdRegsAtLaunch);
    return HK_EUNSUPPORTED;
  }
  return HK_OK;
}

// The layout that serves an instantiation, with its kernels and launch constants.
template <bool CAUSAL>
struct BwdLayout;
template <>
struct BwdLayout<false> {
  static constexpr int kThreads = hk::bwd16::kBwdThreads, kRegsAtLaunch = hk::bwd16::kBwdRegsAtLaunch;
  static constexpr bool kExactRegs = hk::bwd16::kBwdRegsGrown != hk::bwd16::kBwdRegsAtLaunch;
  template <int D> static constexpr auto dkdv() { return &hk::bwd16::attn_bwd_dkdv_kernel<D, false>; }
  template <int D> static constexpr auto dq() { return &hk::bwd16::attn_bwd_dq_kernel<D, false>; }
};
template <>
struct BwdLayout<true> {
  static constexpr int kThreads = hk::bwd8::kBwdThreads, kRegsAtLaunch = hk::bwd8::kBwdRegsAtLaunch;
  static constexpr bool kExactRegs = hk::bwd8::kBwdRegsGrown != hk::bwd8::kBwdRegsAtLaunch;
  template <int D> static constexpr auto dkdv() { return &hk::bwd8::attn_bwd_dkdv_kernel<D, true>; }
  template <int D> static constexpr auto dq() { return &hk::bwd8::attn_bwd_dq_kernel<D, true>; }
};

template <typename Kernel>
int prepare_bwd_kernel(Kernel* fn, int dyn_bytes, const char* name, int regs_at_launch, bool exact) {
  HK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn_bytes));
  cudaFuncAttributes attr;
  HK_CUDA(cudaFuncGetAttributes(&attr, fn));
  // With register re-balancing between warps (the 8-warp layout) the count at launch has to be exact, as for the
  // forward kernel: refuse to launch a build it would not add up in. Without it any count that fits is fine.
  if (exact ? attr.numRegs != regs_at_launch : attr.numRegs > regs_at_launch) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s compiled to %d registers, expected %d", name, attr.numRegs,
             regs_at_launch);
    return HK_EUNSUPPORTED;
  }
  if (attr.sharedSizeBytes != 0) {  // the kernels assume their dynamic shared memory starts the CTA's window
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s has %zu bytes of static shared memory, expected none", name,
             attr.sharedSizeBytes);
    return HK_EUNSUPPORTED;
  }
  return HK_OK;
}

template <int D, bool CAUSAL>
int prepare_bwd_kernels() {
  using Lay = BwdLayout<CAUSAL>;
  int rc = prepare_bwd_kernel(Lay::template dkdv<D>(), hk::BwdSmem<D>::kDynBytes, "attn_bwd_dkdv_kernel",
                              Lay::kRegsAtLaunch, Lay::kExactRegs);
  if (rc != HK_OK) return rc;
  return prepare_bwd_kernel(Lay::template dq<D>(), hk::BwdSmem<D>::kDynBytes, "attn_bwd_dq_kernel", Lay::kRegsAtLaunch,
                            Lay::kExactRegs);
}

int init_device(int device) {
  DeviceState& st = g_dev[device];
  cudaDeviceProp prop;
  HK_CUDA(cudaGetDeviceProperties(&prop, device));
  st.sm_count = prop.multiProcessorCount;
  st.cc_major = prop.major;
  if (prop.major != 10) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "device %d is sm_%d%d; this library needs sm_100", device, prop.major,
             prop.minor);
    return HK_EUNSUPPORTED;
  }
  int rc;
  if ((rc = prepare_fwd_kernel<128, false>()) != HK_OK) return rc;
  if ((rc = prepare_fwd_kernel<128, true>()) != HK_OK) return rc;
  if ((rc = prepare_fwd_kernel<64, false>()) != HK_OK) return rc;
  if ((rc = prepare_fwd_kernel<64, true>()) != HK_OK) return rc;
  if ((rc = hk::prepare_decode_kernels(g_cuda_err, sizeof(g_cuda_err))) != HK_OK) return rc;
  if ((rc = prepare_bwd_kernels<128, false>()) != HK_OK) return rc;
  if ((rc = prepare_bwd_kernels<128, true>()) != HK_OK) return rc;
  if ((rc = prepare_bwd_kernels<64, false>()) != HK_OK) return rc;
  if ((rc = prepare_bwd_kernels<64, true>()) != HK_OK) return rc;
  // the one allocation this library makes: the status word (last, so that a failure above leaves nothing behind)
  int* word = nullptr;
  HK_CUDA(cudaMalloc(&word, sizeof(int)));
  cudaError_t e = cudaMemset(word, 0, sizeof(int));
  if (e != cudaSuccess) {
    cudaFree(word);
    return cuda_fail(e, "cudaMemset(status word)");
  }
  st.status = word;
  return HK_OK;
}

// Makes a device current for the duration of one entry point and puts the caller's current device back when the
// entry point returns (the reference launcher never touches the current device; a torch program whose current
// device is another GPU must not find it changed).
class DeviceScope {
 public:
  DeviceScope() = default;
  DeviceScope(const DeviceScope&) = delete;
  DeviceScope& operator=(const DeviceScope&) = delete;
  ~DeviceScope() {
    if (prev_ >= 0 && prev_ != cur_) cudaSetDevice(prev_);
  }
  // Switches to `device` (< 0: stay on the current one) and reports the index in use through *resolved.
  int enter_raw(int device, int* resolved) {
    HK_CUDA(cudaGetDevice(&prev_));
    if (device < 0) device = prev_;
    if (device >= kMaxDevices) return HK_EINVAL;
    if (device != prev_) HK_CUDA(cudaSetDevice(device));
    cur_ = device;
    *resolved = device;
    return HK_OK;
  }
  // enter_raw plus the device's state, initialised on first use. A failed initialisation is not remembered: the
  // next call tries again (the failing thread finds the reason in hk_last_cuda_error()).
  int enter(int device, DeviceState** out) {
    int rc = enter_raw(device, &device);
    if (rc != HK_OK) return rc;
    DeviceState& st = g_dev[device];
    {
      std::lock_guard<std::mutex> lock(st.mu);
      if (!st.ready) {
        rc = init_device(device);
        if (rc != HK_OK) return rc;
        st.ready = true;
      }
    }
    *out = &st;
    return HK_OK;
  }

 private:
  int prev_ = -1, cur_ = -1;
};

#ifdef HK_TRACE
long long* g_trace_buf = nullptr;
int g_trace_bwd_kernel = 0;  // which backward kernel stamps: 0 = dK/dV, 1 = dQ
#endif

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int unsupported_decode_shape(int S, int H_KV, int max_pages) {
  snprintf(g_cuda_err, sizeof(g_cuda_err),
           "paged decode supports S <= 65535, H_KV <= 65535 and max_pages_per_seq <= %d (got S=%d, H_KV=%d, "
           "max_pages_per_seq=%d)", hk::kMaxCombineSplits * hk::kChunkPagesMin, S, H_KV, max_pages);
  return HK_EUNSUPPORTED;
}

// Device status word -> HK_* code.
int status_to_code(int word) {
  switch (word) {
    case hk::kStatusOk: return HK_OK;
    case hk::kStatusSmemAlign: return HK_EUNSUPPORTED;
    case hk::kStatusBadPage: return HK_EBADPAGE;
    case hk::kStatusBadLen: return HK_EBADLEN;
    default: return HK_ETIMEOUT;
  }
}

// 4-D map over a contiguous bf16 [B, N, heads, D] tensor, box = 64 columns x 1 head x 128 rows,
// 128-byte swizzle (rows of the box are 128 B, the layout tcgen05 descriptors expect).
// `st` = element strides of the batch, sequence and head dimensions (the D dimension is contiguous); every
// stride must be a multiple of 8 elements (16 bytes), which TMA requires.
int make_bnhd_map(CUtensorMap* map, const void* base, int B, int N, int heads, int D, const long long* st,
                  int box_rows = hk::kBlockM) {
  EncodeTiledFn enc = get_encode();
  if (!enc) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled not available from the driver");
    return HK_ECUDA;
  }
  cuuint64_t dims[4] = {cuuint64_t(D), cuuint64_t(heads), cuuint64_t(N), cuuint64_t(B)};
  cuuint64_t strides[3] = {cuuint64_t(st[2]) * 2, cuuint64_t(st[1]) * 2, cuuint64_t(st[0]) * 2};
  cuuint32_t box[4] = {64, 1, cuuint32_t(box_rows), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled failed with CUresult %d", int(r));
    return HK_ECUDA;
  }
  return HK_OK;
}

__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    hk::ptx::mbar_init(&bar, 1);
    hk::ptx::fence_mbar_init();
  }
  __syncthreads();
  // the limit is given in nanoseconds; 2 cycles per nanosecond is the SM's maximum clock, rounded up
  const bool ok = hk::ptx::mbar_wait(&bar, 0, &abort_flag, limit_ns * 2);  // nobody ever arrives
  if (!ok && threadIdx.x == 0) atomicCAS(status, hk::kStatusOk, hk::kStatusTimeout);
}

template <int D, bool CAUSAL>
int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to,
               const hk::FwdParams& p, int grid, cudaStream_t stream) {
  hk::attn_fwd_kernel<D, CAUSAL><<<grid, hk::kFwdThreads, hk::FwdSmem<D, CAUSAL>::kDynBytes, stream>>>(tq, tk, tv, to, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  HK_CUDA(cudaGetLastError());
  return HK_OK;
}

// Sets the fields that say how a kernel's `n_items` work items are dealt to `grid` CTAs - one group (everything)
// unless causal, where a group is `group_units` units of `per_unit` items each - and the divisors of the item
// decode: `per_unit` items per (batch, kv-head) unit, `per_pos` of them per key block or query tile (1 in the dK/dV
// kernel, G in the dQ kernel), `inner` the dQ kernel's second divisor.
void set_bwd_decode(hk::BwdParams& p, int per_unit, int per_pos, int inner, int grid, bool causal) {
  p.group_items = causal ? p.group_units * per_unit : p.n_items;
  const int n_groups = (p.n_items + p.group_items - 1) / p.group_items;
  p.rounds_per_group = (p.group_items + grid - 1) / grid;
  p.total_rounds = p.rounds_per_group * n_groups;
  const int units = p.B * p.H_KV;
  p.G = p.H / p.H_KV;
  p.last_group = (units - 1) / p.group_units;
  p.fd_rounds = hk::FastDiv(p.rounds_per_group);
  p.fd_hkv = hk::FastDiv(p.H_KV);
  p.fd_unit = hk::FastDiv(per_unit);
  p.fd_inner = hk::FastDiv(inner);
  p.fd_group = hk::FastDiv(p.group_units * per_unit);
  p.fd_in_grp = hk::FastDiv(p.group_units * per_pos);
  p.fd_in_grp_last = hk::FastDiv((units - p.last_group * p.group_units) * per_pos);
}

template <int D, bool CAUSAL>
int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
               hk::BwdParams p, int B, int N, int NK, int H, int H_KV, int sm_count, cudaStream_t stream) {
  const int nbq = (N + hk::kBlockM - 1) / hk::kBlockM;   // query tiles
  const int nbk = (NK + hk::kBlockN - 1) / hk::kBlockN;  // key blocks
  if (static_cast<long long>(B) * H * nbq > 0x3fffffffll || static_cast<long long>(B) * H_KV * nbk > 0x3fffffffll)
    return HK_EINVAL;  // work items are indexed with int
  p.n_items = B * H_KV * nbk;
  int grid = p.n_items < sm_count ? p.n_items : sm_count;
  set_bwd_decode(p, nbk, 1, 1, grid, CAUSAL);
  if (CAUSAL) {
    // key blocks are dealt in pairs (j, nbk - 1 - j) of equal cost, two rounds per pair
    const int per_unit = (nbk + 1) / 2;
    p.n_pairs = B * H_KV * per_unit;
    p.fd_pairs = hk::FastDiv(per_unit);
    grid = p.n_pairs < sm_count ? p.n_pairs : sm_count;
    p.total_rounds = 2 * ((p.n_pairs + grid - 1) / grid);
  }
#ifdef HK_TRACE
  long long* const trace_buf = p.trace;
  p.trace = g_trace_bwd_kernel == 0 ? trace_buf : nullptr;
#endif
  using Lay = BwdLayout<CAUSAL>;
  Lay::template dkdv<D>()<<<grid, Lay::kThreads, hk::BwdSmem<D>::kDynBytes, stream>>>(tq, tk, tv, tdo, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  HK_CUDA(cudaGetLastError());
  p.n_items = B * H * nbq;
  grid = p.n_items < sm_count ? p.n_items : sm_count;
  set_bwd_decode(p, (H / H_KV) * nbq, H / H_KV, CAUSAL ? H / H_KV : nbq, grid, CAUSAL);
#ifdef HK_TRACE
  p.trace = g_trace_bwd_kernel == 1 ? trace_buf : nullptr;
#endif
  Lay::template dq<D>()<<<grid, Lay::kThreads, hk::BwdSmem<D>::kDynBytes, stream>>>(tq, tk, tv, tdo, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  HK_CUDA(cudaGetLastError());
  return HK_OK;
}

}  // namespace

extern "C" {

#ifdef HK_TRACE
void hk_debug_set_trace(long long* buf) { g_trace_buf = buf; }
void hk_debug_set_trace_bwd_kernel(int which) { g_trace_bwd_kernel = which; }
#endif

int hk_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int N, int H, int H_KV,
                int D, int causal, float softmax_scale, int device, void* cuda_stream) {
  const long long qs[3] = {(long long)N * H * D, (long long)H * D, D};
  const long long ks[3] = {(long long)N * H_KV * D, (long long)H_KV * D, D};
  return hk_attn_fwd_strided(q, k, v, o, lse, B, N, H, H_KV, D, qs, ks, ks, causal, softmax_scale, device, cuda_stream);
}

int hk_attn_fwd_strided(const void* q, const void* k, const void* v, void* o, float* lse, int B, int N, int H,
                        int H_KV, int D, const long long* q_strides, const long long* k_strides,
                        const long long* v_strides, int causal, float softmax_scale, int device,
                        void* cuda_stream) {
  return hk_attn_fwd_varlen(q, k, v, o, lse, B, N, H, H_KV, D, q_strides, k_strides, v_strides, nullptr, causal,
                            softmax_scale, device, cuda_stream);
}

int hk_attn_fwd_varlen(const void* q, const void* k, const void* v, void* o, float* lse, int B, int N, int H,
                       int H_KV, int D, const long long* q_strides, const long long* k_strides,
                       const long long* v_strides, const int32_t* kv_lens, int causal, float softmax_scale,
                       int device, void* cuda_stream) {
  return hk_attn_fwd_cross(q, k, v, o, lse, B, N, N, H, H_KV, D, q_strides, k_strides, v_strides, kv_lens, causal,
                           softmax_scale, device, cuda_stream);
}

// Shared tail of the forward entries. Contiguous K/V: k, v are [B, NK, H_KV, D] with strides; paged K/V
// (block_table != null): k, v are the page pools [num_pages, 16, H_KV, D] and NK = max_pages * 16.
static int fwd_launch(const void* q, const void* k, const void* v, void* o, float* lse, int B, int N, int NK, int H,
                      int H_KV, int D, const long long* q_strides, const long long* k_strides,
                      const long long* v_strides, const int32_t* kv_lens, const int32_t* block_table, int max_pages,
                      int num_pages, int causal, float softmax_scale, int device, void* cuda_stream) {
  DeviceState* st = nullptr;
  DeviceScope scope;
  int rc = scope.enter(device, &st);
  if (rc != HK_OK) return rc;

  CUtensorMap tq, tk, tv, to;
  if ((rc = make_bnhd_map(&tq, q, B, N, H, D, q_strides)) != HK_OK) return rc;
  {
    // O is written by TMA from a swizzled staging tile, a [128 rows x 64 columns] box at a time
    const long long os[3] = {(long long)N * H * D, (long long)H * D, D};
    if ((rc = make_bnhd_map(&to, o, B, N, H, D, os)) != HK_OK) return rc;
  }
  if (block_table) {
    // the pools as [num_pages * 16 rows, H_KV, D], fetched one page (16 rows) at a time
    const long long ps[3] = {(long long)num_pages * 16 * H_KV * D, (long long)H_KV * D, D};
    if ((rc = make_bnhd_map(&tk, k, 1, num_pages * 16, H_KV, D, ps, 16)) != HK_OK) return rc;
    if ((rc = make_bnhd_map(&tv, v, 1, num_pages * 16, H_KV, D, ps, 16)) != HK_OK) return rc;
  } else {
    if ((rc = make_bnhd_map(&tk, k, B, NK, H_KV, D, k_strides)) != HK_OK) return rc;
    if ((rc = make_bnhd_map(&tv, v, B, NK, H_KV, D, v_strides)) != HK_OK) return rc;
  }

  const int G = H / H_KV;
  const int nqb = (N + hk::kBlockM - 1) / hk::kBlockM;
  hk::FwdParams p;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.B = B;
  p.N = N;
  p.NK = NK;
  p.H = H;
  p.H_KV = H_KV;
  p.pair_heads = (G % 2 == 0) ? 1 : 0;
  {
    // causal sweep groups: as many (batch, kv-head) units as keep K and V of the group within HK_GROUP_MB (the
    // whole tensor at once re-reads K/V 2.6 times at N = 8192)
    const long long kv_bytes = 4ll * NK * D;  // K and V of one unit, bf16
#ifndef HK_GROUP_MB
#define HK_GROUP_MB 32
#endif
    long long u = (static_cast<long long>(HK_GROUP_MB) << 20) / kv_bytes;
    p.group_units = int(u < 1 ? 1 : (u > B * H_KV ? B * H_KV : u));
  }
  if (static_cast<long long>(B) * H * nqb > 0x3fffffffll) return HK_EINVAL;  // work items are indexed with int
  p.n_items = p.pair_heads ? B * H_KV * (G / 2) * nqb : B * H_KV * G * ((nqb + 1) / 2);
  p.scale = softmax_scale > 0.f ? softmax_scale : 1.0f / std::sqrt(float(D));
  p.scale_log2 = p.scale * 1.4426950408889634f;
  p.kv_lens = kv_lens;
  p.block_table = block_table;
  p.max_pages = max_pages;
  p.num_pages = num_pages;
  p.status = st->status;
#ifdef HK_TRACE
  p.trace = g_trace_buf;
#endif
  const int grid = p.n_items < st->sm_count ? p.n_items : st->sm_count;
  {
    // rounds in which the items are dealt to the CTAs: one group (everything) unless causal
    const int per_unit = p.n_items / (B * H_KV);
    p.group_items = causal ? p.group_units * per_unit : p.n_items;
    const int n_groups = (p.n_items + p.group_items - 1) / p.group_items;
    p.rounds_per_group = (p.group_items + grid - 1) / grid;
    p.total_rounds = p.rounds_per_group * n_groups;
  }
  hk::set_item_decode(p);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (D == 128) return causal ? launch_fwd<128, true>(tq, tk, tv, to, p, grid, stream)
                              : launch_fwd<128, false>(tq, tk, tv, to, p, grid, stream);
  return causal ? launch_fwd<64, true>(tq, tk, tv, to, p, grid, stream)
                : launch_fwd<64, false>(tq, tk, tv, to, p, grid, stream);
}

int hk_attn_fwd_cross(const void* q, const void* k, const void* v, void* o, float* lse, int B, int N, int NK, int H,
                      int H_KV, int D, const long long* q_strides, const long long* k_strides,
                      const long long* v_strides, const int32_t* kv_lens, int causal, float softmax_scale,
                      int device, void* cuda_stream) {
  if (!q || !k || !v || !o || !lse || !q_strides || !k_strides || !v_strides) return HK_EINVAL;
  if (B <= 0 || N <= 0 || NK <= 0 || H <= 0 || H_KV <= 0) return HK_EINVAL;
  if (D != 64 && D != 128) return HK_EUNSUPPORTED;
  if (H % H_KV != 0) return HK_EINVAL;
  for (int i = 0; i < 3; ++i) {
    const long long s3[3] = {q_strides[i], k_strides[i], v_strides[i]};
    for (long long st_i : s3)
      if (st_i <= 0 || st_i % 8 != 0 || st_i >= (1ll << 39)) return HK_EINVAL;
  }
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || (reinterpret_cast<uintptr_t>(lse) & 3))
    return HK_EINVAL;
  return fwd_launch(q, k, v, o, lse, B, N, NK, H, H_KV, D, q_strides, k_strides, v_strides, kv_lens, nullptr, 0, 0,
                    causal, softmax_scale, device, cuda_stream);
}

int hk_attn_fwd_paged(const void* q, const void* k_pages, const void* v_pages, const int32_t* block_table,
                      const int32_t* ctx_lens, void* o, float* lse, int S, int T, int H, int H_KV, int D,
                      int page_size, int max_pages_per_seq, int num_pages, int causal, float softmax_scale,
                      int device, void* cuda_stream) {
  if (!q || !k_pages || !v_pages || !block_table || !ctx_lens || !o || !lse) return HK_EINVAL;
  if (S <= 0 || T <= 0 || H <= 0 || H_KV <= 0 || max_pages_per_seq <= 0 || num_pages <= 0) return HK_EINVAL;
  if ((D != 64 && D != 128) || page_size != 16) return HK_EUNSUPPORTED;
  if (H % H_KV != 0) return HK_EINVAL;
  if (static_cast<long long>(num_pages) * 16 > 0x7fffffffll || static_cast<long long>(max_pages_per_seq) * 16 > 0x3fffffffll)
    return HK_EINVAL;
  if (!aligned16(q) || !aligned16(k_pages) || !aligned16(v_pages) || !aligned16(o) ||
      (reinterpret_cast<uintptr_t>(lse) & 3))
    return HK_EINVAL;
  const long long qs[3] = {(long long)T * H * D, (long long)H * D, D};
  return fwd_launch(q, k_pages, v_pages, o, lse, S, T, max_pages_per_seq * 16, H, H_KV, D, qs, qs, qs, ctx_lens,
                    block_table, max_pages_per_seq, num_pages, causal, softmax_scale, device, cuda_stream);
}

int hk_attn_bwd_prep(const void* o, const void* d_o, float* delta, int B, int N, int H, int D, int device,
                     void* cuda_stream) {
  if (!o || !d_o || !delta) return HK_EINVAL;
  if (B <= 0 || N <= 0 || H <= 0) return HK_EINVAL;
  if (D != 64 && D != 128) return HK_EUNSUPPORTED;
  if (!aligned16(o) || !aligned16(d_o) || (reinterpret_cast<uintptr_t>(delta) & 3)) return HK_EINVAL;
  DeviceState* st = nullptr;
  DeviceScope scope;
  int rc = scope.enter(device, &st);
  if (rc != HK_OK) return rc;
  const long long rows = static_cast<long long>(B) * N * H;
  const int rows_per_block = 8 * (32 / (D / 8));  // 8 warps, D/8 lanes per row
  const long long blocks = (rows + rows_per_block - 1) / rows_per_block;
  if (blocks > 0x7fffffffll) return HK_EINVAL;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  const auto* po = static_cast<const __nv_bfloat16*>(o);
  const auto* pd = static_cast<const __nv_bfloat16*>(d_o);
  if (D == 128) hk::attn_bwd_prep_kernel<128><<<unsigned(blocks), 256, 0, stream>>>(po, pd, delta, B, N, H);
  else hk::attn_bwd_prep_kernel<64><<<unsigned(blocks), 256, 0, stream>>>(po, pd, delta, B, N, H);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  HK_CUDA(cudaGetLastError());
  return HK_OK;
}

int hk_attn_bwd(const void* q, const void* k, const void* v, const void* d_o, const float* lse, const float* delta,
                void* dq, void* dk, void* dv, int B, int N, int H, int H_KV, int D, int causal, float softmax_scale,
                int dq_layout, int device, void* cuda_stream) {
  return hk_attn_bwd_varlen(q, k, v, d_o, lse, delta, dq, dk, dv, B, N, H, H_KV, D, nullptr, causal, softmax_scale,
                            dq_layout, device, cuda_stream);
}

int hk_attn_bwd_varlen(const void* q, const void* k, const void* v, const void* d_o, const float* lse,
                       const float* delta, void* dq, void* dk, void* dv, int B, int N, int H, int H_KV, int D,
                       const int32_t* kv_lens, int causal, float softmax_scale, int dq_layout, int device,
                       void* cuda_stream) {
  return hk_attn_bwd_cross(q, k, v, d_o, lse, delta, dq, dk, dv, B, N, N, H, H_KV, D, kv_lens, causal, softmax_scale,
                           dq_layout, device, cuda_stream);
}

int hk_attn_bwd_cross(const void* q, const void* k, const void* v, const void* d_o, const float* lse,
                      const float* delta, void* dq, void* dk, void* dv, int B, int N, int NK, int H, int H_KV, int D,
                      const int32_t* kv_lens, int causal, float softmax_scale, int dq_layout, int device,
                      void* cuda_stream) {
  if (!q || !k || !v || !d_o || !lse || !delta || !dq || !dk || !dv) return HK_EINVAL;
  if (B <= 0 || N <= 0 || NK <= 0 || H <= 0 || H_KV <= 0) return HK_EINVAL;
  if (D != 64 && D != 128) return HK_EUNSUPPORTED;
  if (H % H_KV != 0) return HK_EINVAL;
  if (dq_layout != HK_DQ_BNHD && dq_layout != HK_DQ_BHND) return HK_EINVAL;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(d_o) || !aligned16(dq) || !aligned16(dk) ||
      !aligned16(dv) || (reinterpret_cast<uintptr_t>(lse) & 3) || (reinterpret_cast<uintptr_t>(delta) & 3))
    return HK_EINVAL;
  DeviceState* st = nullptr;
  DeviceScope scope;
  int rc = scope.enter(device, &st);
  if (rc != HK_OK) return rc;

  const long long qs[3] = {(long long)N * H * D, (long long)H * D, D};
  const long long ks[3] = {(long long)NK * H_KV * D, (long long)H_KV * D, D};
  CUtensorMap tq, tk, tv, tdo;
  if ((rc = make_bnhd_map(&tq, q, B, N, H, D, qs)) != HK_OK) return rc;
  if ((rc = make_bnhd_map(&tk, k, B, NK, H_KV, D, ks)) != HK_OK) return rc;
  if ((rc = make_bnhd_map(&tv, v, B, NK, H_KV, D, ks)) != HK_OK) return rc;
  if ((rc = make_bnhd_map(&tdo, d_o, B, N, H, D, qs)) != HK_OK) return rc;

  hk::BwdParams p;
  p.lse = lse;
  p.delta = delta;
  p.dq = static_cast<__nv_bfloat16*>(dq);
  p.dk = static_cast<__nv_bfloat16*>(dk);
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.dq_stride_b = (long long)N * H * D;
  p.dq_stride_n = dq_layout == HK_DQ_BNHD ? (long long)H * D : D;
  p.dq_stride_h = dq_layout == HK_DQ_BNHD ? D : (long long)N * D;
  p.B = B;
  p.N = N;
  p.NK = NK;
  p.H = H;
  p.H_KV = H_KV;
  p.n_items = 0;
  {
    // causal sweep groups: units whose Q, dO, K and V together stay within ~64 MB of L2
    const int G = H / H_KV;
    const long long unit_bytes = 4ll * G * N * D + 4ll * NK * D;
    long long u = (64ll << 20) / unit_bytes;
    p.group_units = int(u < 1 ? 1 : (u > B * H_KV ? B * H_KV : u));
  }
  p.scale = softmax_scale > 0.f ? softmax_scale : 1.0f / std::sqrt(float(D));
  p.scale_log2 = p.scale * 1.4426950408889634f;
  p.kv_lens = kv_lens;
  p.status = st->status;
#ifdef HK_TRACE
  p.trace = g_trace_buf;
#endif
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (D == 128) return causal ? launch_bwd<128, true>(tq, tk, tv, tdo, p, B, N, NK, H, H_KV, st->sm_count, stream)
                              : launch_bwd<128, false>(tq, tk, tv, tdo, p, B, N, NK, H, H_KV, st->sm_count, stream);
  return causal ? launch_bwd<64, true>(tq, tk, tv, tdo, p, B, N, NK, H, H_KV, st->sm_count, stream)
                : launch_bwd<64, false>(tq, tk, tv, tdo, p, B, N, NK, H, H_KV, st->sm_count, stream);
}

int hk_attn_dq_shuffle(const void* dq_bhnd, void* dq_bnhd, int B, int N, int H, int D, int device,
                       void* cuda_stream) {
  if (!dq_bhnd || !dq_bnhd || dq_bhnd == dq_bnhd) return HK_EINVAL;
  if (B <= 0 || N <= 0 || H <= 0 || D <= 0 || D % 8 != 0) return HK_EINVAL;
  if (!aligned16(dq_bhnd) || !aligned16(dq_bnhd)) return HK_EINVAL;
  DeviceState* st = nullptr;
  DeviceScope scope;
  int rc = scope.enter(device, &st);
  if (rc != HK_OK) return rc;
  const int vec = D / 8;
  const long long total = static_cast<long long>(B) * N * H * vec;
  const long long blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffll) return HK_EINVAL;
  hk::attn_dq_shuffle_kernel<<<unsigned(blocks), 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint4*>(dq_bhnd), static_cast<uint4*>(dq_bnhd), B, N, H, vec);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  HK_CUDA(cudaGetLastError());
  return HK_OK;
}

static int rotary_launch(const void* x, void* o, const void* sin, const void* cos, long long rows, int N, int D,
                         int rotary_dim, int n_div, int pos0, int device, void* cuda_stream) {
  if (!x || !o || !sin || !cos) return HK_EINVAL;
  if (rows <= 0 || N <= 0 || D <= 0 || pos0 < 0) return HK_EINVAL;
  if (rotary_dim <= 0) rotary_dim = D;
  if (D % 8 != 0 || rotary_dim % 16 != 0 || rotary_dim > D) return HK_EUNSUPPORTED;
  if (!aligned16(x) || !aligned16(o) || !aligned16(sin) || !aligned16(cos)) return HK_EINVAL;
  DeviceState* st = nullptr;
  DeviceScope scope;
  int rc = scope.enter(device, &st);
  if (rc != HK_OK) return rc;
  hk::RotaryParams p;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.o = static_cast<__nv_bfloat16*>(o);
  p.cos = static_cast<const __nv_bfloat16*>(cos);
  p.sin = static_cast<const __nv_bfloat16*>(sin);
  p.rows = rows;
  p.N = N;
  p.D = D;
  p.R = rotary_dim;
  p.n_div = n_div;
  p.pos0 = pos0;
  const long long units = p.rows * (rotary_dim / 16 + (D - rotary_dim) / 8);
  const long long blocks = (units + 255) / 256;
  if (blocks > 0x7fffffffll) return HK_EINVAL;
  hk::rotary_kernel<<<unsigned(blocks), 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  HK_CUDA(cudaGetLastError());
  return HK_OK;
}

int hk_rotary(const void* x, void* o, const void* sin, const void* cos, int B, int H, int N, int D, int rotary_dim,
              int device, void* cuda_stream) {
  if (B <= 0 || H <= 0) return HK_EINVAL;
  return rotary_launch(x, o, sin, cos, static_cast<long long>(B) * H * N, N, D, rotary_dim, 1, 0, device, cuda_stream);
}

int hk_rotary_bnhd(const void* x, void* o, const void* sin, const void* cos, int B, int N, int H, int D,
                   int rotary_dim, int pos_offset, int device, void* cuda_stream) {
  if (B <= 0 || H <= 0) return HK_EINVAL;
  return rotary_launch(x, o, sin, cos, static_cast<long long>(B) * N * H, N, D, rotary_dim, H, pos_offset, device,
                       cuda_stream);
}

size_t hk_attn_paged_decode_workspace_bytes(int S, int H, int D, int max_pages_per_seq, int page_size) {
  return hk::decode_workspace_bytes(S, H, D, max_pages_per_seq, page_size);
}

int hk_attn_paged_decode(const void* q, const void* k_pages, const void* v_pages, const int32_t* block_table,
                         const int32_t* ctx_lens, void* o, float* lse, int S, int H, int H_KV, int D,
                         int page_size, int max_pages_per_seq, int num_pages, float softmax_scale,
                         void* workspace, size_t workspace_bytes, int device, void* cuda_stream) {
  if (!q || !k_pages || !v_pages || !block_table || !ctx_lens || !o || !lse) return HK_EINVAL;
  if (S <= 0 || H <= 0 || H_KV <= 0 || max_pages_per_seq <= 0 || num_pages <= 0) return HK_EINVAL;
  if (D != 128 || page_size != 16) return HK_EUNSUPPORTED;
  if (H % H_KV != 0) return HK_EINVAL;
  const int G = H / H_KV;
  if (G < 1 || G > 8) return HK_EUNSUPPORTED;  // the heads of a group sit in the 8 usable rows of one MMA tile
  if (!aligned16(q) || !aligned16(k_pages) || !aligned16(v_pages) || !aligned16(o)) return HK_EINVAL;
  if (!hk::decode_shape_supported(S, H_KV, max_pages_per_seq)) return unsupported_decode_shape(S, H_KV, max_pages_per_seq);
  const size_t need = hk::decode_workspace_bytes(S, H, D, max_pages_per_seq, page_size);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255)) return HK_EWORKSPACE;
  DeviceState* st = nullptr;
  DeviceScope scope;
  int rc = scope.enter(device, &st);
  if (rc != HK_OK) return rc;
  hk::DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_pages = static_cast<const __nv_bfloat16*>(k_pages);
  p.v_pages = static_cast<const __nv_bfloat16*>(v_pages);
  p.block_table = block_table;
  p.ctx_lens = ctx_lens;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.S = S;
  p.H = H;
  p.H_KV = H_KV;
  p.max_pages = max_pages_per_seq;
  p.num_pages = num_pages;
  p.scale = softmax_scale > 0.f ? softmax_scale : 1.0f / std::sqrt(float(D));
  p.scale_log2 = p.scale * 1.4426950408889634f;
  p.workspace = workspace;
  p.status = st->status;
  int launched = 0;
  cudaError_t e = hk::launch_paged_decode(p, st->sm_count, static_cast<cudaStream_t>(cuda_stream), &launched);
  g_launches.fetch_add(launched, std::memory_order_relaxed);
  if (e != cudaSuccess) return cuda_fail(e, "paged decode launch");
  return HK_OK;
}

int hk_paged_kv_append(const void* k_new, const void* v_new, void* k_pages, void* v_pages,
                       const int32_t* block_table, const int32_t* start_pos, int S, int T, int H_KV, int D,
                       int page_size, int max_pages_per_seq, int num_pages, int device, void* cuda_stream) {
  if (!k_new || !v_new || !k_pages || !v_pages || !block_table || !start_pos) return HK_EINVAL;
  if (S <= 0 || T <= 0 || H_KV <= 0 || D <= 0 || max_pages_per_seq <= 0 || num_pages <= 0) return HK_EINVAL;
  if (page_size != hk::kPageTokens) return HK_EUNSUPPORTED;
  if ((H_KV * D) % 8 != 0 || T > 65535 || S > 65535) return HK_EINVAL;
  if (!aligned16(k_new) || !aligned16(v_new) || !aligned16(k_pages) || !aligned16(v_pages)) return HK_EINVAL;
  DeviceState* st = nullptr;
  DeviceScope scope;
  int rc = scope.enter(device, &st);
  if (rc != HK_OK) return rc;
  hk::AppendParams p;
  p.k_new = static_cast<const __nv_bfloat16*>(k_new);
  p.v_new = static_cast<const __nv_bfloat16*>(v_new);
  p.k_pages = static_cast<__nv_bfloat16*>(k_pages);
  p.v_pages = static_cast<__nv_bfloat16*>(v_pages);
  p.block_table = block_table;
  p.start_pos = start_pos;
  p.S = S;
  p.T = T;
  p.row_vec16 = H_KV * D * 2 / 16;
  p.max_pages = max_pages_per_seq;
  p.num_pages = num_pages;
  p.status = st->status;
  const long long groups = (static_cast<long long>(S) * T + hk::kAppendUnroll - 1) / hk::kAppendUnroll;
  const long long max_blocks = static_cast<long long>(st->sm_count) * 16;  // 16 x 128 threads fill an SM
  const unsigned blocks = static_cast<unsigned>(groups < max_blocks ? groups : max_blocks);
  hk::paged_kv_append_kernel<<<blocks, 128, 0, static_cast<cudaStream_t>(cuda_stream)>>>(p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  HK_CUDA(cudaGetLastError());
  return HK_OK;
}

int hk_paged_kv_append_rotary(const void* k_new, const void* v_new, void* k_pages, void* v_pages,
                              const int32_t* block_table, const int32_t* start_pos, const void* sin, const void* cos,
                              int S, int T, int H_KV, int D, int rotary_dim, int cos_rows, int page_size,
                              int max_pages_per_seq, int num_pages, int device, void* cuda_stream) {
  if (!k_new || !v_new || !k_pages || !v_pages || !block_table || !start_pos || !sin || !cos) return HK_EINVAL;
  if (S <= 0 || T <= 0 || H_KV <= 0 || D <= 0 || max_pages_per_seq <= 0 || num_pages <= 0 || cos_rows <= 0)
    return HK_EINVAL;
  if (page_size != hk::kPageTokens) return HK_EUNSUPPORTED;
  if (rotary_dim <= 0) rotary_dim = D;
  if (D % 8 != 0 || rotary_dim % 16 != 0 || rotary_dim > D) return HK_EUNSUPPORTED;
  if (T > 65535 || S > 65535) return HK_EINVAL;
  if (!aligned16(k_new) || !aligned16(v_new) || !aligned16(k_pages) || !aligned16(v_pages) || !aligned16(sin) ||
      !aligned16(cos))
    return HK_EINVAL;
  DeviceState* st = nullptr;
  DeviceScope scope;
  int rc = scope.enter(device, &st);
  if (rc != HK_OK) return rc;
  hk::AppendRotaryParams q;
  q.a.k_new = static_cast<const __nv_bfloat16*>(k_new);
  q.a.v_new = static_cast<const __nv_bfloat16*>(v_new);
  q.a.k_pages = static_cast<__nv_bfloat16*>(k_pages);
  q.a.v_pages = static_cast<__nv_bfloat16*>(v_pages);
  q.a.block_table = block_table;
  q.a.start_pos = start_pos;
  q.a.S = S;
  q.a.T = T;
  q.a.row_vec16 = H_KV * D * 2 / 16;
  q.a.max_pages = max_pages_per_seq;
  q.a.num_pages = num_pages;
  q.a.status = st->status;
  q.cos = static_cast<const __nv_bfloat16*>(cos);
  q.sin = static_cast<const __nv_bfloat16*>(sin);
  q.cos_rows = cos_rows;
  q.H_KV = H_KV;
  q.D = D;
  q.R = rotary_dim;
  const long long tokens = static_cast<long long>(S) * T;
  const long long max_blocks = static_cast<long long>(st->sm_count) * 16;  // 16 x 128 threads fill an SM
  const unsigned blocks = static_cast<unsigned>(tokens < max_blocks ? tokens : max_blocks);
  hk::paged_kv_append_rotary_kernel<<<blocks, 128, 0, static_cast<cudaStream_t>(cuda_stream)>>>(q);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  HK_CUDA(cudaGetLastError());
  return HK_OK;
}

int hk_last_device_status(int device) {
  DeviceState* st = nullptr;
  DeviceScope scope;
  int rc = scope.enter(device, &st);
  if (rc != HK_OK) return rc;
  HK_CUDA(cudaDeviceSynchronize());
  int word = 0;
  HK_CUDA(cudaMemcpy(&word, st->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (word != 0) HK_CUDA(cudaMemset(st->status, 0, sizeof(int)));
  return status_to_code(word);
}

int hk_selftest_fastdiv(void) {
  // host only: the multiply-and-shift division of the item decode against the division it replaces, for every
  // divisor up to 4096, divisors around every power of two, and dividends at the edges of [0, 2^31)
  auto check = [](int d) {
    const hk::FastDiv fd(d);
    const long long top = 0x7fffffffll;
    const long long probes[] = {0, 1, d - 1ll, d, d + 1ll, 2ll * d - 1, 2ll * d, 1000003ll * d + d - 1, top - d, top - 1, top,
                                0x3fffffffll, 123456789ll, 2000000011ll};
    for (long long n : probes) {
      if (n < 0 || n > top) continue;
      if (fd.div_host(int(n)) != int(n / d)) return false;
    }
    return true;
  };
  for (int d = 1; d <= 4096; ++d)
    if (!check(d)) return HK_EINVAL;
  for (int k = 1; k < 31; ++k)
    for (int e = -1; e <= 1; ++e) {
      const long long d = (1ll << k) + e;
      if (d >= 1 && d <= 0x7fffffffll && !check(int(d))) return HK_EINVAL;
    }
  return HK_OK;
}

int hk_selftest_bounded_wait(int device, unsigned limit_us) {
  DeviceState* st = nullptr;
  DeviceScope scope;
  int rc = scope.enter(device, &st);
  if (rc != HK_OK) return rc;
  if (limit_us == 0 || limit_us > 1000000u) return HK_EINVAL;
  bounded_wait_selftest_kernel<<<1, 32>>>(st->status, static_cast<unsigned long long>(limit_us) * 1000ull);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  HK_CUDA(cudaGetLastError());
  return hk_last_device_status(device);
}

unsigned long long hk_kernel_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* hk_strerror(int code) {
  switch (code) {
    case HK_OK: return "ok";
    case HK_EINVAL: return "invalid argument (shape, null or misaligned pointer)";
    case HK_EUNSUPPORTED: return "unsupported configuration or device";
    case HK_ECUDA: return "CUDA call failed";
    case HK_ETIMEOUT: return "bounded device-side wait expired";
    case HK_EWORKSPACE: return "workspace missing, misaligned or too small";
    case HK_EBADPAGE: return "block-table entry outside the page pool";
    case HK_EBADLEN: return "context length beyond the block table's capacity (clamped)";
    default: return "unknown error code";
  }
}

const char* hk_last_cuda_error(void) { return g_cuda_err; }

}  // extern "C"

// ---------------------------------------------------------------------------------------------------
// Allocation-free paged decode: scratch and status live in the library image instead of in memory the
// caller or this library would have to allocate (see hk_attn_paged_decode_static in hk_attn.h).
// In host code `g_decode_static_scratch` is only a handle for the runtime, not a device address; the
// address each device gave the array is looked up once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_decode_static_scratch[HK_DECODE_STATIC_SCRATCH_BYTES];
static __device__ int g_decode_static_status;

namespace {

struct StaticDecodeState {
  std::mutex mu;
  bool ready = false;       // a failed set-up is retried by the next call
  int sm_count = 0;
  void* scratch = nullptr;  // device address of g_decode_static_scratch on this device
  int* status = nullptr;    // device address of g_decode_static_status on this device
};
StaticDecodeState g_static_dev[kMaxDevices];

// Runs once per device, with that device current. Nothing in here allocates.
int init_static_decode(int device) {
  StaticDecodeState& st = g_static_dev[device];
  cudaDeviceProp prop;
  HK_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "device %d is sm_%d%d; this library needs sm_100", device, prop.major,
             prop.minor);
    return HK_EUNSUPPORTED;
  }
  st.sm_count = prop.multiProcessorCount;
  HK_CUDA(cudaGetSymbolAddress(&st.scratch, g_decode_static_scratch));
  HK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&st.status), g_decode_static_status));
  if (!st.scratch || !st.status || (reinterpret_cast<uintptr_t>(st.scratch) & 255)) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "static decode scratch has no usable device address");
    return HK_ECUDA;
  }
  return hk::prepare_decode_kernels(g_cuda_err, sizeof(g_cuda_err));
}

}  // namespace

extern "C" int hk_attn_paged_decode_static(const void* q, const void* k_pages, const void* v_pages,
                                           const int32_t* block_table, const int32_t* ctx_lens, void* o, float* lse,
                                           int S, int H, int H_KV, int D, int page_size, int max_pages_per_seq,
                                           int num_pages, float softmax_scale, int device, void* cuda_stream,
                                           int* status_out) {
  if (!q || !k_pages || !v_pages || !block_table || !ctx_lens || !o || !lse) return HK_EINVAL;
  if (S <= 0 || H <= 0 || H_KV <= 0 || max_pages_per_seq <= 0 || num_pages <= 0) return HK_EINVAL;
  if (D != 128 || page_size != 16) return HK_EUNSUPPORTED;
  if (H % H_KV != 0) return HK_EINVAL;
  const int G = H / H_KV;
  if (G < 1 || G > 8) return HK_EUNSUPPORTED;  // the heads of a group sit in the 8 usable rows of one MMA tile
  if (!aligned16(q) || !aligned16(k_pages) || !aligned16(v_pages) || !aligned16(o)) return HK_EINVAL;
  if (!hk::decode_shape_supported(S, H_KV, max_pages_per_seq)) return unsupported_decode_shape(S, H_KV, max_pages_per_seq);
  const size_t need = hk::decode_workspace_bytes(S, H, D, max_pages_per_seq, page_size);
  if (need == 0 || need > HK_DECODE_STATIC_SCRATCH_BYTES) {
    snprintf(g_cuda_err, sizeof(g_cuda_err),
             "problem needs %zu bytes of scratch, the built-in array holds %u: use hk_attn_paged_decode", need,
             unsigned(HK_DECODE_STATIC_SCRATCH_BYTES));
    return HK_EWORKSPACE;
  }
  DeviceScope scope;  // the caller's current device is put back on return
  {
    const int rc = scope.enter_raw(device, &device);
    if (rc != HK_OK) return rc;
  }
  StaticDecodeState& st = g_static_dev[device];
  {
    std::lock_guard<std::mutex> lock(st.mu);
    if (!st.ready) {
      const int rc = init_static_decode(device);
      if (rc != HK_OK) return rc;
      st.ready = true;
    }
  }

  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  // the status word is shared by all calls and keeps the last call's value: start this call from zero
  HK_CUDA(cudaMemsetAsync(st.status, 0, sizeof(int), stream));
  hk::DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_pages = static_cast<const __nv_bfloat16*>(k_pages);
  p.v_pages = static_cast<const __nv_bfloat16*>(v_pages);
  p.block_table = block_table;
  p.ctx_lens = ctx_lens;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.S = S;
  p.H = H;
  p.H_KV = H_KV;
  p.max_pages = max_pages_per_seq;
  p.num_pages = num_pages;
  p.scale = softmax_scale > 0.f ? softmax_scale : 1.0f / std::sqrt(float(D));
  p.scale_log2 = p.scale * 1.4426950408889634f;
  p.workspace = st.scratch;  // the looked-up device address, never the host-side symbol
  p.status = st.status;
  int launched = 0;
  cudaError_t e = hk::launch_paged_decode(p, st.sm_count, stream, &launched);
  g_launches.fetch_add(launched, std::memory_order_relaxed);
  if (e != cudaSuccess) return cuda_fail(e, "paged decode launch");
  if (status_out) {
    int word = 0;
    HK_CUDA(cudaMemcpyAsync(&word, st.status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    HK_CUDA(cudaStreamSynchronize(stream));
    *status_out = status_to_code(word);
  }
  return HK_OK;
}

