// Host side of the persistent decode kernel (decode_kernel.cuh): work planning
// (K-slices, grid, shared-memory budget) and launch.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>

#include "decode_kernel.cuh"
#include "kernels.h"

namespace mlxr {

using namespace decode;

static unsigned long long* g_trace = nullptr;  // set by mlxr_debug_set_trace_buffer
void set_decode_trace(void* p) { g_trace = (unsigned long long*)p; }
void* get_decode_trace() { return g_trace; }
static std::atomic<int> g_launch_mode{MLXR_DECODE_LAUNCH_OVERLAPPED};
void set_decode_launch_mode(int mode) { g_launch_mode.store(mode); }
static std::atomic<unsigned long long> g_wait_ns{2000000000ull};   // limit of every device-side wait
void set_wait_limit_ns(unsigned long long ns) { g_wait_ns.store(ns ? ns : 1ull); }
unsigned long long wait_limit_ns() { return g_wait_ns.load(); }

// Device properties, per device (a process may drive several GPUs).
struct DevProps { int num_sms = 0; int max_smem = 0; };
static std::mutex g_props_mu;
static DevProps g_props[64];

// ---- tensor maps -----------------------------------------------------------------------------
// A packed matrix [rows][row_bytes] is described to the TMA unit as a 2-D tensor of 8-byte
// elements with a box of 36 x 8 (288 bytes x 8 rows).  cuTensorMapEncodeTiled is a pure host
// function fetched from the driver at run time (no link against libcuda); maps are cached per
// (pointer, rows, row_bytes) because weights are long-lived.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static int weight_tensor_map(const void* w, int rows, int row_bytes, CUtensorMap* out) {
  static EncodeTiledFn encode = nullptr;
  static std::mutex mu;
  static std::map<std::tuple<const void*, int, int>, CUtensorMap> cache;
  std::lock_guard<std::mutex> lk(mu);
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    MLXR_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (!fn || q != cudaDriverEntryPointSuccess) { set_error("cuTensorMapEncodeTiled is not available in this driver"); return MLXR_ERR_CUDA; }
    encode = (EncodeTiledFn)fn;
  }
  const auto key = std::make_tuple(w, rows, row_bytes);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return MLXR_OK; }
  const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 8), (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(kRowStride / 8), 8};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(w), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d) for a %d x %d byte matrix", (int)r, rows, row_bytes); return MLXR_ERR_CUDA; }
  if (cache.size() > 4096) cache.clear();
  cache[key] = *out;
  return MLXR_OK;
}

static int device_props(DevProps* out) {
  int dev = 0;
  MLXR_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) { set_error("device index %d outside 0..63", dev); return MLXR_ERR_INVALID_ARGUMENT; }
  std::lock_guard<std::mutex> lk(g_props_mu);
  DevProps& d = g_props[dev];
  if (!d.num_sms) {
    int sms = 0, smem = 0;
    MLXR_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    MLXR_CUDA_TRY(cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    d.max_smem = smem;
    d.num_sms = sms;
  }
  *out = d;
  return MLXR_OK;
}

bool decode_supported(int qt, int M, int K, const void* const* w, int nmat) {
  if (qt != MLXR_Q4_K && qt != MLXR_Q4_0) return false;
  if (M < 1 || M > 8 || K < 512 || K % 256 != 0) return false;   // a TMA box is two 256-blocks wide
  for (int i = 0; i < nmat; i++)
    if (((uintptr_t)w[i]) & 15u) return false;
  return true;
}

// Choose the number of K-slices S for a phase running on G CTAs with ng groups each
// (G % S == 0).  Cost = segments streamed by the busiest CTA; the split-K fix-up and slices
// with fewer segments than warps in a group are penalised.
static int choose_slices(int ntiles, int nseg, int G, int ng, int M, int xrows, int max_x_bytes, bool fixed_grid) {
  double best = 1e30;
  int bestS = 0;
  for (int S = 1; S <= std::min(nseg, 16); S *= 2) {   // powers of two: slice and lane by shift and mask
    if (fixed_grid && (G % S != 0)) continue;
    const int g = fixed_grid ? G : (G / S) * S;
    if (g < 1) continue;
    const int segs = (nseg + S - 1) / S;
    if (xrows * M * (segs * 256 + 32) > max_x_bytes) continue;
    if (S > 1 && ntiles > 2000) continue;  // tile counters live in a fixed pool
    const int lanes = (g / S) * ng;        // (CTA, group) pairs sharing the tiles of one slice
    int tiles_cta0 = 0;                    // CTA 0 owns lanes 0 .. ng-1: the busiest
    for (int gi = 0; gi < ng; gi++)
      if (gi < ntiles) tiles_cta0 += (ntiles - 1 - gi) / lanes + 1;
    double cost = (double)tiles_cta0 * segs;
    if (S > 1) cost *= 1.3;                // every tile pays a fix-up round trip through L2
    if (segs < kGroupWarps) cost *= 1.25;  // warps without a segment idle
    if (cost < best) { best = cost; bestS = S; }
  }
  return bestS;
}

template <int QT, typename T, int NT, int NG, bool PAIRS>
static int launch_inst(const Params& P, const SmemPlan& plan, int G, const DevProps& props, cudaStream_t st) {
  auto kern = decode_kernel<QT, T, NT, NG, PAIRS>;
  constexpr int kThreads = NG * kGroupWarps * 32;
  // Once per (device, instantiation): raise the shared-memory limit and check that a CTA of the
  // largest plan is resident on every SM, i.e. that a grid of one CTA per SM is co-resident when
  // the device runs nothing else (chained phases wait for each other's output).
  static std::mutex mu;
  static bool attr_done[64] = {};
  int dev = 0;
  MLXR_CUDA_TRY(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lk(mu);
    if (!attr_done[dev & 63]) {
      MLXR_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, props.max_smem));
      int per_sm = 0;
      MLXR_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, (size_t)props.max_smem));
      if (per_sm < 1) { set_error("decode kernel: a CTA with %d bytes of shared memory is not resident on this device", props.max_smem); return MLXR_ERR_UNSUPPORTED; }
      attr_done[dev & 63] = true;
    }
  }
  // launch mode: 0 cooperative, 1 plain, 2 plain with programmatic overlap
  int mode = g_launch_mode.load();
  if (const char* e = tune_env("MLXR_DEC_LAUNCH")) mode = atoi(e);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = (size_t)plan.total;
  cfg.stream = st;
  cudaLaunchAttribute at[2];
  int na = 0;
  if (mode == 0 || mode == 3) { at[na].id = cudaLaunchAttributeCooperative; at[na].val.cooperative = 1; na++; }
  if (mode >= 2) { at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[na].val.programmaticStreamSerializationAllowed = 1; na++; }
  cfg.attrs = at;
  cfg.numAttrs = na;
  MLXR_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, P, plan));
  count_launch();
  return MLXR_OK;
}

// Launch one or two chained phases.  sync: workspace sync words (zero-initialised once);
// word 0 is the grid-barrier counter whose host mirror is *bar_host.
static int launch_decode_impl(const DecodeLinear* lin, int nphases, int M, int qt, int dtype, void* scratch,
                              size_t scratch_bytes, uint32_t* sync, uint32_t* bar_host, int* status, cudaStream_t st,
                              const DecodeTp* tp, int force_groups);

int launch_decode(const DecodeLinear* lin, int nphases, int M, int qt, int dtype, void* scratch,
                  size_t scratch_bytes, uint32_t* sync, uint32_t* bar_host, int* status, cudaStream_t st,
                  const DecodeTp* tp) {
  return launch_decode_impl(lin, nphases, M, qt, dtype, scratch, scratch_bytes, sync, bar_host, status, st, tp, 0);
}

// force_groups: 0 = choose, 1 or 2 = that many warp groups per CTA
static int launch_decode_impl(const DecodeLinear* lin, int nphases, int M, int qt, int dtype, void* scratch,
                              size_t scratch_bytes, uint32_t* sync, uint32_t* bar_host, int* status, cudaStream_t st,
                              const DecodeTp* tp, int force_groups) {
  DevProps props;
  if (int r = device_props(&props)) return r;
  const int g_num_sms = props.num_sms, g_max_smem = props.max_smem;
  if (nphases > 1 && !(nphases == 2 && lin[0].interleave && lin[0].y_tagged && lin[1].x_tagged && lin[1].x == lin[0].y_tagged && !lin[1].gamma)) {
    set_error("decode kernel: chained phases need the tagged hand-over buffer between them");
    return MLXR_ERR_INVALID_ARGUMENT;
  }
  Params P;
  memset(&P, 0, sizeof(P));
  P.nphases = nphases;
  P.M = M;
  P.seq_ctl = nphases > 1 ? sync : nullptr;
  P.wait_ns = g_wait_ns.load();
  P.flags = 0;
  if (const char* e = tune_env("MLXR_DEC_FLAGS")) P.flags = (uint32_t)atoi(e);
  P.status = status;
  P.trace = g_trace;
  P.tp_world = 0;
  if (tp && tp->world > 1) {
    const DecodeLinear& last = lin[nphases - 1];
    if (last.nmat != 1 || last.interleave || last.epi[0] != 3 || (size_t)M * last.rows[0] > kTpSlotElems ||
        (last.rows[0] + kTileRows - 1) / kTileRows > kTpFlagsPerRank) {
      set_error("decode kernel: this shape cannot take the fused exchange");
      return MLXR_ERR_UNSUPPORTED;
    }
    for (int i = 0; i < kTpMaxWorld; i++) P.tp_peer[i] = tp->peer[i];
    P.tp_rank = tp->rank;
    P.tp_world = tp->world;
    P.tp_ctl = tp->ctl;
    P.tp_y = tp->y;
  }
  // batch <= 2 with Q4_K: pairs in the MMA columns, one n-tile per batch row
  bool pairs = (qt == MLXR_Q4_K && M <= 2);
  if (const char* e = tune_env("MLXR_DEC_PAIRS")) pairs = pairs && atoi(e) != 0;
  const int NT = pairs ? M : (M <= 4 ? 1 : 2);
  const int xrows = 2;
  const int MB = 4 * NT;
  const int auxw = qt == MLXR_Q4_K ? 4 : 8;
  int G = g_num_sms;
  // shared memory left for the x slice when the rings keep at least two stages per warp
  auto x_budget = [&](int ng) {
    const int fixed = ng * kSlots * (kGroupWarps + 1) * kTileRows * MB * 4 + 2048 + 256;
    return g_max_smem - 2 * ng * kGroupWarps * kStageBytes - fixed - M * 64 * (auxw + 1) * 4;
  };
  // Two warp groups per CTA unless one group gets by with fewer K-slices: beyond batch 2 the
  // activations compete with the rings for shared memory, and a K split over CTAs (a fix-up
  // through L2 per tile) costs more than the second group gains.
  int NG = 2;
  if (force_groups == 1 || force_groups == 2) NG = force_groups;
  else if (const char* e = tune_env("MLXR_DEC_GROUPS")) { const int v = atoi(e); if (v == 1 || v == 2) NG = v; }
  else if (M > 2) {
    int worst[3] = {0, 0, 0};
    for (int ng = 1; ng <= 2; ng++)
      for (int i = 0; i < nphases; i++) {
        const DecodeLinear& L = lin[i];
        int rows = 0;
        for (int j = 0; j < L.nmat; j++) rows += L.rows[j];
        const int nt = L.interleave ? (L.rows[0] + 7) / 8 : (rows + kTileRows - 1) / kTileRows;
        const int sl = choose_slices(nt, L.K / 256, G, ng, M, xrows, x_budget(ng), nphases > 1 || i > 0);
        worst[ng] = std::max(worst[ng], sl <= 0 ? 1 << 20 : sl);
      }
    if (worst[1] < worst[2]) NG = 1;
  }
  const int max_x = x_budget(NG);
  int max_slice_segs = 0;
  size_t scratch_off = 0;
  int counter_off = 16;
  for (int i = 0; i < nphases; i++) {
    const DecodeLinear& L = lin[i];
    Phase& ph = P.ph[i];
    int total_rows = 0;
    for (int j = 0; j < 3; j++) {
      ph.w[j] = (const uint8_t*)L.w[j];
      ph.rows[j] = j < L.nmat ? L.rows[j] : 0;
      ph.y[j] = L.y[j];
      ph.bias[j] = L.bias[j];
      ph.epi[j] = L.epi[j];
      if (j < L.nmat) total_rows += L.rows[j];
    }
    ph.nmat = L.nmat;
    for (int j = 0; j < L.nmat; j++) {
      if (L.nmat > 1 && !L.interleave && L.rows[j] % 8 != 0) { set_error("decode kernel: stacked matrices need row counts that are multiples of 8"); return MLXR_ERR_UNSUPPORTED; }
      if (int r = weight_tensor_map(L.w[j], L.rows[j], (L.K / 256) * kSegBytes, &P.tmap[i][j])) return r;
    }
    ph.interleave = L.interleave;
    ph.n_total = L.interleave ? L.rows[0] : total_rows;
    ph.K = L.K;
    const int nseg = L.K / 256;
    ph.row_bytes = nseg * kSegBytes;
    ph.ntiles = L.interleave ? (ph.n_total + 7) / 8 : (ph.n_total + kTileRows - 1) / kTileRows;
    int S = choose_slices(ph.ntiles, nseg, G, NG, M, xrows, max_x, nphases > 1 || i > 0);
    if (const char* e = tune_env("MLXR_DEC_S")) { const int v = atoi(e); if (v >= 1 && v <= nseg && (v & (v - 1)) == 0 && (nphases == 1 || G % v == 0)) S = v; }
    if (S <= 0) {
      if (NG == 2 && force_groups == 0 && !tune_env("MLXR_DEC_GROUPS"))   // no room beside 16 rings: one group
        return launch_decode_impl(lin, nphases, M, qt, dtype, scratch, scratch_bytes, sync, bar_host, status, st, tp, 1);
      set_error("decode kernel: x slice does not fit shared memory (K=%d, M=%d)", L.K, M);
      return MLXR_ERR_UNSUPPORTED;
    }
    if (P.tp_world > 1 && i == nphases - 1 && S > 1) {
      // a K split of the exchanging phase needs a flag and a system-scope fence per tile inside the
      // hot loop (measured: 172 us instead of 103 us on the 70B-shaped block over 2 GPUs): leave
      // such shapes to the two-kernel form
      set_error("decode kernel: the fused exchange is not used when the last phase is split over CTAs");
      return MLXR_ERR_UNSUPPORTED;
    }
    if (nphases == 1) G = (G / S) * S;
    ph.S = S;
    ph.s_shift = 0;
    while ((1 << ph.s_shift) < S) ph.s_shift++;
    ph.segs_base = nseg / S;
    ph.segs_extra = nseg % S;
    ph.max_slice_segs = ph.segs_base + (ph.segs_extra ? 1 : 0);
    max_slice_segs = std::max(max_slice_segs, ph.max_slice_segs);
    ph.x = L.x;
    ph.gamma = L.gamma;
    ph.eps = L.eps;
    ph.cos_t = (const __half*)L.cos_t;
    ph.sin_t = (const __half*)L.sin_t;
    ph.positions = L.positions;
    ph.head_dim = L.head_dim;
    ph.max_seq = L.max_seq;
    ph.pos_offset = L.pos_offset;
    ph.y_tagged = (unsigned long long*)L.y_tagged;
    ph.x_tagged = L.x_tagged;
    // second of two chained phases: tile lanes run from the last (CTA, group) pair downwards, so
    // that the pairs with one tile more in the first phase are the ones left without a tile here
    ph.reverse = (nphases == 2 && i == 1) ? 1 : 0;
    if (S > 1) {
      const size_t bytes = (size_t)S * ph.ntiles * kTileRows * MB * sizeof(float);
      if (scratch_off + bytes > scratch_bytes) { set_error("decode kernel: split-K scratch too small"); return MLXR_ERR_WORKSPACE; }
      ph.partials = (float*)((char*)scratch + scratch_off);
      scratch_off += (bytes + 255) & ~(size_t)255;
      if (counter_off + ph.ntiles > kSyncWords) { set_error("decode kernel: too many tiles for split-K"); return MLXR_ERR_WORKSPACE; }
      ph.counters = sync + counter_off;
      counter_off += ph.ntiles;
    }
  }
  for (int i = 0; i < nphases; i++) {
    Phase& ph = P.ph[i];
    ph.lane_step = (G / ph.S) * NG;
    ph.lane_q = (ph.ntiles - 1) / ph.lane_step;
    ph.lane_r = (ph.ntiles - 1) % ph.lane_step;
  }
  // shared-memory plan: as many ring stages per warp as fit
  int stages = kMaxStages;
  if (const char* e = tune_env("MLXR_DEC_STAGES")) { const int v = atoi(e); if (v >= 2 && v <= kMaxStages) stages = v; }
  SmemPlan plan = make_plan(NG, stages, max_slice_segs, M, MB, auxw, pairs ? 1 : 0);
  while (plan.total > g_max_smem && stages > 2) {
    stages--;
    plan = make_plan(NG, stages, max_slice_segs, M, MB, auxw, pairs ? 1 : 0);
  }
  if (plan.total > g_max_smem) { set_error("decode kernel: shared memory plan does not fit"); return MLXR_ERR_UNSUPPORTED; }
  int rc = MLXR_OK;
#define INST(QT, T, NTV, NGV)                                                                      \
  do {                                                                                             \
    if (pairs) { if constexpr (QT == MLXR_Q4_K) rc = launch_inst<QT, T, NTV, NGV, true>(P, plan, G, props, st); } \
    else rc = launch_inst<QT, T, NTV, NGV, false>(P, plan, G, props, st);                            \
  } while (0)
#define BY_NT(QT, T)                                                                   \
  do {                                                                                 \
    if (NT == 1) { if (NG == 2) INST(QT, T, 1, 2); else INST(QT, T, 1, 1); }           \
    else { if (NG == 2) INST(QT, T, 2, 2); else INST(QT, T, 2, 1); }                   \
  } while (0)
#define BY_T(QT)                                                         \
  do {                                                                   \
    if (dtype == MLXR_F16) BY_NT(QT, __half);                            \
    else if (dtype == MLXR_BF16) BY_NT(QT, __nv_bfloat16);               \
    else BY_NT(QT, float);                                               \
  } while (0)
  if (qt == MLXR_Q4_K) BY_T(MLXR_Q4_K); else BY_T(MLXR_Q4_0);
#undef BY_T
#undef BY_NT
#undef INST
  (void)bar_host;
  return rc;
}

}  // namespace mlxr
