// Host side of the persistent decode kernel (decode_kernel.cuh): work planning
// (K-slices, grid, shared-memory budget) and launch.
#include <algorithm>
#include <cstring>

#include "decode_kernel.cuh"
#include "kernels.h"

namespace mlxr {

using namespace decode;

static int g_num_sms = 0;
static int g_max_smem = 0;

static int device_props() {
  if (g_num_sms) return MLXR_OK;
  int dev = 0;
  MLXR_CUDA_TRY(cudaGetDevice(&dev));
  MLXR_CUDA_TRY(cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev));
  MLXR_CUDA_TRY(cudaDeviceGetAttribute(&g_max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
  return MLXR_OK;
}

bool decode_supported(int qt, int M, int K, const void* const* w, int nmat) {
  if (qt != MLXR_Q4_K && qt != MLXR_Q4_0) return false;
  if (M < 1 || M > 16 || K <= 0 || K % 256 != 0) return false;
  for (int i = 0; i < nmat; i++)
    if (((uintptr_t)w[i]) & 15u) return false;
  return true;
}

// Choose the number of K-slices S for a phase running on G CTAs (G % S == 0).  Cost =
// rounds of items per CTA x segments per item; slices that leave consumer warps idle
// (fewer than 6 segments per chunk) and the split-K fix-up are penalised.
static int choose_slices(int ntiles, int nseg, int G, int mcols, int max_x_bytes, bool fixed_grid) {
  double best = 1e30;
  int bestS = 0;
  for (int S = 1; S <= std::min(nseg, 16); S++) {
    if (fixed_grid ? (G % S != 0) : false) continue;
    const int g = fixed_grid ? G : (G / S) * S;
    if (g < 1) continue;
    const int segs = (nseg + S - 1) / S;
    if (mcols * (segs * 512 + 64) > max_x_bytes) continue;
    if (S > 1 && ntiles > 2000) continue;  // tile counters live in a fixed pool
    const int rounds = (ntiles * S + g - 1) / g;
    const int nchunks = (segs + kMaxChunkSegs - 1) / kMaxChunkSegs;
    const int csegs = segs / nchunks;
    double cost = (double)rounds * segs;
    if (csegs < 6) cost *= 1.0 + 0.04 * (6 - csegs);
    if (S > 1) cost *= 1.05;
    if (cost < best) { best = cost; bestS = S; }
  }
  return bestS;
}


template <int QT, typename T, int NT>
static int launch_inst(const Params& P, const SmemPlan& plan, int G, bool cooperative, cudaStream_t st) {
  auto kern = decode_kernel<QT, T, NT>;
  static bool attr_done[64] = {};
  int dev = 0;
  MLXR_CUDA_TRY(cudaGetDevice(&dev));
  if (!attr_done[dev & 63]) {
    MLXR_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, g_max_smem));
    attr_done[dev & 63] = true;
  }
  if (cooperative) {
    void* args[] = {(void*)&P, (void*)&plan};
    MLXR_CUDA_TRY(cudaLaunchCooperativeKernel((void*)kern, dim3(G), dim3(kThreads), args, (size_t)plan.total, st));
    count_launch();
  } else {
    kern<<<G, kThreads, plan.total, st>>>(P, plan);
    MLXR_LAUNCH_CHECK("decode_kernel");
  }
  return MLXR_OK;
}

// Launch one or two chained phases.  sync: workspace sync words (zero-initialised once);
// word 0 is the grid-barrier counter whose host mirror is *bar_host.
int launch_decode(const DecodeLinear* lin, int nphases, int M, int qt, int dtype, void* scratch,
                  size_t scratch_bytes, uint32_t* sync, uint32_t* bar_host, int* status, cudaStream_t st) {
  if (int r = device_props()) return r;
  Params P;
  memset(&P, 0, sizeof(P));
  P.nphases = nphases;
  P.M = M;
  P.gridbar = sync;
  P.bar_base = *bar_host;
  P.status = status;
  const int NT = M <= 8 ? 1 : 2;
  const int MC = 8 * NT;
  int G = g_num_sms;
  const int ring_min = 4 * kStageBytes;
  const int fixed = MC * kConsumerWarps * kTileRows * 4 + kTileRows * MC * 4 + 1024;
  const int max_x = g_max_smem - ring_min - fixed - MC * 64 * 4;
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
    ph.interleave = L.interleave;
    ph.n_total = L.interleave ? L.rows[0] : total_rows;
    ph.K = L.K;
    const int nseg = L.K / 256;
    ph.row_bytes = nseg * kSegBytes;
    ph.ntiles = L.interleave ? (ph.n_total + 7) / 8 : (ph.n_total + kTileRows - 1) / kTileRows;
    const int S = choose_slices(ph.ntiles, nseg, G, M, max_x, nphases > 1 || i > 0);
    if (S <= 0) { set_error("decode kernel: x slice does not fit shared memory (K=%d, M=%d)", L.K, M); return MLXR_ERR_UNSUPPORTED; }
    if (nphases == 1) G = (G / S) * S;
    ph.S = S;
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
    if (S > 1) {
      const size_t bytes = (size_t)S * ph.ntiles * kTileRows * MC * sizeof(float);
      if (scratch_off + bytes > scratch_bytes) { set_error("decode kernel: split-K scratch too small"); return MLXR_ERR_WORKSPACE; }
      ph.partials = (float*)((char*)scratch + scratch_off);
      scratch_off += (bytes + 255) & ~(size_t)255;
      if (counter_off + ph.ntiles > kSyncWords) { set_error("decode kernel: too many tiles for split-K"); return MLXR_ERR_WORKSPACE; }
      ph.counters = sync + counter_off;
      counter_off += ph.ntiles;
    }
  }
  // shared-memory plan: as many ring stages as fit
  int stages = 12;
  SmemPlan plan = make_plan(stages, max_slice_segs * 256, max_slice_segs, MC, M);
  while (plan.total > g_max_smem && stages > 2) {
    stages--;
    plan = make_plan(stages, max_slice_segs * 256, max_slice_segs, MC, M);
  }
  if (plan.total > g_max_smem) { set_error("decode kernel: shared memory plan does not fit"); return MLXR_ERR_UNSUPPORTED; }
  const bool coop = nphases > 1;
  int rc = MLXR_OK;
#define INST(QT, T, NTV) rc = launch_inst<QT, T, NTV>(P, plan, G, coop, st)
#define BY_NT(QT, T) do { if (NT == 1) INST(QT, T, 1); else INST(QT, T, 2); } while (0)
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
  if (rc == MLXR_OK && nphases > 1) *bar_host += (uint32_t)G * (uint32_t)(nphases - 1);
  return rc;
}

}  // namespace mlxr
