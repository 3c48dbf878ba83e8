// The C ABI (include/mlxr_b200.h): argument validation, workspace management, kernel
// selection.  Nothing here computes on the CPU: every compute entry point launches CUDA
// kernels or fails.
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace mlxr {

// ---- error text ------------------------------------------------------------------------
static thread_local char g_err[512] = "";
static std::atomic<uint64_t> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
  return MLXR_ERR_CUDA;
}
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

// ---- per-(device, stream) workspace ----------------------------------------------------
// Scratch for intermediates (normalised activations, h = SiLU(g)*u, split-K partials),
// self-cleaning counters and a status word.  Created on first use for a (device, stream)
// pair, grown on demand, freed by mlxr_release_workspaces().  Calls on one stream are
// ordered, so one workspace per stream is race-free.
struct Workspace {
  void* buf = nullptr;       // compute scratch
  size_t bytes = 0;
  void* stage = nullptr;     // device staging of host-buffer calls
  size_t stage_bytes = 0;
  void* part = nullptr;      // split-K partial sums of the tensor-core GEMM (never aliases buf)
  size_t part_bytes = 0;
  void* tagged = nullptr;    // h of the decode MLP block as {payload, sequence number} words; zero-filled when
  size_t tagged_bytes = 0;   // allocated and written by nothing else, so a stale word never carries a live number
  uint32_t* sync = nullptr;  // kSyncWords zero-initialised words (counters, barriers)
  int* status = nullptr;     // device status word
  int* status_host = nullptr;  // pinned mirror
  uint32_t bar_host = 0;     // host mirror of sync[0], the decode kernel's grid-barrier counter
};
static std::mutex g_ws_mu;
static std::map<std::pair<int, void*>, Workspace> g_ws;

static int grow(void** p, size_t* have, size_t need, cudaStream_t st, bool zero = false) {
  if (need <= *have) return MLXR_OK;
  // wait for work that may still use the old buffer, then replace it
  MLXR_CUDA_TRY(cudaStreamSynchronize(st));
  if (*p) MLXR_CUDA_TRY(cudaFree(*p));
  *p = nullptr;
  *have = 0;
  const size_t cap = (need + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
  MLXR_CUDA_TRY(cudaMalloc(p, cap));
  *have = cap;
  if (zero) MLXR_CUDA_TRY(cudaMemsetAsync(*p, 0, cap, st));
  return MLXR_OK;
}

int get_workspace(cudaStream_t st, size_t need, Workspace** out, size_t need_stage = 0, size_t need_tagged = 0) {
  int dev = 0;
  MLXR_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_ws_mu);
  Workspace& ws = g_ws[{dev, (void*)st}];
  if (!ws.sync) {
    MLXR_CUDA_TRY(cudaMalloc(&ws.sync, kSyncWords * sizeof(uint32_t)));
    MLXR_CUDA_TRY(cudaMemset(ws.sync, 0, kSyncWords * sizeof(uint32_t)));
    MLXR_CUDA_TRY(cudaMalloc(&ws.status, 64));
    MLXR_CUDA_TRY(cudaMemset(ws.status, 0, 64));
    MLXR_CUDA_TRY(cudaMallocHost(&ws.status_host, 64));
    ws.status_host[0] = 0;
  }
  if (int r = grow(&ws.buf, &ws.bytes, need, st)) return r;
  if (int r = grow(&ws.stage, &ws.stage_bytes, need_stage, st)) return r;
  if (int r = grow(&ws.tagged, &ws.tagged_bytes, need_tagged, st, true)) return r;
  *out = &ws;
  return MLXR_OK;
}

int stream_status_word(cudaStream_t st, int** status) {
  Workspace* ws = nullptr;
  if (int r = get_workspace(st, 0, &ws)) return r;
  *status = ws->status;
  return MLXR_OK;
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- validation helpers ----------------------------------------------------------------
static bool qt_has_code(int qt) { return block_elems(qt) != 0; }

static int check_dtype(int dt) {
  if (dt != MLXR_F16 && dt != MLXR_BF16 && dt != MLXR_F32) {
    set_error("dtype must be MLXR_F16, MLXR_BF16 or MLXR_F32 (got %d)", dt);
    return MLXR_ERR_INVALID_ARGUMENT;
  }
  return MLXR_OK;
}

static int check_quant(int qt, int K, int group_size, bool check_group) {
  if (!qt_has_code(qt)) {
    set_error("Unsupported quantization type %d (%s)", qt, mlxr_quant_type_name(qt));
    return MLXR_ERR_UNSUPPORTED;
  }
  const int be = block_elems(qt);
  if (K <= 0 || K % be != 0) {
    set_error("K = %d must be a positive multiple of the %s block size %d", K,
              mlxr_quant_type_name(qt), be);
    return MLXR_ERR_SHAPE;
  }
  if (check_group) {
    const bool kq = (qt == MLXR_Q4_K || qt == MLXR_GGML_Q4_K);
    if (!(group_size == be || (kq && group_size == 32))) {
      set_error("group_size %d does not match format %s (block %d%s)", group_size,
                mlxr_quant_type_name(qt), be, kq ? ", or 32" : "");
      return MLXR_ERR_SHAPE;
    }
  }
  return MLXR_OK;
}

// Kernel selection for one linear.  Fast kernels need 16-byte aligned rows.
// The first kDecodeScratchBytes of a workspace's scratch belong to the decode kernel's
// split-K partial sums; intermediates of the fused entry points start after them.
static int run_linear(const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                      int qt, int dtype, cudaStream_t st) {
  if (M > 0 && N > 0 && stream_gemv_supported(qt, M, K, &w, 1) && !tune_env("MLXR_NO_STREAM")) {
    Workspace* ws = nullptr;
    if (int r = get_workspace(st, 0, &ws)) return r;
    DecodeLinear L;
    memset(&L, 0, sizeof(L));
    L.w[0] = w; L.rows[0] = N; L.nmat = 1; L.K = K; L.x = x; L.y[0] = y; L.bias[0] = bias;
    return launch_stream_gemv(L, M, dtype, ws->status, st);
  }
  if (M >= 3 && N > 0 && smallm_supported(qt, M, N, K, dtype, x, w) && !tune_env("MLXR_NO_SMALLM")) {
    int grid = 0, maxc = 0;
    size_t part = 0;
    if (int r = smallm_plan(M, N, K, &grid, &maxc, &part)) return r;
    Workspace* ws = nullptr;
    if (int r = get_workspace(st, 0, &ws)) return r;
    {
      std::lock_guard<std::mutex> lk(g_ws_mu);
      if (int r = grow(&ws->part, &ws->part_bytes, part, st)) return r;
    }
    return launch_smallm(x, w, nullptr, bias, y, M, N, K, qt, dtype, ws->status, (float*)ws->part, ws->sync + 16, grid, maxc, st);
  }
  if (M > 0 && N > 0 && decode_supported(qt, M, K, &w, 1)) {
    Workspace* ws = nullptr;
    if (int r = get_workspace(st, kDecodeScratchBytes, &ws)) return r;
    DecodeLinear L;
    memset(&L, 0, sizeof(L));
    L.w[0] = w; L.rows[0] = N; L.nmat = 1; L.K = K; L.x = x; L.y[0] = y; L.bias[0] = bias;
    return launch_decode(&L, 1, M, qt, dtype, ws->buf, kDecodeScratchBytes, ws->sync, &ws->bar_host, ws->status, st);
  }
  if (M > 0 && N > 0 && gemv_rows_supported(qt, M, K, x, w) && !tune_env("MLXR_NO_GEMV"))
    return launch_gemv_rows(x, w, bias, y, M, N, K, qt, dtype, st);
  if (M > 0 && N > 0 && prefill_supported(qt, M, N, K, dtype, x, w, y) && !tune_env("MLXR_NO_TC")) {
    const int S = prefill_slices(M, N, K);
    Workspace* ws = nullptr;
    if (int r = get_workspace(st, 0, &ws)) return r;
    if (S > 1) {
      std::lock_guard<std::mutex> lk(g_ws_mu);
      if (int r = grow(&ws->part, &ws->part_bytes, (size_t)S * M * N * sizeof(float), st)) return r;
    }
    return launch_prefill(x, w, bias, y, M, N, K, qt, dtype, ws->status, (float*)ws->part, ws->sync + 16, S, st);
  }
  return launch_qgemm_generic(x, w, bias, y, M, N, K, qt, dtype, st);
}

int mlp_block_tp_fused(const void* x, const void* norm_weight, const void* w_gate, const void* w_up, const void* w_down,
                       int M, int hidden, int inter, int qt, float eps, int dtype, const DecodeTp* tp, cudaStream_t st) {
  const void* wgu[2] = {w_gate, w_up};
  if (M < 1 || !decode_supported(qt, M, hidden, wgu, 2) || !decode_supported(qt, M, inter, &w_down, 1)) return MLXR_ERR_UNSUPPORTED;
  Workspace* ws = nullptr;
  if (int r = get_workspace(st, kDecodeScratchBytes, &ws, 0, decode_tagged_bytes(M, inter, dtype))) return r;
  DecodeLinear L[2];
  memset(L, 0, sizeof(L));
  L[0].w[0] = w_gate; L[0].w[1] = w_up; L[0].rows[0] = L[0].rows[1] = inter; L[0].nmat = 2;
  L[0].interleave = 1; L[0].K = hidden; L[0].x = x; L[0].gamma = norm_weight; L[0].eps = eps;
  L[0].y_tagged = ws->tagged;
  L[1].w[0] = w_down; L[1].rows[0] = hidden; L[1].nmat = 1; L[1].K = inter; L[1].x = ws->tagged; L[1].x_tagged = 1;
  L[1].y[0] = tp->y;
  L[1].epi[0] = 3;
  return launch_decode(L, 2, M, qt, dtype, ws->buf, kDecodeScratchBytes, ws->sync, &ws->bar_host, ws->status, st, tp);
}

}  // namespace mlxr

using namespace mlxr;

extern "C" {

const char* mlxr_version(void) { return "mlxr-b200 0.1 (sm_100a)"; }

const char* mlxr_status_string(int s) {
  switch (s) {
    case MLXR_OK: return "ok";
    case MLXR_ERR_INVALID_ARGUMENT: return "invalid argument";
    case MLXR_ERR_SHAPE: return "shape or format rule violated";
    case MLXR_ERR_UNSUPPORTED: return "unsupported quantization format";
    case MLXR_ERR_CUDA: return "CUDA error";
    case MLXR_ERR_TIMEOUT: return "device-side wait timed out";
    case MLXR_ERR_NCCL: return "NCCL error";
    case MLXR_ERR_WORKSPACE: return "workspace too small or misaligned";
    default: return "unknown status";
  }
}
const char* mlxr_last_error(void) { return g_err; }
uint64_t mlxr_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

size_t mlxr_quantized_weight_size(int N, int K, int qt) {
  const int be = block_elems(qt);
  if (!be || N < 0 || K < 0) return 0;
  return (size_t)N * (size_t)((K + be - 1) / be) * (size_t)block_bytes(qt);
}
float mlxr_bytes_per_weight(int qt) {
  const int be = block_elems(qt);
  return be ? (float)block_bytes(qt) / (float)be : -1.0f;
}
int mlxr_default_group_size(int qt) {
  const int be = block_elems(qt);
  return be ? be : 32;  // the reference returns 32 for every format it has no code for
}
const char* mlxr_quant_type_name(int qt) {
  static const char* names[] = {"Q4_0", "Q4_1", "Q8_0", "Q4_K", "Q6_K", "Q5_0", "Q5_1", "Q8_1", "Q2_K",
                                "Q3_K", "Q5_K", "Q8_K", "IQ2_XXS", "IQ2_XS", "IQ3_XXS", "IQ3_S", "NF4"};
  if (qt == MLXR_GGML_Q4_0) return "GGML_Q4_0";
  if (qt == MLXR_GGML_Q4_K) return "GGML_Q4_K";
  return (qt >= 0 && qt <= 16) ? names[qt] : "Unknown";
}
const char* mlxr_rope_scaling_mode_name(int mode) {
  switch (mode) {
    case MLXR_ROPE_BASE: return "BASE";
    case MLXR_ROPE_NTK: return "NTK";
    case MLXR_ROPE_YARN: return "YARN";
    case MLXR_ROPE_LINEAR: return "LINEAR";
    default: return "Unknown";
  }
}
float mlxr_ntk_scaled_base(float base, float scale, int head_dim, int orig_context) {
  (void)orig_context;
  const float exponent = (float)head_dim / (float)(head_dim - 2);
  const float scaling_factor = scale - (scale - 1);
  return base * std::pow(scaling_factor, exponent);
}

// binary32 -> binary16, round to nearest even (host)
static uint16_t f32_to_f16_host(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7FFFFFFFu;
  if (x >= 0x7F800000u) return (uint16_t)(sign | (x > 0x7F800000u ? 0x7E00u : 0x7C00u));
  if (x >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);  // rounds to >= 65520 -> inf
  if (x < 0x33000001u) return (uint16_t)sign;               // <= 2^-25 -> 0
  int e = (int)(x >> 23) - 127;
  uint32_t m = (x & 0x7FFFFFu) | 0x800000u;
  int shift = e < -14 ? (13 + (-14 - e)) : 13;
  uint32_t r = m >> shift;
  const uint32_t rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (r & 1u))) r++;
  if (e < -14) return (uint16_t)(sign | r);  // subnormal (r may carry into the normal range)
  return (uint16_t)(sign | (((uint32_t)(e + 15) << 10) + (r - 0x400u)));
}

int mlxr_rope_tables_host(uint16_t* cos_f16, uint16_t* sin_f16, int max_seq_len, int head_dim,
                          float base, int mode, float scale_factor, int orig_context) {
  if (!cos_f16 || !sin_f16) { set_error("null table pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (head_dim <= 0 || head_dim % 2 != 0) { set_error("head_dim must be even for RoPE"); return MLXR_ERR_SHAPE; }
  if (max_seq_len < 0) { set_error("max_seq_len must be >= 0"); return MLXR_ERR_SHAPE; }
  const int pairs = head_dim / 2;
  float eff = base;
  if (mode == MLXR_ROPE_NTK) eff = mlxr_ntk_scaled_base(base, scale_factor, head_dim, orig_context);
  for (int pos = 0; pos < max_seq_len; pos++) {
    float position = (float)pos;
    if (mode == MLXR_ROPE_LINEAR) position /= scale_factor;
    for (int p = 0; p < pairs; p++) {
      const float freq_exponent = -2.0f * p / head_dim;
      const float freq = std::pow(eff, freq_exponent);
      const float theta = position * freq;
      const size_t idx = (size_t)pos * pairs + p;
      cos_f16[idx] = f32_to_f16_host(std::cos(theta));
      sin_f16[idx] = f32_to_f16_host(std::sin(theta));
    }
  }
  return MLXR_OK;
}

int mlxr_dequantize(const void* weights, void* out, int N, int K, int qt, int out_dtype, int flags,
                    void* stream) {
  if (int r = check_quant(qt, K, 0, false)) return r;
  if (N < 0) { set_error("N must be >= 0"); return MLXR_ERR_SHAPE; }
  if (out_dtype != MLXR_F16 && out_dtype != MLXR_F32) {
    set_error("dequantize output must be MLXR_F16 or MLXR_F32");
    return MLXR_ERR_INVALID_ARGUMENT;
  }
  if (N > 0 && (!weights || !out)) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (((uintptr_t)out & 15u) || ((uintptr_t)weights & 1u)) {
    set_error("dequantize: out must be 16-byte aligned and weights 2-byte aligned");
    return MLXR_ERR_INVALID_ARGUMENT;
  }
  return launch_dequantize(weights, out, N, K, qt, out_dtype, flags, (cudaStream_t)stream);
}

int mlxr_q_gemm_dequant(const void* x, const void* weights, const void* bias, void* y, int M, int N,
                        int K, int qt, int group_size, int dtype, void* stream) {
  if (int r = check_dtype(dtype)) return r;
  if (M < 0 || N < 0) { set_error("Input shape must be [M, K] with M, N >= 0"); return MLXR_ERR_SHAPE; }
  if (int r = check_quant(qt, K, group_size, true)) return r;
  if (M > 0 && N > 0 && (!x || !weights || !y)) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (((uintptr_t)weights & 1u)) { set_error("weights must be 2-byte aligned"); return MLXR_ERR_INVALID_ARGUMENT; }
  return run_linear(x, weights, bias, y, M, N, K, qt, dtype, (cudaStream_t)stream);
}

int mlxr_rmsnorm(const void* x, const void* weight, const void* residual, void* y, int rows,
                 int hidden, float eps, int dtype, void* stream) {
  if (int r = check_dtype(dtype)) return r;
  if (rows < 0 || hidden < 1) {
    set_error("RMSNorm input must have at least 1 dimension with a non-empty last axis");
    return MLXR_ERR_INVALID_ARGUMENT;
  }
  if (rows > 0 && (!x || !weight || !y)) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  return launch_rmsnorm(x, weight, residual, y, rows, hidden, eps, dtype, (cudaStream_t)stream);
}

int mlxr_swiglu(const void* gate, const void* up, void* out, size_t n, int dtype, void* stream) {
  if (int r = check_dtype(dtype)) return r;
  if (n > 0 && (!gate || !out)) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  return launch_swiglu(gate, up, out, n, dtype, (cudaStream_t)stream);
}

int mlxr_rope_apply(const void* x, const uint16_t* cos_f16, const uint16_t* sin_f16,
                    const int32_t* positions, void* y, int batch, int seq, int heads, int head_dim,
                    int max_seq_len, int mode, float scale_factor, int position_offset, int dtype,
                    int check, void* stream) {
  if (int r = check_dtype(dtype)) return r;
  if (head_dim <= 0 || head_dim % 2 != 0) { set_error("head_dim must be even for RoPE"); return MLXR_ERR_SHAPE; }
  if (batch < 0 || seq < 0 || heads < 0 || max_seq_len < 0) { set_error("negative dimension"); return MLXR_ERR_SHAPE; }
  const size_t tokens = (size_t)batch * seq;
  if (tokens * heads == 0) return MLXR_OK;
  if (!x || !y || !cos_f16 || !sin_f16 || !positions) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  cudaStream_t st = (cudaStream_t)stream;
  Workspace* ws = nullptr;
  if (int r = get_workspace(st, 0, &ws)) return r;
  if (int r = launch_rope(x, cos_f16, sin_f16, positions, y, tokens, heads, head_dim, max_seq_len, mode,
                          scale_factor, position_offset, dtype, ws->status, st))
    return r;
  if (check) {
    MLXR_CUDA_TRY(cudaMemcpyAsync(ws->status_host, ws->status, sizeof(int), cudaMemcpyDeviceToHost, st));
    MLXR_CUDA_TRY(cudaMemsetAsync(ws->status, 0, sizeof(int), st));
    MLXR_CUDA_TRY(cudaStreamSynchronize(st));
    if (ws->status_host[0] != 0) {
      set_error("rope_apply: a position (+offset) lies outside [0, max_seq_len)");
      return MLXR_ERR_SHAPE;
    }
  }
  return MLXR_OK;
}

int mlxr_repack_ggml_q4_0(const void* ggml_blocks, void* mlxr_blocks, int N, int K, void* stream) {
  if (N < 0 || K < 0 || K % 32 != 0) { set_error("K = %d must be a multiple of the Q4_0 block size 32", K); return MLXR_ERR_SHAPE; }
  const size_t nblocks = (size_t)N * (size_t)(K / 32);
  if (nblocks == 0) return MLXR_OK;
  if (!ggml_blocks || !mlxr_blocks) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (((uintptr_t)ggml_blocks & 1u) || ((uintptr_t)mlxr_blocks & 1u)) { set_error("block buffers must be 2-byte aligned"); return MLXR_ERR_INVALID_ARGUMENT; }
  return launch_repack_ggml_q4_0(ggml_blocks, mlxr_blocks, nblocks, (cudaStream_t)stream);
}

int mlxr_rope_tables_f32_host(float* cos_f32, float* sin_f32, int max_seq_len, int dim, float base) {
  if (!cos_f32 || !sin_f32) { set_error("null table pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (dim <= 0 || dim % 2 != 0) { set_error("RotaryEmbedding dimension must be even"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (max_seq_len < 0) { set_error("max_seq_len must be >= 0"); return MLXR_ERR_SHAPE; }
  const int half = dim / 2;
  for (int pos = 0; pos < max_seq_len; pos++)
    for (int i = 0; i < half; i++) {
      const float freq = 1.0f / std::pow(base, (2.0f * i) / dim);
      const float angle = (float)pos * freq;
      cos_f32[(size_t)pos * half + i] = std::cos(angle);
      sin_f32[(size_t)pos * half + i] = std::sin(angle);
    }
  return MLXR_OK;
}

int mlxr_rope_apply_split_half(const void* x, const float* cos_f32, const float* sin_f32, void* y, int batch, int seq,
                               int heads, int head_dim, int max_seq_len, int offset, int dtype, void* stream) {
  if (int r = check_dtype(dtype)) return r;
  if (head_dim <= 0 || head_dim % 2 != 0) { set_error("RotaryEmbedding dimension must be even"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (batch < 0 || seq < 0 || heads < 0 || max_seq_len < 0) { set_error("negative dimension"); return MLXR_ERR_SHAPE; }
  if (offset < 0 || (long long)offset + seq > max_seq_len) {
    set_error("positions %d .. %d lie outside the table of %d rows", offset, offset + seq, max_seq_len);
    return MLXR_ERR_SHAPE;
  }
  if ((size_t)batch * seq * heads == 0) return MLXR_OK;
  if (!x || !y || !cos_f32 || !sin_f32) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  return launch_rope_split_half(x, cos_f32, sin_f32, y, (size_t)batch, seq, heads, head_dim, offset, dtype, (cudaStream_t)stream);
}

int mlxr_linear_dense(const void* x, const void* weight, const void* bias, void* y, int M, int N, int K, int dtype,
                      void* stream) {
  if (int r = check_dtype(dtype)) return r;
  if (M < 0 || N < 0 || K <= 0) { set_error("Linear: bad dimensions M=%d N=%d K=%d", M, N, K); return MLXR_ERR_SHAPE; }
  if (M == 0 || N == 0) return MLXR_OK;
  if (!x || !weight || !y) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  return launch_linear_dense(x, weight, bias, y, M, N, K, dtype, (cudaStream_t)stream);
}

// y_f32: y is float [M, hidden] and receives the unrounded sums (a rank's partial result of a
// tensor-parallel block); otherwise y has the activation dtype.
static int mlp_block_impl(const void* x, const void* norm_weight, const void* w_gate, const void* w_up,
                          const void* w_down, void* y, int M, int hidden, int inter, int qt, float eps,
                          int dtype, bool y_f32, void* stream) {
  if (int r = check_dtype(dtype)) return r;
  if (M < 0 || hidden <= 0 || inter <= 0) { set_error("Input must be 2D [M, hidden_size]"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (int r = check_quant(qt, hidden, 0, false)) return r;
  if (int r = check_quant(qt, inter, 0, false)) return r;
  if (M == 0) return MLXR_OK;
  if (!x || !w_gate || !w_up || !w_down || !y) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  cudaStream_t st = (cudaStream_t)stream;
  const size_t es = dtype_size(dtype);
  const size_t n_bytes = align_up((size_t)M * hidden * es, 256);
  const size_t i_bytes = align_up((size_t)M * inter * es, 256);
  Workspace* ws = nullptr;
  const void* wgu[2] = {w_gate, w_up};
  // batches 3..64 of Q4_K: RMSNorm, then gate/up with the SiLU(gate) * up epilogue and down on the
  // small-batch tensor-core kernel (three launches; the decode kernel is built for batch 1-2)
  const bool small = M >= 3 && smallm_supported(qt, M, inter, hidden, dtype, x, w_gate) &&
                     smallm_supported(qt, M, inter, hidden, dtype, x, w_up) &&
                     smallm_supported(qt, M, hidden, inter, dtype, x, w_down) &&
                     (2 * inter + 127) / 128 <= kSyncWords - 16 && !tune_env("MLXR_NO_SMALLM");
  const bool decode = !small && decode_supported(qt, M, hidden, wgu, 2) && decode_supported(qt, M, inter, &w_down, 1);
  if (int r = get_workspace(st, decode ? kDecodeScratchBytes : kDecodeScratchBytes + n_bytes + 2 * i_bytes, &ws, 0,
                            decode ? decode_tagged_bytes(M, inter, dtype) : 0))
    return r;
  char* base = (char*)ws->buf + kDecodeScratchBytes;
  if (decode) {
    // one persistent launch: [RMSNorm ->] gate/up -> SiLU*up -> down; h [M, inter] passes between the
    // phases through L2 as tagged words (no grid barrier)
    DecodeLinear L[2];
    memset(L, 0, sizeof(L));
    L[0].w[0] = w_gate; L[0].w[1] = w_up; L[0].rows[0] = L[0].rows[1] = inter; L[0].nmat = 2;
    L[0].interleave = 1; L[0].K = hidden; L[0].x = x; L[0].gamma = norm_weight; L[0].eps = eps;
    L[0].y_tagged = ws->tagged;
    L[1].w[0] = w_down; L[1].rows[0] = hidden; L[1].nmat = 1; L[1].K = inter; L[1].x = ws->tagged; L[1].x_tagged = 1;
    L[1].y[0] = y;
    if (y_f32) L[1].epi[0] = 3;
    return launch_decode(L, 2, M, qt, dtype, ws->buf, kDecodeScratchBytes, ws->sync, &ws->bar_host, ws->status, st);
  }
  void* nbuf = base;
  void* gbuf = base + n_bytes;
  void* ubuf = base + n_bytes + i_bytes;
  const void* n = x;
  if (norm_weight) {
    if (int r = launch_rmsnorm(x, norm_weight, nullptr, nbuf, M, hidden, eps, dtype, st)) return r;
    n = nbuf;
  }
  if (small) {
    int grid = 0, maxc = 0;
    size_t part = 0;
    if (int r = smallm_plan(M, 2 * inter, hidden, &grid, &maxc, &part)) return r;
    {
      std::lock_guard<std::mutex> lk(g_ws_mu);
      if (int r = grow(&ws->part, &ws->part_bytes, part, st)) return r;
    }
    if (int r = launch_smallm(n, w_gate, w_up, nullptr, gbuf, M, inter, hidden, qt, dtype, ws->status, (float*)ws->part,
                              ws->sync + 16, grid, maxc, st))
      return r;
    if (!y_f32) return run_linear(gbuf, w_down, nullptr, y, M, hidden, inter, qt, dtype, st);
    if (int r = run_linear(gbuf, w_down, nullptr, nbuf, M, hidden, inter, qt, dtype, st)) return r;
    return launch_cast_to_f32(nbuf, (float*)y, (size_t)M * hidden, dtype, st);
  }
  if (int r = run_linear(n, w_gate, nullptr, gbuf, M, inter, hidden, qt, dtype, st)) return r;
  if (int r = run_linear(n, w_up, nullptr, ubuf, M, inter, hidden, qt, dtype, st)) return r;
  if (int r = launch_swiglu(gbuf, ubuf, gbuf, (size_t)M * inter, dtype, st)) return r;
  if (!y_f32) return run_linear(gbuf, w_down, nullptr, y, M, hidden, inter, qt, dtype, st);
  // generic path: the linear rounds to the activation dtype before the widening cast
  if (int r = run_linear(gbuf, w_down, nullptr, nbuf, M, hidden, inter, qt, dtype, st)) return r;
  return launch_cast_to_f32(nbuf, (float*)y, (size_t)M * hidden, dtype, st);
}

int mlxr_mlp_block(const void* x, const void* norm_weight, const void* w_gate, const void* w_up,
                   const void* w_down, void* y, int M, int hidden, int inter, int qt, float eps,
                   int dtype, void* stream) {
  return mlp_block_impl(x, norm_weight, w_gate, w_up, w_down, y, M, hidden, inter, qt, eps, dtype, false, stream);
}

int mlxr_mlp_block_partial_f32(const void* x, const void* norm_weight, const void* w_gate, const void* w_up,
                               const void* w_down, float* y_partial, int M, int hidden, int inter, int qt,
                               float eps, int dtype, void* stream) {
  return mlp_block_impl(x, norm_weight, w_gate, w_up, w_down, y_partial, M, hidden, inter, qt, eps, dtype, true, stream);
}

int mlxr_mlp_block_dense(const void* x, const void* w_gate, const void* w_up, const void* w_down,
                         const void* bias_gate, const void* bias_up, const void* bias_down, void* y, int M,
                         int hidden, int inter, int dtype, void* stream) {
  if (int r = check_dtype(dtype)) return r;
  if (M < 0 || hidden <= 0 || inter <= 0) { set_error("Input must be 2D [M, hidden_size]"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (M == 0) return MLXR_OK;
  if (!x || !w_gate || !w_up || !w_down || !y) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  cudaStream_t st = (cudaStream_t)stream;
  const size_t i_bytes = align_up((size_t)M * inter * dtype_size(dtype), 256);
  Workspace* ws = nullptr;
  if (int r = get_workspace(st, kDecodeScratchBytes + 2 * i_bytes, &ws)) return r;
  char* gbuf = (char*)ws->buf + kDecodeScratchBytes;
  char* ubuf = gbuf + i_bytes;
  if (int r = launch_linear_dense(x, w_gate, bias_gate, gbuf, M, inter, hidden, dtype, st)) return r;
  if (int r = launch_linear_dense(x, w_up, bias_up, ubuf, M, inter, hidden, dtype, st)) return r;
  if (int r = launch_swiglu(gbuf, ubuf, gbuf, (size_t)M * inter, dtype, st)) return r;
  return launch_linear_dense(gbuf, w_down, bias_down, y, M, hidden, inter, dtype, st);
}

int mlxr_set_decode_launch_mode(int mode) {
  if (mode != MLXR_DECODE_LAUNCH_COOPERATIVE && mode != MLXR_DECODE_LAUNCH_OVERLAPPED)
  {
    set_error("mlxr_set_decode_launch_mode: unknown mode %d", mode);
    return MLXR_ERR_INVALID_ARGUMENT;
  }
  set_decode_launch_mode(mode);
  return MLXR_OK;
}

int mlxr_set_wait_limit_ns(uint64_t ns) {
  if (ns == 0) { set_error("mlxr_set_wait_limit_ns: the limit must be positive"); return MLXR_ERR_INVALID_ARGUMENT; }
  set_wait_limit_ns(ns);
  return MLXR_OK;
}

int mlxr_debug_smallm_partition(long long units, int ctas, int cta, long long unit, long long* begin, long long* end, int* owner) {
  if (units < 1 || ctas < 1 || ctas > units || cta < 0 || cta >= ctas || unit < 0 || unit >= units) {
    set_error("partition: need 1 <= ctas <= units, 0 <= cta < ctas, 0 <= unit < units");
    return MLXR_ERR_INVALID_ARGUMENT;
  }
  smallm_partition(units, ctas, cta, unit, begin, end, owner);
  return MLXR_OK;
}

int mlxr_debug_set_trace_buffer(void* dev_ptr) {
  set_decode_trace(dev_ptr);
  return MLXR_OK;
}

int mlxr_stream_status(void* stream, int* status_out) {
  cudaStream_t st = (cudaStream_t)stream;
  Workspace* ws = nullptr;
  if (int r = get_workspace(st, 0, &ws)) return r;
  MLXR_CUDA_TRY(cudaMemcpyAsync(ws->status_host, ws->status, sizeof(int), cudaMemcpyDeviceToHost, st));
  MLXR_CUDA_TRY(cudaMemsetAsync(ws->status, 0, sizeof(int), st));
  MLXR_CUDA_TRY(cudaStreamSynchronize(st));
  if (status_out) *status_out = ws->status_host[0];
  if (ws->status_host[0] == MLXR_ERR_TIMEOUT) set_error("a bounded device-side wait expired in an earlier kernel on this stream");
  else if (ws->status_host[0] == MLXR_ERR_SHAPE) set_error("a RoPE position (+offset) was outside [0, max_seq_len)");
  return MLXR_OK;
}

int mlxr_qkv_rope(const void* x, const void* norm_weight, const void* wq, const void* wk, const void* wv,
                  const uint16_t* cos_f16, const uint16_t* sin_f16, const int32_t* positions, void* q_out,
                  void* k_out, void* v_out, int M, int hidden, int q_heads, int kv_heads, int head_dim,
                  int max_seq_len, int qt, float eps, int position_offset, int dtype, void* stream) {
  if (int r = check_dtype(dtype)) return r;
  if (M < 0 || hidden <= 0 || q_heads <= 0 || kv_heads <= 0) { set_error("bad dimensions"); return MLXR_ERR_SHAPE; }
  if (head_dim <= 0 || head_dim % 2 != 0) { set_error("head_dim must be even for RoPE"); return MLXR_ERR_SHAPE; }
  if (int r = check_quant(qt, hidden, 0, false)) return r;
  if (M == 0) return MLXR_OK;
  if (!x || !wq || !wk || !wv || !q_out || !k_out || !v_out || !cos_f16 || !sin_f16 || !positions) {
    set_error("null pointer");
    return MLXR_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const size_t es = dtype_size(dtype);
  Workspace* ws = nullptr;
  if (int r = get_workspace(st, kDecodeScratchBytes + align_up((size_t)M * hidden * es, 256), &ws)) return r;
  const void* wqkv[3] = {wq, wk, wv};
  if (stream_gemv_supported(qt, M, hidden, wqkv, 3) && !tune_env("MLXR_NO_STREAM")) {
    DecodeLinear L;
    memset(&L, 0, sizeof(L));
    L.w[0] = wq; L.w[1] = wk; L.w[2] = wv;
    L.rows[0] = q_heads * head_dim; L.rows[1] = L.rows[2] = kv_heads * head_dim; L.nmat = 3;
    L.K = hidden; L.x = x; L.gamma = norm_weight; L.eps = eps;
    L.y[0] = q_out; L.y[1] = k_out; L.y[2] = v_out;
    L.epi[0] = L.epi[1] = 2;
    L.cos_t = cos_f16; L.sin_t = sin_f16; L.positions = positions;
    L.head_dim = head_dim; L.max_seq = max_seq_len; L.pos_offset = position_offset;
    return launch_stream_gemv(L, M, dtype, ws->status, st);
  }
  if (decode_supported(qt, M, hidden, wqkv, 3)) {
    // one launch: [RMSNorm ->] q, k, v stacked along N, RoPE in the epilogue of q and k rows
    DecodeLinear L;
    memset(&L, 0, sizeof(L));
    L.w[0] = wq; L.w[1] = wk; L.w[2] = wv;
    L.rows[0] = q_heads * head_dim; L.rows[1] = L.rows[2] = kv_heads * head_dim; L.nmat = 3;
    L.K = hidden; L.x = x; L.gamma = norm_weight; L.eps = eps;
    L.y[0] = q_out; L.y[1] = k_out; L.y[2] = v_out;
    L.epi[0] = L.epi[1] = 2;
    L.cos_t = cos_f16; L.sin_t = sin_f16; L.positions = positions;
    L.head_dim = head_dim; L.max_seq = max_seq_len; L.pos_offset = position_offset;
    return launch_decode(&L, 1, M, qt, dtype, ws->buf, kDecodeScratchBytes, ws->sync, &ws->bar_host, ws->status, st);
  }
  void* nbuf = (char*)ws->buf + kDecodeScratchBytes;
  const void* n = x;
  if (norm_weight) {
    if (int r = launch_rmsnorm(x, norm_weight, nullptr, nbuf, M, hidden, eps, dtype, st)) return r;
    n = nbuf;
  }
  if (int r = run_linear(n, wq, nullptr, q_out, M, q_heads * head_dim, hidden, qt, dtype, st)) return r;
  if (int r = run_linear(n, wk, nullptr, k_out, M, kv_heads * head_dim, hidden, qt, dtype, st)) return r;
  if (int r = run_linear(n, wv, nullptr, v_out, M, kv_heads * head_dim, hidden, qt, dtype, st)) return r;
  if (int r = launch_rope(q_out, cos_f16, sin_f16, positions, q_out, (size_t)M, q_heads, head_dim, max_seq_len,
                          MLXR_ROPE_BASE, 1.0f, position_offset, dtype, ws->status, st))
    return r;
  return launch_rope(k_out, cos_f16, sin_f16, positions, k_out, (size_t)M, kv_heads, head_dim, max_seq_len,
                     MLXR_ROPE_BASE, 1.0f, position_offset, dtype, ws->status, st);
}

// ---- host-buffer variants ---------------------------------------------------------------
// The staging copies of x and y live in the workspace's own staging buffer, separate
// from the compute scratch.
int mlxr_q_gemm_dequant_host(const void* x_host, const void* weights_dev, const void* bias_dev,
                             void* y_host, int M, int N, int K, int qt, int group_size, int dtype,
                             void* stream) {
  if (int r = check_dtype(dtype)) return r;
  if (M < 0 || N < 0) { set_error("Input shape must be [M, K] with M, N >= 0"); return MLXR_ERR_SHAPE; }
  if (int r = check_quant(qt, K, group_size, true)) return r;
  if (M == 0 || N == 0) return MLXR_OK;
  if (!x_host || !weights_dev || !y_host) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  cudaStream_t st = (cudaStream_t)stream;
  const size_t es = dtype_size(dtype);
  const size_t xb = align_up((size_t)M * K * es, 256), yb = align_up((size_t)M * N * es, 256);
  Workspace* ws = nullptr;
  if (int r = get_workspace(st, 0, &ws, xb + yb)) return r;
  char* xs = (char*)ws->stage;
  char* ys = xs + xb;
  MLXR_CUDA_TRY(cudaMemcpyAsync(xs, x_host, (size_t)M * K * es, cudaMemcpyHostToDevice, st));
  if (int r = run_linear(xs, weights_dev, bias_dev, ys, M, N, K, qt, dtype, st)) return r;
  MLXR_CUDA_TRY(cudaMemcpyAsync(y_host, ys, (size_t)M * N * es, cudaMemcpyDeviceToHost, st));
  MLXR_CUDA_TRY(cudaStreamSynchronize(st));
  return MLXR_OK;
}

// Device-side address of pinned, device-mapped host memory (cudaHostAlloc / cudaHostRegister under
// unified addressing), or null for anything else.  Asked on every call: an address can change
// from pinned to pageable between calls.
static void* mapped_host_pointer(void* p) {
  cudaPointerAttributes a;
  void* out = nullptr;
  if (cudaPointerGetAttributes(&a, p) == cudaSuccess) {
    if (a.type == cudaMemoryTypeHost && a.devicePointer) out = a.devicePointer;
  } else {
    cudaGetLastError();   // pageable memory on old drivers reports an error: not sticky
  }
  return out;
}

int mlxr_mlp_block_host(const void* x_host, const void* norm_weight_dev, const void* w_gate_dev,
                        const void* w_up_dev, const void* w_down_dev, void* y_host, int M, int hidden,
                        int inter, int qt, float eps, int dtype, void* stream) {
  if (int r = check_dtype(dtype)) return r;
  if (M < 0 || hidden <= 0 || inter <= 0) { set_error("Input must be 2D [M, hidden_size]"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (M == 0) return MLXR_OK;
  if (!x_host || !y_host) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  cudaStream_t st = (cudaStream_t)stream;
  const size_t es = dtype_size(dtype);
  const size_t xb = align_up((size_t)M * hidden * es, 256);
  Workspace* ws = nullptr;
  if (int r = get_workspace(st, 0, &ws, 2 * xb)) return r;
  char* xs = (char*)ws->stage;
  char* ys = xs + xb;
  MLXR_CUDA_TRY(cudaMemcpyAsync(xs, x_host, (size_t)M * hidden * es, cudaMemcpyHostToDevice, st));
  // A small result in pinned (device-mapped) host memory is written by the kernel's epilogue
  // directly - posted stores over PCIe - which saves the copy back; everything else is staged.
  void* y_direct = nullptr;
  if ((size_t)M * hidden * es <= 64 * 1024 && !tune_env("MLXR_HOST_STAGE_Y")) y_direct = mapped_host_pointer(y_host);
  if (int r = mlxr_mlp_block(xs, norm_weight_dev, w_gate_dev, w_up_dev, w_down_dev, y_direct ? y_direct : ys, M, hidden,
                             inter, qt, eps, dtype, stream))
    return r;
  if (!y_direct) MLXR_CUDA_TRY(cudaMemcpyAsync(y_host, ys, (size_t)M * hidden * es, cudaMemcpyDeviceToHost, st));
  MLXR_CUDA_TRY(cudaStreamSynchronize(st));
  return MLXR_OK;
}

int mlxr_release_workspaces(void) {
  std::lock_guard<std::mutex> lk(g_ws_mu);
  cudaError_t first = cudaSuccess;
  for (auto& kv : g_ws) {
    cudaSetDevice(kv.first.first);
    cudaDeviceSynchronize();
    Workspace& ws = kv.second;
    cudaError_t e;
    if (ws.buf && (e = cudaFree(ws.buf)) != cudaSuccess && first == cudaSuccess) first = e;
    if (ws.stage && (e = cudaFree(ws.stage)) != cudaSuccess && first == cudaSuccess) first = e;
    if (ws.part && (e = cudaFree(ws.part)) != cudaSuccess && first == cudaSuccess) first = e;
    if (ws.tagged && (e = cudaFree(ws.tagged)) != cudaSuccess && first == cudaSuccess) first = e;
    if (ws.sync && (e = cudaFree(ws.sync)) != cudaSuccess && first == cudaSuccess) first = e;
    if (ws.status && (e = cudaFree(ws.status)) != cudaSuccess && first == cudaSuccess) first = e;
    if (ws.status_host) cudaFreeHost(ws.status_host);
  }
  g_ws.clear();
  if (first != cudaSuccess) return cuda_fail(first, "mlxr_release_workspaces");
  return MLXR_OK;
}

}  // extern "C"
