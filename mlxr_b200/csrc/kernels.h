// Host-side launchers of the CUDA kernels (one per .cu file) and shared constants.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>

namespace mlxr {

// Zero-initialised 32-bit words per workspace for counters and barriers.
constexpr int kSyncWords = 4096;

int launch_dequantize(const void* w, void* out, int N, int K, int qt, int out_dtype, int flags,
                      cudaStream_t st);
int launch_repack_ggml_q4_0(const void* src, void* dst, size_t nblocks, cudaStream_t st);
int launch_qgemm_generic(const void* x, const void* w, const void* bias, void* y, int M, int N,
                         int K, int qt, int dtype, cudaStream_t st);
bool gemv_rows_supported(int qt, int M, int K, const void* x, const void* w);
int launch_gemv_rows(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int qt, int dtype,
                     cudaStream_t st);
int launch_linear_dense(const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                        int dtype, cudaStream_t st);
int launch_rmsnorm(const void* x, const void* w, const void* res, void* y, int rows, int hidden,
                   float eps, int dtype, cudaStream_t st);
// device status word of the (device, stream) workspace: kernels record time-outs there
int stream_status_word(cudaStream_t st, int** status);
int launch_cast_from_f32(const float* x, void* y, size_t n, int dtype, cudaStream_t st);
int launch_cast_to_f32(const void* x, float* y, size_t n, int dtype, cudaStream_t st);
int launch_swiglu(const void* g, const void* u, void* o, size_t n, int dtype, cudaStream_t st);
int launch_rope(const void* x, const uint16_t* cos_t, const uint16_t* sin_t,
                const int32_t* positions, void* y, size_t tokens, int heads, int head_dim,
                int max_seq, int mode, float scale, int offset, int dtype, int* status,
                cudaStream_t st);

int launch_rope_split_half(const void* x, const float* cos_t, const float* sin_t, void* y, size_t batch, int seq,
                           int heads, int head_dim, int offset, int dtype, cudaStream_t st);

// ---- exchange buffer of the tensor-parallel block (tp.cu, decode_kernel.cuh) -------------------
// One per rank, mapped by every peer:
// [flags: kTpMaxWorld x kTpFlagsPerRank uint32][pad to kTpFlagBytes][slots: 2 parities x kTpMaxWorld x kTpSlotElems float]
constexpr int kTpMaxWorld = 8;
constexpr int kTpFlagsPerRank = 1024;              // indexed by CTA (exchange kernel) or by output tile (fused decode)
constexpr size_t kTpSlotElems = 256 * 1024;        // = MLXR_TP_PEER_MAX_ELEMS
constexpr size_t kTpFlagBytes = 64 * 1024;
constexpr size_t kTpXchgBytes = kTpFlagBytes + 2 * kTpMaxWorld * kTpSlotElems * sizeof(float);
// What the decode kernel needs to push its partial sums to the peers and reduce: every rank's
// exchange buffer as mapped in this process, this rank, the world size, the sequence words
// ([0] sequence number, [1] CTAs finished) and the final output [M, hidden] of the activation dtype.
struct DecodeTp {
  char* peer[kTpMaxWorld];
  int rank, world;
  uint32_t* ctl;
  void* y;
};

// ---- persistent decode kernel (decode.cu) ---------------------------------------------------
// One linear (or up to three stacked along N, or gate/up interleaved) of a decode phase.
struct DecodeLinear {
  const void* w[3];
  int rows[3];
  int nmat;
  int interleave;          // gate/up in 8+8 row tiles with the SiLU(gate)*up epilogue
  int K;
  const void* x;           // [M, K]
  const void* gamma;       // RMSNorm weight or null
  float eps;
  void* y[3];
  const void* bias[3];
  int epi[3];              // 0 plain, 2 RoPE, 3 plain fp32 store (y is float*)
  const uint16_t* cos_t;
  const uint16_t* sin_t;
  const int32_t* positions;
  int head_dim, max_seq, pos_offset;
  // Hand-over between two chained phases (gate/up -> down) without a grid barrier: the first
  // phase's SiLU(gate)*up epilogue writes 8-byte words {payload, launch sequence number} to
  // y_tagged ([M][rows / per_word] words; per_word = 2 for 16-bit activations, 1 for float), the
  // second phase has x pointing at the same words and x_tagged = 1.
  void* y_tagged;
  int x_tagged;
};
// Bytes of the tagged hand-over buffer for h [M, inter].
inline size_t decode_tagged_bytes(int M, int inter, int dtype) { return (size_t)M * inter * (dtype == MLXR_F32 ? 8 : 4); }
// Limit of every device-side wait (mbarrier, hand-over words, peer flags), in nanoseconds.
void set_wait_limit_ns(unsigned long long ns);
unsigned long long wait_limit_ns();
// Environment probes for tuning exist only in builds with -DMLXR_TUNING.
#ifdef MLXR_TUNING
inline const char* tune_env(const char* name) { return getenv(name); }
#else
inline const char* tune_env(const char*) { return nullptr; }
#endif
constexpr size_t kDecodeScratchBytes = (size_t)8 << 20;  // split-K partial sums
void set_decode_trace(void* dev_ptr);
void* get_decode_trace();
void set_decode_launch_mode(int mode);
bool decode_supported(int qt, int M, int K, const void* const* w, int nmat);
// tp (optional): the last phase must be a single plain linear with epi 3 (float partial sums); its
// sums then go straight into the peers' exchange buffers and the kernel ends with the reduction.
int launch_decode(const DecodeLinear* lin, int nphases, int M, int qt, int dtype, void* scratch,
                  size_t scratch_bytes, uint32_t* sync, uint32_t* bar_host, int* status, cudaStream_t st,
                  const DecodeTp* tp = nullptr);
// The tensor-parallel block in one launch when the decode kernel takes the shapes (else MLXR_ERR_UNSUPPORTED
// and nothing is launched): inter_local is this rank's share of the intermediate size.
int mlp_block_tp_fused(const void* x, const void* norm_weight, const void* w_gate, const void* w_up, const void* w_down,
                       int M, int hidden, int inter_local, int qt, float eps, int dtype, const DecodeTp* tp,
                       cudaStream_t st);

// ---- streaming decode linear for Q4_K at batch 1 and 2 (stream_gemv.cu) ------------------------
// One launch per linear (or per stacked / interleaved group of linears): many small CTAs, weights
// straight from global memory into tensor-core fragments, bulk L2 prefetch, programmatic stream
// serialization between consecutive launches.  Takes the DecodeLinear description (no tagged
// hand-over: chained linears are separate launches).
bool stream_gemv_supported(int qt, int M, int K, const void* const* w, int nmat);
// next_w / next_bytes (optional): packed weights of the launch the caller issues next on the stream; the
// tail of this launch requests them into L2.
int launch_stream_gemv(const DecodeLinear& L, int M, int dtype, int* status, cudaStream_t st,
                       const void* next_w = nullptr, size_t next_bytes = 0);

// ---- small-batch tensor-core linear (smallm.cu): Q4_K / Q4_0, 1 <= M <= 64, fp16 / bf16 --------------
bool smallm_supported(int qt, int M, int N, int K, int dtype, const void* x, const void* w);
void smallm_partition(long long units, int ctas, int cta, long long unit, long long* begin, long long* end, int* owner);
// grid size, the most CTAs that share one output tile, and the bytes of fp32 partial sums needed;
// rows = weight rows streamed (N, or 2 N for the gate/up form)
int smallm_plan(int M, int rows, int K, int* grid, int* maxc, size_t* partial_bytes);
// w2 == nullptr: Y = X W^T (+ bias); otherwise Y = SiLU(X w^T) * (X w2^T) (gate, up; no bias)
int launch_smallm(const void* x, const void* w, const void* w2, const void* bias, void* y, int M, int N, int K, int qt, int dtype,
                  int* status, float* partials, uint32_t* counters, int grid, int maxc, cudaStream_t st);

// ---- tensor-core GEMM for batch >= 9 on Q4_K with 16-bit activations (prefill.cu) -------------
bool prefill_supported(int qt, int M, int N, int K, int dtype, const void* x, const void* w, const void* y);
int prefill_slices(int M, int N, int K);     // K-slices (grid z); S > 1 needs S*M*N floats of scratch
int launch_prefill(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int qt, int dtype,
                   int* status, float* partials, uint32_t* counters, int S, cudaStream_t st);

}  // namespace mlxr
