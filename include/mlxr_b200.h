/*
 * mlxr_b200.h -- C ABI of the B200 (sm_100a) quantized-linear path.
 *
 * This is the boundary a maintainer of MLXR binds instead of the Metal dispatch inside
 * each Primitive's eval_gpu.  Every entry point takes plain pointers and sizes; device
 * pointers unless a parameter is documented as host memory.  `stream` is a cudaStream_t
 * passed as void* (NULL = the legacy default stream).  Calls are asynchronous on that
 * stream unless documented otherwise, never throw, and return an mlxr_status; the text of
 * the last failure on the calling thread is available from mlxr_last_error().
 *
 * There is no CPU fallback: without a CUDA device every compute entry point returns
 * MLXR_ERR_CUDA.
 *
 * Citations are to the MLXR tree (core/kernels/primitives/..., core/kernels/metal/...).
 */
#ifndef MLXR_B200_H
#define MLXR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define MLXR_API
#else
#define MLXR_API __attribute__((visibility("default")))
#endif

/* ---- status codes ------------------------------------------------------------------
 * The C++ primitive layer maps MLXR_ERR_INVALID_ARGUMENT to std::invalid_argument (what
 * rmsnorm_fused and swiglu_mlp throw: rmsnorm_primitive.mm:309-321,
 * swiglu_mlp_primitive.mm:246-265) and every other failure to std::runtime_error (what
 * q_gemm_dequant and rope_apply throw: q_gemm_dequant_primitive.mm:304-306,490-496,
 * rope_apply_primitive.mm:411-451). */
typedef enum mlxr_status {
  MLXR_OK = 0,
  MLXR_ERR_INVALID_ARGUMENT = 1, /* null pointer, bad dtype, size mismatch           */
  MLXR_ERR_SHAPE = 2,            /* shape / format rule violated                      */
  MLXR_ERR_UNSUPPORTED = 3,      /* quant format without an implementation            */
  MLXR_ERR_CUDA = 4,             /* CUDA runtime error (text in mlxr_last_error)      */
  MLXR_ERR_TIMEOUT = 5,          /* a bounded device-side wait gave up                */
  MLXR_ERR_NCCL = 6,             /* collective library error                          */
  MLXR_ERR_WORKSPACE = 7         /* caller-provided scratch too small / misaligned    */
} mlxr_status;

/* ---- element types of activations -------------------------------------------------- */
typedef enum mlxr_dtype { MLXR_F16 = 0, MLXR_BF16 = 1, MLXR_F32 = 2 } mlxr_dtype;

/* ---- quantization formats ----------------------------------------------------------
 * Values 0..15 are MLXR's `enum class QuantType`
 * (q_gemm_dequant_primitive.h:18-35).  Q4_0, Q4_1, Q8_0 and Q4_K are implemented; Q6_K is
 * not (the reference's dequant_q6_k, q_gemm_dequant.metal:265-286, indexes past its
 * block, so it defines no result to reproduce); 5..15 are names only, as in MLXR.  NF4 does not exist in the
 * reference; it takes the first free value.  Block layouts are MLXR's, which are NOT the
 * canonical ggml ones (q_gemm_dequant_primitive.mm:29-57, q_gemm_dequant.metal:142-286):
 *   Q4_0  18 B / 32:  fp16 scale, 16 bytes; byte i = elements 2i (low nibble), 2i+1 (high)
 *   Q4_1  20 B / 32:  fp16 scale, fp16 min, 16 bytes, same nibble order
 *   Q8_0  34 B / 32:  fp16 scale, 32 int8
 *   Q4_K 144 B / 256: fp16 d, fp16 dmin, scales[12], qs[128]; sub-block s uses qs[16s..]
 *   NF4   34 B / 64:  fp16 absmax, 32 bytes of 4-bit codebook indices (Q4_0 nibble order)
 * A weight matrix is [N rows][K / block] blocks, row-major, no padding. */
typedef enum mlxr_quant_type {
  MLXR_Q4_0 = 0, MLXR_Q4_1 = 1, MLXR_Q8_0 = 2, MLXR_Q4_K = 3, MLXR_Q6_K = 4,
  MLXR_Q5_0 = 5, MLXR_Q5_1 = 6, MLXR_Q8_1 = 7, MLXR_Q2_K = 8, MLXR_Q3_K = 9,
  MLXR_Q5_K = 10, MLXR_Q8_K = 11, MLXR_IQ2_XXS = 12, MLXR_IQ2_XS = 13,
  MLXR_IQ3_XXS = 14, MLXR_IQ3_S = 15,
  MLXR_NF4 = 16,
  /* Extension: the CANONICAL ggml layouts, as a .gguf file stores them (the reference parses such
   * files, daemon/registry/gguf_parser.h:141-211, but its loader skips quantized tensors because
   * its kernels cannot read them, daemon/server/model_loader.cpp:236-245):
   *   GGML_Q4_0  18 B / 32:  fp16 d, qs[16]; element i = low nibble of qs[i], i+16 = high nibble;
   *                          w = (q - 8) * d
   *   GGML_Q4_K 144 B / 256: fp16 d, fp16 dmin, scales[12] = eight 6-bit (scale, min) pairs
   *                          (get_scale_min_k4 packing), qs[128]; 64-element chunk j: elements
   *                          0..31 = low nibbles of qs[32j..32j+31], 32..63 = high nibbles;
   *                          w = (d * sc) * q - dmin * m in float32
   * Dequantized values equal gguf.quants.dequantize bit for bit.  mlxr_dequantize and
   * mlxr_q_gemm_dequant accept them (any batch); canonical Q4_0 can also be turned into MLXR's
   * Q4_0 on the device without loss (mlxr_repack_ggml_q4_0) to run on the fast kernels. */
  MLXR_GGML_Q4_0 = 32, MLXR_GGML_Q4_K = 33
} mlxr_quant_type;

/* RoPEScalingMode, rope_apply_primitive.h:18-23 */
typedef enum mlxr_rope_mode {
  MLXR_ROPE_BASE = 0, MLXR_ROPE_NTK = 1, MLXR_ROPE_YARN = 2, MLXR_ROPE_LINEAR = 3
} mlxr_rope_mode;

/* ---- library / errors -------------------------------------------------------------- */
MLXR_API const char* mlxr_version(void);
MLXR_API const char* mlxr_status_string(int status);
/* Message of the last failing call on this thread ("" if none). */
MLXR_API const char* mlxr_last_error(void);
/* Number of kernel launches this library has issued in this process (all threads). */
MLXR_API uint64_t mlxr_launch_count(void);

/* ---- format helpers (host only, no CUDA) ------------------------------------------- */
/* compute_quantized_weight_size, q_gemm_dequant_primitive.mm:116-135: bytes of an [N, K]
 * packed matrix = N * ceil(K / block) * sizeof(block); 0 for a format without code. */
MLXR_API size_t mlxr_quantized_weight_size(int N, int K, int quant_type);
/* QGemmDequantPrimitive::get_bytes_per_weight, q_gemm_dequant_primitive.mm:63-78;
 * negative for a format without code (the reference throws). */
MLXR_API float mlxr_bytes_per_weight(int quant_type);
/* QGemmDequantPrimitive::get_default_group_size, q_gemm_dequant_primitive.mm:80-92 */
MLXR_API int mlxr_default_group_size(int quant_type);
/* quant_type_name, q_gemm_dequant_primitive.mm:94-114 ("NF4" for the extension value) */
MLXR_API const char* mlxr_quant_type_name(int quant_type);
/* rope_scaling_mode_name, rope_apply_primitive.mm:27-35 */
MLXR_API const char* mlxr_rope_scaling_mode_name(int mode);
/* compute_ntk_scaled_base, rope_apply_primitive.mm:37-47 (as written it returns base) */
MLXR_API float mlxr_ntk_scaled_base(float base, float scale, int head_dim, int orig_context);
/* compute_rope_tables, rope_apply_primitive.mm:49-106.  HOST buffers of
 * max_seq_len * head_dim / 2 binary16 values each; fp32 powf/cosf/sinf, cast to half. */
MLXR_API int mlxr_rope_tables_host(uint16_t* cos_f16, uint16_t* sin_f16, int max_seq_len,
                                   int head_dim, float base, int mode, float scale_factor,
                                   int orig_context);

/* ---- dequantize --------------------------------------------------------------------
 * The reference's dequantizers, bit for bit: dequant_q4_0_cpu / dequant_q4_1_cpu /
 * dequant_q8_0_cpu (q_gemm_dequant_primitive.mm:189-225) for out_dtype MLXR_F32, and the
 * shader's half-precision dequant_q4_0 / _q4_1 / _q8_0 / _q4_k
 * (q_gemm_dequant.metal:142-259) for MLXR_F16.  Q4_K is defined in half only; its
 * MLXR_F32 output is the half result widened.  out is [N, K] row-major.
 * flags bit 0: Q4_K multiply-add with a single rounding (a contracting shader compiler)
 * instead of the default two roundings. */
MLXR_API int mlxr_dequantize(const void* weights, void* out, int N, int K, int quant_type,
                             int out_dtype, int flags, void* stream);

/* ---- q_gemm_dequant ----------------------------------------------------------------
 * Y[M,N] = X[M,K] * dequant(W[N,K])^T (+ bias[N]); the work of
 * QGemmDequantPrimitive::eval_gpu / kernel q_gemm_dequant
 * (q_gemm_dequant_primitive.mm:367-450, q_gemm_dequant.metal:338-486) behind
 * q_gemm_dequant() (q_gemm_dequant_primitive.mm:478-522).  x, y and bias have type
 * `dtype` (fp16 as in the reference; bf16 and fp32 added); accumulation is fp32.
 * group_size must be the format's block size, or 32 for Q4_K (the shader's sub-block
 * addressing, q_gemm_dequant.metal:397-430).  K must be a whole number of
 * blocks (the reference overruns the row otherwise).  The kernel is chosen by shape:
 * streaming decode kernel for small M, tcgen05 tensor-core kernel for large M.
 * Uses the per-(device, stream) workspace of this library, created at the first call. */
MLXR_API int mlxr_q_gemm_dequant(const void* x, const void* weights, const void* bias,
                                 void* y, int M, int N, int K, int quant_type,
                                 int group_size, int dtype, void* stream);

/* ---- rmsnorm_fused -----------------------------------------------------------------
 * y = x * rsqrt(mean(x^2) + eps) * weight, row-wise over [rows, hidden]; fp32 internal,
 * one rounding at the store: kernels rmsnorm_fused / rmsnorm_fused_fp16
 * (rmsnorm.metal:39-156) behind rmsnorm_fused() (rmsnorm_primitive.mm:302-359).
 * residual (may be NULL) is added after the scale: rmsnorm_fused_residual
 * (rmsnorm.metal:165-217). */
MLXR_API int mlxr_rmsnorm(const void* x, const void* weight, const void* residual, void* y,
                          int rows, int hidden, float eps, int dtype, void* stream);

/* ---- swish / swiglu ----------------------------------------------------------------
 * out = gate * sigmoid(gate) * up  (up == NULL: out = gate * sigmoid(gate)), elementwise
 * over n values: swish() / swiglu() at swiglu_mlp_primitive.mm:306-318, sign-split
 * sigmoid as in swiglu_mlp_fused.metal:92-99. */
MLXR_API int mlxr_swiglu(const void* gate, const void* up, void* out, size_t n, int dtype,
                         void* stream);

/* ---- rope_apply --------------------------------------------------------------------
 * Interleaved-pair rotation with binary16 cos/sin tables [max_seq_len, head_dim/2]:
 * RoPEApplyPrimitive::eval_gpu / kernels rope_apply, rope_apply_inplace
 * (rope_apply_primitive.mm:272-370, rope_apply.metal:103-245) behind rope_apply()
 * (rope_apply_primitive.mm:399-475).  x, y: [batch, seq, heads, head_dim] of `dtype`
 * (y may equal x: in place).  positions: int32 [batch] when seq == 1 else [batch, seq];
 * every position + position_offset must lie in [0, max_seq_len) -- checked on the
 * device, a violation leaves that token's output untouched and the call's status word
 * set (reported by mlxr_rope_apply's return value only when `check` is non-zero, which
 * synchronises the stream). */
MLXR_API int mlxr_rope_apply(const void* x, const uint16_t* cos_f16, const uint16_t* sin_f16,
                             const int32_t* positions, void* y, int batch, int seq,
                             int heads, int head_dim, int max_seq_len, int mode,
                             float scale_factor, int position_offset, int dtype,
                             int check, void* stream);

/* RoPE in the split-half ("rotate_half") convention of graph::RotaryEmbedding
 * (core/graph/layers.cpp:113-225), which differs from the rope_apply primitive above: the head
 * is split into its first and second half (x1, x2), the tables are float32 [max_seq_len, dim/2]
 * with freq_i = 1 / base^(2i/dim) and angle = pos * freq_i (compute_freqs, :121-154), positions
 * are the contiguous range offset .. offset + seq, and
 *   y1 = x1*cos - x2*sin,  y2 = x2*cos + x1*sin      (forward, :196-222)
 * with every product and sum rounded to float32 like the composition of MLX ops, then one
 * rounding to `dtype`.  x, y: [batch, seq, heads, head_dim]; y may alias x.  The host function
 * fills the tables (HOST memory) exactly as compute_freqs does. */
MLXR_API int mlxr_rope_tables_f32_host(float* cos_f32, float* sin_f32, int max_seq_len, int dim,
                                       float base);
MLXR_API int mlxr_rope_apply_split_half(const void* x, const float* cos_f32, const float* sin_f32,
                                        void* y, int batch, int seq, int heads, int head_dim,
                                        int max_seq_len, int offset, int dtype, void* stream);

/* y[M, N] = x[M, K] W^T (+ bias) with a DENSE weight [N, K] of the activation dtype:
 * graph::Linear::forward (core/graph/layers.cpp:86-99), the op the quantized linear replaces.
 * fp32 accumulation, one rounding at the store.  Not the quantized hot path. */
MLXR_API int mlxr_linear_dense(const void* x, const void* weight, const void* bias, void* y, int M,
                               int N, int K, int dtype, void* stream);

/* Canonical ggml Q4_0 blocks [N, K] -> MLXR Q4_0 blocks (a permutation of nibbles inside every
 * block: value-preserving).  src and dst may not overlap.  Extension, see MLXR_GGML_Q4_0. */
MLXR_API int mlxr_repack_ggml_q4_0(const void* ggml_blocks, void* mlxr_blocks, int N, int K, void* stream);

/* ---- fused decoder-layer pieces ----------------------------------------------------
 * MLP block: y = down( SiLU(gate(n)) * up(n) ),  n = rmsnorm(x, norm_weight, eps) when
 * norm_weight != NULL else n = x.  The composition MLP::forward
 * (core/graph/layers.cpp:400-420) after RMSNorm::forward (:30-55), i.e.
 * SwiGLUMLPPrimitive::eval_cpu (swiglu_mlp_primitive.mm:47-82) with quantized weights as
 * plan/MetalKernelsPlan.md:109-117 intends.  x, y: [M, hidden]; w_gate, w_up:
 * packed [inter, hidden]; w_down: packed [hidden, inter]; all three in `quant_type`.
 * n and h = SiLU(g)*u are rounded to `dtype` where the composition materialises them;
 * h lives only in this library's workspace (L2-resident at decode sizes).  At decode batches
 * the block is ONE launch: the gate/up CTAs publish h as 8-byte words that carry the launch's
 * sequence number, and the down-projection CTAs poll those words instead of meeting at a grid
 * barrier. */
MLXR_API int mlxr_mlp_block(const void* x, const void* norm_weight, const void* w_gate,
                            const void* w_up, const void* w_down, void* y, int M,
                            int hidden, int inter, int quant_type, float eps, int dtype,
                            void* stream);

/* The same block with the down projection's sums stored unrounded as float [M, hidden]:
 * one rank's partial result when `inter` is this rank's share of the intermediate dimension
 * (w_gate/w_up hold its rows, w_down its K range).  Extension; the reference has no sharded path. */
MLXR_API int mlxr_mlp_block_partial_f32(const void* x, const void* norm_weight, const void* w_gate,
                                        const void* w_up, const void* w_down, float* y_partial,
                                        int M, int hidden, int inter, int quant_type, float eps,
                                        int dtype, void* stream);

/* The same block with DENSE weights of the activation dtype and optional biases: the exact
 * signature of swiglu_mlp() (swiglu_mlp_primitive.h:169-176), i.e.
 * SwiGLUMLPPrimitive::eval_cpu (swiglu_mlp_primitive.mm:47-82).  w_gate, w_up:
 * [inter, hidden]; w_down: [hidden, inter].  Not the quantized hot path: a plain
 * fp32-accumulating kernel kept for interface completeness. */
MLXR_API int mlxr_mlp_block_dense(const void* x, const void* w_gate, const void* w_up,
                                  const void* w_down, const void* bias_gate, const void* bias_up,
                                  const void* bias_down, void* y, int M, int hidden, int inter,
                                  int dtype, void* stream);

/* Synchronise `stream`, then report and clear the device status word of its workspace:
 * MLXR_OK, MLXR_ERR_TIMEOUT (a bounded wait inside a persistent kernel gave up; results of
 * that call are invalid) or MLXR_ERR_SHAPE (a RoPE position outside its table in a fused
 * call).  The return value is the status of this call itself. */
MLXR_API int mlxr_stream_status(void* stream, int* status_out);

/* Limit of every device-side wait of this library (copy barriers, hand-over words between the
 * phases of a persistent kernel, peer flags of the tensor-parallel exchange), in nanoseconds
 * of the GPU's global timer; process-wide, default 2 s, read at each launch.  A wait that
 * reaches the limit gives up, the kernel returns, and MLXR_ERR_TIMEOUT is reported through
 * mlxr_stream_status (the failure-detection design: no wait is unbounded, the context stays
 * usable).  No counterpart in the reference, whose kernels never wait on one another. */
MLXR_API int mlxr_set_wait_limit_ns(uint64_t ns);

/* The decode linear (1 <= M <= 8, Q4_K or Q4_0, K a multiple of 256) with NO device allocation,
 * on the first call or later: the kernel's scratch (split-K partial sums, barrier and counter
 * words, status word) is a fixed 4 MiB array inside the loaded module instead of the
 * per-stream workspace that the other entry points cudaMalloc on first use.  No counterpart
 * in the reference (Metal buffers come from MLX's allocator); it exists for hosts that must
 * not allocate at call time - all device memory already given to their own pool, or a path
 * where an allocation's device-wide synchronisation is not acceptable.
 *   - N <= MLXR_STATIC_MAX_N, otherwise MLXR_ERR_WORKSPACE (nothing is truncated); shapes
 *     outside the decode range give MLXR_ERR_UNSUPPORTED.
 *   - The array exists once per device: calls that overlap in time on one device (different
 *     streams) race on it.  Order them (one stream, or events).
 *   - The first call on a device fetches the array's address, zeroes the words that must
 *     start at zero and sets kernel attributes: make it before any stream capture begins.
 *   - A bounded wait that gives up is recorded in the array's own status word, which
 *     mlxr_stream_status does not read: mlxr_static_status reads and clears it.
 *   - The array is part of the module image: it takes its 4 MiB when the CUDA module is loaded
 *     (at the latest on the first launch or symbol lookup of this library), not at a call.  A
 *     host that hands all free memory to its own pool should touch this library first.
 * Same arithmetic and the same results as mlxr_q_gemm_dequant for these shapes. */
#define MLXR_STATIC_MAX_N 8192
MLXR_API int mlxr_q_gemm_dequant_static(const void* x, const void* weights, const void* bias,
                                        void* y, int M, int N, int K, int quant_type, int dtype,
                                        void* stream);
/* Synchronise `stream`, then report and clear the status word of the static array on the
 * current device (MLXR_OK or MLXR_ERR_TIMEOUT).  Allocates nothing.  No counterpart in the
 * reference. */
MLXR_API int mlxr_static_status(void* stream, int* status_out);

/* How the persistent decode kernel is launched (process-wide; no counterpart in the
 * reference, whose Metal command buffers serialise kernels).
 *   MLXR_DECODE_LAUNCH_OVERLAPPED (default): plain launch with programmatic stream
 *     serialization.  The kernel starts its weight copies while the previous kernel of the
 *     stream drains and waits (griddepcontrol.wait) before it reads activations.  Contract:
 *     weight buffers are model constants - no kernel still in flight on the stream writes
 *     them - and at most one decode launch runs on a device at a time.  The MLP block's
 *     down-projection CTAs wait for words written by the gate/up CTAs of the same launch; the
 *     library checks once per device that one CTA per SM is resident, but two decode launches
 *     on concurrent streams could each hold part of the SMs, in which case the bounded wait
 *     reports MLXR_ERR_TIMEOUT through mlxr_stream_status.
 *   MLXR_DECODE_LAUNCH_COOPERATIVE: cooperative launch (the driver guarantees co-residency
 *     or refuses the launch), no overlap with the previous kernel, no contract. */
enum { MLXR_DECODE_LAUNCH_COOPERATIVE = 0, MLXR_DECODE_LAUNCH_OVERLAPPED = 2 };
MLXR_API int mlxr_set_decode_launch_mode(int mode);

/* Timeline tracing of the persistent decode kernel (off by default).  dev_ptr: device buffer
 * of 16 uint64 per CTA (148 * 16 * 8 bytes is enough), or NULL to switch tracing off.  Each
 * CTA stores %globaltimer (ns) at: [0] start, [1] x prologue done, [2] first weight stage
 * landed, [3] first tile accumulated (phase 0; +4 for phase 1), [15]/[14] end. */
MLXR_API int mlxr_debug_set_trace_buffer(void* dev_ptr);

/* Work partition of the small-batch tensor-core linear (no counterpart in the reference; host
 * arithmetic only, usable without a GPU): `units` work units (tile of 128 weight rows x 256-wide
 * super-block of K, tile-major) are dealt to `ctas` CTAs in contiguous ranges.  Writes the first
 * unit of CTA `cta` and of CTA `cta + 1` to begin / end, and the CTA that owns `unit` to owner
 * (each may be NULL).  MLXR_ERR_INVALID_ARGUMENT unless 1 <= ctas <= units, 0 <= cta < ctas,
 * 0 <= unit < units. */
MLXR_API int mlxr_debug_smallm_partition(long long units, int ctas, int cta, long long unit,
                                         long long* begin, long long* end, int* owner);

/* Attention input projections with RoPE on q and k: n = rmsnorm(x) (norm_weight may be
 * NULL), q = n Wq^T, k = n Wk^T, v = n Wv^T, then rope_apply on q and k
 * (Attention::forward, core/graph/layers.cpp:266-278, with the rope_apply primitive).
 * wq: packed [q_heads*head_dim, hidden]; wk, wv: packed [kv_heads*head_dim, hidden].
 * q_out [M, q_heads, head_dim]; k_out, v_out [M, kv_heads, head_dim]; positions int32 [M]. */
MLXR_API int mlxr_qkv_rope(const void* x, const void* norm_weight, const void* wq,
                           const void* wk, const void* wv, const uint16_t* cos_f16,
                           const uint16_t* sin_f16, const int32_t* positions, void* q_out,
                           void* k_out, void* v_out, int M, int hidden, int q_heads,
                           int kv_heads, int head_dim, int max_seq_len, int quant_type,
                           float eps, int position_offset, int dtype, void* stream);

/* ---- host-buffer entry points (what a CPU-side caller of the primitives sees) -------
 * Same operations with x / y (and positions) in HOST memory: the call copies the inputs
 * to the device, runs, copies the result back and synchronises the stream before it
 * returns.  Weights, norm weights and tables stay device-resident (they are model
 * state).  Pinned host memory avoids a staging copy. */
MLXR_API int mlxr_q_gemm_dequant_host(const void* x_host, const void* weights_dev,
                                      const void* bias_dev, void* y_host, int M, int N,
                                      int K, int quant_type, int group_size, int dtype,
                                      void* stream);
MLXR_API int mlxr_mlp_block_host(const void* x_host, const void* norm_weight_dev,
                                 const void* w_gate_dev, const void* w_up_dev,
                                 const void* w_down_dev, void* y_host, int M, int hidden,
                                 int inter, int quant_type, float eps, int dtype,
                                 void* stream);

/* Free every per-(device, stream) workspace this library created (synchronises). */
MLXR_API int mlxr_release_workspaces(void);

#ifdef __cplusplus
}
#endif
#endif /* MLXR_B200_H */
