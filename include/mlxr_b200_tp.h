/* mlxr_b200 tensor-parallel MLP block: C ABI.
 *
 * The reference runs on one Apple GPU and has no sharded path; this header is the extension
 * that spreads the block of MLP::forward (core/graph/layers.cpp:400-420) over the GPUs of one
 * node, one process per GPU:
 *
 *   rank r of t holds rows [r*I/t, (r+1)*I/t) of w_gate and w_up (packed [I, H]: a plain byte
 *   range) and, for every row of w_down (packed [H, I]), the blocks of columns
 *   [r*I/t, (r+1)*I/t) (a repack into a packed [H, I/t] matrix).  x and the RMSNorm weight are
 *   replicated; each rank computes a full-shape float partial [M, H]; one sum over ranks gives y
 *   on every rank.
 *
 * The sum is either ncclAllReduce or, for small payloads, a one-shot exchange written here:
 * every rank stores its partial into a slot of every peer's exchange buffer (peer stores over
 * NVLink, no multicast), raises a flag, waits (bounded) for the peers' flags and adds the t
 * slots in rank order, so that all ranks obtain bit-identical results.
 *
 * Same conventions as mlxr_b200.h: int status returns, mlxr_last_error() for the message,
 * nothing throws, device pointers unless stated, work enqueued on `stream`. */
#ifndef MLXR_B200_TP_H
#define MLXR_B200_TP_H

#include "mlxr_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct mlxr_tp_ctx mlxr_tp_ctx;

/* How the partial results are summed. */
enum {
  MLXR_TP_EXCHANGE_AUTO = 0,      /* peer one-shot when the payload fits, else NCCL fp32 */
  MLXR_TP_EXCHANGE_NCCL_F32 = 1,  /* ncclAllReduce on float partials (parity mode) */
  MLXR_TP_EXCHANGE_NCCL_ACT = 2,  /* partials rounded to the activation dtype first (half the bytes) */
  MLXR_TP_EXCHANGE_PEER = 3       /* one-shot peer-store exchange; payload limit below */
};

/* Largest M*hidden the peer exchange accepts (floats per rank and slot). */
#define MLXR_TP_PEER_MAX_ELEMS (256 * 1024)

/* 128 opaque bytes identifying a communicator (an ncclUniqueId): rank 0 creates it, the host
 * program hands it to the other ranks by its own means (a store, a socket, MPI). Host memory. */
MLXR_API int mlxr_tp_unique_id(void* id128);

/* Collective over all ranks: create the context of `rank` of `world` on the current CUDA
 * device.  Initialises the NCCL communicator, allocates the exchange buffer and maps the
 * peers' buffers (CUDA IPC; all ranks must be processes on one node with peer access).
 * use_peer = 0 skips the exchange buffer (NCCL modes only).
 * The outcome is collective too: a rank whose local step fails (an allocation, an IPC mapping)
 * still joins every collective of the set-up, the ranks agree on the result, and either all
 * return MLXR_OK or all return an error with nothing left allocated.  mlxr_tp_destroy is
 * collective as well: every rank calls it at the same point. */
MLXR_API int mlxr_tp_create(const void* id128, int rank, int world, int use_peer, mlxr_tp_ctx** out);
MLXR_API int mlxr_tp_destroy(mlxr_tp_ctx* ctx);
MLXR_API int mlxr_tp_rank(const mlxr_tp_ctx* ctx);
MLXR_API int mlxr_tp_world(const mlxr_tp_ctx* ctx);

/* ---- shard packer (host memory, no GPU) --------------------------------------------------
 * which: 0 = w_gate or w_up (packed [inter, hidden], rows split), 1 = w_down (packed
 * [hidden, inter], columns split).  inter must be a multiple of world * block elements of the
 * format.  mlxr_tp_shard_bytes returns 0 for an invalid combination. */
MLXR_API size_t mlxr_tp_shard_bytes(int which, int hidden, int inter, int quant_type, int world);
MLXR_API int mlxr_tp_pack_shard(const void* w_full, void* w_shard, int which, int hidden, int inter,
                                int quant_type, int rank, int world);

/* ---- the sharded block ---------------------------------------------------------------------
 * y[M, hidden] = sum over ranks of down_r( SiLU(gate_r(n)) * up_r(n) ), n = rmsnorm(x) (or x).
 * `inter` is the FULL intermediate size; the shard pointers are what mlxr_tp_pack_shard made.
 * All ranks call with the same M, shapes, dtype and exchange mode.  The result is replicated.
 * A peer wait that gives up reports MLXR_ERR_TIMEOUT through mlxr_stream_status(stream). */
MLXR_API int mlxr_tp_mlp_block(mlxr_tp_ctx* ctx, const void* x, const void* norm_weight,
                               const void* w_gate_shard, const void* w_up_shard,
                               const void* w_down_shard, void* y, int M, int hidden, int inter,
                               int quant_type, float eps, int dtype, int exchange, void* stream);

/* Sum float partials [n] over ranks into y (activation dtype) with the chosen exchange: the
 * exchange step of mlxr_tp_mlp_block on its own (row-parallel linears outside the MLP). */
MLXR_API int mlxr_tp_all_reduce(mlxr_tp_ctx* ctx, const float* partial, void* y, size_t n, int dtype,
                                int exchange, void* stream);

/* The one-shot exchange over exchange buffers the CALLER provides (a host that manages its own
 * symmetric memory, or a test that plays the peers): buffers[r] is rank r's buffer as mapped in
 * this process, each mlxr_tp_exchange_buffer_bytes() long, 16-byte aligned, flags zeroed once;
 * ctl: two zero-initialised uint32 of this rank (sequence number, CTAs finished).  Layout of a
 * buffer: uint32 flags[8][1024] (source rank, CTA) in the first 64 KB, then float
 * slots[2][8][MLXR_TP_PEER_MAX_ELEMS] (parity of the call's sequence number, source rank).  Call k
 * (k = 1, 2, ...) of a rank stores its partial into slot [k & 1][rank] of every buffer, sets
 * flags[rank][b] = k there for each of its ceil(n / 1024) (at most 256) CTAs b, waits until
 * flags[r][b] >= k in its own buffer for every r, and adds the slots in rank order.  A wait
 * that reaches the limit of mlxr_set_wait_limit_ns leaves y unwritten for that CTA's elements
 * and reports MLXR_ERR_TIMEOUT through mlxr_stream_status(stream); the sequence number still
 * advances, so the next call is well-formed. */
MLXR_API size_t mlxr_tp_exchange_buffer_bytes(void);
MLXR_API int mlxr_tp_all_reduce_buffers(const float* partial, void* y, size_t n, int dtype, int rank,
                                        int world, void* const* buffers, uint32_t* ctl, void* stream);

#ifdef __cplusplus
}
#endif
#endif
