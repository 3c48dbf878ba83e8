// Tensor-parallel MLP block: shard packer, communicator context, and the exchange step.
//
// One process per GPU.  NCCL is used for set-up (exchange of IPC handles, barriers) and as one of
// the two ways to sum the ranks' partial results; the other is the one-shot peer exchange kernel
// below, which matters at decode sizes where the payload is a few KB and a library all-reduce
// costs more than the weight stream of the block itself.
//
// NCCL is loaded with dlopen at first use, so the library has no link-time dependency on it and
// shares the copy a host framework has already loaded.
#include <dlfcn.h>
#include <nccl.h>

#include <mutex>

#include "../../include/mlxr_b200_tp.h"
#include "common.cuh"
#include "decode_kernel.cuh"   // bounded_wait
#include "kernels.h"

namespace mlxr {
namespace {

// ---- NCCL entry points -----------------------------------------------------------------------
struct Nccl {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};
Nccl g_nccl;
std::mutex g_nccl_mu;

int load_nccl() {
  std::lock_guard<std::mutex> lk(g_nccl_mu);
  if (g_nccl.handle) return MLXR_OK;
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) { set_error("cannot load libnccl.so.2: %s", dlerror()); return MLXR_ERR_NCCL; }
#define MLXR_SYM(field, name)                                                      \
  *(void**)(&g_nccl.field) = dlsym(h, name);                                       \
  if (!g_nccl.field) { set_error("libnccl lacks %s", name); return MLXR_ERR_NCCL; }
  MLXR_SYM(GetUniqueId, "ncclGetUniqueId");
  MLXR_SYM(CommInitRank, "ncclCommInitRank");
  MLXR_SYM(CommDestroy, "ncclCommDestroy");
  MLXR_SYM(AllReduce, "ncclAllReduce");
  MLXR_SYM(AllGather, "ncclAllGather");
  MLXR_SYM(GetErrorString, "ncclGetErrorString");
#undef MLXR_SYM
  g_nccl.handle = h;
  return MLXR_OK;
}

#define MLXR_NCCL_TRY(expr)                                                              \
  do {                                                                                   \
    ncclResult_t r_ = (expr);                                                            \
    if (r_ != ncclSuccess) {                                                             \
      set_error("NCCL error %d (%s) at %s", (int)r_, g_nccl.GetErrorString(r_), #expr);  \
      return MLXR_ERR_NCCL;                                                              \
    }                                                                                    \
  } while (0)

ncclDataType_t nccl_dtype(int dtype) {
  return dtype == MLXR_F16 ? ncclFloat16 : dtype == MLXR_BF16 ? ncclBfloat16 : ncclFloat32;
}

// ---- exchange buffer layout (one per rank, mapped by every peer) --------------------------------
// layout constants shared with the decode kernel's fused exchange (kernels.h)
constexpr int kMaxWorld = kTpMaxWorld;
constexpr int kMaxCtas = 256;                      // CTAs of the exchange kernel (flag index < kTpFlagsPerRank)
constexpr size_t kSlotElems = kTpSlotElems;
constexpr size_t kFlagBytes = kTpFlagBytes;
constexpr size_t kXchgBytes = kTpXchgBytes;
static_assert(kTpSlotElems == MLXR_TP_PEER_MAX_ELEMS, "header and kernel disagree on the slot size");
static_assert(kMaxCtas <= kTpFlagsPerRank, "flag index range");

struct PeerTable {
  char* base[kMaxWorld];
};

__device__ __forceinline__ float* slot_ptr(char* base, int parity, int src) {
  return reinterpret_cast<float*>(base + kFlagBytes) + ((size_t)parity * kMaxWorld + src) * kSlotElems;
}
__device__ __forceinline__ uint32_t* flag_ptr(char* base, int src, int cta) {
  return reinterpret_cast<uint32_t*>(base) + src * kTpFlagsPerRank + cta;
}

// One-shot all-reduce.  CTA b owns elements [b*chunk, (b+1)*chunk): it stores its rank's values
// into slot `rank` of every rank's buffer (its own included), raises flag (rank, b) there, waits
// for the flags (r, b) of all ranks r in its own buffer, and adds the world slots in rank order.
// The sequence number lives in device memory (ctl[0]) and is advanced by the last CTA to finish
// (ctl[1] counts them), so a captured launch replays correctly.  Two slot parities alternate: a
// peer can be at most one call ahead, since finishing a call needs this rank's flag of that call.
template <typename T>
__global__ void __launch_bounds__(256) tp_exchange_kernel(const float* __restrict__ partial, T* __restrict__ y,
                                                          size_t n, size_t chunk, int rank, int world,
                                                          PeerTable peers, uint32_t* ctl, int* status,
                                                          unsigned long long wait_ns) {
  const int b = blockIdx.x, tid = threadIdx.x;
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(ctl) + 1u;
  const int parity = (int)(seq & 1u);
  const size_t e0 = (size_t)b * chunk, e1 = min(n, e0 + chunk);
  __shared__ int dead;
  if (tid == 0) dead = 0;
  // push (the next rank first, so that the t ranks do not all write to the same peer at once)
  for (int i = 0; i < world; i++) {
    const int p = (rank + 1 + i) % world;
    float* dst = slot_ptr(peers.base[p], parity, rank);
    for (size_t e = e0 + (size_t)tid * 4; e < e1; e += 256 * 4)
      *reinterpret_cast<float4*>(dst + e) = *reinterpret_cast<const float4*>(partial + e);
  }
  __threadfence_system();
  __syncthreads();
  if (tid < world) {
    uint32_t* f = flag_ptr(peers.base[tid], rank, b);
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(seq) : "memory");
  }
  if (tid < world) {
    const uint32_t* f = flag_ptr(peers.base[rank], tid, b);
    // bounded by time (the limit every device-side wait of this library shares)
    const bool ok = decode::bounded_wait([&] {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      return (int32_t)(v - seq) >= 0;
    }, wait_ns);
    if (!ok) dead = 1;
  }
  __syncthreads();
  if (!dead) {
    char* mine = peers.base[rank];
    for (size_t e = e0 + (size_t)tid * 4; e < e1; e += 256 * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < world; r++) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(slot_ptr(mine, parity, r) + e));
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      y[e] = Act<T>::from_f(acc.x);
      y[e + 1] = Act<T>::from_f(acc.y);
      y[e + 2] = Act<T>::from_f(acc.z);
      y[e + 3] = Act<T>::from_f(acc.w);
    }
  } else if (tid == 0) {
    atomicExch(status, MLXR_ERR_TIMEOUT);
  }
  // the last CTA to finish advances the sequence number for the next launch
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(ctl + 1, 1u) == gridDim.x - 1u) {
      ctl[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(ctl) = seq;
    }
  }
}

}  // namespace
}  // namespace mlxr

using namespace mlxr;

struct mlxr_tp_ctx {
  int rank = 0, world = 1, device = 0;
  ncclComm_t comm = nullptr;
  float* partial = nullptr;       // this rank's float partial [M, hidden]
  size_t partial_elems = 0;
  char* xchg = nullptr;           // this rank's exchange buffer (null without the peer exchange)
  PeerTable peers;                // every rank's exchange buffer as mapped here
  uint32_t* ctl = nullptr;        // [0] sequence number, [1] CTAs finished, [2] barrier / agreement word
  char* handles_dev = nullptr;    // scratch for the handle all-gather (inside the control block)
  bool ready = false;             // set-up finished on this rank (destroy meets the peers only then)
};

namespace {

int ctx_barrier(mlxr_tp_ctx* c, cudaStream_t st) {
  // a one-float all-reduce as the barrier across ranks
  MLXR_NCCL_TRY(g_nccl.AllReduce(c->ctl + 2, c->ctl + 2, 1, ncclFloat32, ncclSum, c->comm, st));
  MLXR_CUDA_TRY(cudaStreamSynchronize(st));
  return MLXR_OK;
}

int ensure_partial(mlxr_tp_ctx* c, size_t elems) {
  if (elems <= c->partial_elems) return MLXR_OK;
  MLXR_CUDA_TRY(cudaDeviceSynchronize());
  if (c->partial) MLXR_CUDA_TRY(cudaFree(c->partial));
  c->partial = nullptr;
  c->partial_elems = 0;
  MLXR_CUDA_TRY(cudaMalloc(&c->partial, elems * sizeof(float)));
  c->partial_elems = elems;
  return MLXR_OK;
}

}  // namespace

extern "C" {

int mlxr_tp_unique_id(void* id128) {
  if (!id128) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (int r = load_nccl()) return r;
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  ncclUniqueId id;
  MLXR_NCCL_TRY(g_nccl.GetUniqueId(&id));
  memcpy(id128, &id, sizeof(id));
  return MLXR_OK;
}

int mlxr_tp_create(const void* id128, int rank, int world, int use_peer, mlxr_tp_ctx** out) {
  if (!id128 || !out) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) {
    set_error("rank %d / world %d outside 1..%d", rank, world, kMaxWorld);
    return MLXR_ERR_INVALID_ARGUMENT;
  }
  if (int r = load_nccl()) return r;
  mlxr_tp_ctx* c = new mlxr_tp_ctx();
  c->rank = rank;
  c->world = world;
  for (int i = 0; i < kMaxWorld; i++) c->peers.base[i] = nullptr;
  auto cuda_step = [&](cudaError_t e, const char* what) -> int {
    if (e == cudaSuccess) return MLXR_OK;
    set_error("CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
    return MLXR_ERR_CUDA;
  };
  // Set-up is collective and so is its outcome: a rank whose local step fails (an allocation, an
  // IPC mapping) still takes part in every collective below, and the ranks agree on the result
  // (minimum over ranks of a success flag) before anyone returns.  Otherwise the peers of a rank
  // that left early would sit in a collective it never joins.  Only two failures cannot be
  // shared: the 4 KB control block (allocated before the communicator exists) and
  // ncclCommInitRank itself, which NCCL fails on all ranks together.
  if (int rc = cuda_step(cudaGetDevice(&c->device), "cudaGetDevice")) { delete c; return rc; }
  // control block: [0] sequence number, [1] CTAs finished, [2] float used by barriers and the
  // agreement step; from byte 1024: the IPC handles of all ranks
  if (int rc = cuda_step(cudaMalloc(&c->ctl, 4096), "cudaMalloc(ctl)")) { delete c; return rc; }
  if (int rc = cuda_step(cudaMemset(c->ctl, 0, 4096), "cudaMemset(ctl)")) { cudaFree(c->ctl); delete c; return rc; }
  c->handles_dev = reinterpret_cast<char*>(c->ctl) + 1024;
  int local_rc = MLXR_OK;        // first local failure (its text stays in mlxr_last_error)
  auto step = [&](int rc) { if (rc && !local_rc) local_rc = rc; return rc == MLXR_OK; };
  step(ensure_partial(c, kSlotElems));
  const bool want_peer = use_peer && world > 1;
  cudaIpcMemHandle_t mine;
  memset(&mine, 0, sizeof(mine));
  if (want_peer) {
    if (step(cuda_step(cudaMalloc(&c->xchg, kXchgBytes), "cudaMalloc(exchange buffer)")) &&
        step(cuda_step(cudaMemset(c->xchg, 0, kFlagBytes), "cudaMemset(flags)")))
      step(cuda_step(cudaIpcGetMemHandle(&mine, c->xchg), "cudaIpcGetMemHandle"));
    step(cuda_step(cudaMemcpy(c->handles_dev + (size_t)rank * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice), "cudaMemcpy(handle)"));
  }
  step(cuda_step(cudaDeviceSynchronize(), "cudaDeviceSynchronize"));
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  {
    ncclResult_t r = g_nccl.CommInitRank(&c->comm, world, id, rank);
    if (r != ncclSuccess) {
      set_error("NCCL error %d (%s) at ncclCommInitRank", (int)r, g_nccl.GetErrorString(r));
      c->comm = nullptr;
      mlxr_tp_destroy(c);
      return MLXR_ERR_NCCL;
    }
  }
  auto nccl_step = [&](ncclResult_t r, const char* what) -> int {
    if (r == ncclSuccess) return MLXR_OK;
    set_error("NCCL error %d (%s) at %s", (int)r, g_nccl.GetErrorString(r), what);
    return MLXR_ERR_NCCL;
  };
  if (want_peer) {
    // every rank joins the gather, whatever happened to it locally
    step(nccl_step(g_nccl.AllGather(c->handles_dev + (size_t)rank * sizeof(mine), c->handles_dev, sizeof(mine), ncclInt8,
                                    c->comm, (cudaStream_t)0), "ncclAllGather(handles)"));
    step(cuda_step(cudaDeviceSynchronize(), "cudaDeviceSynchronize"));
    cudaIpcMemHandle_t all[kMaxWorld];
    if (!local_rc && step(cuda_step(cudaMemcpy(all, c->handles_dev, (size_t)world * sizeof(mine), cudaMemcpyDeviceToHost), "cudaMemcpy(handles)"))) {
      for (int p = 0; p < world && !local_rc; p++) {
        if (p == rank) { c->peers.base[p] = c->xchg; continue; }
        void* ptr = nullptr;
        if (step(cuda_step(cudaIpcOpenMemHandle(&ptr, all[p], cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")))
          c->peers.base[p] = (char*)ptr;
      }
    }
  }
  // agreement: minimum over ranks of "my set-up succeeded"
  {
    const float ok_local = local_rc ? 0.0f : 1.0f;
    float ok_all = 0.0f;
    int rc = cuda_step(cudaMemcpy(c->ctl + 2, &ok_local, sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy(flag)");
    if (!rc) rc = nccl_step(g_nccl.AllReduce(c->ctl + 2, c->ctl + 2, 1, ncclFloat32, ncclMin, c->comm, (cudaStream_t)0), "ncclAllReduce(agreement)");
    if (!rc) rc = cuda_step(cudaMemcpy(&ok_all, c->ctl + 2, sizeof(float), cudaMemcpyDeviceToHost), "cudaMemcpy(flag)");
    const float zero = 0.0f;
    cudaMemcpy(c->ctl + 2, &zero, sizeof(float), cudaMemcpyHostToDevice);
    if (rc || ok_all < 0.5f) {
      // all ranks arrive here together: nobody is left inside a collective
      if (!local_rc && !rc) set_error("mlxr_tp_create: set-up failed on another rank");
      const int ret = local_rc ? local_rc : (rc ? rc : MLXR_ERR_CUDA);
      c->ready = false;
      mlxr_tp_destroy(c);
      return ret;
    }
  }
  // nobody stores into a peer's buffer before every rank has cleared its flags and mapped all
  if (int rc = ctx_barrier(c, (cudaStream_t)0)) { mlxr_tp_destroy(c); return rc; }
  c->ready = true;
  *out = c;
  return MLXR_OK;
}

int mlxr_tp_destroy(mlxr_tp_ctx* c) {
  if (!c) return MLXR_OK;
  cudaDeviceSynchronize();
  // peers may still be reading this rank's buffer: meet them first (skipped if set-up failed early)
  if (c->ready) ctx_barrier(c, (cudaStream_t)0);
  for (int p = 0; p < c->world; p++)
    if (p != c->rank && c->peers.base[p]) cudaIpcCloseMemHandle(c->peers.base[p]);
  if (c->ready) ctx_barrier(c, (cudaStream_t)0);
  if (c->xchg) cudaFree(c->xchg);
  if (c->partial) cudaFree(c->partial);
  if (c->ctl) cudaFree(c->ctl);
  if (c->comm) g_nccl.CommDestroy(c->comm);
  delete c;
  return MLXR_OK;
}

int mlxr_tp_rank(const mlxr_tp_ctx* c) { return c ? c->rank : -1; }
int mlxr_tp_world(const mlxr_tp_ctx* c) { return c ? c->world : -1; }

// ---- shard packer ------------------------------------------------------------------------------
size_t mlxr_tp_shard_bytes(int which, int hidden, int inter, int qt, int world) {
  const int be = block_elems(qt), bb = block_bytes(qt);
  if (!be || world < 1 || hidden <= 0 || inter <= 0 || hidden % be != 0 || inter % (world * be) != 0) return 0;
  if (which == 0) return (size_t)(inter / world) * (size_t)(hidden / be) * bb;
  if (which == 1) return (size_t)hidden * (size_t)(inter / world / be) * bb;
  return 0;
}

int mlxr_tp_pack_shard(const void* w_full, void* w_shard, int which, int hidden, int inter, int qt, int rank,
                       int world) {
  if (!w_full || !w_shard) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (rank < 0 || rank >= world) { set_error("rank %d outside world %d", rank, world); return MLXR_ERR_INVALID_ARGUMENT; }
  const size_t total = mlxr_tp_shard_bytes(which, hidden, inter, qt, world);
  if (!total) {
    set_error("cannot shard %s [hidden %d, inter %d] over %d ranks: inter must be a multiple of world x block size",
              mlxr_quant_type_name(qt), hidden, inter, world);
    return MLXR_ERR_SHAPE;
  }
  const int be = block_elems(qt), bb = block_bytes(qt);
  const uint8_t* src = (const uint8_t*)w_full;
  uint8_t* dst = (uint8_t*)w_shard;
  if (which == 0) {
    memcpy(dst, src + (size_t)rank * total, total);   // rows [rank*I/t, (rank+1)*I/t)
  } else {
    const size_t row_full = (size_t)(inter / be) * bb, row_shard = row_full / world;
    for (int r = 0; r < hidden; r++) memcpy(dst + (size_t)r * row_shard, src + (size_t)r * row_full + (size_t)rank * row_shard, row_shard);
  }
  return MLXR_OK;
}

// ---- exchange ------------------------------------------------------------------------------------
int mlxr_tp_all_reduce(mlxr_tp_ctx* c, const float* partial, void* y, size_t n, int dtype, int exchange, void* stream) {
  if (!c || !partial || !y) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (dtype != MLXR_F16 && dtype != MLXR_BF16 && dtype != MLXR_F32) { set_error("bad dtype %d", dtype); return MLXR_ERR_INVALID_ARGUMENT; }
  cudaStream_t st = (cudaStream_t)stream;
  if (n == 0) return MLXR_OK;
  if (c->world == 1) return launch_cast_from_f32(partial, y, n, dtype, st);
  const bool peer_ok = c->xchg && n <= kSlotElems && n % 4 == 0;
  if (exchange == MLXR_TP_EXCHANGE_AUTO) exchange = peer_ok ? MLXR_TP_EXCHANGE_PEER : MLXR_TP_EXCHANGE_NCCL_F32;
  if (exchange == MLXR_TP_EXCHANGE_PEER) {
    if (!peer_ok) {
      set_error("peer exchange needs a context created with use_peer, n %% 4 == 0 and n <= %zu (got %zu)", kSlotElems, n);
      return MLXR_ERR_SHAPE;
    }
    int* status = nullptr;
    if (int r = stream_status_word(st, &status)) return r;
    int grid = (int)((n + 1023) / 1024);
    if (grid > kMaxCtas) grid = kMaxCtas;
    size_t chunk = (n + grid - 1) / grid;
    chunk = (chunk + 3) / 4 * 4;
    MLXR_DISPATCH_DTYPE(dtype, T, {
      tp_exchange_kernel<T><<<grid, 256, 0, st>>>(partial, (T*)y, n, chunk, c->rank, c->world, c->peers, c->ctl, status,
                                                  wait_limit_ns());
    });
    MLXR_LAUNCH_CHECK("tp_exchange_kernel");
    return MLXR_OK;
  }
  if (exchange == MLXR_TP_EXCHANGE_NCCL_F32) {
    if (int r = ensure_partial(c, n)) return r;
    float* buf = c->partial;
    if (dtype == MLXR_F32) {
      MLXR_NCCL_TRY(g_nccl.AllReduce(partial, y, n, ncclFloat32, ncclSum, c->comm, st));
      return MLXR_OK;
    }
    MLXR_NCCL_TRY(g_nccl.AllReduce(partial, buf, n, ncclFloat32, ncclSum, c->comm, st));
    return launch_cast_from_f32(buf, y, n, dtype, st);
  }
  if (exchange == MLXR_TP_EXCHANGE_NCCL_ACT) {
    if (int r = launch_cast_from_f32(partial, y, n, dtype, st)) return r;
    MLXR_NCCL_TRY(g_nccl.AllReduce(y, y, n, nccl_dtype(dtype), ncclSum, c->comm, st));
    return MLXR_OK;
  }
  set_error("unknown exchange mode %d", exchange);
  return MLXR_ERR_INVALID_ARGUMENT;
}

size_t mlxr_tp_exchange_buffer_bytes(void) { return kXchgBytes; }

int mlxr_tp_all_reduce_buffers(const float* partial, void* y, size_t n, int dtype, int rank, int world,
                               void* const* buffers, uint32_t* ctl, void* stream) {
  if (!partial || !y || !buffers || !ctl) { set_error("null pointer"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (dtype != MLXR_F16 && dtype != MLXR_BF16 && dtype != MLXR_F32) { set_error("bad dtype %d", dtype); return MLXR_ERR_INVALID_ARGUMENT; }
  if (world < 2 || world > kMaxWorld || rank < 0 || rank >= world) {
    set_error("rank %d / world %d outside 2..%d", rank, world, kMaxWorld);
    return MLXR_ERR_INVALID_ARGUMENT;
  }
  if (n == 0) return MLXR_OK;
  if (n > kSlotElems || n % 4 != 0) {
    set_error("peer exchange needs n %% 4 == 0 and n <= %zu (got %zu)", kSlotElems, n);
    return MLXR_ERR_SHAPE;
  }
  PeerTable peers;
  for (int i = 0; i < kMaxWorld; i++) peers.base[i] = i < world ? (char*)buffers[i] : nullptr;
  for (int i = 0; i < world; i++)
    if (!peers.base[i] || ((uintptr_t)peers.base[i] & 15u)) { set_error("exchange buffer %d is null or not 16-byte aligned", i); return MLXR_ERR_INVALID_ARGUMENT; }
  cudaStream_t st = (cudaStream_t)stream;
  int* status = nullptr;
  if (int r = stream_status_word(st, &status)) return r;
  int grid = (int)((n + 1023) / 1024);
  if (grid > kMaxCtas) grid = kMaxCtas;
  size_t chunk = (n + grid - 1) / grid;
  chunk = (chunk + 3) / 4 * 4;
  MLXR_DISPATCH_DTYPE(dtype, T, {
    tp_exchange_kernel<T><<<grid, 256, 0, st>>>(partial, (T*)y, n, chunk, rank, world, peers, ctl, status, wait_limit_ns());
  });
  MLXR_LAUNCH_CHECK("tp_exchange_kernel");
  return MLXR_OK;
}

int mlxr_tp_mlp_block(mlxr_tp_ctx* c, const void* x, const void* norm_weight, const void* wg, const void* wu,
                      const void* wd, void* y, int M, int hidden, int inter, int qt, float eps, int dtype,
                      int exchange, void* stream) {
  if (!c) { set_error("null context"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (M < 0 || hidden <= 0 || inter <= 0) { set_error("Input must be 2D [M, hidden_size]"); return MLXR_ERR_INVALID_ARGUMENT; }
  if (!mlxr_tp_shard_bytes(0, hidden, inter, qt, c->world)) {
    set_error("cannot shard %s [hidden %d, inter %d] over %d ranks", mlxr_quant_type_name(qt), hidden, inter, c->world);
    return MLXR_ERR_SHAPE;
  }
  if (M == 0) return MLXR_OK;
  const size_t n = (size_t)M * hidden;
  if (c->world > 1 && c->xchg && (exchange == MLXR_TP_EXCHANGE_AUTO || exchange == MLXR_TP_EXCHANGE_PEER) &&
      n <= kSlotElems && !tune_env("MLXR_TP_NO_FUSE")) {
    // decode shapes: one launch computes the rank's share, stores its sums into every rank's
    // exchange buffer from the epilogue and ends with the reduction
    DecodeTp tp;
    for (int i = 0; i < kMaxWorld; i++) tp.peer[i] = c->peers.base[i];
    tp.rank = c->rank;
    tp.world = c->world;
    tp.ctl = c->ctl;
    tp.y = y;
    const int rc = mlp_block_tp_fused(x, norm_weight, wg, wu, wd, M, hidden, inter / c->world, qt, eps, dtype, &tp,
                                      (cudaStream_t)stream);
    if (rc != MLXR_ERR_UNSUPPORTED) return rc;
  }
  // the NCCL float path reduces out of place into a second region of the partial buffer
  if (int r = ensure_partial(c, 2 * n > kSlotElems ? 2 * n : kSlotElems)) return r;
  if (int r = mlxr_mlp_block_partial_f32(x, norm_weight, wg, wu, wd, c->partial, M, hidden, inter / c->world, qt,
                                         eps, dtype, stream))
    return r;
  cudaStream_t st = (cudaStream_t)stream;
  if (c->world > 1 && (exchange == MLXR_TP_EXCHANGE_NCCL_F32 ||
                       (exchange == MLXR_TP_EXCHANGE_AUTO && !(c->xchg && n <= kSlotElems && n % 4 == 0)))) {
    float* red = c->partial + n;
    MLXR_NCCL_TRY(g_nccl.AllReduce(c->partial, red, n, ncclFloat32, ncclSum, c->comm, st));
    return launch_cast_from_f32(red, y, n, dtype, st);
  }
  return mlxr_tp_all_reduce(c, c->partial, y, n, dtype, exchange, stream);
}

}  // extern "C"
