#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl mine|reference]
                    [--workload mlp_decode|...] [--batch M]

One "step" = one pass of the Llama-3-8B-shaped Q4_K decode MLP block (RMSNorm -> gate/up ->
SiLU*up -> down; hidden 4096, intermediate 14336, bf16 activations) over a batch of M
synthetic tokens (default M = 1, the configuration the HBM target is quoted on).  Weights
are random N(0, 0.02) quantized to MLXR-layout Q4_K (no checkpoints exist offline);
activations are N(0, 1).  Prints ONE JSON line.

value     tokens/s with activations resident in HBM, CUDA-event timed, max over ranks
e2e       same metric through the host-buffer C-ABI entry point (mlxr_mlp_block_host):
          x copied host->device and y device->host inside the timed region, every step
roofline  algorithmic bytes of one step / measured step time vs the measured HBM peak
cpu_baseline  the oracle's restatement of the reference CPU path (full dequant + scalar
          triple loop, one thread) timed on this box's host cores

parity    the first step is checked against the oracle composition (and, on several GPUs, for
          identical results on all ranks) before anything is timed; failure ends the run
secondary the other parts of the benchmark definition (prefill Q-GEMM TFLOP/s, GEMV GB/s per
          format, the TinyLlama- and the 70B-shaped block), each with its own roofline

Weights rotate through several device copies so that consecutive steps cannot be served
from the 126 MB L2 (the block's weights are 99 MB).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

H, I = 4096, 14336            # Llama-3-8B MLP (the default workload)
SIZES = {"hidden": H, "inter": I}
# DRAM bytes (read + write) of one decode_kernel launch from an ncu capture of this workload,
# keyed by (hidden, inter, batch); see profiles/
TRAFFIC = {(4096, 14336, 1): 105265152}
QT_Q4_K = 3
EPS = 1e-5
SEED = 1234


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def algorithmic_bytes(M: int, hidden: int = H, inter: int = I) -> int:
    """Packed weights once + x in + y out (bf16) + norm weight; h and scratch excluded."""
    w = 3 * hidden * inter * 144 // 256
    return w + 2 * M * hidden * 2 + hidden * 2


def make_inputs(M: int, hidden: int = H, inter: int = I, qt: int = QT_Q4_K):
    from mlxr_b200.quantize import quantize
    g = lambda i: np.random.Generator(np.random.PCG64(SEED + i))
    wg = quantize((g(1).standard_normal((inter, hidden)) * 0.02).astype(np.float32), qt)
    wu = quantize((g(2).standard_normal((inter, hidden)) * 0.02).astype(np.float32), qt)
    wd = quantize((g(3).standard_normal((hidden, inter)) * 0.02).astype(np.float32), qt)
    x = g(4).standard_normal((M, hidden)).astype(np.float32)
    gamma = (1 + 0.1 * g(5).standard_normal(hidden)).astype(np.float32)
    return wg, wu, wd, x, gamma


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while running."""

    def __init__(self, index: int):
        self.samples = []
        self.stop_flag = False
        self.thread = None
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.max_mhz = None

    def _run(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.ok:
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()

    def window(self, t0, t1):
        """Summary of the samples taken between two perf_counter readings (sampling continues)."""
        return self._summary([s for s in list(self.samples) if t0 <= s[0] <= t1])

    def stop(self, t0=None, t1=None):
        self.stop_flag = True
        if self.thread:
            self.thread.join(timeout=1.0)
        sel = [s for s in self.samples if t0 is not None and t0 <= s[0] <= t1] or self.samples
        return self._summary(sel)

    def _summary(self, sel):
        if not sel:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
                 0x80: "hw_power_brake"}
        bits = 0
        for smp in sel:
            bits |= smp[2]
        return {"sm_mhz": float(np.median([smp[1] for smp in sel])), "sm_max_mhz": self.max_mhz,
                "reasons": [n for b, n in names.items() if bits & b], "samples": len(sel)}


def cpu_baseline(M: int, budget_s: float = 20.0):
    """Oracle port of the reference CPU path (QGemmDequantPrimitive::eval_cpu: full dequant to
    fp32, then the scalar m/n/k loop, single thread) for the whole MLP block at batch M,
    repeated while the time budget lasts.  Returns (record, seconds per step, repetitions)."""
    H, I = SIZES["hidden"], SIZES["inter"]
    from oracle import oracle as O
    wg, wu, wd, x, gamma = make_inputs(M, H, I)
    xb = O.round_to(x, O.BF16)
    gb = O.round_to(gamma, O.BF16)

    def step():
        n = O.round_to(O.rmsnorm(xb, gb, EPS), O.BF16)
        g = O.round_to(O.qgemm_cpu(n, wg, I, QT_Q4_K), O.BF16)
        u = O.round_to(O.qgemm_cpu(n, wu, I, QT_Q4_K), O.BF16)
        h = O.round_to(O.swiglu(g, u), O.BF16)
        return O.round_to(O.qgemm_cpu(h, wd, H, QT_Q4_K), O.BF16)

    times = []
    t_end = time.perf_counter() + budget_s
    while (time.perf_counter() < t_end and len(times) < 20) or not times:
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    t = float(np.median(times))
    return {"value": M / t, "unit": "tokens/s", "cores": 1, "kind": "port",
            "sample": f"full MLP block at batch {M}, {len(times)} repetitions, median {t * 1e3:.1f} ms/step "
                      f"(oracle restatement of eval_cpu: full dequant + scalar loop; the reference's own "
                      f"eval_cpu throws for Q4_K)"}, t, len(times)


def cpu_baseline_all_cores(M: int, budget_s: float = 10.0):
    """The same block as a fair CPU composition on all host cores: the oracle's dequantizers, then
    fp32 BLAS matrix products and fp32 elementwise steps (oracle.mlp_block).  A stated baseline."""
    H, I = SIZES["hidden"], SIZES["inter"]
    from oracle import oracle as O
    wg, wu, wd, x, gamma = make_inputs(M, H, I)
    xb = O.round_to(x, O.BF16)
    gb = O.round_to(gamma, O.BF16)
    times = []
    t_end = time.perf_counter() + budget_s
    while (time.perf_counter() < t_end and len(times) < 10) or not times:
        t0 = time.perf_counter()
        O.mlp_block(xb, gb, wg, wu, wd, I, QT_Q4_K, EPS, O.BF16)
        times.append(time.perf_counter() - t0)
    t = float(np.median(times))
    return {"value": M / t, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"full MLP block at batch {M}, {len(times)} repetitions, median {t * 1e3:.1f} ms/step "
                      f"(oracle dequantizers + fp32 BLAS products on all host cores)"}


def run_reference(args):
    """The reference arm: the reference's CPU path for the same block (oracle port of eval_cpu, one
    thread: that path is single-threaded by construction), a bounded number of repetitions.  The
    line reports the repetitions actually run as `steps`."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    M = args.batch
    want = max(1, min(args.steps, 5))
    cb, t, reps = cpu_baseline(M, budget_s=min(60.0, 12.0 * want))
    line = {
        "impl": "reference", "metric": "mlp_decode_tokens_per_s", "value": cb["value"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": reps, "steps_requested": args.steps, "warmup": 0, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_dict(M, max(1, args.gpus), args.exchange if args.gpus > 1 else None),
        "cpu_baseline": cb,
        "cpu_baseline_all_cores": None if args.no_cpu else cpu_baseline_all_cores(M, budget_s=8.0),
        "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def config_dict(M, n_gpus, exchange=None):
    """The workload's name: the same dict for both arms (nothing that depends on the run)."""
    H, I = SIZES["hidden"], SIZES["inter"]
    name = {(4096, 14336): "Llama-3-8B", (8192, 28672): "Llama-3-70B", (2048, 5632): "TinyLlama"}.get((H, I), "custom")
    d = {"workload": f"{name}-shaped Q4_K decode MLP block (hidden {H}, intermediate {I}, RMSNorm prologue, "
                     f"SwiGLU), batch {M}, bf16 activations",
         "batch": M, "quant": "Q4_K (MLXR layout)",
         "parallelism": "single GPU" if n_gpus == 1 else f"tp{n_gpus} (gate/up rows and down columns sharded, one sum over ranks per step)",
         "l2": "weights rotate over several device copies per GPU (more than 700 MB per GPU; L2 is 126 MB)"}
    if exchange:
        d["exchange"] = exchange
    return d


def timed_graph(step, K, W, stream, min_seconds=0.25, max_repeats=400, dist=None):
    """Capture K calls of step(i, stream_handle) into one CUDA graph on `stream` and replay it until
    at least `min_seconds` of device time have been timed (every replay between its own pair of
    CUDA events on the launching stream).  Returns (median ms per step, repeats, launches counted
    during capture, timed seconds, (t0, t1) wall-clock bracket for the clock sampler)."""
    import torch
    from mlxr_b200._capi import lib
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        for i in range(W):
            step(i, stream.cuda_stream)
        stream.synchronize()
        l0 = lib.mlxr_launch_count()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(K):
                step(W + i, torch.cuda.current_stream().cuda_stream)
        launches = lib.mlxr_launch_count() - l0
        graph.replay()          # untimed: the first replay uploads the graph
        stream.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        times = []
        total = 0.0
        t0 = time.perf_counter()
        while True:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            graph.replay()
            e1.record(stream)
            stream.synchronize()
            ms = e0.elapsed_time(e1)
            times.append(ms)
            total += ms
            more = total < min_seconds * 1e3 and len(times) < max_repeats
            if dist is not None:
                # every rank replays the same number of times: rank 0 alone decides when to stop
                flag = torch.tensor([1.0 if more else 0.0], device="cuda")
                dist.broadcast(flag, 0)
                more = flag.item() != 0.0
            if not more:
                break
        t1 = time.perf_counter()
    torch.cuda.synchronize()
    return float(np.median(times)) / K, len(times), int(launches), total * 1e-3, (t0, t1)


def random_packed(N, K, qt, device, seed):
    """Packed weights for TIMING ONLY: random block bytes with every fp16 field set to a small
    finite constant (quantizing N(0, 0.02) matrices of the larger secondary workloads on the host
    would take minutes; the kernels' time does not depend on the values)."""
    import torch
    be, bb = {0: (32, 18), 2: (32, 34), 3: (256, 144), 16: (64, 34)}[qt]
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w = torch.randint(0, 256, (N * (K // be), bb), dtype=torch.uint8, device=device, generator=g)
    w[:, 0] = 0x1F
    w[:, 1] = 0x20           # fp16 0x201F = 0.0080
    if qt == 3:
        w[:, 2] = 0x1F
        w[:, 3] = 0x1C       # dmin = 0.0040
    return w.reshape(-1)


def secondary_measurements(world, rank, local, ctx, args, dist):
    """The other parts of the benchmark definition, each as its own small measurement with its own
    roofline: prefill Q-GEMM (TFLOP/s against the measured bf16 peak), the M = 1 GEMV per format
    (GB/s against the measured HBM peak), the TinyLlama-shaped block, the small-batch range (one
    linear at batch 8 / 16 / 32 / 64, the Llama-3-8B-shaped block at batch 8 and 32), and the
    Llama-3-70B-shaped block at batch 1 and 32 on this number of GPUs.  Single-GPU entries run on
    rank 0 only."""
    import torch
    from mlxr_b200._capi import check, lib
    hbm, tf, which = measured_peaks()
    dev = torch.device("cuda", local)
    out = []
    side = torch.cuda.Stream()
    sampler = ClockSampler(local)
    sampler.start()

    def clocks_of(bracket):
        c = sampler.window(*bracket)
        return c

    def linear_entry(fmt, M, N, K, min_s):
        qt = FORMATS[fmt]
        wbytes = int(lib.mlxr_quantized_weight_size(N, K, qt))
        copies = max(2, int(np.ceil(300e6 / wbytes))) if M <= 64 else 1
        ws = [random_packed(N, K, qt, dev, 100 + i) for i in range(copies)]
        xcopies = 1 if M <= 64 else max(2, int(np.ceil(300e6 / (M * K * 2))))
        xs = [torch.randn((M, K), device=dev, dtype=torch.float32).bfloat16() for _ in range(min(xcopies, 8))]
        y = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        gs = lib.mlxr_default_group_size(qt)

        def step(i, st):
            check(lib.mlxr_q_gemm_dequant(xs[i % len(xs)].data_ptr(), ws[i % len(ws)].data_ptr(), None, y.data_ptr(), M, N, K, qt, gs, 1, st))

        K_steps = 50 if M <= 64 else 5
        ms, reps, launches, secs, bracket = timed_graph(step, K_steps, 3, side, min_seconds=min_s)
        ab = wbytes + 2 * M * (K + N)
        flops = 2.0 * M * N * K
        gbs, tfl = ab / (ms * 1e-3) / 1e9, flops / (ms * 1e-3) / 1e12
        tensor = M >= 256
        roof = ({"bound": "tensor", "achieved": tfl, "peak": tf, "unit": "TFLOP/s", "frac": tfl / tf, "traffic": None}
                if tensor else
                {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm, "traffic": None})
        roof["peak_source"] = which
        return {"name": f"{'prefill Q-GEMM' if tensor else 'decode GEMV'} {fmt} [{M}, {K}] x [{N}, {K}]^T",
                "metric": "prefill_qgemm_tflops" if tensor else "qgemv_hbm_gbs", "value": tfl if tensor else gbs,
                "unit": "TFLOP/s" if tensor else "GB/s", "us_per_step": ms * 1e3, "steps": K_steps, "repeats": reps,
                "gpu_launches": launches, "roofline": roof, "clocks": clocks_of(bracket), "data": "random packed blocks (timing only)"}

    def block_entry(name, hidden, inter, qt, M, dtype_code, tdt, min_s, tp):
        n_gpus = world if tp else 1
        wsz_gu = int(lib.mlxr_quantized_weight_size(inter // n_gpus, hidden, qt))
        wsz_d = int(lib.mlxr_quantized_weight_size(hidden, inter // n_gpus, qt))
        per_copy = 2 * wsz_gu + wsz_d
        copies = max(1, int(np.ceil(300e6 / per_copy)))
        sets = [(random_packed(inter // n_gpus, hidden, qt, dev, 200 + 3 * i), random_packed(inter // n_gpus, hidden, qt, dev, 201 + 3 * i),
                 random_packed(hidden, inter // n_gpus, qt, dev, 202 + 3 * i)) for i in range(copies)]
        x = torch.randn((M, hidden), device=dev, dtype=torch.float32).to(tdt)
        if tp and n_gpus > 1:
            dist.broadcast(x, 0)
        gam = torch.ones(hidden, device=dev, dtype=tdt)
        y = torch.empty_like(x)

        def step(i, st):
            a, b, c = sets[i % copies]
            if tp and n_gpus > 1:
                check(lib.mlxr_tp_mlp_block(ctx._h, x.data_ptr(), gam.data_ptr(), a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                            y.data_ptr(), M, hidden, inter, qt, EPS, dtype_code, 0, st))
            else:
                check(lib.mlxr_mlp_block(x.data_ptr(), gam.data_ptr(), a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                         y.data_ptr(), M, hidden, inter, qt, EPS, dtype_code, st))

        K_steps = 20
        ms, reps, launches, secs, bracket = timed_graph(step, K_steps, 3, side, min_seconds=min_s, dist=dist if (tp and n_gpus > 1) else None)
        if tp and n_gpus > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        ab = per_copy + 2 * M * hidden * 2 + hidden * 2
        gbs = ab / (ms * 1e-3) / 1e9
        return {"name": name, "metric": "mlp_decode_tokens_per_s", "value": M / (ms * 1e-3), "unit": "tokens/s",
                "n_gpus": n_gpus, "us_per_step": ms * 1e3, "steps": K_steps, "repeats": reps, "gpu_launches": launches,
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm, "traffic": None,
                             "per": "GPU", "algorithmic_bytes_per_step": ab, "peak_source": which},
                "clocks": clocks_of(bracket), "data": "random packed blocks (timing only)"}

    if rank == 0:
        out.append(linear_entry("q4_k", 2048, 14336, 4096, 0.05))
        out.append(linear_entry("q4_k", 8192, 14336, 4096, 0.05))
        for fmt in ("q4_k", "q4_0", "q8_0", "nf4"):
            out.append(linear_entry(fmt, 1, 14336, 4096, 0.03))
        out.append(block_entry("TinyLlama-shaped Q4_0 decode MLP block, batch 1, fp16", 2048, 5632, 0, 1, 0, torch.float16, 0.03, False))
        # the small-batch range (batch 8 / 32 / 64 of the decode configuration): one linear and the block
        for M in (8, 16, 32, 64):
            out.append(linear_entry("q4_k", M, 14336, 4096, 0.03))
        for M in (8, 32):
            out.append(block_entry(f"Llama-3-8B-shaped Q4_K decode MLP block, batch {M}, bf16", 4096, 14336, QT_Q4_K, M, 1,
                                   torch.bfloat16, 0.03, False))
    # the 70B-shaped block on this number of GPUs (every rank takes part)
    for M in (1, 32):
        e = block_entry(f"Llama-3-70B-shaped Q4_K decode MLP block, batch {M}, bf16, {world} GPU(s)", 8192, 28672, QT_Q4_K, M, 1,
                        torch.bfloat16, 0.05, True)
        if rank == 0:
            out.append(e)
    sampler.stop()
    return out


def run_mine(args):
    import torch
    import torch.distributed as dist

    import mlxr_b200 as mx
    from mlxr_b200._capi import check, lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    M = args.batch
    K, W = args.steps, max(args.warmup, 3)
    H, I = SIZES["hidden"], SIZES["inter"]
    # enough distinct weight copies per GPU that consecutive steps cannot be served from L2
    shard_mb = 3 * H * I * 144 // 256 // world / 1e6
    copies = int(min(64, max(8, np.ceil(800.0 / shard_mb))))

    wg_full, wu_full, wd_full, x, gamma = make_inputs(M, H, I)
    wg, wu, wd = wg_full, wu_full, wd_full
    dev = torch.device("cuda", local)
    ctx = None
    exchange = {"auto": 0, "nccl_f32": 1, "nccl_act": 2, "peer": 3}[args.exchange]
    if world > 1:
        import mlxr_b200.tp as tp
        ctx = tp.TPContext()
        wg, wu, wd = tp.shard_mlp_weights(wg, wu, wd, H, I, QT_Q4_K, rank, world)
    wsets = []
    for _ in range(copies):
        wsets.append(tuple(torch.from_numpy(a).to(dev) for a in (wg, wu, wd)))
    xt = torch.from_numpy(x).bfloat16().to(dev)
    gt = torch.from_numpy(gamma).bfloat16().to(dev)
    y = torch.empty_like(xt)
    status = ctypes.c_int(0)

    def step(i, st):
        a, b, c = wsets[i % copies]
        if ctx is None:
            check(lib.mlxr_mlp_block(xt.data_ptr(), gt.data_ptr(), a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                     y.data_ptr(), M, H, I, QT_Q4_K, EPS, 1, st))
        else:
            check(lib.mlxr_tp_mlp_block(ctx._h, xt.data_ptr(), gt.data_ptr(), a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                        y.data_ptr(), M, H, I, QT_Q4_K, EPS, 1, exchange, st))

    # ---- parity gate, before anything is timed: the result of one step against the oracle's
    # composition on rank 0, and - for the exchanges that add the ranks' sums in rank order -
    # bit-identical results on all ranks.  A failure ends the run with a non-zero exit code.
    st0 = torch.cuda.current_stream().cuda_stream
    step(0, st0)
    torch.cuda.synchronize()
    parity = {"tol": 2e-2}
    if world > 1:
        ys = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(ys, y)
        identical = all(torch.equal(ys[0], t) for t in ys)
        parity["ranks_identical"] = bool(identical)
        parity["ranks_identical_required"] = exchange in (0, 3)
    if rank == 0:
        from oracle import oracle as O
        ref = O.mlp_block(O.round_to(x, O.BF16), O.round_to(gamma, O.BF16), wg_full, wu_full, wd_full, I, QT_Q4_K, EPS, O.BF16)
        parity["rel_l2"] = O.rel_l2(y.float().cpu().numpy(), ref)
        parity["against"] = "oracle composition of the unsharded block (fp32, bf16 rounding at each materialised array)"
    ok = torch.tensor([1.0], device=dev)
    if rank == 0 and not (parity["rel_l2"] <= parity["tol"]):
        ok[0] = 0.0
    if world > 1 and parity["ranks_identical_required"] and not parity["ranks_identical"]:
        ok[0] = 0.0
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if ok.item() == 0.0:
        if rank == 0:
            print(json.dumps({"error": "parity gate failed", "parity": parity}))
        sys.exit(3)

    # The K timed steps are captured once into a CUDA graph and replayed: at ~20-30 us per
    # step a Python/ctypes launch loop would measure the host, not the GPU.  The graph is replayed
    # until a quarter of a second of device time has been timed; the value is the median replay.
    # The NCCL exchange modes are timed with plain launches instead (a library collective per step
    # dominates there).
    use_graph = ctx is None or exchange in (0, 3)
    side = torch.cuda.Stream()
    sampler = ClockSampler(local)
    sampler.start()
    if use_graph:
        ms_step, repeats, launches, timed_s, bracket = timed_graph(step, K, W, side, min_seconds=0.25,
                                                                   dist=dist if world > 1 else None)
    else:
        with torch.cuda.stream(side):
            for i in range(W):
                step(i, side.cuda_stream)
            side.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            l0 = lib.mlxr_launch_count()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record(side)
            for i in range(K):
                step(W + i, side.cuda_stream)
            e1.record(side)
            side.synchronize()
            t1 = time.perf_counter()
            launches = lib.mlxr_launch_count() - l0
        ms_step, repeats, timed_s, bracket = e0.elapsed_time(e1) / K, 1, e0.elapsed_time(e1) * 1e-3, (t0, t1)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop(*bracket)
    if world > 1:
        t = torch.tensor([ms_step], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t.item())
    st = torch.cuda.current_stream().cuda_stream

    # end to end: host buffers, copies inside the timed region, every step
    xh = torch.from_numpy(x).bfloat16().pin_memory()
    yh = torch.empty((M, H), dtype=torch.bfloat16).pin_memory()

    def step_host(i):
        a, b, c = wsets[i % copies]
        if ctx is None:
            check(lib.mlxr_mlp_block_host(xh.data_ptr(), gt.data_ptr(), a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                          yh.data_ptr(), M, H, I, QT_Q4_K, EPS, 1, st))
        else:
            # every rank copies the replicated x in, runs its share and the exchange, reads y back
            xt.copy_(xh, non_blocking=True)
            check(lib.mlxr_tp_mlp_block(ctx._h, xt.data_ptr(), gt.data_ptr(), a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                        y.data_ptr(), M, H, I, QT_Q4_K, EPS, 1, exchange, st))
            yh.copy_(y, non_blocking=True)
            torch.cuda.current_stream().synchronize()

    for i in range(W):
        step_host(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    Ke = max(K, 200)
    th0 = time.perf_counter()
    for i in range(Ke):
        step_host(i)
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - th0) / Ke
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())

    # what was timed must have run clean: finite output, no bounded wait gave up
    assert torch.isfinite(y.float()).all()
    check(lib.mlxr_stream_status(side.cuda_stream, ctypes.byref(status)))
    assert status.value == 0, f"device status {status.value} after the timed region"

    secondary = None
    if not args.no_secondary:
        secondary = secondary_measurements(world, rank, local, ctx, args, dist if world > 1 else None)

    if rank == 0:
        hbm, _, which = measured_peaks()
        # per GPU: its share of the weights plus the replicated activations
        ab = (algorithmic_bytes(M, H, I) - 2 * M * H * 2 - H * 2) // world + 2 * M * H * 2 + H * 2
        achieved = ab / (ms_step * 1e-3) / 1e9
        cb = cb_all = None
        if world == 1 and not args.no_cpu:
            cb, _, _ = cpu_baseline(M, budget_s=args.cpu_seconds)
            cb_all = cpu_baseline_all_cores(M, budget_s=8.0)
        line = {
            "metric": "mlp_decode_tokens_per_s", "value": M / (ms_step * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_step,
            "repeats": repeats, "timed_seconds": timed_s,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(M, world, args.exchange if world > 1 else None),
            "weight_copies_per_gpu": copies,
            "parity": parity,
            "e2e": {"value": M / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": M * H * 2, "d2h_bytes_per_step": M * H * 2,
                    "ms_per_step": e2e_s * 1e3, "steps": Ke},
            "gpu_launches": int(launches) * int(repeats),
            "gpu_launches_per_replay": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                         "traffic": TRAFFIC.get((H, I, M)) if world == 1 else None, "peak_source": which,
                         "algorithmic_bytes_per_step": ab, "per": "GPU",
                         "kernel": "decode_kernel (one persistent launch per step: RMSNorm + gate/up + SwiGLU + down)"
                                   + ("" if world == 1 else " + exchange of the ranks' sums"),
                         "timing": "CUDA events around " + (f"each of {repeats} CUDA-graph replays of the K steps (median)" if use_graph else "K plain launches")},
            "cpu_baseline": cb,
            "cpu_baseline_all_cores": cb_all,
            "secondary": secondary,
        }
        print(json.dumps(line))
    if ctx is not None:
        ctx.close()
    if world > 1:
        dist.destroy_process_group()


def run_prefill(args):
    """Prefill Q-GEMM: Y[M, N] = X[M, K] * dequant(W[N, K])^T, Q4_K weights, bf16 activations,
    one linear of the Llama-3-8B MLP (N = inter, K = hidden by default; --transpose for the
    down projection).  value = TFLOP/s (2 M N K per step); the bound is the tensor pipe."""
    import torch

    import mlxr_b200 as mx
    from mlxr_b200._capi import check, lib

    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if int(os.environ.get("RANK", "0")) != 0:
        return                      # a single linear has no exchange step: replicas only
    M = args.batch
    N, K = (SIZES["hidden"], SIZES["inter"]) if args.transpose else (SIZES["inter"], SIZES["hidden"])
    steps, W = args.steps, max(args.warmup, 3)
    from mlxr_b200.quantize import quantize
    g = lambda i: np.random.Generator(np.random.PCG64(SEED + i))
    w = torch.from_numpy(quantize((g(1).standard_normal((N, K)) * 0.02).astype(np.float32), QT_Q4_K)).cuda()
    copies = max(2, int(np.ceil(300e6 / (M * K * 2))))          # rotate X so that it does not sit in L2
    xs = [torch.from_numpy(g(10 + i).standard_normal((M, K)).astype(np.float32)).bfloat16().cuda() for i in range(min(copies, 8))]
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream

    def step(i):
        check(lib.mlxr_q_gemm_dequant(xs[i % len(xs)].data_ptr(), w.data_ptr(), None, y.data_ptr(), M, N, K, QT_Q4_K, 256, 1, st))

    for i in range(W):
        step(i)
    torch.cuda.synchronize()
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    l0 = lib.mlxr_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(steps):
        step(W + i)
    e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    launches = lib.mlxr_launch_count() - l0
    clocks = sampler.stop(t0, t1)
    ms_step = e0.elapsed_time(e1) / steps
    status = ctypes.c_int(0)
    check(lib.mlxr_stream_status(st, ctypes.byref(status)))
    assert status.value == 0 and torch.isfinite(y.float()).all()

    xh = xs[0].cpu().pin_memory()
    yh = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    ke = max(3, min(steps, 20))
    for i in range(2):
        check(lib.mlxr_q_gemm_dequant_host(xh.data_ptr(), w.data_ptr(), None, yh.data_ptr(), M, N, K, QT_Q4_K, 256, 1, st))
    torch.cuda.synchronize()
    th0 = time.perf_counter()
    for i in range(ke):
        check(lib.mlxr_q_gemm_dequant_host(xh.data_ptr(), w.data_ptr(), None, yh.data_ptr(), M, N, K, QT_Q4_K, 256, 1, st))
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - th0) / ke

    _, tf, which = measured_peaks()
    flops = 2.0 * M * N * K
    achieved = flops / (ms_step * 1e-3) / 1e12
    line = {
        "metric": "prefill_qgemm_tflops", "value": achieved, "unit": "TFLOP/s", "n_gpus": 1, "steps": steps, "warmup": W,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"prefill Q-GEMM [{M}, {K}] x Q4_K [{N}, {K}]^T, bf16 activations, fp32 accumulation "
                               f"(tcgen05 / TMEM)", "batch": M, "quant": "Q4_K (MLXR layout)", "parallelism": "single GPU",
                   "l2": f"X rotates over {len(xs)} device copies; W (33 MB packed) is L2-resident by design"},
        "e2e": {"value": flops / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2,
                "ms_per_step": e2e_s * 1e3},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": tf, "unit": "TFLOP/s", "frac": achieved / tf,
                     "traffic": None, "peak_source": which + " (burst bf16 figure)", "flops_per_step": flops,
                     "kernel": "qgemm_tc_kernel", "timing": "CUDA events around K plain launches"},
        "cpu_baseline": None,
    }
    print(json.dumps(line))


FORMATS = {"q4_0": 0, "q8_0": 2, "q4_k": 3, "nf4": 16}


def time_graph(step, K, W):
    """Capture K calls of step(i) into one CUDA graph on a side stream and time one replay with
    CUDA events (ms per step).  Removes the Python launch loop from small-kernel timings."""
    import torch
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        for i in range(W):
            step(i, side.cuda_stream)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for i in range(K):
                step(W + i, torch.cuda.current_stream().cuda_stream)
        graph.replay()
        side.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(side)
        graph.replay()
        e1.record(side)
        side.synchronize()
    return e0.elapsed_time(e1) / K, side


def linear_case(fmt, M, N, K, steps, warmup, cache):
    """One quantized linear Y[M,N] = X[M,K] W[N,K]^T: algorithmic GB/s and TFLOP/s."""
    import torch
    from mlxr_b200._capi import check, lib
    from mlxr_b200.quantize import quantize
    qt = FORMATS[fmt]
    key = (fmt, N, K)
    if key not in cache:
        if ("w", N, K) not in cache:
            cache[("w", N, K)] = (np.random.Generator(np.random.PCG64(SEED + 1)).standard_normal((N, K)) * 0.02).astype(np.float32)
        packed = torch.from_numpy(quantize(cache[("w", N, K)], qt))
        copies = max(2, int(np.ceil(400e6 / packed.numel()))) if M <= 64 else 1
        cache[key] = [packed.cuda() for _ in range(min(copies, 16))]
    ws = cache[key]
    x = torch.from_numpy(np.random.Generator(np.random.PCG64(SEED + 4)).standard_normal((M, K)).astype(np.float32)).bfloat16().cuda()
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    gs = lib.mlxr_default_group_size(qt)

    def step(i, st):
        check(lib.mlxr_q_gemm_dequant(x.data_ptr(), ws[i % len(ws)].data_ptr(), None, y.data_ptr(), M, N, K, qt, gs, 1, st))

    ms, side = time_graph(step, steps, max(warmup, 3))
    status = ctypes.c_int(0)
    check(lib.mlxr_stream_status(side.cuda_stream, ctypes.byref(status)))
    assert status.value == 0 and torch.isfinite(y.float()).all()
    wbytes = ws[0].numel()
    ab = wbytes + 2 * M * (K + N)
    hbm, tf, which = measured_peaks()
    gbs, tfl = ab / (ms * 1e-3) / 1e9, 2.0 * M * N * K / (ms * 1e-3) / 1e12
    tensor_bound = 2.0 * M * N * K / (tf * 1e12) > ab / (hbm * 1e9)
    return {"metric": "qlinear", "format": fmt, "M": M, "N": N, "K": K, "us": ms * 1e3, "GB/s": gbs, "TFLOP/s": tfl,
            "bound": "tensor" if tensor_bound else "hbm", "frac": (tfl / tf) if tensor_bound else (gbs / hbm),
            "peak_source": which, "weight_copies": len(ws)}


def run_sweep(args):
    """The format sweep and the decode / prefill linears of the Llama-3-8B shapes: one JSON line
    per case (not the contract line; a measurement table for the design notes)."""
    import torch
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cache = {}
    cases = []
    for fmt in ("q8_0", "q4_0", "q4_k", "nf4"):
        for M in (1, 16, 2048):
            cases.append((fmt, M, 14336, 4096))
    for M in (8, 32, 64, 512, 8192):
        cases.append(("q4_k", M, 14336, 4096))
    for M in (1, 8, 2048):
        cases.append(("q4_k", M, 4096, 14336))
    for fmt, M, N, K in cases:
        steps = 200 if M <= 64 else 10
        print(json.dumps(linear_case(fmt, M, N, K, steps, 5, cache)), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="mine", choices=["mine", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary measurements (prefill, GEMV per format, other blocks)")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--hidden", type=int, default=H)
    ap.add_argument("--inter", type=int, default=I)
    ap.add_argument("--workload", default="mlp_decode", choices=["mlp_decode", "prefill", "linear", "sweep"])
    ap.add_argument("--format", default="q4_k", choices=["q4_0", "q8_0", "q4_k", "nf4"])
    ap.add_argument("--transpose", action="store_true", help="prefill: the down-projection shape (N = hidden, K = inter)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "nccl_f32", "nccl_act", "peer"],
                    help="how the ranks' partial sums are added (N > 1)")
    args = ap.parse_args()
    SIZES["hidden"], SIZES["inter"] = args.hidden, args.inter
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "sweep":
        run_sweep(args)
    elif args.workload == "linear":
        import torch
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        N, K = (SIZES["hidden"], SIZES["inter"]) if args.transpose else (SIZES["inter"], SIZES["hidden"])
        print(json.dumps(linear_case(args.format, args.batch, N, K, min(args.steps, 500), args.warmup, {})))
    elif args.workload == "prefill":
        if args.batch == 1:
            args.batch = 2048
        run_prefill(args)
    else:
        run_mine(args)


if __name__ == "__main__":
    main()
