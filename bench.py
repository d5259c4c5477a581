#!/usr/bin/env python
"""Benchmark of the mLSTM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (configuration 4): the model-scale training step of the parallel (matmul) mLSTM,
forward + backward of the GLOBAL problem B=16, NH=8, S=4096, D=256 in bf16 (seeded synthetic data:
q, k, v ~ N(0, 1/D), f ~ N(3, 1), i ~ N(0, 1), dh ~ N(0, 1)).  A "step" is one forward + backward over
all 128 (batch, head) slices.  With N GPUs the slices are split contiguously, 128/N per rank, with no
data-path collective (strong scaling); one process per GPU, launched by torch.distributed.run for N > 1.

One JSON line is printed by rank 0.  `value` is tokens/s with inputs resident in HBM; `e2e` is the same
step through the library's public entry points with pinned HOST buffers, the host->device copies of the
inputs and the device->host copies of the results inside the timed region.  `secondary` carries, measured
in the same run outside the headline's timed region: the step through the drop-in autograd function
(fp32 h), a longer back-to-back run under the power cap, the other configurations (1, 2, 3, 5) each with
time, rate, roofline fraction and parity against the CPU oracle, and for N > 1 the weak-scaling figure
and the sequence-parallel long-context forward.

`--impl reference` times the CPU path (the oracle port of the reference's PyTorch functions, since the
reference's Python cannot travel to the GPU box) on the host cores on a bounded sample.
`--workload cfgK` runs one configuration alone (used for profiler captures of small cases).
"""
import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(B=16, NH=8, S=4096, D=256)
METRIC = "mlstm_matmul_fwd_bwd_tokens_per_s"
PKG_NAME = "xlstm-triton-cuda-implementation_b200"
WORKLOAD4 = "cfg4: mLSTM matmul fwd+bwd B=16 NH=8 S=4096 D=256 bf16, fp32 accumulate"


def algorithmic_flops(B, NH, S, D):
    """Causal pairs P = S(S+1)/2 per slice, 2*D flops per pair and contraction; forward 2
    contractions, backward 5 (QK^T recompute, dH V^T, dV, dQ, dK)."""
    pairs = S * (S + 1) // 2
    return 4 * D * pairs * B * NH, 10 * D * pairs * B * NH


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return dict(burst=float(p["bf16_tflops"]), sustained=float(p["bf16_tflops_sustained"]),
                    hbm_gbs=float(p["hbm_gbs"]), source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm_gbs=6650.0, source="fallback")


def config_for(world, B):
    """The `config` object, identical in both arms."""
    full = B == CFG["B"]
    return {"workload": WORKLOAD4 if full else "cfg4 shape at a reduced batch B=%d (profiler case, not the benchmark)" % B,
            "global_batch": B, "heads": CFG["NH"], "seq_len": CFG["S"], "head_dim": CFG["D"],
            "parallelism": f"{B * CFG['NH']} (batch, head) slices split contiguously over {world} GPU(s), no collective",
            "l2": "inputs (1.08 GB per step over all ranks) larger than L2; secondary workloads that fit in L2 flush it"}


class ClockSampler:
    """SM clock and throttle-reason samples taken in-process through NVML while the timed region runs
    (two light queries every 10 ms; a polling nvidia-smi process disturbed sub-millisecond kernels)."""
    # NVML clocks-event bits; the last three are not throttling, but they explain a clock below the maximum
    # (a clock limit somebody set on the device, a boost group, a display setting)
    REASONS = (("hw_slowdown", 0x8), ("sw_power_cap", 0x4), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40),
               ("hw_power_brake_slowdown", 0x80), ("applications_clocks_setting", 0x2), ("sync_boost", 0x10),
               ("display_clock_setting", 0x100))

    def __init__(self, index):
        self.index, self.samples, self.stop_flag, self.thread = int(index), [], False, None
        self.nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.index
            if vis:
                entry = vis.split(",")[self.index].strip()
                idx = int(entry) if entry.isdigit() else self.index
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.nvml = pynvml
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nvml = None
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _loop(self):
        n = self.nvml
        while not self.stop_flag:
            try:
                clk = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                reasons = int(n.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                self.samples.append((time.time(), clk, reasons))
            except Exception:
                pass
            time.sleep(0.010)

    def window(self, lo, hi):
        """Summary of the samples taken between two wall-clock times."""
        if self.nvml is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"], "samples": 0}
        sm, seen = [], set()
        for ts, clk, reasons in list(self.samples):
            if not (lo <= ts <= hi + 0.03):
                continue
            sm.append(clk)
            for name, bit in self.REASONS:
                if reasons & bit:
                    seen.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.sm_max, "reasons": sorted(seen),
                "samples": len(sm)}

    def stop(self):
        if self.nvml is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_oracle_step(slices, threads, f_mean=3.0):
    """Forward + closed-form backward of the CPU oracle (fp32) on `slices` (b,h) slices of the
    workload; returns seconds."""
    import torch
    from oracle import mlstm_oracle as orc
    torch.set_num_threads(threads)
    S, D = CFG["S"], CFG["D"]
    g = torch.Generator().manual_seed(0)
    mk = lambda *s: torch.randn(*s, generator=g)
    q, k, v = ((mk(1, slices, S, D) * D ** -0.5).bfloat16() for _ in range(3))
    f, i = (f_mean + mk(1, slices, S)).bfloat16(), mk(1, slices, S).bfloat16()
    dh = mk(1, slices, S, D).bfloat16()
    t0 = time.perf_counter()
    for s in range(slices):  # one slice at a time: the S x S temporaries are 64 MB each
        sl = lambda t: t[:, s:s + 1]
        orc.matmul_forward(sl(q), sl(k), sl(v), sl(f), sl(i), dtype=torch.float32)
        orc.matmul_backward(sl(dh), sl(q), sl(k), sl(v), sl(f), sl(i), dtype=torch.float32)
    return time.perf_counter() - t0


def run_reference(args, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sample_slices = 1
    times = []
    for s in range(args.warmup + args.steps):
        dt = cpu_oracle_step(sample_slices, threads)
        if s >= args.warmup:
            times.append(dt)
    tokens_per_slice = CFG["S"] / CFG["NH"]  # a token is one (batch, position) over all heads
    per_step = sum(times) / len(times)
    value = sample_slices * tokens_per_slice / per_step
    sample = (f"{sample_slices} of {CFG['B'] * CFG['NH']} (batch, head) slices per step (the rate per slice does not depend "
              "on how many are run), fp32 on bf16-rounded inputs; the reference's own Python path has no build to carry "
              "to this box, so this is the oracle port of it")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_for(args.gpus, CFG["B"]),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------------ helpers
class Ctx:
    def __init__(self, local_rank, rank, world):
        import importlib
        import torch
        self.torch = torch
        self.pkg = importlib.import_module(PKG_NAME)
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
        torch.cuda.set_device(local_rank)
        self.dev = torch.device("cuda", local_rank)
        self.rank, self.world, self.dist = rank, world, None
        if world > 1:
            import torch.distributed as dist
            # the one collective here is a 0.5 MB all-gather: in-switch multicast buys nothing, and without it no rank's
            # memory is bound to a multicast object if another rank dies
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        self.peaks = measured_peaks()
        self.flush = None

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def flush_l2(self):
        if self.flush is None:
            self.flush = self.torch.empty(256 << 20, dtype=self.torch.uint8, device=self.dev)
        self.flush.zero_()

    def max_over_ranks(self, values):
        t = self.torch.tensor(values, device=self.dev, dtype=self.torch.float64)
        if self.dist is not None:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()


L2_BYTES = 126e6   # B200: inputs smaller than this are flushed out of L2 between timed iterations


def time_small(ctx, fn, iters=10, warmup=3, flush=True):
    """Mean CUDA-event time (ms) of fn() over `iters` calls, max over ranks.  flush: L2 is flushed before every call
    and every call is timed by itself (workloads that fit in L2)."""
    torch = ctx.torch
    for _ in range(warmup):
        fn()
    if not flush:
        # inputs larger than L2: the calls run back to back inside one timed region
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx.barrier()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        ctx.barrier()
        return ctx.max_over_ranks([e0.elapsed_time(e1) / iters])[0]
    total = 0.0
    for _ in range(iters):
        if flush:
            ctx.flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx.barrier()
        e0.record()
        fn()
        e1.record()
        ctx.barrier()
        total += e0.elapsed_time(e1)
    return ctx.max_over_ranks([total / iters])[0]


def cfg4_inputs(torch, batches, f_mean=3.0):
    """The global problem is defined batch by batch (generator seeded with 1234 + batch index), so that any
    rank can make exactly its own part of it."""
    NH, S, D = CFG["NH"], CFG["S"], CFG["D"]
    out = {k: [] for k in ("q", "k", "v", "f", "i", "dh")}
    for b in batches:
        g = torch.Generator().manual_seed(1234 + b)
        mk = lambda *s: torch.randn(*s, generator=g)
        out["q"].append((mk(1, NH, S, D) * D ** -0.5).bfloat16())
        out["k"].append((mk(1, NH, S, D) * D ** -0.5).bfloat16())
        out["v"].append((mk(1, NH, S, D) * D ** -0.5).bfloat16())
        out["f"].append((f_mean + mk(1, NH, S)).bfloat16())
        out["i"].append(mk(1, NH, S).bfloat16())
        out["dh"].append(mk(1, NH, S, D).bfloat16())
    return {k: torch.cat(v, 0).contiguous() for k, v in out.items()}


def roofline_tensor(ctx, flops, ms, clocks=None, region_s=None):
    """Achieved TFLOP/s against both measured peaks.  `frac` is the burst one when the timed region is short
    and ran at an unthrottled clock (numerator and denominator then share a clock regime), else the sustained one."""
    p = ctx.peaks
    ach = flops / (ms * 1e-3) / 1e12
    burst_regime = True
    if region_s is not None and region_s >= 1.0:
        burst_regime = False
    if clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz") and clocks["sm_mhz"] < 0.97 * clocks["sm_max_mhz"]:
        burst_regime = False
    peak = p["burst"] if burst_regime else p["sustained"]
    return {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
            "frac_burst": ach / p["burst"], "frac_sustained": ach / p["sustained"],
            "peak_source": f"{p['source']} bf16 cuBLAS, {'burst' if burst_regime else 'sustained'} figure"}


def roofline_hbm(ctx, nbytes, ms):
    p = ctx.peaks
    ach = nbytes / (ms * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": ach, "peak": p["hbm_gbs"], "unit": "GB/s", "frac": ach / p["hbm_gbs"],
            "peak_source": f"{p['source']} copy"}


# ------------------------------------------------------------------------------------------------ secondary workloads
def sec_cfg1(ctx):
    """C++ driver single-head fp16 forward, S=640, D=128, U[-1,1) inputs; parity: the C restatement of mlstmCpu."""
    torch, pkg, dev = ctx.torch, ctx.pkg, ctx.dev
    import numpy as np
    S, D = 640, 128
    g = torch.Generator().manual_seed(100)
    u = lambda *s: (torch.rand(*s, generator=g) * 2 - 1).half()
    host = {"q": u(S, D), "k": u(S, D), "v": u(S, D), "f": u(S), "i": u(S)}
    d = {k: v.to(dev) for k, v in host.items()}
    L = pkg._lib.lib()
    ws = pkg._lib.workspace(L.mlstm_forward_f16_workspace(S, D), dev)
    hbuf = torch.empty(S, D, dtype=torch.float16, device=dev)

    def fn():
        rc = L.mlstm_forward_f16(d["q"].data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(), d["f"].data_ptr(), d["i"].data_ptr(),
                                 hbuf.data_ptr(), S, D, ws.data_ptr(), ws.numel(), pkg._lib.stream_ptr(dev))
        pkg._lib.check(rc, "mlstm_forward_f16")
    ms = time_small(ctx, fn)
    out = {"workload": "cfg1: C++ driver single-head fp16 forward S=640 D=128", "ms": ms, "value": S / (ms * 1e-3),
           "unit": "tokens/s", "roofline": roofline_tensor(ctx, 4 * D * (S * (S + 1) // 2), ms),
           "note": "5 row tiles of work on 148 SMs: latency-bound by construction"}
    if ctx.rank == 0:
        lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "libmlstm_oracle.so"))
        arrs = [host[k].float().numpy().copy() for k in ("q", "k", "v", "f", "i")]
        H = np.zeros((S, D), dtype=np.float32)
        p = lambda a_: a_.ctypes.data_as(ctypes.c_void_p)
        t0 = time.perf_counter()
        lib.mlstm_cpu_forward(*[p(a_) for a_ in arrs], p(H), ctypes.c_uint(S), ctypes.c_uint(D), ctypes.c_int(1))
        dt = time.perf_counter() - t0
        diff = np.abs(hbuf.float().cpu().numpy() - H)
        out["parity_max_abs_rel"] = float(diff.max() / np.abs(H).max())
        out["parity_elements_beyond_0.01"] = int((diff > 0.01).sum())
        out["cpu_baseline"] = {"value": S / dt, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
                               "sample": f"whole workload, C restatement of mlstmCpu, {dt:.3f} s"}
    return out


def sec_cfg2(ctx):
    """The reference demo of the matmul path: fp32, B=1, NH=4, S=2048, D=64, through Triton_mLSTM.apply + backward."""
    torch, pkg, dev = ctx.torch, ctx.pkg, ctx.dev
    from oracle import mlstm_oracle as orc
    B, NH, S, D = 1, 4, 2048, 64
    g = torch.Generator().manual_seed(0)
    mk = lambda *s: torch.randn(*s, generator=g)
    host = {"q": mk(B, NH, S, D), "k": mk(B, NH, S, D), "v": mk(B, NH, S, D), "f": mk(B, NH, S), "i": mk(B, NH, S)}
    dh = mk(B, NH, S, D)
    d = {k: v.to(dev).requires_grad_(True) for k, v in host.items()}
    dhd = dh.to(dev)

    def fn():
        for t in d.values():
            t.grad = None
        h = pkg.Triton_mLSTM.apply(d["q"], d["k"], d["v"], d["f"], d["i"], 32, 8)
        h.backward(dhd)
        return h
    ms = time_small(ctx, fn)
    ff, fb = algorithmic_flops(B, NH, S, D)
    out = {"workload": "cfg2: Triton_mLSTM.apply + backward, fp32, B=1 NH=4 S=2048 D=64, SB=32", "ms": ms,
           "value": B * S / (ms * 1e-3), "unit": "tokens/s", "roofline": roofline_tensor(ctx, ff + fb, ms),
           "math": pkg.fp32_math_mode(D)}
    if ctx.rank == 0:
        h = fn().detach().cpu()
        ref_h = orc.matmul_forward(*(host[k] for k in ("q", "k", "v", "f", "i")))
        ref_g = orc.matmul_backward(dh, *(host[k] for k in ("q", "k", "v", "f", "i")))
        errs = {"h": orc.max_abs_rel(h, ref_h)}
        for n, r in zip(("q", "k", "v", "f", "i"), ref_g):
            errs["d" + n] = orc.max_abs_rel(d[n].grad.cpu(), r)
        out["parity_max_abs_rel"] = max(errs.values())
        out["parity_by_output"] = errs
    return out


def sec_wide_head(ctx):
    """Head dimension above 256 in the matmul path (not one of the named configurations): bf16, B=4, NH=8, S=2048,
    D=512 through Triton_mLSTM.apply + backward; both directions take the two-pass tensor-core form."""
    torch, pkg, dev = ctx.torch, ctx.pkg, ctx.dev
    from oracle import mlstm_oracle as orc
    B, NH, S, D = 4, 8, 2048, 512
    g = torch.Generator().manual_seed(0)
    mk = lambda *s: torch.randn(*s, generator=g)
    host = {"q": (mk(B, NH, S, D) * D ** -0.5).bfloat16(), "k": (mk(B, NH, S, D) * D ** -0.5).bfloat16(),
            "v": (mk(B, NH, S, D) * D ** -0.5).bfloat16(), "f": (3.0 + mk(B, NH, S)).bfloat16(), "i": mk(B, NH, S).bfloat16()}
    dh = mk(B, NH, S, D)
    d = {k: v.to(dev).requires_grad_(True) for k, v in host.items()}
    dhd = dh.to(dev)

    def fn():
        for t in d.values():
            t.grad = None
        h = pkg.Triton_mLSTM.apply(d["q"], d["k"], d["v"], d["f"], d["i"], 32, 8)
        h.backward(dhd)
        return h
    ms = time_small(ctx, fn)
    ff, fb = algorithmic_flops(B, NH, S, D)
    out = {"workload": "Triton_mLSTM.apply + backward, bf16, B=4 NH=8 S=2048 D=512 (two-pass form in both directions)",
           "ms": ms, "value": B * S / (ms * 1e-3), "unit": "tokens/s", "roofline": roofline_tensor(ctx, ff + fb, ms)}
    if ctx.rank == 0:
        h = fn().detach()
        sl = (slice(1, 2), slice(3, 4))     # one (batch, head) slice against the oracle
        one = {k: v[sl] for k, v in host.items()}
        ref_h = orc.matmul_forward(*(one[k] for k in ("q", "k", "v", "f", "i")))
        ref_g = orc.matmul_backward(dh[sl], *(one[k] for k in ("q", "k", "v", "f", "i")))
        errs = {"h": orc.max_abs_rel(h[sl].cpu(), ref_h)}
        for n, r in zip(("q", "k", "v", "f", "i"), ref_g):
            errs["d" + n] = orc.max_abs_rel(d[n].grad[sl].float().cpu(), r)
        out["parity_max_abs_rel"] = max(errs.values())
        out["parity_sample"] = "slice (batch 1, head 3); tolerance 1e-2"
    return out


def sec_cfg5_train(ctx, S=65536):
    """Configuration 5's shape with gradients: chunkwise forward + chunkwise backward through mlstm_chunkwise's autograd
    (one GPU).  Parity: dq depends on the past only, so dq of the first 2048 positions of head 0 is compared with the
    closed-form backward of the oracle on that prefix."""
    torch, pkg, dev = ctx.torch, ctx.pkg, ctx.dev
    from oracle import mlstm_oracle as orc
    B, NH, D, L = 1, 8, 128, 256
    host = cfg5_segment(torch, S, 1, 0)
    g = torch.Generator().manual_seed(5)
    dh = torch.randn(B, NH, S, D, generator=g)
    d = {k: v.to(dev).requires_grad_(True) for k, v in host.items()}
    dhd = dh.to(dev)

    def fn():
        for t in d.values():
            t.grad = None
        h = pkg.mlstm_chunkwise(d["q"], d["k"], d["v"], d["f"], d["i"], chunk_size=L)
        h.backward(dhd)
        return h
    ms = time_small(ctx, fn)
    # credited like the parallel form: 2 contractions forward, 5 backward, each intra-block (triangles) + state part
    intra = 2 * D * (L * (L + 1) // 2) * (S // L)
    inter = 2 * S * D * D
    flops = (2 + 5) * (intra + inter) * B * NH
    out = {"workload": f"chunkwise forward + backward bf16 B=1 NH=8 S={S} D=128 chunk 256 (mlstm_chunkwise autograd)", "ms": ms,
           "value": B * S / (ms * 1e-3), "unit": "tokens/s", "roofline": roofline_tensor(ctx, flops, ms)}
    if ctx.rank == 0:
        fn()
        n = 2048
        one = {k: v[:, :1, :n] for k, v in host.items()}
        ref = orc.matmul_backward(dh[:, :1, :n], *(one[k] for k in ("q", "k", "v", "f", "i")))
        out["parity_max_abs_rel"] = orc.max_abs_rel(d["q"].grad[:, :1, :n].float().cpu(), ref[0])
        out["parity_sample"] = "dq of head 0, positions [0, 2048), against the oracle's closed-form backward of that prefix"
    return out


def sec_cfg3(ctx):
    """The reference demo of the scan path: fp32, B=1, NH=4, S=2048, D=1024 with output gate."""
    torch, pkg, dev = ctx.torch, ctx.pkg, ctx.dev
    from oracle import mlstm_oracle as orc
    B, NH, S, D = 1, 4, 2048, 1024
    g = torch.Generator().manual_seed(0)
    mk = lambda *s: torch.randn(*s, generator=g)
    host = {"q": mk(B, NH, S, D), "k": mk(B, NH, S, D), "v": mk(B, NH, S, D), "f": mk(B, NH, S), "i": mk(B, NH, S),
            "o": mk(B, NH, S, D)}
    d = {k: v.to(dev) for k, v in host.items()}
    fn = lambda: pkg.mlstm_scan(d["q"], d["k"], d["v"], d["f"], d["i"], d["o"], reduce_block_size=4, value_block_size=4)
    in_bytes = sum(t.numel() * t.element_size() for t in d.values())
    ms = time_small(ctx, fn, flush=in_bytes < L2_BYTES)   # 167.8 MB of inputs: larger than L2, no flush needed
    nbytes = (5 * B * NH * S * D + 2 * B * NH * S) * 4          # q, k, v, o read + h written once, fp32
    flops = 4 * D * (S * (S + 1) // 2) * B * NH
    out = {"workload": "cfg3: mlstm_scan forward with output gate, fp32, B=1 NH=4 S=2048 D=1024", "ms": ms,
           "value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "roofline": roofline_hbm(ctx, nbytes, ms),
           "tensor_tflops": flops / (ms * 1e-3) / 1e12,
           "l2": "inputs (167.8 MB) larger than L2: no flush between iterations",
           "math": "tf32 operands (fp32 read as tf32, gated matrix rounded to tf32), fp32 accumulate"}
    if ctx.rank == 0:
        hd = 2
        h = fn()[:, hd].cpu()
        ref = orc.scan_forward(*(host[k][:, hd] for k in ("q", "k", "v", "f", "i", "o")), dtype=torch.float64)
        out["parity_max_abs_rel"] = orc.max_abs_rel(h, ref)
        out["parity_check_fail_fraction"] = orc.check(h, ref)[1]
        out["parity_sample"] = "head 2 of 4 against the recurrent oracle (one step per time index, fp64)"
        steps_cpu = 96
        sl = {k: v[:, :1, :steps_cpu] for k, v in host.items()}
        t0 = time.perf_counter()
        orc.scan_forward(sl["q"], sl["k"], sl["v"], sl["f"], sl["i"], sl["o"], dtype=torch.float32)
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": nbytes * (steps_cpu / (NH * S)) / dt / 1e9, "unit": "GB/s", "cores": os.cpu_count() or 1,
                               "kind": "port", "sample": f"{steps_cpu} time steps of one head of the recurrent oracle, {dt:.2f} s"}
    return out


def cfg5_segment(torch, S, world, r, heads=slice(None)):
    """Segment r of `world` of the long sequence (all heads, or a selection): seeded per segment so that any
    rank can rebuild any part of the sequence."""
    B, NH, D = 1, 8, 128
    n = S // world
    g = torch.Generator().manual_seed(5000 + 97 * world + r)
    mk = lambda *s: torch.randn(*s, generator=g)
    x = {"q": (mk(B, NH, n, D) * D ** -0.5).bfloat16(), "k": (mk(B, NH, n, D) * D ** -0.5).bfloat16(),
         "v": (mk(B, NH, n, D) * D ** -0.5).bfloat16(), "f": (3.0 + mk(B, NH, n)).bfloat16(), "i": mk(B, NH, n).bfloat16()}
    return {k: v[:, heads].contiguous() for k, v in x.items()}


def sec_cfg5(ctx, S=65536, parity=True):
    """Long-context chunkwise forward, bf16, B=1, NH=8, D=128, chunk 256; sequence-parallel for N > 1 (rank r holds
    the r-th contiguous segment).  Parity is taken on the LAST rank's segment, whose result depends on every carry."""
    torch, pkg, dev = ctx.torch, ctx.pkg, ctx.dev
    from oracle import mlstm_oracle as orc
    B, NH, D, L = 1, 8, 128, 256
    n = S // ctx.world
    d = {k: v.to(dev) for k, v in cfg5_segment(torch, S, ctx.world, ctx.rank).items()}
    if ctx.world > 1:
        fn = lambda: pkg.mlstm_chunkwise_sequence_parallel(d["q"], d["k"], d["v"], d["f"], d["i"], chunk_size=L,
                                                           h_dtype=torch.bfloat16)
    else:
        fn = lambda: pkg.mlstm_chunkwise(d["q"], d["k"], d["v"], d["f"], d["i"], chunk_size=L, h_dtype=torch.bfloat16)
    ms = time_small(ctx, fn)
    flops = (4 * D * (L * (L + 1) // 2) * (S // L) + 4 * S * D * D) * B * NH      # intra + inter, whole job
    out = {"workload": f"cfg5: chunkwise mLSTM forward bf16 B=1 NH=8 S={S} D=128 chunk 256"
                       + (f", sequence-parallel over {ctx.world} GPUs (one all-gather of 0.53 MB per rank)" if ctx.world > 1 else ""),
           "ms": ms, "value": B * S / (ms * 1e-3), "unit": "tokens/s"}
    # q, k, v read and h written once (16-bit), f and i read: at this head dimension the chunkwise form is bound by
    # memory (539 MB against 68.9 GFLOP: 82 us at the measured copy rate, 42 us at the measured tensor rate)
    nbytes = (4 * B * NH * S * D + 2 * B * NH * S) * 2
    out["roofline"] = roofline_hbm(ctx, nbytes / ctx.world, ms)
    out["roofline_tensor"] = roofline_tensor(ctx, flops / ctx.world, ms)
    if parity:
        err = 0.0
        h = fn().float().cpu()
        if ctx.rank == ctx.world - 1:
            segs = [cfg5_segment(torch, S, ctx.world, r, heads=slice(0, 1)) for r in range(ctx.world)]
            x = {k: torch.cat([sg[k] for sg in segs], 2) for k in segs[0]}
            one = torch.full(x["q"].shape, 1.2784645, dtype=torch.float32)        # silu(1.2784645...) = 1
            ref = orc.scan_forward(x["q"], x["k"], x["v"], x["f"], x["i"], one, dtype=torch.float64)
            ref = ref / torch.nn.functional.silu(torch.tensor(1.2784645, dtype=torch.float64))
            base = S - n
            spots = sorted({0, (n // L // 2) * L, n - L})
            err = max(orc.max_abs_rel(h[:, :1, lo:lo + L], ref[:, :, base + lo:base + lo + L]) for lo in spots)
            out["parity_sample"] = (f"head 0 of the last segment (positions [{base}, {S})) against the recurrent oracle "
                                    f"(fp64, one step per time index, run over the whole sequence), compared on the "
                                    f"blocks starting at {[base + lo for lo in spots]}")
        out["parity_max_abs_rel"] = ctx.max_over_ranks([err])[0]
    return out


def sec_cfg4_parity(ctx):
    """Four (batch, head) slices spread over the batch of the timed problem (f ~ N(3,1)) and four slices with
    f ~ N(0,1), forward + backward against the fp32 CPU oracle on the same bf16-rounded inputs."""
    torch, pkg, dev = ctx.torch, ctx.pkg, ctx.dev
    from oracle import mlstm_oracle as orc
    out = {}
    for regime, f_mean in (("f~N(3,1)", 3.0), ("f~N(0,1)", 0.0)):
        host = cfg4_inputs(torch, [0, 5, 10, 15], f_mean=f_mean)
        d = {k: v.to(dev) for k, v in host.items()}
        h, m, b = pkg.mlstm_matmul_forward(d["q"], d["k"], d["v"], d["f"], d["i"], h_dtype=torch.bfloat16)
        grads = pkg.mlstm_matmul_backward(d["dh"], d["q"], d["k"], d["v"], d["f"], d["i"], h, m, b)
        worst = {}
        for bi, hd in ((0, 0), (1, 3), (2, 5), (3, 7)):
            sl = {k: v[bi:bi + 1, hd:hd + 1] for k, v in host.items()}
            rh = orc.matmul_forward(sl["q"], sl["k"], sl["v"], sl["f"], sl["i"], dtype=torch.float32)
            rg = orc.matmul_backward(sl["dh"], sl["q"], sl["k"], sl["v"], sl["f"], sl["i"], dtype=torch.float32)
            errs = {"h": orc.max_abs_rel(h[bi:bi + 1, hd:hd + 1].float(), rh)}
            for n, got, r in zip(("dq", "dk", "dv", "df", "di"), grads, rg):
                errs[n] = orc.max_abs_rel(got[bi:bi + 1, hd:hd + 1].float(), r)
            for n, e in errs.items():
                worst[n] = max(worst.get(n, 0.0), e)
        out[regime] = worst
    return {"parity_max_abs_rel": max(max(v.values()) for v in out.values()), "by_regime": out,
            "parity_sample": "slices (batch 0, head 0), (5, 3), (10, 5), (15, 7) per regime; tolerance 1e-2"}


def run_workload(args, ctx):
    """One configuration alone, printed as one line (profiler captures and ad-hoc runs)."""
    fn = {"cfg1": sec_cfg1, "cfg2": sec_cfg2, "cfg3": sec_cfg3, "cfg5": sec_cfg5, "d512": sec_wide_head, "cfg5train": sec_cfg5_train}[args.workload]
    sec = fn(ctx) if args.workload != "cfg5" else sec_cfg5(ctx, S=args.seq or 65536)
    if ctx.rank == 0:
        line = {"metric": args.workload + "_" + sec["unit"].replace("/", "_per_"), "value": sec["value"], "unit": sec["unit"],
                "n_gpus": ctx.world, "steps": 10, "warmup": 3, "ms_per_step": sec["ms"], "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "data": "synthetic", "config": {"workload": sec["workload"]},
                "roofline": sec["roofline"], "detail": sec}
        print(json.dumps(line))


# ------------------------------------------------------------------------------------------------ headline
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary workloads (profiler captures)")
    ap.add_argument("--batch", type=int, default=None,
                    help="cfg4 only: a smaller global batch of the same shape (profiler captures); the line's config says so")
    ap.add_argument("--seq", type=int, default=None, help="cfg5 only: sequence length (default 65536)")
    ap.add_argument("--workload", default="cfg4", choices=["cfg4", "cfg5", "cfg3", "cfg2", "cfg1", "d512", "cfg5train"],
                    help="cfg4 (default, the headline); the others run one secondary configuration alone")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    ctx = Ctx(local_rank, rank, world)
    torch, pkg, dev, dist = ctx.torch, ctx.pkg, ctx.dev, ctx.dist
    if args.workload != "cfg4":
        run_workload(args, ctx)
        if dist is not None:
            dist.destroy_process_group()
        return

    B, NH, S, D = CFG["B"], CFG["NH"], CFG["S"], CFG["D"]
    if args.batch is not None:
        if not 1 <= args.batch <= CFG["B"]:
            raise SystemExit("--batch must be between 1 and %d" % CFG["B"])
        B = args.batch
    if (B * NH) % world:
        raise SystemExit("the number of ranks must divide the %d (batch, head) slices" % (B * NH))
    warmup = max(args.warmup, 3)
    # this rank's contiguous range of the global problem's flattened (batch, head) slices
    lo, hi = pkg.slice_range(B * NH, rank, world)
    n_local = hi - lo
    need = sorted({s // NH for s in range(lo, hi)})
    glob = cfg4_inputs(torch, need)
    off = need[0] * NH
    host = {k: v.reshape((1, len(need) * NH) + tuple(v.shape[2:]))[:, lo - off:hi - off].contiguous().pin_memory()
            for k, v in glob.items()}
    del glob
    d = {k: v.to(dev, non_blocking=True) for k, v in host.items()}
    torch.cuda.synchronize()

    def step(t):
        h, m, b = pkg.mlstm_matmul_forward(t["q"], t["k"], t["v"], t["f"], t["i"], h_dtype=torch.bfloat16)
        grads = pkg.mlstm_matmul_backward(t["dh"], t["q"], t["k"], t["v"], t["f"], t["i"], h, m, b)
        return (h,) + tuple(grads)

    sampler = ClockSampler(local_rank)  # started early: the first samples take a while to arrive
    sampler.start()
    h = m = b = None
    for _ in range(warmup):  # same tensor lifetimes as the timed loop, so the allocator reaches its steady state
        h, m, b = pkg.mlstm_matmul_forward(d["q"], d["k"], d["v"], d["f"], d["i"], h_dtype=torch.bfloat16)
        pkg.mlstm_matmul_backward(d["dh"], d["q"], d["k"], d["v"], d["f"], d["i"], h, m, b)
    ctx.barrier()

    # ---- device-resident timing, with separate events around the forward and the backward call
    def timed_region(steps):
        nonlocal h, m, b
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
        t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx.barrier()
        w0 = time.time()
        t_begin.record()
        for s in range(steps):
            ev[s][0].record()
            h, m, b = pkg.mlstm_matmul_forward(d["q"], d["k"], d["v"], d["f"], d["i"], h_dtype=torch.bfloat16)
            ev[s][1].record()
            pkg.mlstm_matmul_backward(d["dh"], d["q"], d["k"], d["v"], d["f"], d["i"], h, m, b)
            ev[s][2].record()
        t_end.record()
        ctx.barrier()
        w1 = time.time()
        fwd = sum(e[0].elapsed_time(e[1]) for e in ev) / steps
        bwd = sum(e[1].elapsed_time(e[2]) for e in ev) / steps
        return t_begin.elapsed_time(t_end), fwd, bwd, sampler.window(w0, w1)

    elapsed_ms, fwd_ms, bwd_ms, clocks = timed_region(args.steps)
    del h, m, b
    h = m = b = None

    # ---- end to end: pinned host buffers in, results back to pinned host buffers, every step.
    # Three streams, as a training input pipeline would run it: the inputs of step s+1 travel to the device while
    # step s computes and the results of step s-1 travel back (PCIe is full duplex; the copies dominate a step).
    # Every step's host->device and device->host copies lie inside the timed region.
    s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dev_in = [{k: torch.empty(v.shape, dtype=v.dtype, device=dev) for k, v in host.items()} for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    cmp_done = [torch.cuda.Event() for _ in range(2)]
    out_host = None
    e2e_begin, e2e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = 0
    e2e_steps = args.steps
    for s in range(1 + e2e_steps):
        if s == 1:
            ctx.barrier()
            e2e_begin.record()
            for st in (s_in, s_cmp, s_out):
                st.wait_event(e2e_begin)
        k = s & 1
        with torch.cuda.stream(s_in):
            if s >= 2:
                s_in.wait_event(cmp_done[k])          # step s-2 has read this input buffer
            for name, v in host.items():
                dev_in[k][name].copy_(v, non_blocking=True)
            in_ready[k].record(s_in)
        with torch.cuda.stream(s_cmp):
            s_cmp.wait_event(in_ready[k])
            outs = step(dev_in[k])
            cmp_done[k].record(s_cmp)
        if out_host is None:
            out_host = [torch.empty(o.shape, dtype=o.dtype, pin_memory=True) for o in outs]
            d2h = sum(o.numel() * o.element_size() for o in outs)
        with torch.cuda.stream(s_out):
            s_out.wait_event(cmp_done[k])
            for dst, src in zip(out_host, outs):
                dst.copy_(src, non_blocking=True)
                src.record_stream(s_out)              # allocated on the compute stream, read here
        del outs
    cur = torch.cuda.current_stream()
    for st in (s_in, s_cmp, s_out):
        cur.wait_stream(st)
    e2e_end.record()
    ctx.barrier()
    e2e_ms = e2e_begin.elapsed_time(e2e_end)
    del dev_in, out_host

    elapsed_ms, e2e_ms, fwd_ms, bwd_ms = ctx.max_over_ranks([elapsed_ms, e2e_ms, fwd_ms, bwd_ms])
    byte_totals = ctx.torch.tensor([float(h2d), float(d2h)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(byte_totals)
    h2d_all, d2h_all = (int(x) for x in byte_totals.tolist())

    # ---- secondary measurements (outside the headline's timed regions)
    secondary = {}
    if not args.no_secondary:
        # the same step through the drop-in autograd function: fp32 h out, fp32 dh in, as the reference's API has it
        t = {k: d[k].detach().requires_grad_(True) for k in ("q", "k", "v", "f", "i")}
        dh32 = d["dh"].float()

        def dropin():
            for x in t.values():
                x.grad = None
            hh = pkg.Triton_mLSTM.apply(t["q"], t["k"], t["v"], t["f"], t["i"], 16, 8)
            hh.backward(dh32)
        ms_dropin = time_small(ctx, dropin, iters=10, warmup=3, flush=False)
        for x in t.values():
            x.grad = None
        del t, dh32
        ff, fb = algorithmic_flops(B, NH, S, D)
        secondary["cfg4_dropin"] = {
            "workload": "the headline step through Triton_mLSTM.apply(q,k,v,f,i,SB,NUM_WARPS) + h.backward(dh): fp32 h and dh",
            "ms": ms_dropin, "value": B * S / (ms_dropin * 1e-3), "unit": "tokens/s",
            "roofline": roofline_tensor(ctx, (ff + fb) / world, ms_dropin)}
        # a longer back-to-back run: the clock settles under the board's power cap
        long_steps = max(150, args.steps)
        l_ms, l_fwd, l_bwd, l_clk = timed_region(long_steps)
        l_ms = ctx.max_over_ranks([l_ms])[0]
        h = m = b = None
        secondary["cfg4_sustained"] = {
            "workload": f"{long_steps} headline steps back to back", "ms": l_ms / long_steps,
            "value": B * S / (l_ms / long_steps * 1e-3), "unit": "tokens/s", "clocks": l_clk,
            "roofline": roofline_tensor(ctx, (ff + fb) / world, l_ms / long_steps, l_clk, l_ms * 1e-3)}
        if world > 1 and B == CFG["B"]:
            # weak scaling: every rank runs the whole configuration on its own data (what one GPU does at N = 1)
            hostw = cfg4_inputs(torch, [0, 1])   # timing only: two batches repeated to the full batch
            dw = {k: v.to(dev).repeat((CFG["B"] // 2,) + (1,) * (v.dim() - 1)).contiguous() for k, v in hostw.items()}
            del hostw

            def weak():
                hh, mm, bb = pkg.mlstm_matmul_forward(dw["q"], dw["k"], dw["v"], dw["f"], dw["i"], h_dtype=torch.bfloat16)
                pkg.mlstm_matmul_backward(dw["dh"], dw["q"], dw["k"], dw["v"], dw["f"], dw["i"], hh, mm, bb)
            ms_w = time_small(ctx, weak, iters=10, warmup=3, flush=False)
            del dw
            secondary["cfg4_weak"] = {"workload": "every rank runs the whole configuration 4 on its own data (weak scaling)",
                                      "ms": ms_w, "value": CFG["B"] * S * world / (ms_w * 1e-3), "unit": "tokens/s"}
        del d
        torch.cuda.empty_cache()
        if B == CFG["B"]:
            if rank == 0:
                secondary["cfg4_parity"] = sec_cfg4_parity(ctx)
            secondary["cfg5"] = sec_cfg5(ctx)
            if world > 1:
                secondary["cfg5_long"] = sec_cfg5(ctx, S=262144, parity=False)
            if world == 1:
                secondary["cfg1"] = sec_cfg1(ctx)
                secondary["cfg2"] = sec_cfg2(ctx)
                secondary["cfg3"] = sec_cfg3(ctx)
                secondary["cfg5_long"] = sec_cfg5(ctx, S=262144, parity=False)
                secondary["wide_head_d512"] = sec_wide_head(ctx)
                secondary["cfg5_train"] = sec_cfg5_train(ctx)
    sampler.stop()

    if rank == 0:
        tokens_per_step = B * S
        ms_per_step = elapsed_ms / args.steps
        value = tokens_per_step / (ms_per_step * 1e-3)
        e2e_value = tokens_per_step / (e2e_ms / e2e_steps * 1e-3)
        ff, fb = algorithmic_flops(B, NH, S, D)
        roof = roofline_tensor(ctx, (ff + fb) / world, fwd_ms + bwd_ms, clocks, elapsed_ms * 1e-3)
        roof.update({
            "kernel": "mlstm_tc_pass_pair (FWD, DQ, DK, DV launches of one step, with the gate passes), per GPU",
            # DRAM bytes per launch from the ncu capture in profiles/ (B=4 case, scaled by slices)
            "traffic": 1.18e9 / world, "traffic_source": "ncu, B=4 case scaled by slices, average of the four passes",
            "fwd_tflops": ff / world / (fwd_ms * 1e-3) / 1e12, "bwd_tflops": fb / world / (bwd_ms * 1e-3) / 1e12,
            "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "timed_region_s": elapsed_ms * 1e-3,
            "ms_times_mhz": (fwd_ms + bwd_ms) * clocks["sm_mhz"] if clocks.get("sm_mhz") else None})
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config_for(world, B),
            "slices_per_gpu": n_local,
            "tflops_algorithmic": (ff + fb) / (ms_per_step * 1e-3) / 1e12,
            "roofline": roof,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d_all, "d2h_bytes_per_step": d2h_all,
                    "ms_per_step": e2e_ms / e2e_steps,
                    "pipeline": "3 streams per rank: H2D of step s+1, compute of step s and D2H of step s-1 overlap; bytes summed over ranks"},
            "gpu_launches": 8 * args.steps,
            "clocks": clocks,
        }
        if secondary:
            line["secondary"] = secondary
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            cpu_oracle_step(1, threads)  # warm-up
            slices = 4
            dt = cpu_oracle_step(slices, threads)
            line["cpu_baseline"] = {"value": slices * (S / NH) / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
                                    "sample": f"{slices} of {B * NH} (batch, head) slices, fwd+bwd, fp32 on bf16-rounded inputs, {dt:.2f} s"}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
