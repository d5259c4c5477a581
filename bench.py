#!/usr/bin/env python
"""Benchmark of the mLSTM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the model-scale training step of the parallel (matmul) mLSTM, forward + backward at
B=16, NH=8, S=4096, D=256 in bf16 per GPU (seeded synthetic data: q, k, v ~ N(0, 1/D), f ~ N(3, 1),
i ~ N(0, 1), dh ~ N(0, 1)).  A "step" is one forward + backward over the whole batch.  Every
(batch, head) slice is independent, so with N GPUs every rank runs the same per-GPU batch on its
own data with no data-path collective (weak scaling); one process per GPU, launched by
torch.distributed.run for N > 1.

One JSON line is printed by rank 0.  `value` is tokens/s with inputs resident in HBM; `e2e` is the
same step through the library's public entry points with pinned HOST buffers, the host->device
copies of the inputs and the device->host copies of the results inside the timed region.

`--impl reference` times the CPU path (the oracle port of the reference's PyTorch functions, since the
reference's Python cannot travel to the GPU box) on the host cores on a bounded sample.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(B=16, NH=8, S=4096, D=256)
METRIC = "mlstm_matmul_fwd_bwd_tokens_per_s"


def algorithmic_flops(B, NH, S, D):
    """Causal pairs P = S(S+1)/2 per slice, 2*D flops per pair and contraction; forward 2
    contractions, backward 5 (QK^T recompute, dH V^T, dV, dQ, dK)."""
    pairs = S * (S + 1) // 2
    fwd = 4 * D * pairs * B * NH
    bwd = 10 * D * pairs * B * NH
    return fwd, bwd


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return dict(tflops=float(p["bf16_tflops_sustained"]), hbm_gbs=float(p["hbm_gbs"]), source="measured (sustained)")
    return dict(tflops=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """SM clock and throttle-reason samples taken in-process through NVML while the timed region runs
    (two light queries every 10 ms; a polling nvidia-smi process disturbed sub-millisecond kernels)."""
    REASONS = (("hw_slowdown", 0x8), ("sw_power_cap", 0x4), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40))

    def __init__(self, index):
        self.index, self.samples, self.stop_flag, self.thread = int(index), [], False, None
        self.window = [None, None]  # wall-clock bounds of the timed region
        self.nvml = None

    def mark(self, which):
        self.window[which] = time.time()

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

    def stop(self):
        if self.nvml is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"], "samples": 0}
        self.stop_flag = True
        self.thread.join(timeout=2)
        lo, hi = self.window
        sm, seen = [], set()
        for ts, clk, reasons in self.samples:
            if lo is not None and hi is not None and not (lo <= ts <= hi + 0.03):
                continue
            sm.append(clk)
            for name, bit in self.REASONS:
                if reasons & bit:
                    seen.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.sm_max, "reasons": sorted(seen),
                "samples": len(sm)}


def cpu_oracle_step(slices, threads):
    """Forward + closed-form backward of the CPU oracle (fp32) on `slices` (b,h) slices of the
    workload; returns seconds."""
    import torch
    from oracle import mlstm_oracle as orc
    torch.set_num_threads(threads)
    S, D = CFG["S"], CFG["D"]
    g = torch.Generator().manual_seed(0)
    mk = lambda *s: torch.randn(*s, generator=g)
    q, k, v = ((mk(1, slices, S, D) * D ** -0.5).bfloat16() for _ in range(3))
    f, i = (3.0 + mk(1, slices, S)).bfloat16(), mk(1, slices, S).bfloat16()
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
    sample = f"{sample_slices} of {CFG['B'] * CFG['NH']} (batch, head) slices per step, fp32 on bf16-rounded inputs"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "cfg4: mLSTM matmul fwd+bwd B=16 NH=8 S=4096 D=256 bf16", "sample": sample},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_forward_workload(args, rank, world, local_rank):
    """The forward-only configurations, same JSON contract as the headline workload."""
    import ctypes
    import importlib
    import torch
    from oracle import mlstm_oracle as orc
    pkg = importlib.import_module("xlstm-triton-cuda-implementation_b200")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    g = torch.Generator().manual_seed(0)
    mk = lambda *s: torch.randn(*s, generator=g)
    peaks = measured_peaks()
    name = args.workload
    scaling = "weak"
    if name == "cfg5":
        B, NH, S, D = 1, 8, 65536, 128
        full = {"q": (mk(B, NH, S, D) * D ** -0.5).bfloat16(), "k": (mk(B, NH, S, D) * D ** -0.5).bfloat16(),
                "v": (mk(B, NH, S, D) * D ** -0.5).bfloat16(), "f": (3.0 + mk(B, NH, S)).bfloat16(), "i": mk(B, NH, S).bfloat16()}
        a, b = rank * S // world, (rank + 1) * S // world   # contiguous segment of this rank
        host = {k: v[:, :, a:b].contiguous() for k, v in full.items()}
        scaling = "strong"
        if world > 1:
            fn = lambda t: pkg.mlstm_chunkwise_sequence_parallel(t["q"], t["k"], t["v"], t["f"], t["i"], chunk_size=256,
                                                                 h_dtype=torch.bfloat16)
        else:
            fn = lambda t: pkg.mlstm_chunkwise(t["q"], t["k"], t["v"], t["f"], t["i"], chunk_size=256, h_dtype=torch.bfloat16)
        L = 256
        flops = (4 * D * (L * (L + 1) // 2) * (S // L) + 4 * S * D * D) * B * NH      # intra + inter, whole job
        units, unit, metric = B * S, "tokens/s", "mlstm_chunkwise_fwd_tokens_per_s"
        workload = "cfg5: chunkwise mLSTM forward B=1 NH=8 S=65536 D=128 bf16, chunk 256"
        bound, alg = "tensor", flops
        launches = 5 if world == 1 else 7
    elif name == "cfg3":
        B, NH, S, D = 1, 4, 2048, 1024
        host = {"q": mk(B, NH, S, D), "k": mk(B, NH, S, D), "v": mk(B, NH, S, D), "f": mk(B, NH, S), "i": mk(B, NH, S),
                "o": mk(B, NH, S, D)}
        fn = lambda t: pkg.mlstm_scan(t["q"], t["k"], t["v"], t["f"], t["i"], t["o"], reduce_block_size=4, value_block_size=4)
        alg = (5 * B * NH * S * D + 2 * B * NH * S) * 4                                   # 4 reads + 1 write, fp32
        units, unit, metric = alg / 1e9, "GB/s", "mlstm_scan_fwd_GB_per_s"
        workload = "cfg3: mLSTM scan forward with output gate B=1 NH=4 S=2048 D=1024 fp32"
        bound = "hbm"
        launches = 2
    else:
        S, D = 640, 128
        u = lambda *s: (torch.rand(*s, generator=g) * 2 - 1).half()
        host = {"q": u(S, D), "k": u(S, D), "v": u(S, D), "f": u(S), "i": u(S)}
        L_ = pkg._lib.lib()
        ws = pkg._lib.workspace(L_.mlstm_forward_f16_workspace(S, D), dev)
        hbuf = torch.empty(S, D, dtype=torch.float16, device=dev)

        def fn(t):
            rc = L_.mlstm_forward_f16(t["q"].data_ptr(), t["k"].data_ptr(), t["v"].data_ptr(), t["f"].data_ptr(),
                                      t["i"].data_ptr(), hbuf.data_ptr(), S, D, ws.data_ptr(), ws.numel(),
                                      pkg._lib.stream_ptr(dev))
            pkg._lib.check(rc, "mlstm_forward_f16")
            return hbuf
        alg = 4 * D * (S * (S + 1) // 2)
        units, unit, metric = S, "tokens/s", "mlstm_forward_f16_tokens_per_s"
        workload = "cfg1: C++ driver single-head fp16 forward S=640 D=128"
        bound = "tensor"
        launches = 2
    host = {k: v.pin_memory() for k, v in host.items()}
    d = {k: v.to(dev) for k, v in host.items()}
    small = sum(v.numel() * v.element_size() for v in host.values()) < 200e6
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if small else None

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    warmup = max(args.warmup, 3)
    out = None
    for _ in range(warmup):
        out = fn(d)          # held like in the timed loop, so the allocator reaches its steady state
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    sampler.mark(0)
    total_ms = 0.0
    for _ in range(args.steps):
        if flush is not None:
            flush.zero_()                       # inputs fit in L2: flush it between timed iterations
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        out = fn(d)
        e1.record()
        barrier()
        total_ms += e0.elapsed_time(e1)
    sampler.mark(1)
    clocks = sampler.stop()
    out_host = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
    e2e_ms = 0.0
    for _ in range(args.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        t = {k: v.to(dev, non_blocking=True) for k, v in host.items()}
        out_host.copy_(fn(t), non_blocking=True)
        e1.record()
        barrier()
        e2e_ms += e0.elapsed_time(e1)
    times = torch.tensor([total_ms, e2e_ms], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = times.tolist()
    if rank == 0:
        ms = total_ms / args.steps
        value = units / (ms * 1e-3)
        if bound == "tensor":
            achieved, peak, runit = alg / (ms * 1e-3) / 1e12, peaks["tflops"], "TFLOP/s"
        else:
            achieved, peak, runit = alg / (ms * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
        line = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": warmup,
                "ms_per_step": ms, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
                "dtype": {"cfg5": "bf16", "cfg3": "f32", "cfg1": "f16"}[name], "data": "synthetic",
                "config": {"workload": workload, "l2": "L2 flushed between timed iterations" if small else "inputs larger than L2"},
                "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": runit, "frac": achieved / peak,
                             "peak_source": peaks["source"], "traffic": None},
                "e2e": {"value": units / (e2e_ms / args.steps * 1e-3), "unit": unit,
                        "h2d_bytes_per_step": sum(v.numel() * v.element_size() for v in host.values()),
                        "d2h_bytes_per_step": out_host.numel() * out_host.element_size()},
                "gpu_launches": launches * args.steps, "clocks": clocks}
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            torch.set_num_threads(threads)
            if name == "cfg1":
                lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "libmlstm_oracle.so"))
                arrs = [host[k].float().numpy().copy() for k in ("q", "k", "v", "f", "i")]
                import numpy as np
                H = np.zeros((S, D), dtype=np.float32)
                p = lambda a_: a_.ctypes.data_as(ctypes.c_void_p)
                t0 = time.perf_counter()
                lib.mlstm_cpu_forward(*[p(a_) for a_ in arrs], p(H), ctypes.c_uint(S), ctypes.c_uint(D), ctypes.c_int(1))
                dt = time.perf_counter() - t0
                line["cpu_baseline"] = {"value": S / dt, "unit": unit, "cores": threads, "kind": "port",
                                        "sample": f"whole workload, C restatement of mlstmCpu with OpenMP, {dt:.3f} s"}
            else:
                steps_cpu = 96   # recurrent oracle, one head, a bounded number of time steps
                sl = {k: v[:, :1, :steps_cpu].float() for k, v in host.items()}
                o = sl.get("o", torch.zeros_like(sl["q"]))
                t0 = time.perf_counter()
                orc.scan_forward(sl["q"], sl["k"], sl["v"], sl["f"], sl["i"], o, dtype=torch.float32)
                dt = time.perf_counter() - t0
                frac = steps_cpu / (host["q"].shape[1] * host["q"].shape[2])   # of all (head, position) pairs
                line["cpu_baseline"] = {"value": units * frac / dt, "unit": unit, "cores": threads, "kind": "port",
                                        "sample": f"{steps_cpu} time steps of one head of the recurrent oracle, {dt:.2f} s"}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=None,
                    help="cfg4 only: a smaller batch of the same shape (profiler captures); the line's config says so")
    ap.add_argument("--workload", default="cfg4", choices=["cfg4", "cfg5", "cfg3", "cfg1"],
                    help="cfg4 (default, the headline): matmul fwd+bwd; cfg5: chunkwise forward S=65536, "
                         "sequence-parallel for N>1; cfg3: scan forward fp32 D=1024; cfg1: C++ single-head fp16 forward")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload != "cfg4":
        run_forward_workload(args, rank, world, local_rank)
        return

    import importlib
    import torch
    pkg = importlib.import_module("xlstm-triton-cuda-implementation_b200")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    B, NH, S, D = CFG["B"], CFG["NH"], CFG["S"], CFG["D"]
    if args.batch is not None:
        if not 1 <= args.batch <= CFG["B"]:
            raise SystemExit("--batch must be between 1 and %d" % CFG["B"])
        B = args.batch
    warmup = max(args.warmup, 3)
    g = torch.Generator().manual_seed(1234 + rank)
    mk = lambda *s: torch.randn(*s, generator=g)
    host = {
        "q": (mk(B, NH, S, D) * D ** -0.5).bfloat16(), "k": (mk(B, NH, S, D) * D ** -0.5).bfloat16(),
        "v": (mk(B, NH, S, D) * D ** -0.5).bfloat16(), "f": (3.0 + mk(B, NH, S)).bfloat16(),
        "i": mk(B, NH, S).bfloat16(), "dh": mk(B, NH, S, D).bfloat16(),
    }
    host = {k: v.pin_memory() for k, v in host.items()}
    d = {k: v.to(dev, non_blocking=True) for k, v in host.items()}
    torch.cuda.synchronize()

    def step(t):
        h, m, b = pkg.mlstm_matmul_forward(t["q"], t["k"], t["v"], t["f"], t["i"], h_dtype=torch.bfloat16)
        grads = pkg.mlstm_matmul_backward(t["dh"], t["q"], t["k"], t["v"], t["f"], t["i"], h, m, b)
        return (h,) + tuple(grads)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)  # started early: the first samples take a while to arrive
    sampler.start()
    h = m = b = None
    for _ in range(warmup):  # same tensor lifetimes as the timed loop, so the allocator reaches its steady state
        h, m, b = pkg.mlstm_matmul_forward(d["q"], d["k"], d["v"], d["f"], d["i"], h_dtype=torch.bfloat16)
        pkg.mlstm_matmul_backward(d["dh"], d["q"], d["k"], d["v"], d["f"], d["i"], h, m, b)
    barrier()

    # ---- device-resident timing, with separate events around the forward and the backward call
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    host_fwd = host_bwd = 0.0
    sampler.mark(0)
    t_begin.record()
    for s in range(args.steps):
        ev[s][0].record()
        c0 = time.perf_counter()
        h, m, b = pkg.mlstm_matmul_forward(d["q"], d["k"], d["v"], d["f"], d["i"], h_dtype=torch.bfloat16)
        c1 = time.perf_counter()
        ev[s][1].record()
        pkg.mlstm_matmul_backward(d["dh"], d["q"], d["k"], d["v"], d["f"], d["i"], h, m, b)
        host_bwd += time.perf_counter() - c1
        host_fwd += c1 - c0
        ev[s][2].record()
    t_end.record()
    barrier()
    sampler.mark(1)
    clocks = sampler.stop()
    elapsed_ms = t_begin.elapsed_time(t_end)
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / args.steps
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / args.steps
    del h, m, b

    # ---- end to end: pinned host buffers in, results back to pinned host buffers, every step.
    # Three streams, as a training input pipeline would run it: the inputs of step s+1 travel to the device while
    # step s computes and the results of step s-1 travel back (PCIe is full duplex; the copies dominate a step).
    # Every step's host->device and device->host copies lie inside the timed region.
    del d
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
            barrier()
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
    barrier()
    e2e_ms = e2e_begin.elapsed_time(e2e_end)

    times = torch.tensor([elapsed_ms, e2e_ms, fwd_ms, bwd_ms], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, fwd_ms, bwd_ms = times.tolist()

    if rank == 0:
        tokens_per_step = B * S * world
        ms_per_step = elapsed_ms / args.steps
        value = tokens_per_step / (ms_per_step * 1e-3)
        e2e_value = tokens_per_step / (e2e_ms / e2e_steps * 1e-3)
        ff, fb = algorithmic_flops(B, NH, S, D)
        peaks = measured_peaks()
        achieved = (ff + fb) / ((fwd_ms + bwd_ms) * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": ("cfg4: mLSTM matmul fwd+bwd B=16 NH=8 S=4096 D=256 bf16, fp32 accumulate" if B == CFG["B"] else
                                    "cfg4 shape at a reduced batch B=%d (profiler case, not the benchmark)" % B),
                       "per_gpu_batch": B, "global_batch": B * world, "heads": NH, "seq_len": S, "head_dim": D,
                       "parallelism": f"dp{world} over (batch, head) slices, no collective",
                       "l2": "inputs (%.2f GB per step) larger than L2" % (h2d / 1e9)},
            "tflops_algorithmic": (ff + fb) * world / (ms_per_step * 1e-3) / 1e12,
            "roofline": {"bound": "tensor", "kernel": "mlstm_tc_pass_pair (FWD, DQ, DK, DV launches of one step, with the gate passes)",
                         "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["tflops"],
                         "peak_source": peaks["source"],
                         # DRAM bytes per launch from the ncu capture in profiles/ (B=4 case, scaled by slices)
                         "traffic": 1.18e9, "traffic_source": "ncu, B=4 case x4, average of the four passes",
                         "fwd_tflops": ff / (fwd_ms * 1e-3) / 1e12, "bwd_tflops": fb / (bwd_ms * 1e-3) / 1e12,
                         "fwd_ms": fwd_ms, "bwd_ms": bwd_ms},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / e2e_steps,
                    "pipeline": "3 streams: H2D of step s+1, compute of step s and D2H of step s-1 overlap"},
            "gpu_launches": 8 * args.steps,
            "host_submit_ms": {"fwd": host_fwd / args.steps * 1e3, "bwd": host_bwd / args.steps * 1e3},
            "clocks": clocks,
        }
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
