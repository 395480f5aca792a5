"""Benchmark of the attention forward+backward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 2|4] [--impl reference]

Default (--config 2, BASELINE config 2 per GPU): one step = the SSSL group of the default model:
four attention layers of B=16, H=4, T=2048, head_dim=128 (bf16 operands, fp32 accumulate, RoPE base
10000 applied to Q/K, fp32 gradients), three with a 1024-key sliding window and one full causal,
forward for all four then backward for all four.  Each layer has its own Q/K/V/dO/O/gradient
tensors (1.4 GB per GPU in total, far beyond the 126 MB L2).  Under torchrun every rank runs the
same per-GPU workload on its own (batch, head) units (weak scaling, no data-path collective); the
time is the max over ranks of a CUDA-event interval and the value is the whole-job algorithmic
TFLOP/s (14 * D * visible (q,k) pairs * B * H per layer).

--config 4 (BASELINE config 4, long context): B=4, H=16, T=8192; the 1024-key window and the full
causal mask are timed separately (`value` is the windowed one, `full_causal` the other).

Besides the headline the line carries: `roofline` (per-kernel achieved TFLOP/s against the measured
bf16 peak), `sustained` (the same step back to back for at least three seconds, with the clocks
seen), `config5` (BASELINE config 5: the global B=128, H=8 workload split over the ranks by
(batch, head) units, strong scaling), `e2e` (host buffers in, host buffers out) and, on one GPU,
`cpu_baseline` (the reference's algorithm on the host cores).
"""
from __future__ import annotations

import argparse
import copy
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

D = 128
METRIC = "attn_fwd_bwd_tflops_windowed_causal"
# name -> (B per GPU, H, T, per-layer windows of one step)
CONFIGS = {
    2: dict(B=16, H=4, T=2048, windows=(1024, 1024, 1024, 2048),      # config.mojo:49-55, one SSSL group
            workload="BASELINE config 2 per GPU: default-model attention fwd+bwd, SSSL group "
                     "(3 x window 1024 + 1 x full causal), RoPE on Q/K"),
    4: dict(B=4, H=16, T=8192, windows=(1024,),
            workload="BASELINE config 4 per GPU: long-context attention fwd+bwd, T=8192, window 1024 "
                     "(full causal timed separately), RoPE on Q/K"),
}
C5 = dict(B=128, H=8, T=2048, windows=(1024, 1024, 1024, 2048))       # BASELINE config 5 (global)

# DRAM bytes per launch (dram__bytes_read.sum, dram__bytes_write.sum) from an ncu capture of
# full-size launches: B=16, H=4, T=2048, W=1024, 64 (b,h) units; other unit counts scale it.
NCU_DRAM = {
    "attn_fwd": (126.5e6, 8.8e6), "attn_bwd_dq": (276.3e6, 50.3e6), "attn_bwd_dkv": (157.9e6, 83.1e6),
    "source": "ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum --clock-control none -k regex:attn_ "
              "-s 36 -c 12 on `bench.py --steps 2 --warmup 3 --no-e2e --no-cpu --no-sustained --no-config5 "
              "--no-phases` (B=16 H=4 T=2048; mean of the three W=1024 launches of each kernel; "
              "scaled by the unit count)",
}


def pairs(t: int, w: int) -> int:
    """Visible (q, k) pairs per (b, h): keys q-w..q, or all k <= q when the window covers T."""
    if w <= 0 or w >= t - 1:
        return t * (t + 1) // 2
    return (w + 1) * (w + 2) // 2 + (t - w - 1) * (w + 1)


def flops(per_pair: int, t: int, windows, b: int, h: int) -> float:
    return sum(float(per_pair) * D * pairs(t, w) * b * h for w in windows)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return d["bf16_tflops"], d["bf16_tflops_sustained"], d["hbm_gbs"], "measured"
    return 1590.0, 1400.0, 6650.0, "fallback"


class ClockSampler:
    """SM clock and throttle-reason samples (read-only NVML queries, every 20 ms) taken by a
    background thread while a timed region runs."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap"}

    def __init__(self, index: int):
        import threading
        self.samples, self.bits, self.max_mhz, self.err = [], 0, None, None
        self._stop = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # noqa: BLE001 - any NVML failure just disables sampling
            self.err = repr(e)
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                self.bits |= int(self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
            except Exception as e:  # noqa: BLE001
                self.err = repr(e)
                return
            self._stop.wait(0.02)

    def stop(self):
        if self.err and not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable: " + self.err]}
        self._stop.set()
        self.thread.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(n for b, n in self.REASONS.items() if self.bits & b), "samples": len(s)}


# --------------------------------------------------------------------------------------
# CPU arm: the oracle port (the reference has no CPU implementation and cannot be built)
# --------------------------------------------------------------------------------------
def cpu_sample(cfg_id: int):
    """A bounded sample of the workload: whole (b, h) units, all layers of the step."""
    c = CONFIGS[cfg_id]
    if cfg_id == 2:
        return dict(B=2, H=4, T=c["T"], windows=c["windows"], of=f"8 of {c['B'] * c['H']} units")
    return dict(B=1, H=2, T=c["T"], windows=c["windows"], of=f"2 of {c['B'] * c['H']} units")


def cpu_sample_inputs(s):
    from oracle import oracle as orc
    orc.use_all_cores()
    q, k, v, do = orc.make_inputs(s["B"], s["T"], s["H"], D, seed=0, bf16=True)
    return orc, (q, k, v, do), orc.rope_table(s["T"], D)


def cpu_time_once(orc, tensors, tables, windows) -> float:
    t0 = time.perf_counter()
    for w in windows:
        orc.attention_path(*tensors[:3], tensors[3], w, rope=tables)
    return time.perf_counter() - t0


def cpu_baseline(cfg_id: int):
    s = cpu_sample(cfg_id)
    orc, tensors, tables = cpu_sample_inputs(s)
    cpu_time_once(orc, tensors, tables, s["windows"])                      # warm-up (page-in, thread pool)
    dt = min(cpu_time_once(orc, tensors, tables, s["windows"]) for _ in range(2))
    return {"value": flops(14, s["T"], s["windows"], s["B"], s["H"]) / dt / 1e12, "unit": "TFLOP/s",
            "cores": orc.num_threads(), "kind": "port",
            "sample": f"oracle port, B={s['B']} H={s['H']} T={s['T']} D={D}, windows {list(s['windows'])} "
                      f"({s['of']}), fwd+bwd, {dt:.2f} s"}


def run_reference(args):
    """--impl reference: the reference's algorithm on the host cores.  The reference is
    GPU-only Mojo with no toolchain here, so the timed code is the C restatement of its
    kernels (oracle port), all host threads, on a bounded sample of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    s = cpu_sample(args.config)
    orc, tensors, tables = cpu_sample_inputs(s)
    for _ in range(min(args.warmup, 2)):
        cpu_time_once(orc, tensors, tables, s["windows"])
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_time_once(orc, tensors, tables, s["windows"])
    dt = (time.perf_counter() - t0) / steps
    val = flops(14, s["T"], s["windows"], s["B"], s["H"]) / dt / 1e12
    cb = {"value": val, "unit": "TFLOP/s", "cores": orc.num_threads(), "kind": "port",
          "sample": f"B={s['B']} H={s['H']} T={s['T']} D={D} windows {list(s['windows'])} per step ({s['of']})"}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 2), "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": CONFIGS[args.config]["workload"] + " (bounded sample)", "B": s["B"], "H": s["H"],
                   "T": s["T"], "D": D, "windows": list(s["windows"])},
        "tokens_per_s": s["B"] * s["T"] * len(s["windows"]) / dt,
        "cpu_baseline": cb,
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------
def bind_to_gpu_numa_node(local: int):
    """Best effort: run this rank (and so allocate its pinned host buffers) on the CPUs of the NUMA
    node its GPU hangs off, so that eight ranks do not all stage through one memory controller.
    Returns a short description for the output line; failing at any step leaves things as they are."""
    try:
        import pynvml
        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(local)).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        if len(bus.split(":")[0]) == 8:
            bus = bus[4:]
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        if node < 0:
            return "numa node unknown"
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return f"gpu on node {node}, none of its cpus allowed here"
        os.sched_setaffinity(0, allowed)
        return f"bound to node {node} ({len(allowed)} cpus)"
    except Exception as e:  # noqa: BLE001
        return "not bound: " + type(e).__name__


def run_gpu(args):
    import torch

    import autoresearch_b200 as ab
    from autoresearch_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    numa = bind_to_gpu_numa_node(local)
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    ab.lib()  # fail loudly if libarattn.so is missing

    cfg = CONFIGS[args.config]
    B, H, T = args.batch or cfg["B"], cfg["H"], cfg["T"]
    windows = cfg["windows"]
    nl = len(windows)
    cos_h, sin_h = ab.precompute_rope(T, D)
    tables = (torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev))
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    peak_burst, peak_sust, hbm_gbs, peak_src = measured_peaks()

    def randn(b, t, h):
        return torch.randn(b, t, h, D, device=dev, generator=gen).to(torch.bfloat16)

    def make_layer(b, t, h, w, grad_dtype=torch.float32):
        L = {"w": w, "q": randn(b, t, h), "k": randn(b, t, h), "v": randn(b, t, h), "do": randn(b, t, h)}
        L["o"] = torch.empty_like(L["q"])
        L["lse"] = torch.empty(b, t, h, device=dev, dtype=torch.float32)
        L["d"] = torch.empty(b, t, h, device=dev, dtype=torch.float32)
        for n in ("dq", "dk", "dv"):
            L[n] = torch.empty(b, t, h, D, device=dev, dtype=grad_dtype)
        if args.rope == "saved":      # the reference's data flow: rotate once, save, reuse in backward
            L["q_rot"], L["k_rot"] = torch.empty_like(L["q"]), torch.empty_like(L["k"])
        L["p"] = ab.AttnParams(window=w, rope=tables, rope_prepass=args.rope == "prepass", grad_dtype=grad_dtype,
                               q_rot=L.get("q_rot"), k_rot=L.get("k_rot"))
        return L

    def fwd(L, p=None):
        ab.attn_fwd(L["q"], L["k"], L["v"], p or L["p"], out=L["o"], lse=L["lse"])

    def bwd(L, p=None):
        ab.attn_bwd(L["q"], L["k"], L["v"], L["o"], L["do"], L["lse"], p or L["p"], d_buf=L["d"],
                    dq=L["dq"], dk=L["dk"], dv=L["dv"])

    def make_step(layers):
        def step():
            for L in layers:
                fwd(L)
            for L in reversed(layers):
                bwd(L)
        return step

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, iters):
        """Device time of `iters` calls of fn in ms (CUDA events on the launching stream)."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    graph_note = {"timing": "CUDA graph replay"}

    def timed_graph(fn, iters):
        """Device time in ms of `iters` calls of fn, captured once into a CUDA graph and replayed: the
        kernels run back to back with no host call between them, so launches of 20 us are timed on the
        device and not on the host that issues them.  Falls back to plain event timing (and says so)
        if the capture is refused."""
        try:
            g = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.graph(g, stream=side):
                for _ in range(iters):
                    fn()
            torch.cuda.current_stream().wait_stream(side)
            g.replay()                                  # untimed: first replay uploads the graph
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1)
        except Exception as exc:                        # noqa: BLE001
            graph_note["timing"] = f"events around direct launches (graph capture refused: {type(exc).__name__})"
            torch.cuda.synchronize()
            return timed(fn, iters)

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def check_status():
        if _lib.lib().ar_device_status() != _lib.AR_OK:
            raise SystemExit("device status: " + _lib.lib().ar_last_error().decode())

    # ---- headline: K steps, barrier + synchronize on both sides, max over ranks ----------------
    layers = [make_layer(B, T, H, w) for w in windows]
    step = make_step(layers)
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    ms_total = timed(step, args.steps)
    barrier()
    clocks = sampler.stop() if sampler else None
    check_status()
    ms_step = max_over_ranks(ms_total) / args.steps
    step_fl = flops(14, T, windows, B, H)
    value = step_fl * world / (ms_step * 1e-3) / 1e12
    line_extra = {}

    # ---- the same step with bf16 gradients (what a torch caller of bf16 tensors gets back) -------
    # The headline keeps the reference's fp32 gradient tensors; this is the same work with half the
    # gradient bytes written.
    if not args.no_phases:
        glayers = [make_layer(B, T, H, w, grad_dtype=torch.bfloat16) for w in windows]
        gstep = make_step(glayers)
        for _ in range(3):
            gstep()
        barrier()
        ms_g = max_over_ranks(timed(gstep, args.steps)) / args.steps
        line_extra["bf16_gradients"] = {"value": step_fl * world / (ms_g * 1e-3) / 1e12, "unit": "TFLOP/s",
                                        "ms_per_step": ms_g, "note": "dQ, dK, dV written as bf16 instead of fp32 (through a write-out laid out for "
                                                "fp32 rows: the bf16 rows leave in 32-byte pieces)"}
        del glayers, gstep
        check_status()

    # ---- config 4 only: the full causal mask, timed the same way -----------------------------
    if args.config == 4:
        full = [make_layer(B, T, H, 0)]
        fstep = make_step(full)
        for _ in range(3):
            fstep()
        barrier()
        ms_full = max_over_ranks(timed(fstep, args.steps)) / args.steps
        fl_full = flops(14, T, (0,), B, H)
        line_extra["full_causal"] = {"value": fl_full * world / (ms_full * 1e-3) / 1e12, "unit": "TFLOP/s",
                                     "ms_per_step": ms_full, "frac_of_burst_peak": fl_full / (ms_full * 1e-3) / 1e12 / peak_burst,
                                     "tokens_per_s": world * B * T / (ms_full * 1e-3)}
        del full, fstep
        check_status()

    # ---- per-kernel device times (same tensors, same stream) for the roofline -----------------
    roofline = None
    if not args.no_phases:
        reps = 5

        def only(**kw):
            ps = []
            for L in layers:
                p = copy.copy(L["p"])
                p.skip_d, p.skip_dq, p.skip_dkv = kw.get("d", True), kw.get("dq", True), kw.get("dkv", True)
                ps.append(p)
            return lambda: [bwd(L, p) for L, p in zip(layers, ps)]

        # forward on Q, K that are already rotated: the attention kernel without the rotation launch
        plain = [ab.AttnParams(window=L["w"]) for L in layers]
        phase = {"attn_fwd": timed_graph(lambda: [fwd(L, p) for L, p in zip(layers, plain)], reps) / reps}
        phase["fwd_total(rope+attn_fwd)"] = timed_graph(lambda: [fwd(L) for L in layers], reps) / reps
        # rope pre-pass of q, k inside the backward call (none in "saved" mode: the call launches nothing)
        prepass_ms = timed_graph(only(), reps) / reps if args.rope != "saved" else 0.0
        # In the step the dQ kernel also computes D = rowsum(O*dO) and the key-stationary statistics the
        # dK/dV kernel streams; timed alone, the dK/dV launch is preceded by the stand-alone re-layout.
        phase["attn_bwd_dq"] = timed_graph(only(d=False, dq=False), reps) / reps - prepass_ms
        phase["attn_bwd_dkv"] = timed_graph(only(dkv=False), reps) / reps - prepass_ms
        check_status()
        # Peak: the burst figure while the sampled clock sat at its maximum with no power-cap bit,
        # the sustained one when the power cap was seen (these short loops run at the burst clock).
        capped = bool(clocks and "sw_power_cap" in clocks.get("reasons", []))
        peak, peak_name = (peak_sust, "bf16_tflops_sustained") if capped else (peak_burst, "bf16_tflops")
        # executed-useful FLOPs per kernel on exact visible pairs: fwd QK^T+PV = 4D; dq kernel
        # S, dP, dQ = 6D; dkv kernel S^T, dP^T, dV, dK = 8D (S and dP are recomputed in both).
        per_pair = {"attn_fwd": 4, "attn_bwd_dq": 6, "attn_bwd_dkv": 8}
        kernels = {}
        for name, pp in per_pair.items():
            ach = flops(pp, T, windows, B, H) / (phase[name] * 1e-3) / 1e12
            rd, wr = NCU_DRAM[name]
            kernels[name] = {"flop_per_pair": pp * D, "ms_per_step": round(phase[name], 4), "launches_per_step": nl,
                             "achieved": ach, "frac": ach / peak,
                             "traffic": (rd + wr) * (B * H) / 64.0 if T == 2048 else None}
        # forward rotation of Q and K (one launch per layer): the backward entry point with all three of
        # its stages skipped and no saved rotated tensors launches exactly that kernel, into scratch
        rope_only = []
        for L in layers:
            p = ab.AttnParams(window=L["w"], rope=tables, skip_d=True, skip_dq=True, skip_dkv=True)
            rope_only.append(p)
        rope_fn = lambda: [bwd(L, p) for L, p in zip(layers, rope_only)]    # noqa: E731
        rope_fn()                                  # first use allocates the scratch
        rope_ms = timed_graph(rope_fn, 4 * reps) / (4 * reps)
        nbytes = 4 * B * T * H * D * 2 * nl       # 2 tensors read + 2 written, bf16
        kernels["rope_pair_bf16_128"] = {"bound": "hbm", "ms_per_step": round(rope_ms, 4), "launches_per_step": nl,
                                         "achieved": nbytes / (rope_ms * 1e-3) / 1e9, "unit": "GB/s",
                                         "frac": nbytes / (rope_ms * 1e-3) / 1e9 / hbm_gbs, "peak": hbm_gbs, "bytes": nbytes // nl}
        # the HBM-bound kernels around the path, each through its C-ABI entry point at this size:
        # algorithmic bytes (tensors read + written once) over the device time of one launch
        n_el = B * T * H * D
        f32 = [torch.randn(B, T, H, D, device=dev, generator=gen) for _ in range(3)]
        b16 = [torch.empty(B, T, H, D, device=dev, dtype=torch.bfloat16) for _ in range(3)]
        dsc = torch.empty(B, T, H, device=dev)
        L_ = _lib.lib()

        def st_():
            return torch.cuda.current_stream().cuda_stream      # the capturing stream inside a graph capture

        def hbm_kernel(name, fn, nbytes, what):
            fn()
            ms = timed_graph(fn, 10) / 10
            kernels[name] = {"bound": "hbm", "ms_per_launch": round(ms, 4), "achieved": nbytes / (ms * 1e-3) / 1e9,
                             "unit": "GB/s", "frac": nbytes / (ms * 1e-3) / 1e9 / hbm_gbs, "peak": hbm_gbs, "bytes": nbytes,
                             "what": what}

        hbm_kernel("qk_norm_rope_cast_128", lambda: _lib.check(L_.ar_qk_norm_rope_cast(
            b16[0].data_ptr(), b16[1].data_ptr(), b16[2].data_ptr(), None, None, f32[0].data_ptr(), f32[1].data_ptr(),
            f32[2].data_ptr(), _lib.AR_F32, tables[0].data_ptr(), tables[1].data_ptr(), B * T, H, D, T, 1e-5, st_())),
            n_el * (3 * 4 + 3 * 2), "ar_qk_norm_rope_cast: fp32 q, k, v in, bf16 rotated+normalised q, k and bf16 v out")
        hbm_kernel("rope_cast<f32,f32>", lambda: ab.rope_fwd(f32[0], f32[0], tables[0], tables[1], B * T, H, D, T),
                   n_el * 8, "ar_rope_fwd in place on one fp32 tensor")
        hbm_kernel("precompute_d128<f32>", lambda: ab.flash_attn_bwd_precompute_d(dsc, f32[1], f32[2], B, T, H, D),
                   n_el * 8 + B * T * H * 4, "ar_flash_attn_bwd_precompute_d on fp32 O, dO")
        del f32, b16, dsc
        # the projections either side of the path (linear_fwd / _bwd_dx / _bwd_dw, ops.mojo:110, 870, 953) at
        # this config's token count: one head group's projection (N = K = H*D) as the reference launches
        # it, and q, k, v as one N = 3*H*D product; bf16 in and out, operand sets cycled so that no
        # launch finds its operands in L2
        Mtok, C = B * T, H * D

        def gemm_kernel(name, call, N, K, what):
            sets = max(2, int(192e6 / (2.0 * Mtok * (N + K))) + 1)
            xs = [torch.randn(Mtok, K, device=dev, generator=gen).bfloat16() for _ in range(sets)]
            dys = [torch.randn(Mtok, N, device=dev, generator=gen).bfloat16() for _ in range(sets)]
            wt = (torch.randn(N, K, device=dev, generator=gen) * 0.05).bfloat16()
            dws = torch.zeros(N, K, device=dev)
            it = [0]

            def fn():
                i = it[0] % sets
                it[0] += 1
                call(xs[i], dys[i], wt, dws, Mtok, N, K)
            fn()
            ms = timed_graph(lambda: [fn() for _ in range(sets)], 5) / (5 * sets)
            fl = 2.0 * Mtok * N * K
            kernels[name] = {"bound": "tensor", "ms_per_launch": round(ms, 4), "achieved": fl / (ms * 1e-3) / 1e12,
                             "unit": "TFLOP/s", "frac": fl / (ms * 1e-3) / 1e12 / peak, "peak": peak,
                             "M": Mtok, "N": N, "K": K, "what": what}

        for tag, N in (("", C), ("_qkv", 3 * C)):
            gemm_kernel("linear_fwd" + tag, lambda x, dy, w_, dw, M, N, K: ab.linear_fwd(dy, x, w_, M, N, K), N, C,
                        "ar_linear_fwd, bf16 in and out")
            gemm_kernel("linear_bwd_dx" + tag, lambda x, dy, w_, dw, M, N, K: ab.linear_bwd_dx(x, dy, w_, M, N, K), N, C,
                        "ar_linear_bwd_dx, bf16 in and out")
            gemm_kernel("linear_bwd_dw" + tag, lambda x, dy, w_, dw, M, N, K: ab.linear_bwd_dw(dw, dy, x, M, N, K), N, C,
                        "ar_linear_bwd_dw, bf16 in, fp32 accumulated")
        dominant = max(per_pair, key=lambda n: phase[n])
        kd = kernels[dominant]
        roofline = {"bound": "tensor", "kernel": dominant, "achieved": kd["achieved"], "peak": peak, "unit": "TFLOP/s",
                    "frac": kd["frac"], "traffic": kd["traffic"], "traffic_source": NCU_DRAM["source"],
                    "peak_source": f"{peak_name}, {peak_src}" + (" (sw_power_cap sampled)" if capped else
                                                                 " (clock at max, no power-cap bit sampled)"),
                    "launch_ms": phase[dominant] / nl, "kernel_timing": graph_note["timing"],
                    "kernels": kernels,
                    # the whole path on the 14*D the metric credits (the split backward executes 14*D
                    # for its 10*D), against the same peak
                    "path": {"flop_per_pair_credited": 14 * D, "flop_per_pair_executed": 18 * D,
                             "achieved": value / world, "frac": value / world / peak}}

    # ---- sustained: the same step back to back for at least three seconds ------------------------
    sustained = None
    if not args.no_sustained:
        n_sus = max(args.steps, int(3000.0 / ms_step) + 1)
        barrier()
        s2 = ClockSampler(local) if rank == 0 else None
        ms_sus = max_over_ranks(timed(step, n_sus)) / n_sus
        ck = s2.stop() if s2 else None
        check_status()
        tf = step_fl * world / (ms_sus * 1e-3) / 1e12
        sustained = {"value": tf, "unit": "TFLOP/s", "steps": n_sus, "ms_per_step": ms_sus, "seconds": ms_sus * n_sus * 1e-3}
        if ck and ck.get("sm_mhz"):
            sustained.update({"sm_mhz_median": ck["sm_mhz"], "sm_max_mhz": ck["sm_max_mhz"], "reasons": ck["reasons"],
                              "power_capped": "sw_power_cap" in ck["reasons"],
                              "value_at_max_clock": tf * ck["sm_max_mhz"] / ck["sm_mhz"],
                              "frac_of_sustained_peak": tf / world / peak_sust})

    # ---- BASELINE config 5: the global B=128, H=8 workload sharded over the ranks -----------------
    config5 = None
    if args.config == 2 and not args.no_config5 and not args.batch:
        del layers, step
        torch.cuda.empty_cache()
        b0, nb, h0, nh = ab.shard_units(C5["B"], C5["H"], world, rank)    # contiguous batch slab, all heads
        assert nh == C5["H"] and h0 == 0
        L5 = make_layer(nb, C5["T"], C5["H"], 0)        # one tensor set (0.4 GB per tensor at N=1, beyond L2)
        ps = [copy.copy(L5["p"]) for _ in C5["windows"]]
        for p, w in zip(ps, C5["windows"]):
            p.window = w

        def step5():
            for p in ps:
                fwd(L5, p)
            for p in reversed(ps):
                bwd(L5, p)

        for _ in range(3):
            step5()
        barrier()
        n5 = max(3, min(args.steps, 10))
        ms5 = max_over_ranks(timed(step5, n5)) / n5
        barrier()
        check_status()
        fl5 = flops(14, C5["T"], C5["windows"], C5["B"], C5["H"])
        config5 = {"workload": "BASELINE config 5: B=128 H=8 T=2048 D=128 bf16, SSSL group, (batch, head) units "
                               f"split over {world} rank(s) in contiguous batch slabs, no collective",
                   "scaling": "strong", "units_total": C5["B"] * C5["H"], "units_per_rank": nb * nh,
                   "ms_per_step": ms5, "value": fl5 / (ms5 * 1e-3) / 1e12, "unit": "TFLOP/s",
                   "tokens_per_s": C5["B"] * C5["T"] * len(C5["windows"]) / (ms5 * 1e-3), "steps": n5}
        del L5
        torch.cuda.empty_cache()
        layers = [make_layer(B, T, H, w) for w in windows] if not args.no_e2e else None

    # ---- end to end: host buffers -> H2D -> fwd+bwd through the public API -> D2H --------
    e2e = None
    if not args.no_e2e:
        gb = torch.bfloat16
        host_in = [{n: torch.empty(B, T, H, D, dtype=gb).pin_memory() for n in ("q", "k", "v", "do")} for _ in windows]
        for hl, L in zip(host_in, layers):
            for n in hl:
                hl[n].copy_(L[n])
        host_out = [{n: torch.empty(B, T, H, D, dtype=gb).pin_memory() for n in ("o", "dq", "dk", "dv")} for _ in windows]

        # Two complete device buffer sets (inputs, saved rotated Q/K, O, LSE, D, bf16 gradients), used
        # by alternate steps, and three streams: while one step's kernels run, the next step's inputs
        # arrive and the previous step's results leave (PCIe is full duplex).  Every step still
        # copies all of its inputs in and all of its results out; the timed interval ends only after
        # the last device->host copy has finished.
        def make_set():
            st = []
            for w in windows:
                S = {n: torch.empty(B, T, H, D, device=dev, dtype=gb) for n in
                     ("q", "k", "v", "do", "o", "dq", "dk", "dv", "q_rot", "k_rot")}
                S["lse"] = torch.empty(B, T, H, device=dev, dtype=torch.float32)
                S["d"] = torch.empty(B, T, H, device=dev, dtype=torch.float32)
                rot = args.rope == "saved"
                S["p"] = ab.AttnParams(window=w, rope=tables, rope_prepass=args.rope == "prepass", grad_dtype=gb,
                                       q_rot=S["q_rot"] if rot else None, k_rot=S["k_rot"] if rot else None)
                st.append(S)
            return st

        sets = [make_set(), make_set()]
        s_main = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        ev_in = [[torch.cuda.Event() for _ in windows] for _ in range(2)]
        ev_bwd = [[torch.cuda.Event() for _ in windows] for _ in range(2)]
        ev_free = [torch.cuda.Event() for _ in range(2)]     # the set's results have left the device
        for e in ev_free:
            e.record(s_main)

        def e2e_step(k):
            cur, par = sets[k & 1], k & 1
            s_in.wait_event(ev_free[par])                     # step k-2 is completely done with this set
            with torch.cuda.stream(s_in):
                for i, (hl, S) in enumerate(zip(host_in, cur)):
                    for n in hl:
                        S[n].copy_(hl[n], non_blocking=True)
                    ev_in[par][i].record(s_in)
            for i, S in enumerate(cur):
                s_main.wait_event(ev_in[par][i])
                ab.attn_fwd(S["q"], S["k"], S["v"], S["p"], out=S["o"], lse=S["lse"])
            for i in reversed(range(nl)):
                S = cur[i]
                ab.attn_bwd(S["q"], S["k"], S["v"], S["o"], S["do"], S["lse"], S["p"], d_buf=S["d"],
                            dq=S["dq"], dk=S["dk"], dv=S["dv"])
                ev_bwd[par][i].record(s_main)
                s_out.wait_event(ev_bwd[par][i])
                with torch.cuda.stream(s_out):
                    for n in ("o", "dq", "dk", "dv"):
                        host_out[i][n].copy_(S[n], non_blocking=True)
            ev_free[par].record(s_out)

        def e2e_run(n_steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record(s_main)
            for k in range(n_steps):
                e2e_step(k)
            s_main.wait_event(ev_free[0])
            s_main.wait_event(ev_free[1])
            e1.record(s_main)
            torch.cuda.synchronize()
            return e0.elapsed_time(e1)

        e2e_steps = max(2, min(args.steps, 10))
        e2e_run(2)
        barrier()
        ms_e2e = max_over_ranks(e2e_run(e2e_steps)) / e2e_steps
        check_status()
        nbytes = B * T * H * D * 2
        e2e = {"value": step_fl * world / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": 4 * nl * nbytes, "d2h_bytes_per_step": 4 * nl * nbytes,
               "ms_per_step": ms_e2e, "tokens_per_s": world * B * T * nl / (ms_e2e * 1e-3),
               "host_copy_gbs_per_gpu_each_way": 4 * nl * nbytes / (ms_e2e * 1e-3) / 1e9, "host_numa": numa,
               "note": "pinned host q,k,v,dO in; o,dq,dk,dv (bf16) out; steps pipelined over two device "
                       "buffer sets and three streams (H2D, kernels, D2H); timed until the last D2H copy is done; "
                       "bound by the host<->device copies, not by the kernels"}

    cpu = cpu_baseline(args.config) if (rank == 0 and world == 1 and not args.no_cpu) else None
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    # kernels per layer: forward attention 1 (+1 launch rotating Q and K unless rotate-on-load);
    # backward: dQ (which also computes D and the key-stationary statistics) 1, dK/dV 1
    # (+1 rotation launch unless the forward saved the rotated Q, K)
    launches_per_step = nl * ((1 + (0 if args.rope == "fused" else 1)) + 2 + (0 if args.rope == "saved" else 1))
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg["workload"],
                   "B_per_gpu": B, "H": H, "T": T, "D": D, "windows": list(windows), "global_batch": B * world,
                   "grad_dtype": "f32", "rope": {"saved": "fwd: rotate Q/K once into saved bf16 buffers; bwd: reuse them, inverse rotation fused into dQ/dK stores",
                            "fused": "fwd: rotate-on-load; bwd: pre-pass + fused inverse",
                            "prepass": "pre-pass in both passes"}[args.rope],
                   "parallelism": f"(batch,head) units sharded over {world} rank(s), no collective",
                   "l2": f"working set {(5 * 2 + 2 * 2 + 3 * 4) * B * T * H * D * nl / 1e9:.1f} GB per GPU (inputs larger than L2), "
                         "distinct tensors per layer"},
        "tokens_per_s": world * B * T * nl / (ms_step * 1e-3),
        "frac_of_peak": {"burst": value / world / peak_burst, "sustained": value / world / peak_sust,
                         "nominal_2250": value / world / 2250.0, "source": peak_src},
        "clocks": clocks, "gpu_launches": launches_per_step * args.steps,
    }
    line.update(line_extra)
    for key, obj in (("roofline", roofline), ("sustained", sustained), ("config5", config5), ("e2e", e2e),
                     ("cpu_baseline", cpu)):
        if obj is not None:
            line[key] = obj
    print(json.dumps(line))


def run_config3(args):
    """BASELINE config 3: forward + backward of the reference's small GPT (depth 8, d_model 512, 4 heads of
    128, vocabulary 8192, T=2048, B=16 per GPU; token ids uniform, seeded) with the attention path on
    libarattn.so and the other layers as torch operations; under torchrun each rank takes its own batch
    and the gradients are all-reduced in per-layer buckets over NCCL.  Reports tokens/s of the whole step
    and the share of the step's device time spent in the attention calls."""
    import torch

    import autoresearch_b200 as ab
    from autoresearch_b200 import train_step as ts

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    cfg = ab.GPTConfig()                       # depth 8, 512 wide, 4 heads of 128, vocabulary 8192, T = 2048
    B, T = args.batch or 16, cfg.sequence_len
    weights = ts.init_weights(cfg, dev, test_init=True)     # non-zero c_proj / mlp_proj (test_forward.mojo:48-63)
    attn = ts.LibraryAttention(cfg, T, dev)
    step = ts.TrainStep(cfg, weights, attn, reference_quirks=True, process_group=True if world > 1 else None,
                        projections=args.projections)
    gen = torch.Generator(device=dev).manual_seed(7 + rank)
    ids = torch.randint(0, cfg.vocab_size, (B, T), device=dev, generator=gen)
    targets = torch.cat([ids[:, 1:], torch.randint(0, cfg.vocab_size, (B, 1), device=dev, generator=gen)], dim=1)
    steps = max(1, min(args.steps, 10))
    loss = None
    for _ in range(3):
        step.zero_grads()
        loss = step.step(ids, targets)
    attn.attention_ms()                        # reset
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step.zero_grads()
        loss = step.step(ids, targets)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    attn_ms = attn.attention_ms() / steps
    ab.check_device_status()
    if dist is not None:
        t = torch.tensor([ms, attn_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, attn_ms = float(t[0]), float(t[1])
        dist.destroy_process_group()
    if rank != 0:
        return
    windows = [cfg.window_size(i) for i in range(cfg.n_layer)]
    attn_flops = flops(14, T, windows, B, cfg.n_head)
    n_param = sum(v.numel() for v in weights.values())
    print(json.dumps({
        "metric": "gpt_train_step_tokens_per_s", "value": world * B * T / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": 3, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "BASELINE config 3 per GPU: small-GPT forward + backward, attention on libarattn.so, the "
                               "other layers torch operations on an fp32 residual stream", "B_per_gpu": B, "T": T,
                   "n_layer": cfg.n_layer, "n_embd": cfg.n_embd, "n_head": cfg.n_head, "vocab": cfg.vocab_size,
                   "windows": windows, "parameters": n_param, "backward": "as the reference computes it",
                   "projections": "ar_linear_* (libarattn.so)" if args.projections == "library" else "torch matmul",
                   "parallelism": f"data parallel over {world} rank(s), per-layer gradient buckets all-reduced with NCCL"},
        "loss": float(loss),
        "attention": {"ms_per_step": attn_ms, "share_of_step": attn_ms / ms,
                      "tflops": attn_flops / (attn_ms * 1e-3) / 1e12,
                      "calls": "prologue (rope + qk-norm + cast) + forward + backward, 8 layers"},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4],
                    help="BASELINE config: 2 = default-model SSSL group (the headline), 3 = full small-GPT train step, "
                         "4 = long context T=8192")
    ap.add_argument("--batch", type=int, default=0,
                    help="batch per GPU instead of the config's (a small case for profilers); 0 = the config's")
    ap.add_argument("--rope", default="saved", choices=["saved", "fused", "prepass"],
                    help="saved: forward rotates Q/K once into saved buffers that backward reuses; "
                         "fused: forward rotates on load, backward rotates in a pre-pass; "
                         "prepass: both passes rotate in a pre-pass")
    ap.add_argument("--projections", default="library", choices=["library", "torch"],
                    help="config 3: the model's matmuls through ar_linear_* or through torch")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-phases", action="store_true", help="skip the per-kernel timing behind `roofline`")
    ap.add_argument("--no-sustained", action="store_true", help="skip the three-second back-to-back run")
    ap.add_argument("--no-config5", action="store_true", help="skip the config-5 strong-scaling object")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.config == 3:
            args.config = 2      # the host-core arm times the attention path, which is what it restates
        run_reference(args)
    elif args.config == 3:
        run_config3(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
