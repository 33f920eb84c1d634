#!/usr/bin/env python3
"""Benchmark of the masked flash-attention forward (``mha_fwd_with_mask``) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload standard]
                    [--impl ours|reference|reference-cuda] [--scaling weak|strong]

One step = one forward pass of the operator over one batch of the workload
(default "standard": d128 B4 H16 S2048 bf16, 10 % random -inf mask -- the
configuration the headline metric is quoted on).  Prints ONE JSON line on rank 0.

* ``value``    TFLOPS = 4*B*H*Sq*Sk*d / t (dense convention, mask ignored;
               reference benchmark/benchmark_fa.py:135-137), kernel launched through
               the C ABI with every input resident in HBM, summed over ranks.
* ``e2e``      the same metric through ``ops.mha_fwd_with_mask`` with the inputs in
               pinned host memory: H2D copies, the operator and the D2H copy of the
               result are all inside the timed region.
* ``roofline`` achieved TFLOP/s (or GB/s for the HBM-bound workload) of the
               attention kernel from CUDA events on the launching stream over the
               timed region, against the measured peak in MEASURED_PEAKS.json.
* ``cpu_baseline`` the reference's own C++ CPU attention (oracle/_ref, compiled
               from its csrc/fa/cpu sources) on the host cores, on a bounded sample.

* ``all_configs`` (default workload only) the other four benchmark configurations, measured
               after the headline region with the same method: microseconds, TFLOPS, GB/s, the
               roofline fraction that binds, and the error against the CPU oracle on one
               (batch, head) slice.

With ``--gpus N`` (launched under torchrun) every rank runs the workload on its
own batch shard -- (batch, head) units are independent, there is no collective on
the data path -- so scaling is weak; the time is the max over ranks.  The same line
then also carries ``strong_scaling`` (ONE problem's (batch, kv-head) units spread over
the ranks, no collective) and ``cross_gpu_splitkv`` (the long-context shape with its keys
split across the ranks, one NCCL all-gather of the fp32 partials + LSE merge, checked
against the oracle).  ``--scaling strong`` makes the strong-scaled run the headline.

``--impl reference`` times the reference's CPU implementation of the same
workload (rank 0 only) and prints the same line shape with "impl": "reference".
``--impl reference-cuda`` times the reference's own CUDA extension (its sm8x kernels
built for sm_100a, loaded from ``baseline/_ref/fa_so``) on the same inputs with the
same method, in a process that never loads this package's operator; it prints an
``unavailable`` line where that library is absent.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from custom_ops_b200.workloads import WORKLOADS, dtype_tag, make_inputs, to_bits  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# dram__bytes_read.sum + dram__bytes_write.sum of one attention-kernel launch, from
# the ncu captures summarised under profiles/ (None until a capture exists).
LEAD_IN_STEPS = 2      # untimed steps between the barrier and the first timed step (clock ramp)

# (constants from a capture, not measured live: they say which capture they come from)
NCU_TRAFFIC_BYTES = {
    "standard": 152.1e6,        # 134.69 MB read + 17.46 MB written (profiles/fa_mask_fwd_kernel_standard.md)
    "splitkv_long": 281.6e6,    # 277.46 MB read + 4.11 MB written (profiles/fa_mask_fwd_kernel_splitkv_long.md)
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {k: float(p[k]) for k in FALLBACK_PEAKS}, "measured"
    except Exception:  # noqa: BLE001
        return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and clock-event (throttle) reasons during the timed region.

    In-process NVML reads (``pynvml``) on a thread: a polling ``nvidia-smi`` child, the other
    way to get them, stalled the GPU for milliseconds now and then and showed up as outlier
    steps.  Falls back to that child only where the NVML binding is missing.
    """

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    PERIOD_S = 0.05

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []          # (sm MHz, max sm MHz, set of reasons)
        self.nvml = None
        self.handle = None
        self._stop = threading.Event()
        self.thread = None

    # ---- NVML path
    def _nvml_open(self) -> bool:
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = self.index
            if visible:
                ids = [x.strip() for x in visible.split(",") if x.strip()]
                if self.index < len(ids) and ids[self.index].isdigit():
                    phys = int(ids[self.index])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.nvml = pynvml
            return True
        except Exception:  # noqa: BLE001
            self.nvml = None
            return False

    def _nvml_sample(self):
        n = self.nvml
        sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
        smax = n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)
        get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            n.nvmlDeviceGetCurrentClocksThrottleReasons
        mask = get(self.handle)
        reasons = set()
        for name, attrs in (("hw_slowdown", ("nvmlClocksEventReasonHwSlowdown", "nvmlClocksThrottleReasonHwSlowdown")),
                            ("hw_thermal_slowdown", ("nvmlClocksEventReasonHwThermalSlowdown",
                                                     "nvmlClocksThrottleReasonHwThermalSlowdown")),
                            ("sw_thermal_slowdown", ("nvmlClocksEventReasonSwThermalSlowdown",
                                                     "nvmlClocksThrottleReasonSwThermalSlowdown")),
                            ("sw_power_cap", ("nvmlClocksEventReasonSwPowerCap", "nvmlClocksThrottleReasonSwPowerCap"))):
            for a in attrs:
                bit = getattr(n, a, None)
                if bit is not None:
                    if mask & bit:
                        reasons.add(name)
                    break
        return float(sm), float(smax), reasons

    def _nvml_loop(self):
        while not self._stop.is_set():
            try:
                self.lines.append(self._nvml_sample())
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(self.PERIOD_S)

    # ---- nvidia-smi fallback
    def _smi_read(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.strip().split(",")]
            if len(parts) < 7:
                continue
            try:
                sm, smax = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            self.lines.append((sm, smax, {n for n, v in zip(names, parts[3:7]) if v.lower().startswith("active")}))

    def start(self):
        if self._nvml_open():
            self.thread = threading.Thread(target=self._nvml_loop, daemon=True)
            self.thread.start()
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._smi_read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.nvml is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            source = "nvml"
        elif self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            source = "nvidia-smi"
        else:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML binding and no nvidia-smi"]}
        sm = [x[0] for x in self.lines]
        smax = [x[1] for x in self.lines]
        reasons = set()
        for x in self.lines:
            reasons |= x[2]
        # the idle samples before the first launch sit at the idle clock; the median under
        # load is taken over the upper half of the samples
        sm_load = sorted(sm)[len(sm) // 2:] if len(sm) > 3 else sm
        return {"sm_mhz": statistics.median(sm_load) if sm_load else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": source}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# --------------------------------------------------------------------------- reference arm
def cpu_reference_sample(w, steps: int, warmup: int):
    """Times the reference's CPU attention on one batch element of workload ``w``
    (its kernels parallelise over heads only, csrc/fa/cpu/fa_fwd_cpu.cpp:203-204)."""
    import numpy as np
    from oracle import oracle

    sample = w.with_batch(1)
    q, k, v, m = make_inputs(sample, seed=42)
    qb, kb, vb, mb = to_bits(q), to_bits(k), to_bits(v), to_bits(m)
    dt = dtype_tag(q)
    cores = os.cpu_count() or 1
    if oracle.load_ref() is not None:
        kind, isa = "reference", oracle.ref_best_isa()
        threads = min(sample.H, cores)
        fn = lambda: oracle.ref_cpu_attn(qb, kb, vb, mb, dt, isa=isa, n_threads=threads)  # noqa: E731
        what = f"reference csrc/fa/cpu kernel ({isa}), fp32, {threads} threads over heads"
    elif oracle.load_port() is not None:
        kind, threads = "port", cores
        fn = lambda: oracle.port_attn(qb, kb, vb, mb, dt, quantize_p=False, n_threads=threads)  # noqa: E731
        what = f"C restatement of the reference semantics, fp32, {threads} threads"
    else:
        raise RuntimeError("neither oracle/_ref nor the oracle port is built")
    # The kernels take fp32 buffers; widening the 16-bit inputs is part of the call,
    # as it is in the reference's own CPU wrapper (csrc/fa/cpu/fa_fwd_cpu.cpp:243-276).
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        out = fn()
        times.append(time.perf_counter() - t0)
    assert np.isfinite(out).all()
    t = statistics.median(times)
    return {"value": sample.flops / t / 1e12, "unit": "TFLOPS", "cores": threads, "kind": kind,
            "sample": f"{what}; one batch element of '{w.name}' (B=1 of {w.B}), "
                      f"median of {steps} runs, {t * 1e3:.1f} ms each",
            "host_cores": cores, "ms": t * 1e3}


def torch_fp32_cpu_sample(w):
    """The same masked attention in fp32 torch on the host cores, one batch element."""
    sample = w.with_batch(1)
    q, k, v, m = make_inputs(sample, seed=42)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = sample.H // sample.Hk

    def fn():
        kk = k.float().repeat_interleave(g, dim=1)
        vv = v.float().repeat_interleave(g, dim=1)
        s = torch.matmul(q.float(), kk.transpose(-2, -1)) / (sample.d ** 0.5) + m.float()
        return torch.matmul(torch.softmax(s, dim=-1), vv)

    fn()
    times = []
    for _ in range(3):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    return {"value": sample.flops / t / 1e12, "unit": "TFLOPS", "cores": cores,
            "sample": f"fp32 torch softmax(QK^T*scale+mask)V, one batch element of '{w.name}', "
                      f"median of 3, {t * 1e3:.1f} ms"}


def run_reference_arm(args, w):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    base = cpu_reference_sample(w, max(1, args.steps), max(1, min(args.warmup, 2)))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "TFLOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": base["ms"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w.name, "shape": shape_str(w), "sample": "B=1 of the workload"},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "TFLOPS", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)



# --------------------------------------------------------------------------- shared measurement
def oracle_slice_error(out, q_h, k_h, v_h, m_h, b: int, h: int):
    """max-abs / mean-abs of one (batch, head) slice of ``out`` against the fp32 CPU oracle
    softmax(QK^T*scale+mask)V (the checker; never on the measured path)."""
    from oracle import oracle

    g = q_h.shape[1] // k_h.shape[1]
    qs, ks, vs, ms = q_h[b:b + 1, h:h + 1], k_h[b:b + 1, h // g:h // g + 1], v_h[b:b + 1, h // g:h // g + 1], m_h[b:b + 1]
    dt = dtype_tag(q_h)
    args = (to_bits(qs), to_bits(ks), to_bits(vs), to_bits(ms), dt)
    ref = oracle.port_attn(*args, quantize_p=False) if oracle.load_port() is not None else oracle.attn_fp32(*args)
    got = out[b:b + 1, h:h + 1].float().cpu().numpy()
    mx, mean = oracle.errors(got, ref)
    return float(mx), float(mean)


def visited_fraction(w, m_h, region_rows: int = 256) -> float:
    """Share of (region_rows query rows, 128-key block) regions that hold a visible key:
    256-row query pairs, or 128-row tiles where grouped heads run in pairs
    (``FaMaskFwdPlan.head_pairs``)."""
    mp = -(-w.Sq // region_rows)
    nb = -(-w.Sk // 128)
    fin = ~torch.isneginf(m_h.float())
    pad = torch.zeros(m_h.shape[0], 1, mp * region_rows, nb * 128, dtype=torch.bool)
    pad[:, :, :w.Sq, :w.Sk] = fin[:, :, :w.Sq, :w.Sk]
    return float(pad.view(m_h.shape[0], mp, region_rows, nb, 128).any(dim=4).any(dim=2).float().mean())


def measure_config(name: str, dev, steps: int, peaks, flush):
    """One benchmark configuration, kernel-only through the C ABI with the inputs resident in
    HBM, timed like the headline: L2 evicted before every step (or, for the HBM-bound shape,
    rotating input copies), CUDA events per step on the launching stream."""
    from custom_ops_b200 import _cabi

    w = WORKLOADS[name]
    q_h, k_h, v_h, m_h = make_inputs(w, seed=42)
    q, k, v, m = (t.to(dev) for t in (q_h, k_h, v_h, m_h))
    out = torch.empty_like(q)
    rotate = name == "splitkv_long"
    sets = [(k, v, m)] + ([(k.clone(), v.clone(), m.clone()) for _ in range(3)] if rotate else [])
    dt = _cabi.BF16 if w.dtype == torch.bfloat16 else _cabi.FP16
    cargs = [_cabi.make_args(q=q.data_ptr(), k=ks.data_ptr(), v=vs.data_ptr(), mask=ms.data_ptr(),
                             out=out.data_ptr(), batch=w.B, heads=w.H, heads_k=w.Hk, seqlen_q=w.Sq,
                             seqlen_k=w.Sk, head_dim=w.d, dtype=dt, device=dev.index)
             for ks, vs, ms in sets]
    plan = _cabi.plan(cargs[0])
    nbytes = _cabi.workspace_bytes(cargs[0])
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev)
    n = [0]

    def step():
        _cabi.forward(cargs[n[0] % len(cargs)], ws.data_ptr(), nbytes, stream.cuda_stream)
        n[0] += 1

    for _ in range(5):
        if not rotate:
            flush.zero_()
        step()
    torch.cuda.synchronize(dev)
    launches0 = _cabi.launch_count()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(-LEAD_IN_STEPS, steps):
        if not rotate:
            flush.zero_()
        if i == 0:
            launches0 = _cabi.launch_count()
        if i >= 0:
            starts[i].record(stream)
        step()
        if i >= 0:
            ends[i].record(stream)
    torch.cuda.synchronize(dev)
    launches = _cabi.launch_count() - launches0
    ms = [a.elapsed_time(b) for a, b in zip(starts, ends)]
    mean_ms = sum(ms) / len(ms)
    mx, mean = oracle_slice_error(out, q_h, k_h, v_h, m_h, w.B - 1, w.H - 1)
    visited = visited_fraction(w, m_h, 128 if plan.head_pairs else 256) if plan.tile_skip else 1.0
    # The same steps for a caller that vouches for the mask's content (FaMaskFwdArgs.mask_version):
    # the tile-skip pre-pass then runs once, not per call.
    remembered = None
    if plan.tile_skip and not plan.mask_repitched and not rotate:
        vargs = _cabi.make_args(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), mask=m.data_ptr(),
                                out=out.data_ptr(), batch=w.B, heads=w.H, heads_k=w.Hk, seqlen_q=w.Sq,
                                seqlen_k=w.Sk, head_dim=w.d, dtype=dt, device=dev.index, mask_version=1)
        for _ in range(4):
            flush.zero_()
            _cabi.forward(vargs, ws.data_ptr(), nbytes, stream.cuda_stream)
        torch.cuda.synchronize(dev)
        l0 = _cabi.launch_count()
        for i in range(steps):
            flush.zero_()
            starts[i].record(stream)
            _cabi.forward(vargs, ws.data_ptr(), nbytes, stream.cuda_stream)
            ends[i].record(stream)
        torch.cuda.synchronize(dev)
        vms = [a.elapsed_time(b) for a, b in zip(starts, ends)]
        vmx, _ = oracle_slice_error(out, q_h, k_h, v_h, m_h, w.B - 1, w.H - 1)
        remembered = {"us": sum(vms) / len(vms) * 1e3, "us_min": min(vms) * 1e3,
                      "kernels_per_step": (_cabi.launch_count() - l0) / steps, "max_abs_vs_oracle": vmx}
    # The same attention with the mask given as a rule (this workload's mask is "causal, window of
    # 512 keys"): no mask in memory, no pre-pass (fa_mask_fwd_sm100_rule).
    by_rule = None
    if w.mask_kind == "causal_window":
        rout = torch.empty_like(q)
        rargs = _cabi.make_args(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), mask=0, out=rout.data_ptr(),
                                batch=w.B, heads=w.H, heads_k=w.Hk, seqlen_q=w.Sq, seqlen_k=w.Sk, head_dim=w.d,
                                dtype=dt, device=dev.index)
        rws = torch.empty(_cabi.RULE_WORKSPACE_BYTES, dtype=torch.uint8, device=dev)
        for _ in range(4):
            flush.zero_()
            _cabi.forward_rule(rargs, 1, 512, 0, stream.cuda_stream, rws.data_ptr(), _cabi.RULE_WORKSPACE_BYTES)
        torch.cuda.synchronize(dev)
        l0 = _cabi.launch_count()
        for i in range(steps):
            flush.zero_()
            starts[i].record(stream)
            _cabi.forward_rule(rargs, 1, 512, 0, stream.cuda_stream, rws.data_ptr(), _cabi.RULE_WORKSPACE_BYTES)
            ends[i].record(stream)
        torch.cuda.synchronize(dev)
        rms = [a.elapsed_time(b) for a, b in zip(starts, ends)]
        rmx, _ = oracle_slice_error(rout, q_h, k_h, v_h, m_h, w.B - 1, w.H - 1)
        by_rule = {"us": sum(rms) / len(rms) * 1e3, "us_min": min(rms) * 1e3,
                   "kernels_per_step": (_cabi.launch_count() - l0) / steps, "max_abs_vs_oracle": rmx,
                   "max_abs_vs_mask_tensor_run": float((rout.float() - out.float()).abs().max())}
    tflops = w.flops / (mean_ms * 1e-3) / 1e12
    gbs = w.bytes / (mean_ms * 1e-3) / 1e9
    if name == "splitkv_long":
        bound, achieved, peak, unit = "hbm", gbs, peaks["hbm_gbs"], "GB/s"
    elif name == "plumbing":
        bound, achieved, peak, unit = "launch latency", tflops, peaks["bf16_tflops"], "TFLOP/s"
    else:
        bound, achieved, peak, unit = "tensor", tflops * visited, peaks["bf16_tflops"], "TFLOP/s"
    return {"shape": shape_str(w), "us": mean_ms * 1e3, "us_min": min(ms) * 1e3, "us_max": max(ms) * 1e3,
            "tflops_dense_convention": tflops, "gb_per_s": gbs, "bound": bound, "achieved": achieved,
            "unit": unit, "peak": peak, "frac": achieved / peak, "visited_block_fraction": visited,
            "max_abs_vs_oracle": mx, "mean_abs_vs_oracle": mean, "oracle_slice": f"batch {w.B - 1}, head {w.H - 1}",
            "steps": steps, "kernels_per_step": launches / steps, "num_splits": plan.num_splits,
            "grid": plan.grid_x, "mask_repitched": bool(plan.mask_repitched), "head_pairs": bool(plan.head_pairs),
            "with_mask_version": remembered, "mask_as_rule": by_rule,
            "l2": "4 rotating input copies" if rotate else "256 MB zero-fill before every step"}


def measure_strong_scaling(w, dev, steps: int, rank: int, world: int, flush, dist):
    """ONE problem of workload ``w``: its (batch, kv-head) units are spread over the ranks
    (custom_ops_b200.parallel.shard_inputs), every rank runs its sub-problems through the C ABI,
    no collective touches the data path.  Returns (max-over-ranks ms, this rank's slice error)."""
    from custom_ops_b200 import _cabi, parallel

    q_h, k_h, v_h, m_h = make_inputs(w, seed=42)          # the same problem on every rank
    pieces_h = parallel.shard_inputs(q_h, k_h, v_h, m_h, world, rank)
    dt = _cabi.BF16 if w.dtype == torch.bfloat16 else _cabi.FP16
    stream = torch.cuda.current_stream(dev)
    jobs = []
    for qs, ks, vs, ms in pieces_h:
        qd, kd, vd, md = (t.to(dev) for t in (qs, ks, vs, ms))
        od = torch.empty_like(qd)
        a = _cabi.make_args(q=qd.data_ptr(), k=kd.data_ptr(), v=vd.data_ptr(), mask=md.data_ptr(),
                            out=od.data_ptr(), batch=qd.shape[0], heads=qd.shape[1], heads_k=kd.shape[1],
                            seqlen_q=w.Sq, seqlen_k=w.Sk, head_dim=w.d, dtype=dt, device=dev.index)
        nb = _cabi.workspace_bytes(a)
        jobs.append((a, torch.empty(max(nb, 16), dtype=torch.uint8, device=dev), nb, (qd, kd, vd, md, od)))

    def step():
        for a, ws, nb, _ in jobs:
            _cabi.forward(a, ws.data_ptr(), nb, stream.cuda_stream)

    for _ in range(4):
        flush.zero_()
        step()
    torch.cuda.synchronize(dev)
    dist.barrier()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(-LEAD_IN_STEPS, steps):
        flush.zero_()
        if i >= 0:
            starts[i].record(stream)
        step()
        if i >= 0:
            ends[i].record(stream)
    torch.cuda.synchronize(dev)
    ms = sum(a.elapsed_time(b) for a, b in zip(starts, ends)) / steps
    err = (0.0, 0.0)
    if jobs:
        qs, ks, vs, ms_h = pieces_h[-1]
        err = oracle_slice_error(jobs[-1][3][4], qs, ks, vs, ms_h, qs.shape[0] - 1, qs.shape[1] - 1)
    t = torch.tensor([ms, err[0], err[1]], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0]), float(t[1]), float(t[2]), len(jobs)


def measure_cross_gpu_splitkv(dev, steps: int, rank: int, world: int, dist):
    """The long-context shape with its keys split across the ranks: local forward into the
    packed part, exchange, LSE merge; checked against the oracle on one head.  Both exchanges
    are timed: through peer-addressable memory inside the merge kernel, and one NCCL
    all-gather followed by the merge."""
    from custom_ops_b200 import parallel

    w = WORKLOADS["splitkv_long"]
    q_h, k_h, v_h, m_h = make_inputs(w, seed=42)
    lo, hi = parallel.kv_slice_bounds(w.Sk, world, rank)
    q = q_h.to(dev)
    k, v, m = (k_h[:, :, lo:hi].contiguous().to(dev), v_h[:, :, lo:hi].contiguous().to(dev),
               m_h[:, :, :, lo:hi].contiguous().to(dev))
    stream = torch.cuda.current_stream(dev)

    def timed(exchange):
        out = None
        for _ in range(5):
            out = parallel.splitkv_forward(q, k, v, m, exchange=exchange)
        torch.cuda.synchronize(dev)
        mx, mean = oracle_slice_error(out, q_h, k_h, v_h, m_h, 0, w.H - 1)
        dist.barrier()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for i in range(-LEAD_IN_STEPS, steps):
            if i >= 0:
                starts[i].record(stream)
            out = parallel.splitkv_forward(q, k, v, m, exchange=exchange)
            if i >= 0:
                ends[i].record(stream)
        torch.cuda.synchronize(dev)
        ms = sum(a.elapsed_time(b) for a, b in zip(starts, ends)) / steps
        t = torch.tensor([ms, mx, mean], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    nccl_ms, nccl_mx, nccl_mean = timed("nccl")
    # the collective alone, on the same buffers: what that exchange step costs at this size
    scratch = parallel._SplitKVScratch.get(dev, w.B * w.H * w.Sq, w.d, world)
    dist.barrier()
    g0 = torch.cuda.Event(enable_timing=True)
    g1 = torch.cuda.Event(enable_timing=True)
    g0.record(stream)
    for _ in range(steps):
        dist.all_gather_into_tensor(scratch.gathered, scratch.part)
    g1.record(stream)
    torch.cuda.synchronize(dev)
    t = torch.tensor([g0.elapsed_time(g1) / steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    gather_ms = float(t[0])
    # every rank must take the same branch: agree on whether the peer exchange can be set up
    can = torch.tensor([1 if parallel.peer_exchange_available() else 0], device=dev)
    dist.all_reduce(can, op=dist.ReduceOp.MIN)
    peer = None
    peer_note = "symmetric memory not available in this torch build"
    if int(can[0]):
        try:
            peer = timed("peer")
            peer_note = "parts in symmetric memory, read over NVLink by the merge kernel (plain loads, bounded wait)"
        except Exception as e:  # noqa: BLE001
            peer_note = f"peer exchange failed to set up: {str(e)[:160]}"
    best_ms, mx, mean = (peer if peer is not None and peer[0] <= nccl_ms else (nccl_ms, nccl_mx, nccl_mean))
    return {"shape": shape_str(w), "ranks": world, "keys_per_rank": hi - lo, "us": best_ms * 1e3,
            "exchange": "peer" if (peer is not None and peer[0] <= nccl_ms) else "nccl",
            "us_peer_exchange": None if peer is None else peer[0] * 1e3,
            "us_nccl_exchange": nccl_ms * 1e3, "nccl_all_gather_alone_us": gather_ms * 1e3,
            "peer_exchange": peer_note, "part_bytes": scratch.part_floats * 4,
            "gb_per_s": w.bytes / (best_ms * 1e-3) / 1e9,
            "max_abs_vs_oracle": max(mx, nccl_mx), "mean_abs_vs_oracle": max(mean, nccl_mean),
            "oracle_slice": f"batch 0, head {w.H - 1}",
            "l2": "inputs stay in place between steps (each rank's key slice is smaller than L2 from 4 ranks on)",
            "timing": "CUDA events per step on the launching stream, mean over steps, max over ranks"}


# --------------------------------------------------------------------------- reference CUDA arm
def run_reference_cuda_arm(args, w):
    """The reference's own CUDA extension on this GPU (what a B200 runs today: its sm8x cp.async /
    mma.sync family built for sm_100a), same inputs, same timing as the reference's own
    harness (benchmark/benchmark_fa.py:115-132: L2 flush before every iteration, CUDA events).
    Runs in a process of its own so that its recsys_ops::mha_fwd_with_mask registration never
    meets this package's."""
    rank, world, local = dist_env()
    if rank != 0:
        return
    so = os.path.join(ROOT, "baseline", "_ref", "fa_so", "recsys_fa_kernel.so")
    line = {"impl": "reference-cuda", "metric": METRIC if w.name == "standard" else f"masked attn fwd TFLOPS ({shape_str(w)})"}
    if not os.path.exists(so) or not torch.cuda.is_available():
        line["unavailable"] = ("baseline/_ref/fa_so/recsys_fa_kernel.so is not built (the reference's FA group, "
                               "JIT-built once for sm_100a)" if not os.path.exists(so) else "no CUDA device")
        print(json.dumps(line), flush=True)
        return
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    torch.ops.load_library(so)
    op = torch.ops.recsys_ops.mha_fwd_with_mask
    names = [w.name] if args.workload != "standard" or args.only_headline else list(WORKLOADS)
    flush = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.int32, device=dev)
    results = {}
    for name in names:
        wl = WORKLOADS[name]
        q_h, k_h, v_h, m_h = make_inputs(wl, seed=42)
        q, k, v, m = (t.to(dev) for t in (q_h, k_h, v_h, m_h))
        for _ in range(max(3, args.warmup)):
            out = op(q, k, v, m)
        torch.cuda.synchronize(dev)
        ts = []
        for _ in range(args.steps):
            flush.zero_()
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            a.record()
            out = op(q, k, v, m)
            b.record()
            torch.cuda.synchronize(dev)
            ts.append(a.elapsed_time(b))
        mean_ms = sum(ts) / len(ts)
        mx, mean = oracle_slice_error(out, q_h, k_h, v_h, m_h, wl.B - 1, wl.H - 1)
        results[name] = {"shape": shape_str(wl), "us": mean_ms * 1e3, "us_median": statistics.median(ts) * 1e3,
                         "tflops_dense_convention": wl.flops / (mean_ms * 1e-3) / 1e12,
                         "gb_per_s": wl.bytes / (mean_ms * 1e-3) / 1e9,
                         "max_abs_vs_oracle": mx, "mean_abs_vs_oracle": mean}
        del q, k, v, m, out
    head = results[w.name]
    line.update({"value": head["tflops_dense_convention"], "unit": "TFLOPS", "n_gpus": 1, "steps": args.steps,
                 "warmup": max(3, args.warmup), "ms_per_step": head["us"] / 1e3, "higher_is_better": True,
                 "dtype": "bf16" if w.dtype == torch.bfloat16 else "fp16", "data": "synthetic",
                 "config": {"workload": w.name, "shape": shape_str(w),
                            "l2": "256 MB zero-fill before every timed step",
                            "library": "baseline/_ref/fa_so/recsys_fa_kernel.so (reference csrc/fa, -DFA_TARGETS=2, sm_100a)"},
                 "all_configs": results})
    print(json.dumps(line), flush=True)

# --------------------------------------------------------------------------- our arm
METRIC = "masked attn fwd TFLOPS (d128 B4 H16 S2048, 10% random mask)"


def shape_str(w):
    return (f"d{w.d} B{w.B} H{w.H} Hk{w.Hk} Sq{w.Sq} Sk{w.Sk} "
            f"{'bf16' if w.dtype == torch.bfloat16 else 'fp16'} mask={w.mask_kind}")


def run_ours(args, w):
    from custom_ops_b200 import _cabi, ops

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the sm_100a kernels have no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # Default: every rank owns its own batch shard of the same shape (weak scaling).
    # The long-context shape on several GPUs instead splits ONE problem's keys across the
    # ranks (strong scaling): local forward on the key slice, all-gather of the fp32
    # partials + LSE over NCCL, log-sum-exp merge.
    cross_split = (w.name == "splitkv_long" and world > 1)
    # --scaling strong: ONE problem, its (batch, kv-head) units spread over the ranks
    strong = (args.scaling == "strong" and world > 1 and not cross_split)
    q_h, k_h, v_h, m_h = make_inputs(w, seed=42 if (cross_split or strong) else 42 + rank)
    if strong:
        from custom_ops_b200 import parallel
        pieces = parallel.shard_inputs(q_h, k_h, v_h, m_h, world, rank)
        if len(pieces) != 1:
            raise SystemExit("--scaling strong: this rank's units span several batch elements or none; "
                             "use a rank count that divides the (batch, kv-head) units of one batch element")
        q_h, k_h, v_h, m_h = pieces[0]
        w_local = type(w)(w.name, q_h.shape[0], q_h.shape[1], k_h.shape[1], w.Sq, w.Sk, w.d, w.dtype, w.mask_kind,
                          w.sigma)
    elif cross_split:
        from custom_ops_b200 import parallel
        lo, hi = parallel.kv_slice_bounds(w.Sk, world, rank)
        k_h, v_h, m_h = (k_h[:, :, lo:hi].contiguous(), v_h[:, :, lo:hi].contiguous(),
                         m_h[:, :, :, lo:hi].contiguous())
        w_local = type(w)(w.name, w.B, w.H, w.Hk, w.Sq, hi - lo, w.d, w.dtype, w.mask_kind, w.sigma)
    else:
        w_local = w
    wl = w_local if strong else w          # the shape this rank launches
    q_h, k_h, v_h, m_h = (t.pin_memory() for t in (q_h, k_h, v_h, m_h))
    q, k, v, m = (t.to(dev, non_blocking=True) for t in (q_h, k_h, v_h, m_h))
    out = torch.empty_like(q)
    # HBM-bound workload: instead of the zero-fill flush (which leaves 126 MB of dirty lines
    # whose write-back then competes with the kernel's reads), every step reads one of several
    # copies of K, V and the mask, so that none of a step's inputs is in L2 when it starts.
    rotate = (w.name == "splitkv_long" and not cross_split)
    n_sets = 4 if rotate else 1
    sets = [(k, v, m)] + [(k.clone(), v.clone(), m.clone()) for _ in range(n_sets - 1)]
    out_h = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    flush = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.int32, device=dev)

    cargs = _cabi.make_args(
        q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), mask=m.data_ptr(), out=out.data_ptr(),
        batch=wl.B, heads=wl.H, heads_k=wl.Hk, seqlen_q=w.Sq, seqlen_k=w_local.Sk, head_dim=w.d,
        dtype=_cabi.BF16 if w.dtype == torch.bfloat16 else _cabi.FP16, device=local)
    plan = _cabi.plan(cargs)
    cargs_sets = [cargs]
    for ks, vs, ms in sets[1:]:
        cargs_sets.append(_cabi.make_args(
            q=q.data_ptr(), k=ks.data_ptr(), v=vs.data_ptr(), mask=ms.data_ptr(), out=out.data_ptr(),
            batch=wl.B, heads=wl.H, heads_k=wl.Hk, seqlen_q=w.Sq, seqlen_k=w_local.Sk, head_dim=w.d,
            dtype=_cabi.BF16 if w.dtype == torch.bfloat16 else _cabi.FP16, device=local))
    step_no = [0]
    ws_bytes = _cabi.workspace_bytes(cargs)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev)
    launches_per_step = (1 + (1 if plan.num_splits > 1 else 0) + (1 if plan.mask_repitched else 0)
                         + (1 if plan.tile_skip else 0))

    # --mask-as-rule (gqa_window only, whose mask is "causal, window of 512 keys"): the kernel-only
    # steps run the rule forward, which reads no mask at all; for profiling that kernel.
    as_rule = bool(getattr(args, "mask_as_rule", False)) and w.mask_kind == "causal_window" and not cross_split
    rule_ws = torch.empty(_cabi.RULE_WORKSPACE_BYTES, dtype=torch.uint8, device=dev)

    def step_kernel():
        if cross_split:
            return parallel.splitkv_forward(q, k, v, m)
        if as_rule:
            _cabi.forward_rule(cargs, 1, 512, 0, stream.cuda_stream, rule_ws.data_ptr(), _cabi.RULE_WORKSPACE_BYTES)
            return
        _cabi.forward(cargs_sets[step_no[0] % n_sets], ws.data_ptr(), ws_bytes, stream.cuda_stream)
        step_no[0] += 1

    from custom_ops_b200 import mha_fwd_with_mask_from_host

    def step_e2e():
        if cross_split:
            qd = q_h.to(dev, non_blocking=True)
            kd = k_h.to(dev, non_blocking=True)
            vd = v_h.to(dev, non_blocking=True)
            md = m_h.to(dev, non_blocking=True)
            out_h.copy_(parallel.splitkv_forward(qd, kd, vd, md), non_blocking=True)
        else:
            # the package's host-memory entry point: batch elements pipelined over three streams
            # (copy in / operator / copy out), the operator itself unchanged
            mha_fwd_with_mask_from_host(q_h, k_h, v_h, m_h, out_h, device=dev)

    ops.ensure_loaded("fa")
    if not ops.is_available("fa"):
        raise SystemExit(f"operator library failed to load: {ops.load_error('fa')}")

    # clocks are sampled from before the warm-up to after the last timed step
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        t_wait = time.time()
        while not sampler.lines and time.time() - t_wait < 3.0:
            time.sleep(0.05)

    for _ in range(max(3, args.warmup)):
        if not rotate:
            flush.zero_()                   # the warm-up steps are the timed steps, untimed
        step_kernel()
    torch.cuda.synchronize(dev)

    # ---- timed region 1: kernel-only, inputs resident in HBM
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    launches_before = _cabi.launch_count()
    # The synchronise + barrier above leaves the GPU idle long enough to drop its clocks, and the
    # first launch after it then runs several times slower than the rest; two untimed lead-in
    # steps, enqueued back to back with the timed ones, take that ramp.
    for i in range(-LEAD_IN_STEPS, args.steps):
        if not rotate:
            flush.zero_()                   # evict L2 between steps (outside the events)
        if i == 0:
            launches_before = _cabi.launch_count()
        if i >= 0:
            starts[i].record(stream)
        step_kernel()
        if i >= 0:
            ends[i].record(stream)
    barrier()
    kernel_launches = _cabi.launch_count() - launches_before
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    mean_ms = sum(step_ms) / len(step_ms)
    med_ms = statistics.median(step_ms)

    # ---- timed region 2: end to end from pinned host memory through the operator
    for _ in range(2):
        step_e2e()
    barrier()
    t0 = time.perf_counter()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step_e2e()
    e1.record(stream)
    barrier()
    e2e_ms = e0.elapsed_time(e1) / args.steps
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3 / args.steps

    clocks = sampler.stop() if rank == 0 else None
    status = _cabi.device_status(local, clear=True)
    if status != 0:
        raise SystemExit(f"device status word set ({status}): a kernel gave up on a bounded wait")

    if world > 1:
        t = torch.tensor([mean_ms, med_ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        mean_ms, med_ms, e2e_ms = (float(x) for x in t.tolist())

    # ---- after the headline regions: the other configurations and the multi-GPU sub-records
    peaks, peak_src = load_peaks()
    headline_err = oracle_slice_error(out, q_h, k_h, v_h, m_h, wl.B - 1, wl.H - 1) if not cross_split else None
    extra = {}
    sub_steps = max(5, min(args.steps, 10))
    if w.name == "standard" and not args.only_headline:
        del sets
        if world == 1:
            extra["all_configs"] = {name: measure_config(name, dev, sub_steps, peaks, flush)
                                    for name in ("plumbing", "gqa_window", "splitkv_long", "ragged_items")}
        else:
            if not strong:
                s_ms, s_mx, s_mean, n_jobs = measure_strong_scaling(w, dev, sub_steps, rank, world, flush, dist)
                extra["strong_scaling"] = {
                    "shape": shape_str(w), "ranks": world, "us": s_ms * 1e3,
                    "tflops": w.flops / (s_ms * 1e-3) / 1e12, "sub_problems_per_rank": n_jobs,
                    "partition": "(batch, kv-head) units of ONE problem, contiguous range per rank, no collective",
                    "max_abs_vs_oracle": s_mx, "mean_abs_vs_oracle": s_mean,
                    "l2": "256 MB zero-fill before every step",
                    "timing": "CUDA events per step on the launching stream, mean over steps, max over ranks"}
            # (a failure that every rank meets alike - a facility the box does not have - costs
            # this sub-record, not the line)
            try:
                extra["cross_gpu_splitkv"] = measure_cross_gpu_splitkv(dev, sub_steps, rank, world, dist)
            except Exception as exc:  # noqa: BLE001
                extra["cross_gpu_splitkv"] = {"error": f"{type(exc).__name__}: {exc}"}
        status = _cabi.device_status(local, clear=True)
        if status != 0:
            raise SystemExit(f"device status word set ({status}): a kernel gave up on a bounded wait")

    if rank == 0:
        total_flops = w.flops if (cross_split or strong) else w.flops * world
        value = total_flops / (mean_ms * 1e-3) / 1e12
        # Tile skipping: the headline value keeps the dense convention (4*B*H*Sq*Sk*d, mask
        # ignored, like the reference's benchmark); the tensor roofline uses the FLOPs of the
        # key blocks that are actually visited.
        visited_frac = visited_fraction(wl, m_h, 128 if plan.head_pairs else 256) if plan.tile_skip else 1.0
        hbm_bound = w.name == "splitkv_long"
        if hbm_bound:
            achieved = w_local.bytes / (mean_ms * 1e-3) / 1e9
            peak, unit, bound = peaks["hbm_gbs"], "GB/s", "hbm"
        else:
            # per GPU: a rank's own share of the work over the (max-over-ranks) step time
            achieved = wl.flops * visited_frac / (mean_ms * 1e-3) / 1e12
            peak, unit, bound = peaks["bf16_tflops"], "TFLOP/s", "tensor"
        in_bytes = sum(t.numel() * t.element_size() for t in (q_h, k_h, v_h, m_h))
        line = {
            "metric": METRIC if w.name == "standard" else f"masked attn fwd TFLOPS ({shape_str(w)})",
            "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": mean_ms, "median_ms_per_step": med_ms,
            "min_ms_per_step": min(step_ms), "max_ms_per_step": max(step_ms),
            "higher_is_better": True, "scaling": "strong" if (cross_split or strong) else "weak",
            "vs_baseline": None,
            "dtype": "bf16" if w.dtype == torch.bfloat16 else "fp16", "data": "synthetic",
            "config": {"workload": w.name, "shape": shape_str(w), "mask_as_rule": as_rule,
                       "parallelism": (f"keys split across {world} ranks, NCCL all-gather of fp32 "
                                       f"partials + LSE merge" if cross_split else
                                       f"(batch, kv-head) units of one problem spread over {world} rank(s), no collective"
                                       if strong else
                                       f"(batch, head) sharded, {world} rank(s), no collective"),
                       "global_batch": w.B if (cross_split or strong) else w.B * world, "l2": (f"{n_sets} rotating copies of K, V and mask ({n_sets * (w.bytes) / 1e6:.0f} MB in all, L2 is "
                              f"126 MB): no input of a step is in L2 when it starts; no flush kernel"
                              if rotate else "256 MB zero-fill before every timed step"),
                       "timing": ("CUDA events per step on the launching stream, mean over steps, max over ranks; "
                                  f"{LEAD_IN_STEPS} untimed lead-in steps after the barrier"),
                       "num_splits": plan.num_splits, "grid": plan.grid_x,
                       "tile_skip_eligible": bool(plan.tile_skip),
                       "kernels_per_step_max": launches_per_step},
            "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(w.name),
                         "peak_source": f"{peak_src} (MEASURED_PEAKS.json burst figure)"
                         if peak_src == "measured" else "fallback",
                         "algorithmic_flops": w_local.flops, "algorithmic_bytes": w_local.bytes,
                         "visited_block_fraction": visited_frac,
                         "note": "achieved = FLOPs of visited key blocks / kernel time" if not hbm_bound
                                 else "achieved = algorithmic bytes / time of attention + merge kernels"},
            "e2e": {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS",
                    "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_h.numel() * 2,
                    "ms_per_step": e2e_ms, "wall_ms_per_step": e2e_wall_ms,
                    "api": ("custom_ops_b200.parallel.splitkv_forward" if cross_split else
                            "custom_ops_b200.mha_fwd_with_mask_from_host: per batch element H2D, torch op "
                            "recsys_ops::mha_fwd_with_mask, D2H, pipelined over three streams")},
            "gpu_launches": kernel_launches,
            "clocks": clocks,
        }
        if headline_err is not None:
            line["max_abs_vs_oracle"], line["mean_abs_vs_oracle"] = headline_err
        line.update(extra)
        if world == 1 and not args.no_cpu_baseline:
            try:
                base = cpu_reference_sample(w, 3, 1)
                line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
                line["cpu_torch_fp32"] = torch_fp32_cpu_sample(w)
            except Exception as e:  # noqa: BLE001
                line["cpu_baseline"] = {"value": None, "unit": "TFLOPS", "cores": 0, "kind": "port",
                                        "sample": f"unavailable: {e}"}
        print(json.dumps(line), flush=True)

    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="standard", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-cuda"])
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="with --gpus N > 1: weak = every rank its own batch shard (default); strong = one "
                         "problem's (batch, kv-head) units spread over the ranks")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--mask-as-rule", action="store_true",
                    help="--workload gqa_window only: the kernel-only steps give the mask as a rule "
                         "(fa_mask_fwd_sm100_rule) instead of a tensor")
    ap.add_argument("--only-headline", action="store_true",
                    help="skip the all_configs / strong_scaling / cross_gpu_splitkv sub-records")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, w)
    elif args.impl == "reference-cuda":
        run_reference_cuda_arm(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
