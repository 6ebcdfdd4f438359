#!/usr/bin/env python
"""Benchmark of the Prism hot path: one step = forward + full backward (dA+dR, dB) of one Prism
linear layer on one batch of synthetic tokens.

Workload (default ``cfg2_m16384``): K=4096, N=14336, group_size=256, reconn_sz=16, bf16,
silu_gate, M=16384 tokens per GPU -- the configuration the headline metric is quoted on.
With N > 1 GPUs every rank processes its own batch of M tokens (weak scaling) and the parameter
gradients dR and dB are summed over ranks with an NCCL all-reduce inside the timed step.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5
    python bench.py --impl reference            # CPU arm: the reference's pytorch backend on the host cores
    python bench.py --workload cfg4 --gpus N    # GPT-2-small-shaped decoder, every linear a PrismLinear

Rank 0 prints ONE JSON line.  ``value`` = algorithmic TFLOP/s of the whole job with inputs resident
in HBM; ``e2e`` = the same through the public API with the step's inputs (A, dC) coming from pinned
host memory and its results (C, dA, dR, dB) copied back, copies inside the timed region.
Extra objects on the default line: ``sustained`` (the same step back to back for seconds, with the
clocks it settled at), ``small_m_fwd`` (decode-sized forward calls against the HBM roofline),
``train_cfg3`` (the 65536-token fp16 training step with its rows sharded over the ranks),
``cpu_baseline`` (the host-core baseline).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    "cfg2_m16384": dict(M=16384, K=4096, N=14336, gs=256, rs=16, dtype="bf16", act="silu_gate", dc_std=1.0),
    "cfg2_m4096": dict(M=4096, K=4096, N=14336, gs=256, rs=16, dtype="bf16", act="silu_gate", dc_std=1.0),
    "cfg2_m2048": dict(M=2048, K=4096, N=14336, gs=256, rs=16, dtype="bf16", act="silu_gate", dc_std=1.0),
    # cfg 2 with the input shuffle: every group's permutation folded into the parameters, i.e. the kernels run a
    # 64-wide rotation (rs) while the layer's algorithmic work is that of its 16-wide blocks (rs_algo)
    "cfg2_m16384_shuffle": dict(M=16384, K=4096, N=14336, gs=256, rs=64, rs_algo=16, shuffle=True, dtype="bf16",
                                act="silu_gate", dc_std=1.0),
    "cfg3_m8192": dict(M=8192, K=1024, N=16384, gs=256, rs=8, dtype="fp16", act="silu_gate", dc_std=0.1),
    "cfg1": dict(M=1024, K=256, N=1024, gs=256, rs=8, dtype="fp16", act="silu_gate", dc_std=1.0),
}
CFG3 = dict(M=65536, K=1024, N=16384, gs=256, rs=8, dtype="fp16", act="silu_gate", dc_std=0.1)
NOMINAL_TFLOPS = 2250.0
NCCL_CTAS = 8   # CTAs NCCL uses per collective: the all-reduce of dB runs beside the dA+dR kernel on the SMs its grid leaves free


def flops(w):
    dense = 2.0 * w["M"] * w["N"] * w["K"]
    bd = 2.0 * w["M"] * w["K"] * w.get("rs_algo", w["rs"]) * (w["N"] // w["gs"])
    gated = w["act"] is not None
    return {"fwd": dense + bd, "dadr": dense + 2 * bd, "db": dense if gated else 0.0}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return json.load(f), "measured"
    except (OSError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def ncu_traffic(kernel, workload):
    """DRAM read + write bytes per launch from the committed ncu summary table (null when the
    kernel / workload pair has not been captured)."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            table = json.load(f)
    except (OSError, ValueError):
        return None, None
    e = table.get("entries", {}).get(f"{kernel}@{workload}")
    if not e:
        return None, None
    return e.get("bytes_per_launch"), e.get("how")


# --------------------------------------------------------------------------- host placement
def _read(path):
    try:
        with open(path) as f:
            return f.read().strip()
    except OSError:
        return None


def _parse_cpulist(text):
    cpus = set()
    for part in (text or "").split(","):
        if "-" in part:
            a, b = part.split("-")
            cpus.update(range(int(a), int(b) + 1))
        elif part.strip():
            cpus.add(int(part))
    return cpus


def bind_to_gpu_numa_node(device_index):
    """Pin this process (and so its pinned host buffers, first touch) to the CPUs of the NUMA node the
    GPU hangs off: a pinned buffer on the far socket costs PCIe bandwidth."""
    info = {"numa_node": None, "bound": False, "cpus_before": len(os.sched_getaffinity(0))}
    try:
        bus = torch.cuda.get_device_properties(device_index).pci_bus_id
        dom = torch.cuda.get_device_properties(device_index).pci_domain_id
        dev = torch.cuda.get_device_properties(device_index).pci_device_id
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0/numa_node"
        node = _read(path)
        info["numa_node"] = int(node) if node is not None else None
        if info["numa_node"] is not None and info["numa_node"] >= 0:
            cpus = _parse_cpulist(_read(f"/sys/devices/system/node/node{info['numa_node']}/cpulist"))
            cpus &= os.sched_getaffinity(0)
            if cpus:
                os.sched_setaffinity(0, cpus)
                info["bound"] = True
    except Exception as e:   # placement is best effort
        info["error"] = str(e)[:80]
    info["cpus"] = len(os.sched_getaffinity(0))
    return info


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, device_index):
        super().__init__(daemon=True)
        self.samples, self.reasons, self.max_mhz, self.power = [], set(), None, []
        self._stop_evt = threading.Event()
        self.handle = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.handle = None

    def run(self):
        if self.handle is None:
            return
        nv = self.nv
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for b, name in self.REASONS.items():
                    if bits & b:
                        self.reasons.add(name)
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0)
            except Exception:
                pass
            self._stop_evt.wait(0.004)

    def stop(self):
        self._stop_evt.set()
        self.join(2.0)
        s = sorted(self.samples)
        p = sorted(self.power)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "sm_mhz_min": (s[0] if s else None), "sm_mhz_highest": (s[-1] if s else None),
                "reasons": sorted(self.reasons), "samples": len(s),
                "power_w_max": (p[-1] if p else None), "power_w_median": (p[len(p) // 2] if p else None)}


# --------------------------------------------------------------------------- CPU arm
def _reference_backend():
    """The reference's own pytorch backend, staged by oracle/stage_ref.py (git-ignored), or None."""
    path = os.path.join(ROOT, "oracle", "_ref", "cute_prism_pytorch_backend.py")
    if not os.path.exists(path):
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("_staged_reference_pytorch_backend", path)
    mod = importlib.util.module_from_spec(spec)
    try:
        spec.loader.exec_module(mod)
    except Exception:
        return None
    return mod


def cpu_step_fn(w, m_rows, threads):
    """One bounded sample of the workload on the host cores: forward + backward on m_rows tokens in
    fp32, by the reference's pytorch backend when it is staged, else by the oracle port."""
    from oracle import prism_oracle as O
    torch.set_num_threads(threads)
    A, B, R, dC = O.make_inputs(m_rows, w["K"], w["N"], w["gs"], w["rs"], seed=0, b_std=w["K"] ** -0.5,
                                dc_std=w["dc_std"])
    ref = _reference_backend()
    if ref is not None:
        def step():
            ref.pytorch_forward(A, B, R, w["gs"], w["rs"], activation=w["act"])
            ref.pytorch_backward(dC, A, B, R, w["gs"], w["rs"], activation=w["act"])
        return step, "reference"

    def step():
        O.prism_forward(A, B, R, w["gs"], w["rs"], w["act"])
        O.prism_backward(dC, A, B, R, w["gs"], w["rs"], w["act"])
    return step, "port"


def cpu_baseline(w, budget_s=12.0):
    """Host-core baseline on a bounded sample of the workload's tokens.  The sample is as large as the
    budget allows (at most 1024 rows): the reference's backward loops over every rotation block in
    Python, a fixed cost per call that a small sample would over-weigh."""
    threads = len(os.sched_getaffinity(0)) or 1
    m_rows = min(1024, w["M"])
    while True:
        step, kind = cpu_step_fn(w, m_rows, threads)
        t0 = time.perf_counter(); step(); t1 = time.perf_counter() - t0   # also the warm-up
        if t1 <= budget_s / 4 or m_rows <= 64:
            break
        m_rows //= 2
    ts = []
    for _ in range(3):
        t0 = time.perf_counter(); step(); ts.append(time.perf_counter() - t0)
    f = sum(flops(dict(w, M=m_rows)).values())
    what = "the reference's pytorch backend (src/cute_prism/_pytorch_backend.py)" if kind == "reference" else "the fp32 oracle port"
    return {"value": f / min(ts) / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": kind,
            "sample": f"fwd+bwd of {what} in fp32 on {m_rows} of {w['M']} tokens, best of 3"}, m_rows


def run_reference_arm(args, w, wname):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = len(os.sched_getaffinity(0)) or 1
    base, m_rows = cpu_baseline(w, budget_s=6.0)
    step, kind = cpu_step_fn(w, m_rows, threads)
    warm = min(max(args.warmup, 1), 2)
    for _ in range(warm):
        step()
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    val = sum(flops(dict(w, M=m_rows)).values()) / dt / 1e12
    what = "the reference's pytorch backend" if kind == "reference" else "the fp32 oracle port"
    line = {
        "impl": "reference", "metric": "prism_fwd_bwd_tflops", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(wname, w, 1, sample_rows=m_rows),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": kind,
                         "sample": f"each step = fwd+bwd of {what} in fp32 on {m_rows} of {w['M']} tokens"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(wname, w, world, **extra):
    """The same ``config`` keys for both arms."""
    cfg = {"workload": wname, "M_per_gpu": w["M"], "K": w["K"], "N": w["N"], "group_size": w["gs"],
           "reconn_sz": w["rs"], "activation": w["act"],
           "step": "forward + backward(dA+dR, dB)" + (" + NCCL all-reduce(dR, dB)" if world > 1 else "")}
    cfg.update(extra)
    return cfg


# --------------------------------------------------------------------------- GPU arm: pieces
def make_inputs(w, dev, rank, M=None):
    from oracle import prism_oracle as O  # seeded input generator only
    dt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    M = w["M"] if M is None else M
    K, N, gs, rs = w["K"], w["N"], w["gs"], w["rs"]
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    A = torch.randn(M, K, device=dev, generator=gen).to(dt)
    B = (torch.randn(N, K, device=dev, generator=torch.Generator(device=dev).manual_seed(7)) * K ** -0.5).to(dt)
    R = O.orthogonal_R(N // gs, K, w.get("rs_algo", rs), torch.Generator().manual_seed(0)).to(dt).to(dev)
    if w.get("shuffle"):
        from cute_mma_b200 import _shuffle
        masks, _ = _shuffle.build_shuffle_masks(K, N, gs, w["rs_algo"])
        fold = _shuffle.ShuffleFold(masks, K, gs, w["rs_algo"], dev)
        B, R = fold.fold_cols(B, gs), fold.fold_R(R)
    dC = (torch.randn(M, N, device=dev, generator=gen) * w["dc_std"]).to(dt)
    return A, B, R, dC


def make_step(w, A, B, R, dC, world, exchange="auto"):
    """One step on resident inputs: forward, dB (its all-reduce starts at once), dA+dR, all-reduce(dR)."""
    import cute_mma_b200 as cp
    from cute_mma_b200 import _functional as F
    gs, rs, act = w["gs"], w["rs"], w["act"]
    gate = 1 if act else 0
    # with more than one rank the dA+dR grid leaves NCCL the SMs its CTAs need, so that the
    # all-reduce of dB really runs beside the kernel instead of in front of its last CTAs
    dadr_cfg = None
    if world > 1:
        sms = torch.cuda.get_device_properties(A.device).multi_processor_count
        n_ft, pairs = (w["K"] + 127) // 128, (sms - NCCL_CTAS) // 2
        if n_ft <= pairs:
            runs = max(1, pairs // n_ft)
            extra = pairs - n_ft * runs
            dadr_cfg = [runs, 0 if extra > 0 else -1, max(extra, 0)]

    red_b = red_r = None
    if world > 1 and exchange in ("peer", "auto"):
        # the gradient sums over peer memory: the reduce kernels write their fp32 sums straight into buffers all
        # ranks can address, one kernel per rank adds its slice over the ranks in rank order (bit-identical on
        # every rank) and stores it everywhere; the dB exchange runs on a side stream beside the dA+dR kernel.
        # "auto": if the symmetric buffers cannot be set up on some rank, all ranks agree on NCCL instead.
        import torch.distributed as dist
        ok = 1
        try:
            red_b = cp.PeerGradReducer([tuple(B.shape)], out_dtype=A.dtype, ctas=NCCL_CTAS) if gate else None
            red_r = cp.PeerGradReducer([tuple(R.shape)], out_dtype=A.dtype, ctas=NCCL_CTAS)
        except Exception as e:   # noqa: BLE001 -- any set-up failure means "use NCCL", on every rank
            if exchange == "peer":
                raise
            print(f"[bench] peer exchange not available on rank {dist.get_rank()}: {e}", file=sys.stderr, flush=True)
            ok = 0
        flag = torch.tensor([ok], device=A.device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            red_b = red_r = None
    make_step.last_exchange = "peer" if red_r is not None else ("nccl" if world > 1 else None)
    if red_r is not None:
        side = torch.cuda.Stream()

        def step_peer(ev=None):
            if ev: ev[0].record()
            C, _ = cp.forward(A, B, R, gs, rs, activation=act)
            if ev: ev[1].record()
            dB = None
            if gate:
                F._backward_db(dC, A, R, gs, rs, gate, out_dtype=torch.float32, dB_out=red_b.inputs()[0])
                ready = torch.cuda.Event()
                ready.record()
                with torch.cuda.stream(side):
                    side.wait_event(ready)
                    dB = red_b.reduce()[0]
            if ev: ev[2].record()
            dA, _ = F._backward_dadr(dC, A, B, R, gs, rs, gate, tile_cfg=dadr_cfg, dR_dtype=torch.float32,
                                     dR_out=red_r.inputs()[0])
            if ev: ev[3].record()
            dR = red_r.reduce()[0]
            torch.cuda.current_stream().wait_stream(side)
            return C, dA, dR, dB
        return step_peer

    def step(ev=None):
        if ev: ev[0].record()
        C, _ = cp.forward(A, B, R, gs, rs, activation=act)
        if ev: ev[1].record()
        dB = F._backward_db(dC, A, R, gs, rs, gate) if gate else None
        fin_b = cp.allreduce_grads([dB], async_op=True) if world > 1 else None
        if ev: ev[2].record()
        dA, dR = F._backward_dadr(dC, A, B, R, gs, rs, gate, tile_cfg=dadr_cfg)
        if ev: ev[3].record()
        if world > 1:
            fin_r = cp.allreduce_grads([dR], async_op=True)
            fin_b(); fin_r()
        return C, dA, dR, dB
    return step


def timed_steps(step, n_steps, world, sampler_index=None, with_events=True):
    """(ms per step [max over ranks], per-kernel ms, clocks) of exactly n_steps, CUDA events,
    barrier + synchronize on both sides."""
    import torch.distributed as dist
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(n_steps)] if with_events else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(sampler_index) if sampler_index is not None else None
    if sampler:
        sampler.start()
    e0.record()
    for i in range(n_steps):
        step(evs[i] if evs else None)
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    ms = e0.elapsed_time(e1) / n_steps
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    parts = None
    if evs:
        parts = {"prism_fwd": sum(e[0].elapsed_time(e[1]) for e in evs) / n_steps,
                 "prism_bwd_db": sum(e[1].elapsed_time(e[2]) for e in evs) / n_steps,
                 "prism_bwd_dadr": sum(e[2].elapsed_time(e[3]) for e in evs) / n_steps}
    return ms, parts, clocks


def run_e2e(args, w, dev, world, A, B, R, dC, step_flops):
    """The same step through cute_mma_b200.forward / backward with host buffers.  Every step's
    tokens are processed as micro-batches (gradient accumulation).  The host->device copy of
    micro-batch i+1, the kernels of micro-batch i and the device->host copy of micro-batch i-1 run on
    three streams, so PCIe traffic in both directions overlaps the compute; the stream of
    micro-batches runs on across step boundaries and the host waits once, after the last step."""
    import cute_mma_b200 as cp
    dt = A.dtype
    M, K = A.shape
    N = B.shape[0]
    gs, rs, act = w["gs"], w["rs"], w["act"]
    gate = 1 if act else 0
    e_steps = max(2, min(args.steps, 8))
    n_mb = 8 if M % 8 == 0 and M >= 8192 else (4 if M % 4 == 0 and M >= 4096 else 1)
    mb = M // n_mb
    A_h, dC_h = A.cpu().pin_memory(), dC.cpu().pin_memory()
    C_h = torch.empty(M, N, dtype=dt, pin_memory=True)
    dA_h = torch.empty(M, K, dtype=dt, pin_memory=True)
    dR_h = torch.empty(R.shape, dtype=dt, pin_memory=True)
    dB_h = torch.empty(B.shape, dtype=dt, pin_memory=True) if gate else None
    s_in, s_out, s_cmp = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    n_buf = 3
    A_d = [torch.empty(mb, K, dtype=dt, device=dev) for _ in range(n_buf)]
    dC_d = [torch.empty(mb, N, dtype=dt, device=dev) for _ in range(n_buf)]
    dR_acc = [torch.zeros(R.shape, dtype=torch.float32, device=dev) for _ in range(2)]
    dB_acc = [torch.zeros(B.shape, dtype=torch.float32, device=dev) for _ in range(2)] if gate else None
    grads_out = [None, None]   # events: the step's gradients have left the accumulator pair

    # plain copy rates of this box with these buffers (what bounds the end-to-end step)
    def copy_rate(dst, src, reps=3):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize()
        return src.numel() * src.element_size() * reps / (time.perf_counter() - t0) / 1e9
    dC_full = torch.empty_like(dC)
    dC_full.copy_(dC_h, non_blocking=True)
    h2d_gbs = copy_rate(dC_full, dC_h)
    d2h_gbs = copy_rate(C_h, dC_full)
    # the step copies in both directions at once: the two rates with both directions busy (two streams,
    # in the step's byte ratio: the shorter direction is repeated until the longer one is done)
    def both_rates(reps=3):
        up = torch.empty_like(dC)
        sa, sb = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        torch.cuda.synchronize()
        with torch.cuda.stream(sa):
            e[0].record(sa)
            for _ in range(reps):
                up.copy_(dC_h, non_blocking=True)
            e[1].record(sa)
        with torch.cuda.stream(sb):
            e[2].record(sb)
            for _ in range(reps):
                C_h.copy_(dC_full, non_blocking=True)
            e[3].record(sb)
        torch.cuda.synchronize()
        nbytes = dC.numel() * dC.element_size() * reps
        return nbytes / (e[0].elapsed_time(e[1]) * 1e-3) / 1e9, nbytes / (e[2].elapsed_time(e[3]) * 1e-3) / 1e9
    h2d_gbs_both, d2h_gbs_both = both_rates()
    del dC_full

    def e2e_steps(n_steps):
        buf_free = [None] * n_buf
        it = 0
        for st in range(n_steps):
            acc = st % 2
            if grads_out[acc] is not None:
                s_cmp.wait_event(grads_out[acc])
            dR_acc[acc].zero_()
            if gate:
                dB_acc[acc].zero_()
            for i in range(n_mb):
                sl = slice(i * mb, (i + 1) * mb)
                bi = it % n_buf
                with torch.cuda.stream(s_in):
                    if buf_free[bi] is not None:
                        s_in.wait_event(buf_free[bi])      # the kernels that read this buffer are done
                    A_d[bi].copy_(A_h[sl], non_blocking=True)
                    dC_d[bi].copy_(dC_h[sl], non_blocking=True)
                    ready = torch.cuda.Event()
                    ready.record(s_in)
                s_cmp.wait_event(ready)
                Ci, _ = cp.forward(A_d[bi], B, R, gs, rs, activation=act)
                # the fp32 sums of the reduce kernels go straight into the fp32 accumulators
                dAi, dRi, dBi, _ = cp.backward(dC_d[bi], A_d[bi], B, R, gs, rs, activation=act,
                                               dR_dtype=torch.float32, dB_dtype=torch.float32)
                dR_acc[acc].add_(dRi)
                if gate:
                    dB_acc[acc].add_(dBi)
                buf_free[bi] = torch.cuda.Event()
                buf_free[bi].record(s_cmp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(buf_free[bi])
                    C_h[sl].copy_(Ci, non_blocking=True)
                    dA_h[sl].copy_(dAi, non_blocking=True)
                Ci.record_stream(s_out)                    # keep the blocks until the copies have run
                dAi.record_stream(s_out)
                it += 1
            dR_out = dR_acc[acc].to(dt)                    # gradients leave in the parameters' dtype
            dB_out = dB_acc[acc].to(dt) if gate else None
            done = torch.cuda.Event()
            done.record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                dR_h.copy_(dR_out, non_blocking=True)
                dR_out.record_stream(s_out)
                if gate:
                    dB_h.copy_(dB_out, non_blocking=True)
                    dB_out.record_stream(s_out)
                grads_out[acc] = torch.cuda.Event()
                grads_out[acc].record(s_out)
        torch.cuda.synchronize()

    e2e_steps(2)
    t0 = time.perf_counter()
    e2e_steps(e_steps)
    e_ms = (time.perf_counter() - t0) / e_steps * 1e3
    cp.check_device_status()
    h2d = int((A_h.numel() + dC_h.numel()) * 2)
    d2h = int(C_h.numel() * 2 + dA_h.numel() * 2 + dR_h.numel() * 2 + (dB_h.numel() * 2 if gate else 0))
    copy_bound_ms = max(h2d / h2d_gbs, d2h / d2h_gbs) / 1e6
    copy_bound_both_ms = max(h2d / h2d_gbs_both, d2h / d2h_gbs_both) / 1e6
    return {"value": world * step_flops / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e_ms, "steps": e_steps,
            "micro_batches": n_mb,
            "h2d_gbs_achieved": h2d / (e_ms * 1e-3) / 1e9, "d2h_gbs_achieved": d2h / (e_ms * 1e-3) / 1e9,
            "h2d_gbs_plain_copy": h2d_gbs, "d2h_gbs_plain_copy": d2h_gbs,
            "copy_bound_ms": copy_bound_ms, "ms_over_copy_bound": e_ms / copy_bound_ms,
            "h2d_gbs_plain_copy_both_directions": h2d_gbs_both, "d2h_gbs_plain_copy_both_directions": d2h_gbs_both,
            "copy_bound_both_directions_ms": copy_bound_both_ms,
            "ms_over_copy_bound_both_directions": e_ms / copy_bound_both_ms,
            "note": "cute_mma_b200.forward/backward per micro-batch with A, dC from pinned host memory; C, dA "
                    "copied back per micro-batch, dR, dB (accumulated in fp32, cast to 16 bit) once per step; copies "
                    "and kernels of neighbouring micro-batches and steps overlap on three streams, one host wait after "
                    "the last step; copy_bound_ms = the slower direction's bytes at this box's plain pinned-copy rate"}


def run_small_m_sweep(w, dev, B, R, peaks):
    """Streaming kernel (path 2) against the general tiled kernel (path 1) over token counts: the
    measurement behind the default switch-over and the shipped tile-table entries."""
    import cute_mma_b200 as cp
    dt = B.dtype
    N, K = B.shape
    gs, rs, act = w["gs"], w["rs"], w["act"]
    flush = torch.empty(384 * 1024 * 1024, dtype=torch.uint8, device=dev)
    flush_words = flush.view(torch.int32)
    gen = torch.Generator(device=dev).manual_seed(99)
    rows = []
    for m in (1, 8, 16, 32, 48, 64, 96, 128):
        A_s = torch.randn(m, K, device=dev, generator=gen).to(dt)
        row = {"M": m}
        for path, name in ((2, "streaming_us"), (1, "general_us")):
            cfg = [0, 0, 0, path]
            for _ in range(3):
                cp.forward(A_s, B, R, gs, rs, activation=act, tile_cfg=cfg)
            ts = []
            for _ in range(8):
                flush.fill_(1)
                flush_words.sum()
                t0e, t1e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0e.record()
                cp.forward(A_s, B, R, gs, rs, activation=act, tile_cfg=cfg)
                t1e.record()
                torch.cuda.synchronize()
                ts.append(t0e.elapsed_time(t1e) * 1e3)
            ts.sort()
            row[name] = {"min": ts[0], "median": ts[len(ts) // 2]}
        rows.append(row)
    cp.check_device_status()
    return rows


def run_small_m(w, dev, B, R, peaks):
    """Decode-sized forward calls: HBM-bound, minimum traffic B + R + A + C.  L2 (126 MB) would
    otherwise keep most of B (117 MB) between iterations: before every timed call a 384 MB buffer is
    written and then read back once (the read pass leaves L2 full of clean lines of that buffer;
    after the write pass alone the timed call would also pay for writing 126 MB of dirty lines back)."""
    import cute_mma_b200 as cp
    dt = B.dtype
    N, K = B.shape
    gs, rs, act = w["gs"], w["rs"], w["act"]
    flush = torch.empty(384 * 1024 * 1024, dtype=torch.uint8, device=dev)
    flush_words = flush.view(torch.int32)
    gen = torch.Generator(device=dev).manual_seed(99)
    small = []
    for m in (1, 16, 128):
        A_s = torch.randn(m, K, device=dev, generator=gen).to(dt)
        for _ in range(3):
            cp.forward(A_s, B, R, gs, rs, activation=act)
        ts = []
        for _ in range(10):
            flush.fill_(1)
            flush_words.sum()
            t0e, t1e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0e.record()
            cp.forward(A_s, B, R, gs, rs, activation=act)
            t1e.record()
            torch.cuda.synchronize()
            ts.append(t0e.elapsed_time(t1e) * 1e3)
        ts.sort()
        nbytes = (B.numel() + R.numel() + m * K + m * N) * 2
        med = ts[len(ts) // 2]
        small.append({"M": m, "us_median": med, "us_min": ts[0], "bytes": nbytes,
                      "gbs": nbytes / (med * 1e-6) / 1e9,
                      "frac_of_measured_hbm": nbytes / (med * 1e-6) / 1e9 / peaks["hbm_gbs"]})
    cp.check_device_status()
    return {"note": "forward only, cold L2 (384 MB written, then read, before each call), CUDA events, 10 calls",
            "hbm_peak_gbs": peaks["hbm_gbs"], "calls": small}


def run_train_cfg3(dev, rank, world, local_rank, exchange="auto"):
    """The 65536-token fp16 training step (K=1024, N=16384, gs=256, rs=8, silu_gate) with its token rows
    split evenly over the ranks: forward, dB, all-reduce(dB) beside dA+dR, all-reduce(dR).  Strong
    scaling: tokens/s of the whole job; rank 0 also times the unsplit step on its own GPU, which gives
    the speed-up on this very box."""
    import torch.distributed as dist
    w = dict(CFG3)
    rows = w["M"] // world
    wl = dict(w, M=rows)
    A, B, R, dC = make_inputs(wl, dev, rank)
    step = make_step(wl, A, B, R, dC, world, exchange)
    for _ in range(3):
        step()
    n = 6
    ms, parts, _ = timed_steps(step, n, world)
    out = {"workload": "cfg3 (M=65536 split over the ranks)", "rows_per_gpu": rows, "ms_per_step": ms,
           "tokens_per_s": w["M"] / (ms * 1e-3), "tflops": sum(flops(w).values()) / (ms * 1e-3) / 1e12,
           "kernels_ms": parts, "scaling": "strong",
           "exchange": ("NCCL all-reduce of dB (33.5 MB fp16) beside the dA+dR kernel, then of dR (1 MB)"
                        if make_step.last_exchange != "peer" else
                        "prism_peer_reduce over peer memory: fp32 dB sums (67 MB) added in rank order beside the dA+dR kernel, then dR")}
    del A, dC, step
    torch.cuda.empty_cache()
    if world > 1:
        # the unsplit step on one GPU of the same box (every rank runs it, so no rank idles into a timeout)
        A, _, _, dC = make_inputs(w, dev, rank)
        step1 = make_step(w, A, B, R, dC, 1)
        for _ in range(2):
            step1()
        ms1, _, _ = timed_steps(step1, 4, 1)
        t = torch.tensor([ms1], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out["n1_ms_per_step_same_box"] = float(t.item())
        out["speedup_vs_n1"] = float(t.item()) / ms
        del A, dC, step1
        torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------- cfg 4: GPT-2-small-shaped decoder
def run_cfg4(args, dev, rank, world, local_rank):
    """GPT-2-small-shaped decoder (12 layers, d_model 768, 12 heads, sequence 1024, vocabulary 50304,
    random init, bf16) whose attention QKV / attention projection / MLP up / MLP down linears are
    plain-mode PrismLinear(group_size=256, reconn_sz=8): R starts as identity blocks, B frozen, R, the
    biases, the layer norms and the embeddings are trained with AdamW on uniformly random token ids;
    global batch 64 sequences, sequences sharded over the ranks, gradients averaged by all-reduce.
    Attention, norms and the tied LM head are PyTorch ops (outside the Prism path)."""
    import torch.distributed as dist
    import torch.nn as nn
    import torch.nn.functional as TF
    import cute_mma_b200 as cp
    from cute_mma_b200 import _functional as F

    d, heads, layers, seq, vocab, gbatch = 768, 12, 12, 1024, 50304, args.cfg4_sequences
    if gbatch % world:
        raise SystemExit("cfg4: the global batch of 64 sequences must divide over the ranks")
    per_rank = gbatch // world
    micro = min(per_rank, 16)
    n_micro = per_rank // micro

    def plin(i, o):
        return cp.PrismLinear(i, o, group_size=256, reconn_sz=8, activation=None, bias=True)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
            self.qkv, self.proj = plin(d, 3 * d), plin(d, d)
            self.up, self.down = plin(d, 4 * d), plin(4 * d, d)

        def forward(self, x):
            b, t, _ = x.shape
            q, k, v = self.qkv(self.ln1(x)).split(d, dim=2)
            q, k, v = [z.view(b, t, heads, d // heads).transpose(1, 2) for z in (q, k, v)]
            y = TF.scaled_dot_product_attention(q, k, v, is_causal=True)
            x = x + self.proj(y.transpose(1, 2).reshape(b, t, d))
            return x + self.down(TF.gelu(self.up(self.ln2(x))))

    class GPT(nn.Module):
        def __init__(self):
            super().__init__()
            self.wte, self.wpe = nn.Embedding(vocab, d), nn.Embedding(seq, d)
            self.blocks = nn.ModuleList(Block() for _ in range(layers))
            self.ln_f = nn.LayerNorm(d)

        def forward(self, idx, targets):
            pos = torch.arange(idx.shape[1], device=idx.device)
            x = self.wte(idx) + self.wpe(pos)
            for blk in self.blocks:
                x = blk(x)
            logits = TF.linear(self.ln_f(x), self.wte.weight)   # tied head
            return TF.cross_entropy(logits.float().view(-1, vocab), targets.reshape(-1))

    torch.manual_seed(0)
    model = GPT().to(dev).to(torch.bfloat16)
    with torch.no_grad():
        model.wte.weight.normal_(std=0.02)
        model.wpe.weight.normal_(std=0.02)
    params = [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(params, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)

    # time spent inside the library's kernels: events around every call into it
    spans, timing = [], [True]

    def spanned(fn):
        def wrapped(*a, **k):
            if not timing[0]:
                return fn(*a, **k)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn(*a, **k)
            e1.record()
            spans.append((e0, e1))
            return r
        return wrapped
    F.forward, F._backward_dadr, F._backward_db, F.bias_grad = (spanned(F.forward), spanned(F._backward_dadr),
                                                                spanned(F._backward_db), spanned(F.bias_grad))

    static_idx = torch.zeros(n_micro, micro, seq + 1, dtype=torch.long, device=dev)

    def fwd_bwd():
        last = None
        for i in range(n_micro):
            last = model(static_idx[i, :, :-1], static_idx[i, :, 1:]) / n_micro
            last.backward()
        return last

    def finish_step():
        cp.sync_module_grads(model, average=True)
        opt.step()
        opt.zero_grad(set_to_none=False)   # the gradient buffers stay where they are (the graph adds into them)

    def eager_step():
        static_idx.random_(0, vocab, generator=gen)
        loss = fwd_bwd()
        finish_step()
        return loss

    for _ in range(max(args.warmup, 3)):
        eager_step()
    torch.cuda.synchronize()
    cp.check_device_status()
    # one eager step with an event pair around every call into the library: the time inside its kernels
    spans.clear()
    eager_step()
    torch.cuda.synchronize()
    prism_ms = sum(a.elapsed_time(b) for a, b in spans)
    timing[0] = False

    # The forward + backward of all micro-batches as one CUDA graph: at 8 sequences per GPU the step is
    # bound by the host issuing ~10^4 small PyTorch launches, not by the GPU.  The all-reduce and the
    # optimizer stay outside the graph.  If anything on the path cannot be captured the step stays eager.
    graph, graph_note, static_loss = None, "eager", None
    if not args.no_cuda_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    fwd_bwd()
                    opt.zero_grad(set_to_none=False)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_loss = fwd_bwd()
            graph_note = "forward+backward of the step's micro-batches replayed as one CUDA graph"
        except Exception as e:   # noqa: BLE001
            graph, graph_note = None, "eager (capture failed: %s)" % str(e).splitlines()[0][:120]
            torch.cuda.synchronize()
            opt.zero_grad(set_to_none=False)

    def step():
        if graph is None:
            return eager_step()
        static_idx.random_(0, vocab, generator=gen)
        graph.replay()
        finish_step()
        return static_loss

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    steps = max(2, min(args.steps, 10))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0.record()
    for _ in range(steps):
        loss = step()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    cp.check_device_status()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank != 0:
        return
    tokens = gbatch * seq
    # Prism linears only, plain mode: forward (dense + bd) + dA+dR (dense + 2 bd) per layer and token
    fl = 0.0
    for k_, n_ in ((d, 3 * d), (d, d), (d, 4 * d), (4 * d, d)):
        f = flops(dict(M=tokens, K=k_, N=n_, gs=256, rs=8, act=None))
        fl += layers * (f["fwd"] + f["dadr"])
    line = {
        "metric": "train_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "cfg4", "layers": layers, "d_model": d, "heads": heads, "seq_len": seq, "vocab": vocab,
                   "global_batch_sequences": gbatch, "sequences_per_gpu": per_rank, "micro_batch": micro,
                   "prism": "QKV 768->2304, proj 768->768, up 768->3072, down 3072->768: PrismLinear(gs=256, rs=8, plain), "
                            "B frozen; R, biases, layer norms, embeddings trained (AdamW, fused)"},
        "loss": float(loss.item()) * n_micro, "launch": graph_note,
        "prism_kernels_ms_per_step": prism_ms, "prism_share_of_step": prism_ms / ms,
        "prism_tflops_in_kernels": fl / world / (prism_ms * 1e-3) / 1e12 if prism_ms > 0 else None,
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="cfg2_m16384", choices=sorted(WORKLOADS) + ["cfg4"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-small-m", action="store_true")
    ap.add_argument("--no-sustained", action="store_true")
    ap.add_argument("--no-train-cfg3", action="store_true")
    ap.add_argument("--small-m-sweep", action="store_true",
                    help="only time the few-token forward, streaming against general kernel, and print the table")
    ap.add_argument("--grad-exchange", default="auto", choices=["auto", "nccl", "peer"],
                    help="N > 1: how dB / dR are summed over the ranks: this library's kernel over peer memory "
                         "(cute_mma_b200.PeerGradReducer: fp32 sums added in rank order), NCCL all-reduce, or auto: "
                         "peer memory if every rank can set it up, else NCCL")
    ap.add_argument("--no-cuda-graph", action="store_true", help="cfg4: issue the step eagerly")
    ap.add_argument("--cfg4-sequences", type=int, default=64, help="cfg4: global batch in sequences (64 = the configuration)")
    args = ap.parse_args()
    if args.impl == "reference":
        w = WORKLOADS[args.workload if args.workload in WORKLOADS else "cfg2_m16384"]
        run_reference_arm(args, w, args.workload)
        return
    if args.warmup < 3:
        args.warmup = 3

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    placement = bind_to_gpu_numa_node(local_rank)

    import torch.distributed as dist
    import cute_mma_b200 as cp
    from cute_mma_b200 import _lib
    if world > 1:
        # a fixed, small number of NCCL CTAs: the all-reduce of dB runs beside the persistent dA+dR
        # kernel, whose grid leaves exactly these SMs free (see make_step).  Measured on 8 GPUs: the
        # sharded cfg-3 step 1.20 ms against 1.41 ms with NCCL's default CTA count on a full dA+dR grid
        # (the weak-scaling step is the same either way)
        opts = dist.ProcessGroupNCCL.Options()
        opts.config.max_ctas = NCCL_CTAS
        opts.config.min_ctas = NCCL_CTAS
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)
    if args.workload == "cfg4":
        run_cfg4(args, dev, rank, world, local_rank)
        if world > 1:
            dist.destroy_process_group()
        return

    wname = args.workload
    w = WORKLOADS[wname]
    if args.small_m_sweep:
        _, B, R, _ = make_inputs(dict(w, M=16), dev, rank)
        print(json.dumps({"small_m_sweep": run_small_m_sweep(w, dev, B, R, measured_peaks()[0]),
                          "config": workload_config(wname, w, 1)}), flush=True)
        return
    A, B, R, dC = make_inputs(w, dev, rank)
    fl = flops(w)
    step_flops = sum(fl.values())
    step = make_step(w, A, B, R, dC, world, args.grad_exchange)
    exchange_used = make_step.last_exchange
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    cp.check_device_status()

    launches0 = _lib.lib().prism_launch_count()
    ms, parts_ms, clocks = timed_steps(step, args.steps, world, sampler_index=local_rank)
    launches = _lib.lib().prism_launch_count() - launches0
    cp.check_device_status()

    # the same step back to back for a few seconds: the clocks and the rate the GPU settles at
    sustained = None
    if not args.no_sustained:
        n_sus = max(args.steps, int(math.ceil(2500.0 / max(ms, 1e-3))))
        ms_s, parts_s, clocks_s = timed_steps(step, n_sus, world, sampler_index=local_rank)
        sustained = {"steps": n_sus, "seconds": ms_s * n_sus / 1e3, "ms_per_step": ms_s,
                     "value": world * step_flops / (ms_s * 1e-3) / 1e12, "unit": "TFLOP/s",
                     "kernels_ms": parts_s, "clocks": clocks_s}

    train_cfg3 = None
    if not args.no_train_cfg3 and wname == "cfg2_m16384":
        del step
        train_cfg3 = run_train_cfg3(dev, rank, world, local_rank, args.grad_exchange)

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    value = world * step_flops / (ms * 1e-3) / 1e12
    peaks, peak_kind = measured_peaks()
    flops_of = {"prism_bwd_dadr": fl["dadr"], "prism_fwd": fl["fwd"], "prism_bwd_db": fl["db"]}
    dom = max(parts_ms, key=lambda k: parts_ms[k])   # the kernel with the largest share of the step
    achieved = flops_of[dom] / (parts_ms[dom] * 1e-3) / 1e12
    burst, sust = peaks["bf16_tflops"], peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
    # the denominator follows the clocks of the timed region: a short region at (nearly) full SM clock
    # compares with the burst GEMM figure, a power-capped one with the sustained figure
    region_s = ms * args.steps / 1e3
    at_burst = bool(clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz")
                    and clocks["sm_mhz"] >= 0.9 * clocks["sm_max_mhz"] and region_s < 1.0)
    peak = burst if at_burst else sust
    traffic, traffic_how = ncu_traffic(dom, wname)
    roofline = {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_how,
                "peak_source": f"{peak_kind} cuBLAS bf16 GEMM, " + ("burst figure (timed region %.2f s at a median %s MHz)" % (region_s, clocks and clocks.get("sm_mhz")) if at_burst
                                                                   else "sustained figure (timed region %.2f s at a median %s MHz)" % (region_s, clocks and clocks.get("sm_mhz"))),
                "frac_of_burst": achieved / burst, "frac_of_sustained": achieved / sust,
                "frac_of_nominal": achieved / NOMINAL_TFLOPS,
                "ms_per_launch": parts_ms[dom], "kernels_ms": parts_ms,
                "kernels_tflops": {k: (flops_of[k] / (v * 1e-3) / 1e12 if v > 0 else None) for k, v in parts_ms.items()}}

    line = {
        "metric": "prism_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": workload_config(wname, w, world,
                                  l2="inputs larger than L2 (A+B+dC = %.0f MB per step), no flush"
                                     % ((A.numel() + B.numel() + dC.numel()) * 2 / 1e6)),
        "tokens_per_s": world * w["M"] / (ms * 1e-3),
        "frac_of_nominal_peak": value / world / NOMINAL_TFLOPS,
        "frac_of_measured_burst": value / world / burst,
        "frac_of_measured_sustained": value / world / sust,
        "roofline": roofline, "clocks": clocks, "gpu_launches": int(launches), "host": placement,
    }
    if world > 1:
        line["grad_exchange"] = exchange_used
    if sustained:
        sustained["frac_of_measured_sustained"] = sustained["value"] / world / sust
        sustained["frac_of_nominal_peak"] = sustained["value"] / world / NOMINAL_TFLOPS
        line["sustained"] = sustained
    if train_cfg3:
        line["train_cfg3"] = train_cfg3
    if not args.no_e2e:
        line["e2e"] = run_e2e(args, w, dev, world, A, B, R, dC, step_flops)
    if not args.no_small_m and wname.startswith("cfg2"):
        line["small_m_fwd"] = run_small_m(w, dev, B, R, peaks)
    if not args.no_cpu_baseline:
        line["cpu_baseline"], _ = cpu_baseline(w)

    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
