#!/usr/bin/env python
"""Benchmark of the NVFP4 attention forward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl ours|reference]

One "step" is one forward over the (batch, kv-head) units a rank holds.  At N = 1 the workload is
the causal GQA prefill configuration (B=4, Hq=32, Hkv=8, S=8192, D=128, the one the 50 %-of-FP4-peak
target is quoted on).  With N > 1 (launched by torch.distributed.run, one rank per GPU) the SAME
problem is dealt over the ranks: it is quantised once (tensor scales from the whole tensors), its
B * Hkv = 32 units go 32 / 16 / 8 / 4 per GPU (flash_attention_b200.shard), every rank times its
shard with nothing exchanged on the data path, and value = FLOPs of the whole problem / max-over-
ranks time: strong scaling.  Outside the timed region the shards of O and LSE are all-gathered
over NCCL, rank 0 compares them bit for bit with the un-sharded call and checks sampled windows
against exact attention (``verified``).  ``--scaling weak`` runs one whole problem per rank
instead (replicas).

Rank 0 prints ONE JSON line.  ``value`` is measured with inputs resident in HBM (scale factors
already tiled, one kernel launch per step, CUDA events around each launch, L2 flushed between
launches).  ``e2e`` is the same metric through the public Python API with HOST buffers: pinned
host -> device copies of the packed operands and linear scale factors, the scale-factor tiling
kernels, the attention kernel, and the device -> host copy of O and LSE, all inside the timed
region.  ``cpu_baseline`` / ``--impl reference`` time the CPU restatement of the reference's
``attention_ref`` (oracle/nvfp4_oracle.py) on a bounded sample of the same workload.

``--workload sweep`` (head dims 64 / 128 / 192 x sequence lengths x causal) and ``--workload
decode`` (one query token against a long KV cache: decode kernel beside the prefill kernel's
split-KV path, GB/s of K/V) print one JSON line each with a table; ``--kernel ws128`` forces the
128-key prefill kernel on the main workloads.
"""
import argparse
import datetime
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, Hq, Hkv, S, D, causal, v_std, outlier_frac)
    "cfg0": (1, 4, 4, 256, 128, False, 1.0, 0.0),
    "cfg1": (4, 32, 32, 4096, 128, False, 1.0, 0.0),
    "cfg2": (4, 32, 8, 8192, 128, True, 0.5, 0.0),
    "cfg3": (1, 64, 8, 32768, 128, True, 1.0, 0.01),
}
FP4_NOMINAL_TFLOPS = 9000.0   # B200 dense FP4 (4 x the 2.25 PFLOP/s dense bf16)


def parse_workload(name):
    if name in WORKLOADS:
        return WORKLOADS[name]
    if name.startswith("custom:"):  # custom:B,Hq,Hkv,S,causal(0/1)   (D = 128)
        b, hq, hkv, sq, c = (int(x) for x in name[7:].split(","))
        return (b, hq, hkv, sq, 128, bool(c), 1.0, 0.0)
    if name.startswith("sweep:"):  # sweep:D,S,causal(0/1)  with B*H = 128 (H = 16, B = 8)
        d, s, c = (int(x) for x in name[6:].split(","))
        return (8, 16, 16, s, d, bool(c), 1.0, 0.0)
    raise SystemExit(f"unknown workload {name}")


def flops_of(B, Hq, S, D, causal, Dv=None):
    avg = S / 2 if causal else S                  # flash_attn/cute/bench_utils.py:15-38, Sq == Sk
    return B * Hq * 2 * S * avg * (D + (D if Dv is None else Dv))


def algorithmic_bytes(B, Hq, Hkv, S, D, Dv=None):
    Dv = D if Dv is None else Dv
    per = lambda h, d: B * S * h * (d // 2 + d // 16)       # packed values + block scales
    return per(Hq, D) + per(Hkv, D) + per(Hkv, Dv) + B * S * Hq * Dv * 2 + B * Hq * S * 4


def gpu_busy_while_host_enqueues():
    """A ~150 us spin on the GPU in front of a timed call that is synchronised every step: the host
    enqueues the start event, the kernels and the stop event while the GPU is still busy, so the
    event pair brackets device work only and not the host's launch path (for calls of 30-500 us the
    Python side otherwise adds an idle gap to what the events see)."""
    torch.cuda._sleep(300_000)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"bf16_tflops": d["bf16_tflops"], "hbm_gbs": d["hbm_gbs"], "source": "measured",
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"])}
    return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle's restatement of attention_ref on a bounded sample
# ------------------------------------------------------------------------------------------------
def cpu_sample_inputs(wl, seed=0):
    B, Hq, Hkv, S, D, causal, v_std, _ = wl
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, S, 1, D, generator=g).bfloat16()
    k = torch.randn(1, S, 1, D, generator=g).bfloat16()
    v = (torch.randn(1, S, 1, D, generator=g) * v_std).bfloat16()
    from flash_attention_b200 import quantize_qkv
    Q, K, V = quantize_qkv(q, k, v)
    return Q.dequantize(), K.dequantize(), V.dequantize()


def cpu_reference_step(qd, kd, vd, causal):
    from oracle import nvfp4_oracle as orc
    return orc.attention_oracle_a(qd, kd, vd, causal=causal)


def time_cpu(wl, steps, warmup):
    """One step = one (batch, query-head) pair of the workload at full sequence length."""
    B, Hq, Hkv, S, D, causal, _, _ = wl
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    qd, kd, vd = cpu_sample_inputs(wl)
    for _ in range(warmup):
        cpu_reference_step(qd, kd, vd, causal)
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_reference_step(qd, kd, vd, causal)
        ts.append(time.perf_counter() - t0)
    fl = flops_of(1, 1, S, D, causal)
    mean = sum(ts) / len(ts)
    return {"value": fl / mean / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"1 of {B * Hq} (batch, query-head) pairs at full S={S}, D={D}, "
                      f"causal={causal}; {steps} timed passes after {warmup} warm-up; "
                      f"fp32 attention_ref restatement on dequantised NVFP4 inputs",
            "ms_per_pass": mean * 1e3}


def run_reference_arm(args, wl, rank, world):
    if rank != 0:
        return
    B, Hq, Hkv, S, D, causal, _, _ = wl
    steps = max(1, args.steps)
    cb = time_cpu(wl, steps, args.warmup)
    line = {
        "impl": "reference", "metric": "nvfp4_attn_fwd_tflops", "value": cb["value"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_pass"],
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(args.workload, wl, world, args.scaling),
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tokens_per_s": S / (cb["ms_per_pass"] * 1e-3) / Hq,
    }
    print(json.dumps(line), flush=True)


def workload_config(name, wl, world, scaling="strong"):
    """The ``config`` both arms print: same ``workload`` string for the same run."""
    B, Hq, Hkv, S, D, causal, v_std, outl = wl
    if scaling == "strong":
        per = B * Hkv // world if (B * Hkv) % world == 0 else None
        work = (f"one problem B={B}, Hq={Hq}, Hkv={Hkv}, Sq=Sk={S}, D={D}, causal={causal}, its {B * Hkv} "
                f"(batch, kv-head) units dealt over {world} GPU(s), {per} per GPU")
        sharding = (f"(batch, kv-head) units of ONE problem, {per} per GPU, no collective on the data path; NCCL "
                    "all-gather of O / LSE for verification only")
        gb = B
    else:
        work = f"B={B} per GPU (global batch {B * world}), Hq={Hq}, Hkv={Hkv}, Sq=Sk={S}, D={D}, causal={causal}"
        sharding = f"(batch, kv-head) units, {B * Hkv} per GPU (one whole problem per GPU), no collective on the data path"
        gb = B * world
    return {"workload": f"{name}: NVFP4 attention forward, {work}",
            "global_batch": gb, "Hq": Hq, "Hkv": Hkv, "seq_len": S, "head_dim": D,
            "causal": causal, "v_std": v_std, "outlier_frac": outl, "sharding": sharding,
            "l2": "L2 flushed between timed launches (256 MiB write)"}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi clock / throttle-reason samples; only those stamped inside the timed region count."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.QUERY}",
                                       "--format=csv,noheader,nounits", "-lms", "20"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self, t_begin, t_end):
        """t_begin / t_end: datetime.now() taken around the timed region."""
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        rows = [r.strip().split(", ") for r in open(self.f.name) if r.strip()]
        os.unlink(self.f.name)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        parsed = []
        for r in rows:
            if len(r) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(r[0].strip(), "%Y/%m/%d %H:%M:%S.%f")
                parsed.append((ts, float(r[1]), float(r[2]), float(r[3]),
                               [nm for nm, val in zip(names, r[5:9]) if val.strip().lower() == "active"]))
            except ValueError:
                continue
        inside = [x for x in parsed if t_begin <= x[0] <= t_end]
        window = "timed region"
        if not inside:                      # region shorter than the sampling interval
            inside, window = parsed[-3:], "last samples before the region ended"
        sm = [x[1] for x in inside]
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max((x[2] for x in inside), default=None),
                "power_w_max": max((x[3] for x in inside), default=None),
                "samples": len(inside), "samples_total": len(parsed), "window": window,
                "reasons": sorted({nm for x in inside for nm in x[4]})}


def numa_pin(local_rank):
    """Run this rank on the CPUs of its GPU's NUMA node, so that the pinned host buffers it
    allocates afterwards (first touch) sit next to the GPU's PCIe root.  Returns a note."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        bus = pynvml.nvmlDeviceGetPciInfo(h).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        bus = bus.lower()
        if len(bus.split(":")[0]) == 8:           # 00000000:1B:00.0 -> 0000:1b:00.0
            bus = bus[4:]
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        if node < 0:
            return "single NUMA node"
        cpus = open(f"/sys/devices/system/node/node{node}/cpulist").read().strip()
        ids = []
        for part in cpus.split(","):
            a, _, b = part.partition("-")
            ids += list(range(int(a), int(b or a) + 1))
        allowed = sorted(set(ids) & os.sched_getaffinity(0))
        if allowed:
            os.sched_setaffinity(0, allowed)
            return f"NUMA node {node}, cpus {cpus}"
        return f"NUMA node {node} (its cpus are outside this process's affinity mask)"
    except Exception as e:                        # nothing here may stop the benchmark
        return f"not pinned ({type(e).__name__})"


def blocks_of(B, Hq, S, causal):
    """128 x 128 score blocks the kernel visits (whole diagonal blocks count)."""
    m = (S + 127) // 128
    per_head = m * (m + 1) // 2 if causal else m * m
    return B * Hq * per_head


def sampled_window_check(fa, Ql, Kl, Vl, out, lse, samples, causal, group):
    """max relative O error and max LSE error of sampled 128-row windows against exact attention
    (fp64, on the GPU) on the dequantised operands."""
    dev = out.device
    S = Kl.data.shape[1]
    D = Ql.data.shape[-1] * 2
    worst_o, worst_l = 0.0, 0.0
    for (b, h, r0) in samples:
        hk = h // group
        sk = r0 + 128 if causal else S
        qd = fa.dequantize_lastdim(Ql.data[b, r0:r0 + 128, h], Ql.sf[b, r0:r0 + 128, h], Ql.scale).double()
        kd = fa.dequantize_lastdim(Kl.data[b, :sk, hk], Kl.sf[b, :sk, hk], Kl.scale).double()
        vd = fa.dequantize_lastdim(Vl.data[b, hk, :, :sk // 2], Vl.sf[b, hk, :, :sk // 16], Vl.scale).double().T
        s = (qd @ kd.T) / math.sqrt(D)
        if causal:
            rows = torch.arange(r0, r0 + 128, device=dev)[:, None]
            s = s.masked_fill(torch.arange(sk, device=dev)[None, :] > rows, float("-inf"))
        ref_l = torch.logsumexp(s, dim=-1)
        ref_o = torch.softmax(s, dim=-1) @ vd
        got_o, got_l = out[b, r0:r0 + 128, h].double(), lse[b, h, r0:r0 + 128].double()
        worst_o = max(worst_o, ((got_o - ref_o).norm() / ref_o.norm()).item())
        worst_l = max(worst_l, (got_l - ref_l).abs().max().item())
    return worst_o, worst_l


def run_gpu_arm(args, wl, rank, local_rank, world):
    import torch.distributed as dist
    import flash_attention_b200 as fa
    from flash_attention_b200 import shard as sh
    B, Hq, Hkv, S, D, causal, v_std, outl = wl
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    strong = args.scaling == "strong"
    numa_note = numa_pin(local_rank) if world > 1 else "one rank"
    sampler = ClockSampler(local_rank) if rank == 0 else None   # started early: its first sample is slow

    # ---- synthetic inputs.  strong: ONE problem of the workload's size, quantised on rank 0 (tensor
    # scales computed on the whole tensors), broadcast, and every rank keeps its (batch, kv-head)
    # units.  weak: every rank draws its own problem of that size (replicas).
    def draw(seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        q = torch.randn(B, S, Hq, D, generator=g, device=dev, dtype=torch.bfloat16)
        k = torch.randn(B, S, Hkv, D, generator=g, device=dev, dtype=torch.bfloat16)
        v = (torch.randn(B, S, Hkv, D, generator=g, device=dev) * v_std).bfloat16()
        if outl > 0:
            n = max(1, int(round(outl * D)))
            for t in (q, k):
                idx = torch.randperm(D, generator=g, device=dev)[:n]
                t[..., idx] *= 20.0
        return q, k, v

    quant_ms = quant_bytes = None
    if strong:
        u8 = torch.uint8
        shapes = [(B, S, Hq, D // 2), (B, S, Hkv, D // 2), (B, Hkv, D, S // 2),
                  (B, S, Hq, D // 16), (B, S, Hkv, D // 16), (B, Hkv, D, S // 16)]
        scales = torch.zeros(3, dtype=torch.float64, device=dev)
        if rank == 0:
            q, k, v = draw(1000)
            Qf, Kf, Vf = fa.quantize_qkv_fused(q, k, v)          # linear + tiled scale factors
            for _ in range(2):
                fa.quantize_qkv_fused(q, k, v, linear_sf=False)
            qe0, qe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            qe0.record()
            for _ in range(5):
                fa.quantize_qkv_fused(q, k, v, linear_sf=False)
            qe1.record()
            torch.cuda.synchronize()
            quant_ms = qe0.elapsed_time(qe1) / 5
            n_el = q.numel() + k.numel() + v.numel()
            quant_bytes = n_el * (2 + 2) + n_el // 2 + n_el // 16     # two bf16 reads, packed + tiled scales
            del q, k, v
            bufs = [Qf.data, Kf.data, Vf.data, Qf.sf, Kf.sf, Vf.sf]
            scales.copy_(torch.tensor([Qf.scale, Kf.scale, Vf.scale], dtype=torch.float64))
        else:
            bufs = [torch.empty(s_, dtype=u8, device=dev) for s_ in shapes]
        if world > 1:
            for t in bufs:
                dist.broadcast(t, 0)
            dist.broadcast(scales, 0)
        sc = [float(x) for x in scales.cpu()]
        Qg = fa.NVFP4Tensor(bufs[0], bufs[3], sc[0])
        Kg = fa.NVFP4Tensor(bufs[1], bufs[4], sc[1])
        Vg = fa.NVFP4Tensor(bufs[2], bufs[5], sc[2], is_v=True)
        plan = sh.plan_shard(B, Hkv, world, rank)
        Qs, Ks, Vs = sh.shard_operands(Qg, Kg, Vg, plan)          # views: strided head / batch slices
    else:
        q, k, v = draw(1000 + rank)
        Qs, Ks, Vs = fa.quantize_qkv(q, k, v)
        del q, k, v
        plan = sh.Shard(rank, world, 0, B, 0, Hkv)
        Qg, Kg, Vg = Qs, Ks, Vs
    Bs, Hq_s, Hkv_s = Qs.data.shape[0], Qs.data.shape[2], Ks.data.shape[2]
    Qt, Kt, Vt = (fa.NVFP4Tensor(t.data, t.tiled_sf(), t.scale, True, t.is_v) for t in (Qs, Ks, Vs))
    out = torch.empty(Bs, S, Hq_s, D, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(Bs, Hq_s, S, dtype=torch.float32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    variant = fa.VARIANT_WS if args.kernel == "ws128" else fa.VARIANT_AUTO

    def step():
        fa.flash_attn_fp4_func(Qt.data, Kt.data, Vt.data, Qt.sf, Kt.sf, Vt.sf, Qt.scale, Kt.scale,
                               Vt.scale, causal=causal, return_lse=True, out=out, lse=lse,
                               sf_layout="tiled", variant=variant)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    fa.check_status(dev)

    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(args.steps)]
    barrier()
    torch.cuda.nvtx.range_push("timed")          # lets a profiler select the timed region
    t_begin = datetime.datetime.now()
    t_wall0 = time.perf_counter()
    for e0, e1 in evs:
        flush.zero_()
        e0.record()
        step()
        e1.record()
    barrier()
    torch.cuda.nvtx.range_pop()
    t_wall = time.perf_counter() - t_wall0
    dev_ms = sum(e0.elapsed_time(e1) for e0, e1 in evs)
    clocks = sampler.stop(t_begin, datetime.datetime.now()) if sampler else None
    fa.check_status(dev)
    # ---- sustained mode: launches back to back for a few seconds (no flush between them; the
    # operands of one launch exceed L2), clocks sampled throughout: what a serving loop sees once
    # the power cap has pulled the clock down
    sustained = None
    if args.sustained > 0:
        samp2 = ClockSampler(local_rank) if rank == 0 else None
        n_launch = max(10, int(args.sustained * 1e3 / (dev_ms / args.steps)))
        barrier()
        tb = datetime.datetime.now()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(n_launch):
            step()
        s1.record()
        barrier()
        sus_ms = s0.elapsed_time(s1) / n_launch
        sustained = {"launches": n_launch, "ms_per_step": sus_ms,
                     "clocks": samp2.stop(tb, datetime.datetime.now()) if samp2 else None}
        fa.check_status(dev)

    # ---- verification (outside every timed region): all-gather O / LSE of the shards over NCCL,
    # rank 0 compares with the un-sharded call it computes itself (must be bit-identical) and checks
    # sampled windows against exact attention on the dequantised operands
    verified = None
    if strong:
        full_o, full_l = (sh.gather_output(out, lse, plan, B, Hq, Hkv) if world > 1 else (out, lse))
        if rank == 0:
            if world > 1:
                ref_o, ref_l = fa.flash_attn_func(Qg, Kg, Vg, causal=causal, return_lse=True)
                torch.cuda.synchronize()
                same = bool(torch.equal(ref_o, full_o) and torch.equal(ref_l, full_l))
                del ref_o, ref_l
            else:
                same = True
            samples = [(0, 0, 0), (B - 1, Hq - 3, (S // 2 // 128) * 128), (B // 2, Hq // 2, S - 128)]
            err_o, err_l = sampled_window_check(fa, Qg, Kg, Vg, full_o, full_l, samples, causal, Hq // Hkv)
            verified = {"ok": bool(same and err_o < 0.2 and err_l < 1e-3),
                        "sharded_equals_unsharded_bitwise": same, "gathered_with": "nccl all_gather" if world > 1 else "n/a",
                        "max_rel_err_o_vs_exact": err_o, "max_abs_err_lse_vs_exact": err_l,
                        "tolerance": "rel-RMS(O) < 0.2 per sampled 128-row window (4-bit P), |dLSE| < 1e-3"}
        del full_o, full_l

    # ---- end to end through the public API with host buffers (this rank's shard)
    host_in = [t.contiguous().cpu().pin_memory() for t in (Qs.data, Ks.data, Vs.data, Qs.sf, Ks.sf, Vs.sf)]
    host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    host_lse = torch.empty(lse.shape, dtype=lse.dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = host_out.numel() * 2 + host_lse.numel() * 4

    pipe = fa.HostPipeline(Bs, S, S, Hq_s, Hkv_s, D, D, device=dev)

    def e2e_step():
        # public host-buffer API: copy-in, scale tiling, attention and copy-out of row ranges on
        # three streams; every step moves all inputs in and the whole result out
        pipe.run(*host_in, Qs.scale, Ks.scale, Vs.scale, host_out, host_lse, causal=causal)

    e2e_steps = max(2, min(args.steps, 10))
    e2e_step()
    pipe.wait()
    barrier()
    cur = torch.cuda.current_stream(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(cur)
    for _ in range(e2e_steps):
        e2e_step()
    cur.wait_event(pipe.done)
    e1.record(cur)
    barrier()
    pipe.wait()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    fa.check_status(dev)
    mma_rate = fa.measure_fp4_mma_rate(device=dev) if rank == 0 else None
    ex2_rate = fa.measure_ex2_rate(device=dev) if rank == 0 else None

    sus_ms = sustained["ms_per_step"] if sustained else 0.0
    times = torch.tensor([dev_ms, e2e_ms, sus_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, sus_ms = (float(x) for x in times.cpu())
    if rank == 0:
        fl_job = flops_of(B, Hq, S, D, causal) * (1 if strong else world)
        fl_rank = fl_job / world
        ms_per_step = dev_ms / args.steps
        tflops_total = fl_job / (ms_per_step * 1e-3) / 1e12
        tflops_gpu = tflops_total / world
        peaks = measured_peaks()
        fp4_peak = 4.0 * peaks["bf16_tflops"]
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        blocks_rank = blocks_of(Bs, Hq_s, S, causal)
        tiles_rank = Bs * Hq_s * ((S + 127) // 128)
        sm_mhz = (clocks or {}).get("sm_mhz") or 0.0
        clk_per_block = ms_per_step * 1e-3 * sm_mhz * 1e6 / (blocks_rank / sms) if sm_mhz else None
        # exponential roofline: one exp2 per score; the hardware unit's measured rate, the share
        # of the exponentials this build moves to the FMA pipe, and the ceiling that leaves
        emu_mask = fa.lib().fa4_nvfp4_query(101)
        emu_share = bin(emu_mask).count("1") / 8.0
        exp_ceiling = None
        if ex2_rate and sm_mhz:
            clk_floor = 128 * 128 * (1.0 - emu_share) / ex2_rate["per_clk_per_sm"]
            exp_ceiling = sms * 4.0 * 128 * 128 * D * sm_mhz * 1e6 / clk_floor / 1e12
        cfg = dict(workload_config(args.workload, wl, world, args.scaling),
                   kernel="attn_fwd_ws64_kernel (automatic choice)" if args.kernel == "auto"
                   else "attn_fwd_ws_kernel<128> (forced)",
                   B_per_gpu=Bs, units_per_gpu=Bs * Hkv_s, tiles_per_gpu=tiles_rank,
                   tiles_per_cta=tiles_rank / min(sms, tiles_rank),
                   blocks_128x128_per_sm=blocks_rank / sms, host_numa=numa_note)
        line = {
            "metric": "nvfp4_attn_fwd_tflops", "value": tflops_total, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "nvfp4", "data": "synthetic",
            "config": cfg,
            "tflops_per_gpu": tflops_gpu,
            "tokens_per_s": B * S * (1 if strong else world) / (ms_per_step * 1e-3),
            "pct_fp4_peak_nominal": 100.0 * tflops_gpu / FP4_NOMINAL_TFLOPS,
            "clk_per_block": clk_per_block,
            "roofline": {
                "bound": "tensor", "achieved": tflops_gpu, "peak": fp4_peak, "unit": "TFLOP/s",
                "frac": tflops_gpu / fp4_peak,
                "peak_note": f"4 x the {peaks['source']} cuBLAS bf16 burst figure "
                             f"({peaks['bf16_tflops']} TFLOP/s): block-scaled e2m1 MMAs issue at 4x the "
                             f"bf16 rate; nominal dense FP4 is {FP4_NOMINAL_TFLOPS} TFLOP/s",
                "fp4_mma_rate_measured": mma_rate,
                "frac_of_measured_fp4_mma_rate": tflops_gpu / mma_rate["tflops"],
                "exp": {"ex2_per_clk_per_sm_measured": ex2_rate["per_clk_per_sm"] if ex2_rate else None,
                        "emulated_share": emu_share, "ceiling_tflops": exp_ceiling,
                        "frac": tflops_gpu / exp_ceiling if exp_ceiling else None,
                        "note": "one exp2 per score; ceiling = FLOPs of a 128x128 block / (its hardware exp2 / "
                                "measured rate) at the sampled SM clock"},
                **traffic_record(args.workload),
                "algorithmic_bytes": algorithmic_bytes(B, Hq, Hkv, S, D) // (world if strong else 1),
                "hbm_gbs_achieved": algorithmic_bytes(B, Hq, Hkv, S, D) / (world if strong else 1)
                                    / (ms_per_step * 1e-3) / 1e9,
            },
            "e2e": {"value": fl_job / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "h2d_gbs_per_rank": h2d / (e2e_ms * 1e-3) / 1e9, "d2h_gbs_per_rank": d2h / (e2e_ms * 1e-3) / 1e9,
                    "launches_per_step": Bs * len(pipe.ranges) * 5,
                    "pieces_per_step": Bs * len(pipe.ranges),
                    "note": "HostPipeline on this rank's shard: pinned host buffers, copy-in / compute / copy-out of "
                            "query-row ranges on three streams, successive steps overlap; bytes are per rank"},
            "gpu_launches": args.steps,
            "wall_ms_timed_region": t_wall * 1e3,
            "clocks": clocks,
        }
        if verified is not None:
            line["verified"] = verified["ok"]
            line["verification"] = verified
        if quant_ms is not None:
            line["quantizer"] = {"ms": quant_ms, "algorithmic_bytes": quant_bytes,
                                 "gbs": quant_bytes / (quant_ms * 1e-3) / 1e9,
                                 "frac_of_hbm_peak": quant_bytes / (quant_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                 "note": "fused bf16 -> NVFP4 quantiser of q, k, v of the whole problem on rank 0 "
                                         "(6 launches + one scale read-back), outside the timed region"}
        if sustained:
            sus_tf = fl_job / (sus_ms * 1e-3) / 1e12 / world
            sus_peak = 4.0 * peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
            smhz = (sustained["clocks"] or {}).get("sm_mhz") or 0.0
            line["sustained"] = {"seconds_requested": args.sustained, "launches": sustained["launches"],
                                 "ms_per_step": sus_ms, "tflops_per_gpu": sus_tf, "peak": sus_peak,
                                 "frac": sus_tf / sus_peak,
                                 "clk_per_block": sus_ms * 1e-3 * smhz * 1e6 / (blocks_rank / sms) if smhz else None,
                                 "clocks": sustained["clocks"],
                                 "note": "back-to-back launches, no L2 flush (one launch's operands exceed L2); peak = "
                                         "4 x the measured sustained cuBLAS bf16 figure"}
        if world == 1 and not args.no_cpu:
            cb = time_cpu(wl, 3, 1)
            line["cpu_baseline"] = {k2: cb[k2] for k2 in ("value", "unit", "cores", "kind", "sample")}
            line["cpu_baseline"]["note"] = ("a rate on ONE (batch, head) pair; ms_per_step of the CPU arm and of this "
                                            "arm are not comparable, the TFLOP/s are")
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def kernel_source_hash():
    """SHA-256 of the CUDA sources with `//` comments and blank lines removed: what identifies the
    code an ncu capture was taken on (a reworded comment does not make the capture stale)."""
    import hashlib
    import re
    h = hashlib.sha256()
    csrc = os.path.join(ROOT, "flash_attention_b200", "csrc")
    for name in sorted(os.listdir(csrc)):
        h.update(name.encode())
        for line in open(os.path.join(csrc, name), encoding="utf-8"):
            code = re.sub(r"\s*//.*$", "", line.rstrip("\n")).rstrip()
            if code:
                h.update(code.encode() + b"\n")
    return h.hexdigest()


def traffic_record(workload):
    """DRAM bytes per launch of the attention kernel from the ncu capture recorded in
    profiles/traffic.json, with the hash of the kernel sources it was captured on; a capture of
    other sources is reported as stale."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        rec = json.load(open(path)).get(workload)
    except (OSError, ValueError):
        rec = None
    if not rec:
        return {"traffic": None}
    return {"traffic": rec["bytes"], "traffic_note": rec.get("note"),
            "traffic_stale": rec.get("source_sha256") != kernel_source_hash()}


def run_sweep(args):
    """Head-dim and shape sweep (B * H = 128 as B = 8, H = 16): every point is timed like the main
    arm (resident inputs, L2 flush between launches, CUDA events); ONE JSON line with the table.
    With N ranks every point is ONE problem whose 128 (batch, head) units are dealt 128 / N per GPU
    (whole batch entries; the tensor scales come from the whole tensors, which every rank draws
    from the same seed); a point's time is the maximum over the ranks."""
    import torch.distributed as dist
    import flash_attention_b200 as fa
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if 8 % world != 0:
        raise SystemExit("the sweep deals 8 batch entries: 1, 2, 4 or 8 GPUs")
    peaks = measured_peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    steps = max(3, min(args.steps, 20))
    for D in (64, 128, 192):
        Dv = 128 if D == 192 else D               # 192 pairs with a V / O head dim of 128
        for S in (1024, 2048, 4096, 16384):
            for causal in (False, True):
                B, H = 8, 16
                g = torch.Generator(device=dev).manual_seed(7)
                q, k = (torch.randn(B, S, H, D, generator=g, device=dev, dtype=torch.bfloat16) for _ in range(2))
                v = torch.randn(B, S, H, Dv, generator=g, device=dev, dtype=torch.bfloat16)
                Q, K, V = fa.quantize_qkv_fused(q, k, v, linear_sf=False)
                del q, k, v
                b0, b1 = rank * (B // world), (rank + 1) * (B // world)      # this rank's batch entries
                Q, K, V = (fa.NVFP4Tensor(t.data[b0:b1], t.sf[b0:b1], t.scale, True, t.is_v) for t in (Q, K, V))
                out = torch.empty(b1 - b0, S, H, Dv, dtype=torch.bfloat16, device=dev)
                lse = torch.empty(b1 - b0, H, S, dtype=torch.float32, device=dev)

                def step():
                    fa.flash_attn_fp4_func(Q.data, K.data, V.data, Q.sf, K.sf, V.sf, Q.scale, K.scale, V.scale,
                                           causal=causal, return_lse=True, out=out, lse=lse, sf_layout="tiled")
                for _ in range(3):
                    step()
                torch.cuda.synchronize()
                ms = 0.0
                for _ in range(steps):
                    flush.zero_()
                    gpu_busy_while_host_enqueues()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(); step(); e1.record(); e1.synchronize()
                    ms += e0.elapsed_time(e1)
                ms /= steps
                fa.check_status(dev)
                if world > 1:
                    tmax = torch.tensor([ms], dtype=torch.float64, device=dev)
                    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
                    ms = float(tmax.item())
                fl, by = flops_of(B, H, S, D, causal, Dv), algorithmic_bytes(B, H, H, S, D, Dv)
                rows.append({"D": D, "Dv": Dv, "S": S, "causal": causal, "ms": ms, "tflops": fl / ms / 1e9,
                             "pct_fp4_peak_nominal": 100 * fl / ms / 1e9 / world / FP4_NOMINAL_TFLOPS,
                             "frac_of_4x_bf16_measured": fl / ms / 1e9 / world / (4 * peaks["bf16_tflops"]),
                             "hbm_gbs": by / ms / 1e6, "frac_of_hbm_peak": by / ms / 1e6 / world / peaks["hbm_gbs"]})
                del Q, K, V, out, lse
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return
    head = next(r for r in rows if r["D"] == 128 and r["S"] == 4096 and r["causal"])
    print(json.dumps({"metric": "nvfp4_attn_fwd_tflops", "value": head["tflops"], "unit": "TFLOP/s",
                      "n_gpus": world, "steps": steps, "warmup": 3, "ms_per_step": head["ms"],
                      "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4",
                      "data": "synthetic",
                      "config": {"workload": "sweep: D in {64, 128, 192 (with Dv = 128)} x S in {1024, 2048, 4096, "
                                             "16384} x causal / non-causal, B = 8, H = 16 (B * H = 128); "
                                             "headline row D=128, S=4096, causal",
                                 "l2": "L2 flushed between timed launches (256 MiB write)"},
                      "gpu_launches": steps * len(rows), "sweep": rows}), flush=True)


def run_fa4_bf16(args):
    """Same-box comparator: the reference's own Blackwell forward (flash_attn.cute.flash_attn_func,
    flash_attn/cute/interface.py:1753, BF16, CuTe-DSL JIT) on the DEQUANTISED operands of the
    benchmark configurations, rounded to bf16 -- the kernel the NVFP4 path sits beside.  Needs the
    reference's `flash_attn/cute` package installed into baseline/_ref (pip install --no-index
    --no-build-isolation --no-deps --target baseline/_ref <copy of flash_attn/cute>) and a GPU;
    prints {"impl": "fa4_bf16", "unavailable": ...} otherwise.  Timed like the main arm (resident
    inputs, warm-up 5, L2 flush between launches, CUDA events), one JSON line with a table."""
    import types
    ref_root = os.path.join(ROOT, "baseline", "_ref", "flash_attn")
    if not os.path.isdir(os.path.join(ref_root, "cute")):
        print(json.dumps({"impl": "fa4_bf16", "unavailable": "baseline/_ref/flash_attn/cute is not installed"}))
        return
    try:
        # the image also carries another `flash_attn` distribution: bind the name to the installed
        # reference package explicitly
        pkg = types.ModuleType("flash_attn")
        pkg.__path__ = [ref_root]
        sys.modules["flash_attn"] = pkg
        from flash_attn.cute.interface import flash_attn_func as ref_func
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "fa4_bf16", "unavailable": f"import failed: {type(e).__name__}: {e}"[:300]}))
        return
    import flash_attention_b200 as fa
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    steps = max(3, min(args.steps, 20))
    points = [("cfg1", WORKLOADS["cfg1"]), ("cfg2", WORKLOADS["cfg2"])]
    points += [(f"sweep D=128 S={S} causal={c}", (8, 16, 16, S, 128, c, 1.0, 0.0))
               for S in (1024, 2048, 4096, 16384) for c in (False, True)]
    rows = []

    def sm_clock():
        try:
            r = subprocess.run(["nvidia-smi", "--id=0", "--query-gpu=clocks.sm", "--format=csv,noheader,nounits"],
                               capture_output=True, text=True, timeout=10)
            return float(r.stdout.strip().splitlines()[0])
        except Exception:  # noqa: BLE001
            return None

    def timed(fn):
        """mean ms per call and the SM clock sampled while a further batch of calls is in flight.
        Half a second of idle first: the two kernels are timed in turn, and a measurement that
        starts right behind the other kernel's batch inherits its power state (measured: up to 20 %
        on the 0.45 ms points)."""
        torch.cuda.synchronize()
        time.sleep(0.5)
        ms = 0.0
        for _ in range(steps):
            flush.zero_()
            gpu_busy_while_host_enqueues()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record(); e1.synchronize()
            ms += e0.elapsed_time(e1)
        for _ in range(20):
            fn()
        mhz = sm_clock()
        torch.cuda.synchronize()
        return ms / steps, mhz

    for name, (B, Hq, Hkv, S, D, causal, v_std, _) in points:
        g = torch.Generator(device=dev).manual_seed(1000)
        q = torch.randn(B, S, Hq, D, generator=g, device=dev, dtype=torch.bfloat16)
        k = torch.randn(B, S, Hkv, D, generator=g, device=dev, dtype=torch.bfloat16)
        v = (torch.randn(B, S, Hkv, D, generator=g, device=dev) * v_std).bfloat16()
        Q, K, V = fa.quantize_qkv_fused(q, k, v)
        del q, k, v
        qd, kd, vd = (t.dequantize().bfloat16() for t in (Q, K, V))      # (B, S, H, D) bf16
        row = {"workload": name, "B": B, "Hq": Hq, "Hkv": Hkv, "S": S, "D": D, "causal": causal}
        fl = flops_of(B, Hq, S, D, causal)
        # this repository's kernel on the quantised operands
        out = torch.empty(B, S, Hq, D, dtype=torch.bfloat16, device=dev)
        Qt, Kt, Vt = (fa.NVFP4Tensor(t.data, t.tiled_sf(), t.scale, True, t.is_v) for t in (Q, K, V))

        def our_step():
            fa.flash_attn_fp4_func(Qt.data, Kt.data, Vt.data, Qt.sf, Kt.sf, Vt.sf, Qt.scale, Kt.scale, Vt.scale,
                                   causal=causal, out=out, sf_layout="tiled")
        for _ in range(5):
            our_step()
        torch.cuda.synchronize()
        ms, mhz = timed(our_step)
        fa.check_status(dev)
        row.update(nvfp4_ms=ms, nvfp4_tflops=fl / ms / 1e9, nvfp4_sm_mhz=mhz)
        # the reference's BF16 kernel on the dequantised operands
        try:
            holder = {}

            def ref_step():
                holder["r"] = ref_func(qd, kd, vd, causal=causal)
            for _ in range(5):
                ref_step()
            torch.cuda.synchronize()
            ms_ref, mhz_ref = timed(ref_step)
            r = holder["r"]
            ref_out = r[0] if isinstance(r, (tuple, list)) else r
            row.update(fa4_bf16_ms=ms_ref, fa4_bf16_tflops=fl / ms_ref / 1e9, fa4_bf16_sm_mhz=mhz_ref,
                       speedup_vs_fa4_bf16=ms_ref / ms)
            a_, b_ = out[0, :, 0].float(), ref_out[0, :, 0].float()
            row["rel_rms_nvfp4_vs_fa4_bf16_sample"] = float((a_ - b_).norm() / b_.norm())
        except Exception as e:  # noqa: BLE001
            row.update(fa4_bf16_error=f"{type(e).__name__}: {e}"[:300])
        rows.append(row)
        del Q, K, V, Qt, Kt, Vt, qd, kd, vd, out
    head = rows[1]
    print(json.dumps({"impl": "fa4_bf16", "metric": "nvfp4_attn_fwd_tflops", "value": head.get("fa4_bf16_tflops"),
                      "unit": "TFLOP/s", "n_gpus": 1, "steps": steps, "warmup": 5, "ms_per_step": head.get("fa4_bf16_ms"),
                      "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": "the reference's BF16 sm_100 forward on the dequantised operands of cfg1, "
                                             "cfg2 and the D = 128 sweep points, beside this repository's NVFP4 kernel",
                                 "l2": "L2 flushed between timed launches (256 MiB write)"},
                      "table": rows}), flush=True)


def run_decode(args):
    """Decode shapes (one query token per sequence against a long NVFP4 KV cache, GQA 4): the
    transposed decode kernel with chosen key splits beside the prefill kernel's split-KV path.
    HBM-bound work: the figure of merit is bytes of K, V and their scales per second."""
    import flash_attention_b200 as fa
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = measured_peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    steps = max(3, min(args.steps, 20))
    rows = []
    for (B, Sk) in ((4, 32768), (1, 131072), (8, 8192), (64, 4096)):
        Hq, Hkv, D = 32, 8, 128
        g = torch.Generator(device=dev).manual_seed(11)
        q = torch.randn(B, 1, Hq, D, generator=g, device=dev, dtype=torch.bfloat16)
        k = torch.randn(B, Sk, Hkv, D, generator=g, device=dev, dtype=torch.bfloat16)
        v = torch.randn(B, Sk, Hkv, D, generator=g, device=dev, dtype=torch.bfloat16)
        Q, K, V = fa.quantize_qkv_fused(q, k, v, linear_sf=False)
        del q, k, v
        kv_bytes = 2 * B * Hkv * Sk * (D // 2 + D // 16)
        row = {"B": B, "Sk": Sk, "Hq": Hq, "Hkv": Hkv, "kv_bytes": kv_bytes,
               "splits": fa.interface.choose_decode_splits(B, Hkv, Sk, dev)}
        for name, variant in (("decode", fa.VARIANT_DECODE), ("prefill_splitkv", fa.VARIANT_WS)):
            def step():
                fa.flash_attn_fp4_func(Q.data, K.data, V.data, Q.sf, K.sf, V.sf, Q.scale, K.scale, V.scale,
                                       causal=True, return_lse=True, sf_layout="tiled", variant=variant,
                                       num_splits=0)
            for _ in range(3):
                step()
            torch.cuda.synchronize()
            ms = 0.0
            for _ in range(steps):
                flush.zero_()
                gpu_busy_while_host_enqueues()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); step(); e1.record(); e1.synchronize()
                ms += e0.elapsed_time(e1)
            ms /= steps
            fa.check_status(dev)
            row[name] = {"us": ms * 1e3, "kv_gbs": kv_bytes / ms / 1e6,
                         "frac_of_hbm_peak": kv_bytes / ms / 1e6 / peaks["hbm_gbs"]}
            if variant == fa.VARIANT_DECODE:
                # the same call captured in a CUDA graph and replayed back to back, as a serving loop
                # runs its decode steps: no launch gap, no L2 flush (K and V exceed L2 on the first
                # two shapes; on the smaller ones part of them stays cached, which is what such a loop sees)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    step()
                for _ in range(3):
                    graph.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(50):
                    graph.replay()
                e1.record(); e1.synchronize()
                g_ms = e0.elapsed_time(e1) / 50
                fa.check_status(dev)
                row[name].update(graph_replay_us=g_ms * 1e3, graph_replay_kv_gbs=kv_bytes / g_ms / 1e6,
                                 graph_replay_kv_fits_l2=bool(kv_bytes < 126 * 1000 * 1000))
                del graph
        rows.append(row)
        del Q, K, V
    head = rows[0]
    print(json.dumps({"metric": "nvfp4_decode_kv_gbs", "value": head["decode"]["kv_gbs"], "unit": "GB/s",
                      "n_gpus": 1, "steps": steps, "warmup": 3, "ms_per_step": head["decode"]["us"] / 1e3,
                      "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4",
                      "data": "synthetic",
                      "config": {"workload": "decode: Sq = 1, Hq = 32, Hkv = 8, D = 128, causal, (B, Sk) in "
                                             "{(4, 32768), (1, 131072), (8, 8192), (64, 4096)}; headline row "
                                             "B = 4, Sk = 32768; one call = decode kernel + combine kernel",
                                 "l2": "L2 flushed between timed calls (256 MiB write)"},
                      "roofline": {"bound": "hbm", "achieved": head["decode"]["kv_gbs"], "peak": peaks["hbm_gbs"],
                                   "unit": "GB/s", "frac": head["decode"]["frac_of_hbm_peak"], "traffic": None},
                      "gpu_launches": 2 * steps * 2 * len(rows), "decode": rows}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "fa4-bf16"],
                    help="ours: this repository's kernels; reference: the CPU restatement of attention_ref on the "
                         "host cores; fa4-bf16: the reference's own BF16 Blackwell kernel from baseline/_ref on the "
                         "dequantised operands (the same-box comparator)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong (default): ONE problem of the workload's size, its (batch, kv-head) units dealt "
                         "over the GPUs, verified after an NCCL all-gather; weak: one such problem per GPU")
    ap.add_argument("--sustained", type=float, default=0.0,
                    help="also time back-to-back launches for this many seconds (no L2 flush, clocks sampled)")
    ap.add_argument("--kernel", default="auto", choices=["auto", "ws128"],
                    help="auto: the library's choice (the 64-key kernel for these workloads); ws128: force "
                         "the 128-key kernel that serves split-KV")
    args = ap.parse_args()
    if args.gpus > 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1 and args.workload != "decode":
        # not under a launcher: start one rank per GPU ourselves
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port", "29517",
               os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if args.impl == "fa4-bf16":
        if not torch.cuda.is_available():
            print(json.dumps({"impl": "fa4_bf16", "unavailable": "no CUDA device"}))
            return
        return run_fa4_bf16(args)
    if args.workload in ("sweep", "decode"):
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (no CPU fallback)")
        return run_sweep(args) if args.workload == "sweep" else run_decode(args)
    wl = parse_workload(args.workload)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, wl, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback); use --impl reference for the CPU arm")
    run_gpu_arm(args, wl, rank, local_rank, world)


if __name__ == "__main__":
    main()
