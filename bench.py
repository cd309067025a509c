"""Benchmark of the sparse MLA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5|c2s|c4s|c5s] [--impl ours|reference]
                    [--scaling weak|strong] [--no-also] [--no-cpu-baseline]

Default workload "c2": FP8 sparse MLA decode at the DeepSeek-V3.2 shape (b=128, s_q=2, h_q=128,
topk=2048, cache_seqlens uniform in [4096, 32768], 64-token pages in random order, ~2% invalid
indices), synthetic seeded data.  One step = one flash_mla_with_kvcache call (attention kernel +
combine kernel; the tile scheduler's output is cached after the first call, as in the reference's
own timing, tests/kernelkit/bench.py:77-100).  Prints ONE JSON line on rank 0.

On one GPU the default run also measures the other benchmark configurations for a few steps each
(MXFP8 decode "c3", MODEL1 decode "m1", prefill forward "c4", prefill backward "c5", dense bf16 decode "dense", MODEL1 decode over
two caches "m1x") and reports them under "also".

Multi-GPU (launched by torch.distributed.run): every rank owns its own sequences and KV pages
(decode) or its own query tokens (prefill); there is no collective in the data path.  The headline is
weak-scaled (the per-GPU workload is fixed and the global batch is N times it); with more than one
GPU the line also carries a "strong" record, the same global workload cut into N parts (b = 128 / N
requests per GPU for c2), and for the backward the all-reduce of the per-GPU dKV partial sums.

--impl reference times the CPU restatement of the reference's torch oracle (tests/ref.py) on the
host cores, on a bounded sample of the same workload.
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

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from flashmla_b200 import workloads as wl  # noqa: E402

WORKLOADS = {
    "c2": dict(kind="decode", b=128, s_q=2, h_q=128, topk=2048, lo=4096, hi=32768, layout=wl.LAYOUT_V32,
               name="fp8_sparse_decode_v32_b128_sq2_h128_topk2048_sk4096-32768"),
    "c3": dict(kind="decode", b=256, s_q=1, h_q=128, topk=2048, lo=65536, hi=65536, layout=wl.LAYOUT_MXFP8,
               name="mxfp8_sparse_decode_b256_sq1_h128_topk2048_sk65536"),
    "c4": dict(kind="prefill_fwd", s_q=4096, s_kv=32768, h_q=128, topk=2048, offset=28672,
               name="sparse_prefill_fwd_sq4096_skv32768_h128_topk2048"),
    # the c2 shape with the reference's second model shape: d_qk = 512, MODEL1 cache blocks
    "m1": dict(kind="decode", b=128, s_q=2, h_q=128, topk=2048, lo=4096, hi=32768, layout=wl.LAYOUT_MODEL1,
               name="fp8_sparse_decode_model1_d512_b128_sq2_h128_topk2048_sk4096-32768"),
    # reduced copies of c2 / c4 for profiler captures (same kernels and per-unit work, fewer units; inputs still exceed L2)
    "c2s": dict(kind="decode", b=16, s_q=2, h_q=128, topk=2048, lo=4096, hi=32768, layout=wl.LAYOUT_V32,
                name="fp8_sparse_decode_v32_b16_sq2_h128_topk2048_sk4096-32768"),
    "m1s": dict(kind="decode", b=16, s_q=2, h_q=128, topk=2048, lo=4096, hi=32768, layout=wl.LAYOUT_MODEL1,
                name="fp8_sparse_decode_model1_d512_b16_sq2_h128_topk2048_sk4096-32768"),
    "c4s": dict(kind="prefill_fwd", s_q=592, s_kv=32768, h_q=128, topk=2048, offset=28672,
                name="sparse_prefill_fwd_sq592_skv32768_h128_topk2048"),
    "c5": dict(kind="prefill_bwd", s_q=4096, s_kv=32768, h_q=128, topk=2048, offset=28672,
               name="sparse_prefill_bwd_sq4096_skv32768_h128_topk2048"),
    # one pass of the tensor-core backward (592 query tokens), for profiler captures
    "c5s": dict(kind="prefill_bwd", s_q=592, s_kv=32768, h_q=128, topk=2048, offset=28672,
                name="sparse_prefill_bwd_sq592_skv32768_h128_topk2048"),
}
# DRAM bytes (read + write) of one launch of the dominant kernel, from the ncu captures summarised under profiles/
# (captured on the reduced cases c2s / c4s / c5s and scaled by the units a full launch processes)
NCU_TRAFFIC = {"c2": 424.2e6, "c2s": 53.03e6, "c4": 1.32e9, "c4s": 190.7e6}
METRIC = {"decode": "fp8_sparse_mla_decode_tflops", "prefill_fwd": "sparse_prefill_fwd_tflops",
          "prefill_bwd": "sparse_prefill_bwd_tflops"}
KERNEL_NAME = {"decode": "pair_attn_kernel<0,0>", "prefill_fwd": "pair_attn_kernel<1,0>",
               "prefill_bwd": "bwd_scores_kernel + bwd_dq_dkv_kernel (tcgen05; the whole step)"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], basis="measured (burst)")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, basis="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)

            def reader():
                for ln in self.proc.stdout:
                    self.lines.append((time.time(), ln))
            self.thread = threading.Thread(target=reader, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            self.proc.wait(timeout=5)
            self.thread.join(timeout=5)

    def count(self, t0):
        return sum(1 for t, _ in self.lines if t >= t0)

    def summary(self, t0, t1):
        """Median SM clock and the throttle reasons seen in samples taken between t0 and t1 (wall clock)."""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, ln in self.lines:
            if t < t0 or t > t1 + 0.15:
                continue
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def bind_to_gpu_numa_node(local_rank: int) -> str:
    """Binds this process to the CPUs next to its GPU (the PCI device's local_cpulist), so that pinned host buffers
    allocated afterwards come from that NUMA node.  Changes nothing on the GPU; returns a note for the JSON line."""
    try:
        prop = torch.cuda.get_device_properties(local_rank)
        bdf = f"{prop.pci_domain_id:04x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
        cpus = set()
        for part in open(f"/sys/bus/pci/devices/{bdf}/local_cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return f"bound to {len(cpus)} CPUs local to GPU {bdf}"
    except (OSError, ValueError, AttributeError):
        pass
    return "not bound"


def make_workload(cfg, device, seed, units=None):
    if cfg["kind"] == "decode":
        return wl.make_decode_workload(units or cfg["b"], cfg["s_q"], cfg["h_q"], cfg["topk"], cfg["lo"], cfg["hi"],
                                       layout=cfg["layout"], seed=seed, device=device, invalid_frac=0.02, keep_bf16=False)
    return wl.make_prefill_workload(units or cfg["s_q"], cfg["s_kv"], cfg["h_q"], cfg["topk"], seed=seed, device=device,
                                    causal_offset=cfg["offset"])


# ------------------------------------------------------------------------------------------------
# CPU leg: the oracle on the host cores, bounded sample
# ------------------------------------------------------------------------------------------------
def cpu_step(cfg, w_cpu, sample):
    """One pass of the oracle over `sample` requests (decode) or query tokens (prefill). Returns flops done."""
    from oracle import attention, quant
    if cfg["kind"] == "decode":
        idx = w_cpu.indices[:sample]
        b, s_q, topk = idx.shape
        rows = w_cpu.kv_rows.reshape(-1, 1, 1, 656)[idx.clamp_min(0).reshape(-1).long()].view(b * s_q * topk, 1, 1, 656)
        deq = quant.dequantize_rows(rows, w_cpu.layout)
        local = torch.arange(b * s_q * topk, dtype=torch.int32).view(b, s_q, topk).masked_fill(idx < 0, -1)
        attention.sparse_decode(w_cpu.q[:sample], deq, local, w_cpu.sm_scale)
        return 2.0 * cfg["h_q"] * b * s_q * topk * (576 + 512)
    if cfg["kind"] == "prefill_fwd":
        attention.sparse_prefill_fwd(w_cpu.q[:sample], w_cpu.kv, w_cpu.indices[:sample], w_cpu.sm_scale)
        return 2.0 * sample * cfg["topk"] * cfg["h_q"] * (576 + 512)
    attention.sparse_prefill_bwd(w_cpu.q[:sample], w_cpu.kv, w_cpu.dout[:sample], w_cpu.indices[:sample], w_cpu.sm_scale)
    return 2.0 * sample * cfg["topk"] * cfg["h_q"] * (3 * 576 + 2 * 512)


def cpu_workload(cfg, sample, seed):
    """A CPU copy of the first `sample` units of the workload (same distributions, smaller pool)."""
    if cfg["kind"] == "decode":
        return wl.make_decode_workload(sample, cfg["s_q"], cfg["h_q"], cfg["topk"], cfg["lo"], cfg["hi"], layout=cfg["layout"],
                                       seed=seed, device="cpu", invalid_frac=0.02, keep_bf16=False)
    return wl.make_prefill_workload(sample, cfg["s_kv"], cfg["h_q"], cfg["topk"], seed=seed, device="cpu",
                                    causal_offset=cfg["offset"])


def host_threads(world: int) -> int:
    """The host cores this process may use: its share of the machine when several ranks run (torchrun sets
    OMP_NUM_THREADS=1, which would otherwise leave the oracle on one core)."""
    return max(1, len(os.sched_getaffinity(0)) // max(world, 1))


def cpu_baseline(cfg, seed, world, budget_s=12.0):
    cores = host_threads(world)
    torch.set_num_threads(cores)
    sample = 4 if cfg["kind"] == "decode" else 32
    w_cpu = cpu_workload(cfg, sample, seed)
    cpu_step(cfg, w_cpu, min(sample, 1))     # warm-up
    t0 = time.perf_counter()
    flops, reps = 0.0, 0
    while True:
        flops += cpu_step(cfg, w_cpu, sample)
        reps += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    unit = "requests" if cfg["kind"] == "decode" else "query tokens"
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{reps} passes over the first {sample} {unit} of the workload ({dt:.1f} s), torch fp32 oracle, {cores} threads"}


def run_reference(args, cfg, rank, world):
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))     # rank 0 alone runs: it may use every core
    torch.set_num_threads(cores)
    sample = 16 if cfg["kind"] == "decode" else 64
    w_cpu = cpu_workload(cfg, sample, args.seed)
    for _ in range(args.warmup):
        cpu_step(cfg, w_cpu, sample)
    t0 = time.perf_counter()
    flops = 0.0
    for _ in range(args.steps):
        flops += cpu_step(cfg, w_cpu, sample)
    dt = time.perf_counter() - t0
    val = flops / dt / 1e12
    unit = "requests" if cfg["kind"] == "decode" else "query tokens"
    desc = f"each step = first {sample} {unit} of the workload, torch fp32 oracle (restatement of tests/ref.py), {cores} threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC[cfg["kind"]], "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["name"], "sample": desc},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------------
# GPU leg
# ------------------------------------------------------------------------------------------------
class Bench:
    """One workload on this rank's GPU: the device-timed step, the end-to-end step and their bookkeeping."""

    def __init__(self, cfg, dev, seed, units=None):
        import flash_mla
        self.cfg, self.dev, self.kind = cfg, dev, cfg["kind"]
        self.units = units or cfg.get("b", cfg.get("s_q"))
        w = self.w = make_workload(cfg, dev, seed, units)
        fm = flash_mla
        if self.kind == "decode":
            self.sched = fm.get_mla_metadata()[0]
            self.flops, self.alg_bytes, self.launches = w.flops, w.algorithmic_bytes, 2
            self.step = lambda q=w.q, idx=w.indices, mid=None: fm.flash_mla_with_kvcache(
                q, w.kv_rows, None, None, 512, self.sched, None, w.sm_scale, False, True, idx, kvcache_layout=w.layout,
                attn_done_event=mid)
            self.inputs = [w.q, w.indices]
            self.results = lambda r: [r[0], r[1].transpose(1, 2)]
        elif self.kind == "prefill_fwd":
            self.flops, self.alg_bytes, self.launches = w.fwd_flops, None, 1
            self.step = lambda q=w.q, idx=w.indices: fm.flash_mla_sparse_fwd(q, w.kv, idx, w.sm_scale)
            self.inputs = [w.q, w.indices]
            self.results = lambda r: [r[0], r[2]]
        else:
            from flashmla_b200 import interface as itf
            self.flops, self.alg_bytes = w.bwd_flops, None
            # memset + passes of 592 tokens x (scores kernel, dq+dkv kernel) + fp32 -> bf16 cast
            self.passes = -(-self.units // itf.BWD_CHUNK_TOKENS)
            self.launches = 2 * self.passes + 1
            out_f, _, lse_f = fm.flash_mla_sparse_fwd(w.q, w.kv, w.indices, w.sm_scale)
            self.step = lambda q=w.q, idx=w.indices, dout=w.dout, ev=None: fm.flash_mla_sparse_bwd(
                q, w.kv, out_f, dout, idx, lse_f, w.sm_scale, grad_events=ev)
            self.inputs = [w.q, w.indices, w.dout]
            self.results = lambda r: [r[0], r[1]]
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # > 126 MB L2

    # -- device-timed -----------------------------------------------------------------------------
    def timed(self, steps, barrier, mid=False):
        """Per-step CUDA-event timing on the launching stream with an L2 flush before every step.

        A spin kernel is queued first so that the host runs ahead of the device: a step's events then bracket
        device work only, not the host's launch latency (a decode step is shorter than its Python call).
        Returns the per-step times and, with `mid`, the times of the part the inner events bracket."""
        ev = lambda: torch.cuda.Event(enable_timing=True)
        starts, ends = [ev() for _ in range(steps)], [ev() for _ in range(steps)]
        inner = [(ev(), ev()) for _ in range(steps)] if mid else None
        keep = []
        barrier()
        torch.cuda._sleep(int(2e6 * (10 + 1.0 * steps)))      # about (10 + steps) ms at 2 GHz
        for i in range(steps):
            self.flush.fill_(i & 0xff)
            starts[i].record()
            if not mid:
                keep.append(self.step())
            elif self.kind == "decode":
                keep.append(self.step(mid=inner[i][1]))
            else:
                keep.append(self.step(ev=inner[i]))
            ends[i].record()
        barrier()
        total = [s.elapsed_time(e) for s, e in zip(starts, ends)]
        if not mid:
            return total
        if self.kind == "decode":       # start of the step .. event between the attention and the combine kernel
            return total, [s.elapsed_time(m[1]) for s, m in zip(starts, inner)]
        return total, [m[0].elapsed_time(m[1]) for m in inner]      # the first pass's dQ / dKV launch

    # -- end to end ---------------------------------------------------------------------------------
    def prepare_e2e(self):
        """Pinned host copies of the per-step inputs and results, two sets of device input buffers, three streams."""
        self.host_in = [t.cpu().pin_memory() for t in self.inputs]
        first = self.results(self.step())
        torch.cuda.synchronize()
        self.host_out = [[torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in first] for _ in range(2)]
        self.dev_in = [[torch.empty_like(t) for t in self.inputs] for _ in range(2)]
        self.s_in, self.s_out = torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev)
        self.h2d = sum(h.numel() * h.element_size() for h in self.host_in)
        self.d2h = sum(h.numel() * h.element_size() for h in self.host_out[0])

    def e2e(self, steps, barrier):
        """`steps` calls through the public API with every step's inputs copied from pinned host memory and every
        step's results copied back.  The copies run on their own streams with two sets of buffers, so that step
        i+1's host-to-device copy and step i-1's device-to-host copy travel (PCIe is full duplex) while step i
        computes; all of it lies between the two events.  Returns the milliseconds per step."""
        main = torch.cuda.current_stream(self.dev)
        in_done = [torch.cuda.Event() for _ in range(2)]
        free_in = [torch.cuda.Event() for _ in range(2)]      # the compute of the step that read this buffer set is over
        out_done = [torch.cuda.Event() for _ in range(2)]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        keep = []
        barrier()
        start.record(main)
        self.s_in.wait_event(start)
        self.s_out.wait_event(start)
        for i in range(steps):
            k = i & 1
            with torch.cuda.stream(self.s_in):
                if i >= 2:
                    self.s_in.wait_event(free_in[k])
                for d, h in zip(self.dev_in[k], self.host_in):
                    d.copy_(h, non_blocking=True)
                in_done[k].record(self.s_in)
            main.wait_event(in_done[k])
            res = self.results(self.step(*self.dev_in[k]))
            free_in[k].record(main)
            computed = torch.cuda.Event()
            computed.record(main)
            keep.append(res)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(computed)
                for h, t in zip(self.host_out[k], res):
                    h.copy_(t, non_blocking=True)
                out_done[k].record(self.s_out)
        main.wait_stream(self.s_out)
        end.record(main)
        barrier()
        return start.elapsed_time(end) / steps

    def first_call_ms(self):
        """Decode: one call with a fresh FlashMLASchedMeta - plan, tile-scheduler kernel, allocation of the split-KV
        accumulators, then the two kernels - by CUDA events after an L2 flush (the library is loaded and its tensor
        maps are cached: the warm-up calls came before).  The steady-state step reuses the schedule, as the
        reference's own timing does."""
        if self.kind != "decode":
            return None
        import flash_mla
        w = self.w
        ms = []
        for i in range(3):
            fresh = flash_mla.get_mla_metadata()[0]
            self.flush.fill_(i)
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            flash_mla.flash_mla_with_kvcache(w.q, w.kv_rows, None, None, 512, fresh, None, w.sm_scale, False, True, w.indices,
                                             kvcache_layout=w.layout)
            t1.record()
            torch.cuda.synchronize()
            ms.append(t0.elapsed_time(t1))
        return statistics.median(ms)

    # -- host cost of a call ------------------------------------------------------------------------
    def host_us_per_call(self, n=200):
        """Host time of one call (Python + C ABI + launches) with the device kept busy behind it, and of one replay
        of the same call captured in a CUDA graph."""
        if self.kind == "prefill_bwd":
            return None
        self.step(); torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            self.step()
        eager = (time.perf_counter() - t0) / n * 1e6
        torch.cuda.synchronize()
        side = torch.cuda.Stream(self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                captured = self.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            graph.replay()
        replay = (time.perf_counter() - t0) / n * 1e6
        torch.cuda.synchronize()
        del captured
        return {"eager": round(eager, 1), "graph_replay": round(replay, 1),
                "note": "host time per call, device work queued behind it; the eager call encodes no tensor map after the first (they are cached)"}


def measure(bench: Bench, clk: ClockSampler, steps, warmup, barrier, world, dev, all_reduce_max):
    """Warm-up, device-timed steps (measured once more when the clocks were throttled or a step stalled) and the
    attention kernel's own time.  Returns (ms per step, ms of the roofline kernel per launch, clocks)."""
    for _ in range(warmup):
        bench.step()
    torch.cuda.synchronize()
    attempts = []
    for attempt in range(2):
        t0 = time.time()
        ms = ms_k = bench.timed(steps, barrier)
        if bench.kind != "prefill_fwd":
            # a second pass with timing events inside the step: decode - between the attention and the combine kernel
            # (the event turns the combine kernel's dependent launch off, so `value` comes from the first pass);
            # backward - around the first pass's dQ / dKV launch
            _, ms_k = bench.timed(steps, barrier, mid=True)
        t_end = time.time() + 6.0
        while clk.count(t0) < 4 and time.time() < t_end:     # keep the load up until nvidia-smi has delivered samples
            bench.step()
            torch.cuda.synchronize()
        cl = clk.summary(t0, time.time())
        attempts.append((ms, ms_k, cl))
        # a measurement taken under a thermal / hardware slowdown, with SM clocks far below their maximum, or with a
        # step that stalled (another tenant of the host, a host hiccup) is taken once more
        bad = [r for r in cl["reasons"] if r != "sw_power_cap"]
        slow_clock = cl["sm_mhz"] is not None and cl["sm_mhz"] < 0.8 * cl["sm_max_mhz"]
        stalled = max(ms) > 1.5 * statistics.median(ms)
        if all_reduce_max(1 if (bad or slow_clock or stalled) else 0) == 0:   # the ranks decide together: timed() holds barriers
            break
    ms, ms_k, clocks = attempts[-1]
    clocks["attempts"] = len(attempts)
    return ms, ms_k, clocks


def roofline_record(bench: Bench, key, t_step, t_kernel, pk):
    """The roofline object of a workload: the tensor pipe bounds all of them (flops counted with the reference's own
    model, tests/lib.py:345-402)."""
    if bench.kind == "prefill_bwd":
        # t_kernel = the first pass's dQ / dKV launch: its fp32 reductions into dKV are the traffic that matters there
        units = min(bench.units, 592)
        red_bytes = units * bench.cfg["topk"] * 576 * 4.0
        return {"bound": "tensor", "achieved": bench.flops / t_step / 1e12, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                "frac": bench.flops / t_step / 1e12 / pk["bf16_tflops"], "traffic": NCU_TRAFFIC.get(key), "basis": pk["basis"],
                "kernel": KERNEL_NAME[bench.kind], "ms_per_launch": t_step * 1e3,
                "dkv_reduction": {"bytes_per_pass": red_bytes, "ms_dq_dkv_launch": t_kernel * 1e3,
                                  "achieved_gbs": red_bytes / t_kernel / 1e9,
                                  "note": "fp32 red.global.add traffic of the first pass's dQ / dKV launch (592 query tokens x topk x 576 x 4 B) over its CUDA-event time"},
                "note": "the whole step (all launches), 2*h_q*topk*(3*576+2*512) flops per query token"}
    # the captured traffic belongs to the workload's full unit count; a part of it (a strong-scaling shard) moves in proportion
    full = bench.cfg.get("b", bench.cfg.get("s_q"))
    traffic = NCU_TRAFFIC.get(key)
    if traffic is not None and bench.units != full:
        traffic = traffic * bench.units / full
    return {"bound": "tensor", "achieved": bench.flops / t_kernel / 1e12, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
            "frac": bench.flops / t_kernel / 1e12 / pk["bf16_tflops"], "traffic": traffic, "basis": pk["basis"],
            "kernel": "pair_attn_kernel<0,2>" if key in ("m1", "m1s") else KERNEL_NAME[bench.kind], "ms_per_launch": t_kernel * 1e3,
            "note": "the attention kernel alone (one launch per step), 2*h_q*topk*(d_qk+512) flops per query token; "
                    "traffic = DRAM bytes of one launch from the ncu capture under profiles/"}


def dense_decode_record(dev, seed, pk, steps=4, warmup=3, b=128):
    """Dense MLA decode (indices=None; the path the reference's own dense benchmark measures, benchmark/bench_flash_mla.py,
    at b=128, s_q=2, causal, h_q=128, s_k=8192 for every request) timed like the other workloads: CUDA events per step,
    L2 flush before every step.  The step is the whole call: the split-KV attention kernel, which walks the block table
    itself, and the combine kernel."""
    import flash_mla
    s_q, h_q, s_k, page, d = 2, 128, 8192, 64, 576
    g = torch.Generator(device=dev).manual_seed(seed)
    nblk = s_k // page
    block_table = torch.randperm(b * nblk, generator=g, device=dev).to(torch.int32).view(b, nblk)
    q = torch.randn((b, s_q, h_q, d), generator=g, device=dev).to(torch.bfloat16)
    k_cache = (torch.randn((b * nblk, page, 1, d), generator=g, device=dev) / 10).to(torch.bfloat16)
    lens = torch.full((b,), s_k, dtype=torch.int32, device=dev)
    meta = flash_mla.get_mla_metadata()[0]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    step = lambda: flash_mla.flash_mla_with_kvcache(q, k_cache, block_table, lens, 512, meta, None, None, True)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    ms = []
    for i in range(steps):
        flush.fill_(i)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(); step(); t1.record()
        torch.cuda.synchronize()
        ms.append(t0.elapsed_time(t1))
    t = statistics.median(ms) / 1e3
    # causal: row j of a request's s_q rows sees s_k - (s_q - 1 - j) tokens
    seen = sum(s_k - (s_q - 1 - j) for j in range(s_q))
    flops = 2.0 * b * h_q * seen * (576 + 512)
    return {"workload": f"dense_mla_decode_bf16_b{b}_sq2_h128_sk8192_causal", "metric": "dense_mla_decode_tflops", "value": flops / t / 1e12,
            "unit": "TFLOP/s", "steps": steps, "ms_per_step": t * 1e3,
            "kv_gbs": b * s_k * d * 2 / t / 1e9,
            "roofline": {"bound": "tensor", "achieved": flops / t / 1e12, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": flops / t / 1e12 / pk["bf16_tflops"], "traffic": None, "basis": pk["basis"],
                         "kernel": "pair_attn_kernel<0,3> + combine_kernel", "ms_per_launch": t * 1e3}}


def model1_extra_record(dev, seed, pk, steps=6, warmup=3, b=128):
    """MODEL1 decode over two caches at the reference's production shape for it (test_flash_mla_sparse_decoding.py:107-108,
    "MODEL1 CONFIG2": h_q=128, s_q=2, d_qk=512, topk=128 over pages of 256 tokens + extra_topk=1024 over pages of 64,
    16384-token sequences in both) with b=128, timed like the other workloads."""
    import flash_mla
    s_q, h_q, topk, xtopk, s_k = 2, 128, 128, 1024, 16384
    w = wl.make_decode_workload(b, s_q, h_q, topk, s_k, s_k, page=256, layout=wl.LAYOUT_MODEL1, seed=seed, device=str(dev),
                                q_std=1.0, kv_std=0.1, clamp=1.0, sm_scale=512 ** -0.55, keep_bf16=False)
    x = wl.make_decode_workload(b, s_q, h_q, xtopk, s_k, s_k, page=64, layout=wl.LAYOUT_MODEL1, seed=seed + 1, device=str(dev),
                                q_std=1.0, kv_std=0.1, clamp=1.0, keep_bf16=False)
    meta = flash_mla.get_mla_metadata()[0]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    step = lambda: flash_mla.flash_mla_with_kvcache(w.q, w.kv_rows, None, None, 512, meta, None, w.sm_scale, False, True, w.indices,
                                                    None, x.kv_rows, x.indices, None, None, kvcache_layout=wl.LAYOUT_MODEL1)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    ms = []
    for i in range(steps):
        flush.fill_(i)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(); step(); t1.record()
        torch.cuda.synchronize()
        ms.append(t0.elapsed_time(t1))
    t = statistics.median(ms) / 1e3
    flops = 2.0 * b * s_q * h_q * (topk + xtopk) * (512 + 512)
    return {"workload": f"fp8_sparse_decode_model1_two_caches_b{b}_sq2_h128_topk128+1024", "metric": "fp8_sparse_mla_decode_tflops",
            "value": flops / t / 1e12, "unit": "TFLOP/s", "steps": steps, "ms_per_step": t * 1e3,
            "roofline": {"bound": "tensor", "achieved": flops / t / 1e12, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": flops / t / 1e12 / pk["bf16_tflops"], "traffic": None, "basis": pk["basis"],
                         "kernel": "pair_attn_kernel<0,4> + combine_kernel", "ms_per_launch": t * 1e3}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="strong: the headline is the global workload cut into N parts instead of N copies of it")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the other configurations of the default run")
    ap.add_argument("--record", choices=["dense", "m1x"], help="one GPU: run only this side record of the default line and print it "
                    "(for profiler captures; --batch sets its request count)")
    ap.add_argument("--batch", type=int, default=128)
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, cfg, rank, world)
        return
    if args.record:
        dev = torch.device("cuda", local_rank)
        torch.cuda.set_device(dev)
        fn = dense_decode_record if args.record == "dense" else model1_extra_record
        print(json.dumps(fn(dev, args.seed + 11, peaks(), steps=args.steps, warmup=args.warmup, b=args.batch)))
        return

    import torch.distributed as dist
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # The CPU baseline runs on rank 0 before the ranks meet, on rank 0's share of the cores: the other ranks then
    # wait in the rendezvous (a host wait), not in a collective that would keep their GPUs spinning.
    cpu = None
    if rank == 0 and not args.no_cpu_baseline:
        cpu = cpu_baseline(cfg, args.seed, world)
    numa = bind_to_gpu_numa_node(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    args.warmup = max(args.warmup, 3)
    kind = cfg["kind"]
    full_units = cfg.get("b", cfg.get("s_q"))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def all_reduce_max(v):
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    strong_units = max(1, full_units // world)
    head_units = strong_units if args.scaling == "strong" else full_units
    line = None
    # nvidia-smi is started before the warm-up: its start-up queries stall kernel launches for milliseconds
    with ClockSampler(local_rank) as clk:
        bench = Bench(cfg, dev, args.seed + rank, head_units)
        bench.prepare_e2e()
        for _ in range(args.warmup):
            bench.e2e(2, barrier)
        t_wait = time.time() + 5.0
        while not clk.lines and time.time() < t_wait:      # first sample delivered = start-up over
            bench.step()
            torch.cuda.synchronize()
        ms, ms_k, clocks = measure(bench, clk, args.steps, args.warmup, barrier, world, dev, all_reduce_max)
        if os.environ.get("FMLA_BENCH_VERBOSE"):
            print("per-step ms:", [round(x, 3) for x in ms], file=sys.stderr)
        t_step = all_reduce_max(sum(ms)) / args.steps / 1e3
        t_e2e = all_reduce_max(bench.e2e(args.steps, barrier)) / 1e3
        host_us = bench.host_us_per_call() if rank == 0 else None
        pk = peaks()
        if rank == 0:
            t_kernel = sum(ms_k) / args.steps / 1e3
            value = world * bench.flops / t_step / 1e12
            per_gpu = value / world
            line = {
                "metric": METRIC[kind], "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": t_step * 1e3, "higher_is_better": True, "scaling": args.scaling,
                "vs_baseline": (per_gpu / 350.0) if args.workload == "c2" else (per_gpu / 1450.0 if args.workload == "c4" else None),
                "dtype": "bf16", "data": "synthetic",
                "config": {"workload": cfg["name"], "per_gpu_units": head_units, "global_units": head_units * world,
                           "timing": "CUDA events per step on the launching stream, 256 MB L2 flush before every step, max over ranks",
                           "baseline_note": "vs_baseline divides the per-GPU value by the reference README's B200 figure (350 TFLOPS decode / 1450 prefill), whose exact shape is not published"},
                "gpu_launches": bench.launches * args.steps,
                "e2e": {"value": world * bench.flops / t_e2e / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": bench.h2d,
                        "d2h_bytes_per_step": bench.d2h, "ms_per_step": t_e2e * 1e3, "host_binding": numa,
                        "note": "every step's q and indices (and dout) come from pinned host memory and its results go back; copy-in, "
                                "compute and copy-out run on three streams with two buffer sets, so the copies of neighbouring "
                                "steps overlap the compute; the paged KV cache is resident serving state; the inputs exceed L2"},
                "clocks": clocks,
                "roofline": roofline_record(bench, args.workload, t_step, t_kernel, pk),
            }
            if host_us:
                line["host_us_per_call"] = host_us
                line["first_call_ms"] = bench.first_call_ms()
            if bench.alg_bytes is not None:
                line["hbm"] = {"algorithmic_bytes": bench.alg_bytes, "achieved_gbs": bench.alg_bytes / t_step / 1e9,
                               "frac_of_measured_copy": bench.alg_bytes / t_step / 1e9 / pk["hbm_gbs"]}
            if cpu is not None:
                line["cpu_baseline"] = cpu

        # ---- backward on several GPUs: the per-GPU dKV partial sums are added with one NCCL all-reduce after the kernels
        if kind == "prefill_bwd" and world > 1:
            dkv = torch.zeros((cfg["s_kv"], 576), dtype=torch.float32, device=dev)
            for _ in range(3):
                dist.all_reduce(dkv)
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            s.record()
            for _ in range(10):
                dist.all_reduce(dkv)
            e.record()
            torch.cuda.synchronize()
            t_red = all_reduce_max(s.elapsed_time(e) / 10)
            if rank == 0:
                line["dkv_all_reduce"] = {"bytes": dkv.numel() * 4, "ms": t_red, "ms_kernels_plus_reduce": t_step * 1e3 + t_red,
                                          "note": "NCCL all-reduce of the fp32 [s_kv, 576] partial sums, issued after the kernels; "
                                                  "`value` is the kernels alone"}

        # ---- the same global workload cut into N parts (BASELINE's partition: 128 / N requests per GPU)
        if world > 1 and args.scaling == "weak" and strong_units < full_units:
            del bench
            torch.cuda.empty_cache()
            sb = Bench(cfg, dev, args.seed + 100 + rank, strong_units)
            s_ms, s_k, s_clocks = measure(sb, clk, args.steps, args.warmup, barrier, world, dev, all_reduce_max)
            ts = all_reduce_max(sum(s_ms)) / args.steps / 1e3
            if rank == 0:
                line["strong"] = {"value": world * sb.flops / ts / 1e12, "unit": "TFLOP/s", "ms_per_step": ts * 1e3,
                                  "per_gpu_units": strong_units, "global_units": strong_units * world, "clocks": s_clocks,
                                  "roofline_frac_per_gpu": roofline_record(sb, None, ts, sum(s_k) / args.steps / 1e3, pk)["frac"],
                                  "note": "the global workload of one GPU's run cut into N parts; compare with the N = 1 value"}
            del sb
        elif world == 1 and args.workload == "c2" and not args.no_also:
            # ---- the other benchmark configurations, a few steps each
            del bench
            also = {}
            for key, steps in (("c3", 6), ("m1", 6), ("c4", 3), ("c5", 2)):
                torch.cuda.empty_cache()
                c = WORKLOADS[key]
                ob = Bench(c, dev, args.seed + 7)
                o_ms, o_k, o_clocks = measure(ob, clk, steps, 3, barrier, world, dev, all_reduce_max)
                t = sum(o_ms) / steps / 1e3
                rec = {"workload": c["name"], "metric": METRIC[c["kind"]], "value": ob.flops / t / 1e12, "unit": "TFLOP/s",
                       "steps": steps, "ms_per_step": t * 1e3, "clocks": o_clocks,
                       "roofline": roofline_record(ob, key, t, sum(o_k) / steps / 1e3, pk)}
                if ob.alg_bytes is not None:
                    rec["hbm_achieved_gbs"] = ob.alg_bytes / t / 1e9
                also[key] = rec
                del ob
            torch.cuda.empty_cache()
            also["dense"] = dense_decode_record(dev, args.seed + 11, pk)
            also["m1x"] = model1_extra_record(dev, args.seed + 13, pk)
            line["also"] = also
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
