#!/usr/bin/env python
"""Benchmark of the fused SDPA path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of the headline workload: the
Llama-3-8B-shaped grouped-query prefill (bf16 q [4,32,4096,128], k/v [4,8,4096,128],
causal, right padding with per-batch key lengths in [2048,4096], seed 2; "configuration 3").
With N > 1 (launched by torchrun, one rank per GPU) every rank owns its own batch of that
shape -- the (batch x kv head) units are independent, so there is no collective on the data
path -- and the reported value is the sum over ranks divided by the slowest rank's time.

The single JSON line carries

* ``value`` / ``ms_per_step``: the median of five timed blocks of K launches each, inputs
  resident in HBM (337 MB per GPU, larger than L2), CUDA events on the launching stream;
  ``blocks_ms`` lists the five, ``sustained`` is one more block that runs for at least a
  second, each with the SM clocks sampled while it ran;
* ``roofline`` for the prefill kernel (DRAM traffic per launch read from
  ``profiles/traffic.json``, which ``--ingest-ncu`` writes from an ncu capture);
* ``e2e``: the same metric through the public op with pinned host buffers, copies inside the
  timed region, and ``e2e.ceiling``: the same copies without the kernel;
* ``cpu_baseline``: the CPU oracle on this box's cores over a bounded sample;
* ``decode_roofline``: configuration 4 (split-KV decode, HBM bound) at top level;
* under ``extra``: the other configurations (each with its CPU figure where the north star
  asks for one), the (batch x kv head) partition of configuration 3 and of the decode
  configuration over the N ranks, and configuration 5 (long-context ring, also at N = 1)
  with ``ring_check``: sampled rows of the ring result recomputed by the independent
  CUDA-core kernel and by the CPU oracle, forward and backward, with the negative guard.
  A failed check makes the exit code non-zero.

``--impl reference`` times the CPU restatement of upstream's ``_sdpa_math`` path (the
oracle; the upstream file itself cannot travel to the GPU box) on the host cores.
"""

from __future__ import annotations

import argparse
import csv
import json
import math
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "attention TFLOP/s (prefill, aggregate over GPUs); decode HBM GB/s under extra"
WORKLOAD_C3 = ("llama3-8b-shaped GQA prefill bf16 q[4,32,4096,128] kv[4,8,4096,128] causal + right padding "
               "kv_lens~U[2048,4096] (configuration 3)")
CONFIG_C3 = {"workload": WORKLOAD_C3, "l2": "inputs (337 MB per GPU) larger than L2; no flush",
             "partition": "batch x kv-head, one batch of 4 per GPU, no collective"}
L2_BYTES = 126 * 1024 * 1024
TRAFFIC_JSON = os.path.join(ROOT, "profiles", "traffic.json")


# ----------------------------------------------------------------------------- workloads


def c3_inputs(seed: int, device=None, pinned=False):
    """Llama-3-8B-shaped GQA prefill with right padding (configuration 3)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(4, 32, 4096, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(4, 8, 4096, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(4, 8, 4096, 128, generator=g).to(torch.bfloat16)
    lens = torch.randint(2048, 4097, (4,), generator=g).to(torch.int32)
    if pinned:
        q, k, v, lens = (t.pin_memory() for t in (q, k, v, lens))
    if device is not None:
        q, k, v, lens = (t.to(device) for t in (q, k, v, lens))
    return q, k, v, lens


def c3_flops(lens, hq=32, L=4096, e=128) -> float:
    """4 * E * (visible (query, key) pairs): causal square clipped by the key length."""
    pairs = 0
    for n in lens.tolist():
        n = min(int(n), L)
        pairs += hq * (n * (n + 1) // 2 + (L - n) * n)
    return 4.0 * e * pairs


def c2_inputs(device=None):
    g = torch.Generator().manual_seed(1)
    ts = tuple((torch.randn(8, 12, 1024, 64, generator=g) * 0.5).to(torch.bfloat16) for _ in range(3))
    return tuple(t.to(device) for t in ts) if device is not None else ts


C2_FLOPS = 4.0 * 64 * 8 * 12 * (1024 * 1025 // 2)


def c4_inputs(device, batch=64):
    g = torch.Generator().manual_seed(3)
    q = torch.randn(batch, 32, 1, 128, generator=g).to(torch.bfloat16).to(device)
    # the cache itself is drawn on the device: 2 x 1 GiB of host randn would dominate start-up
    gd = torch.Generator(device=device).manual_seed(3)
    k = torch.randn(batch, 8, 8192, 128, generator=gd, device=device, dtype=torch.bfloat16)
    v = torch.randn(batch, 8, 8192, 128, generator=gd, device=device, dtype=torch.bfloat16)
    lens = torch.randint(512, 8193, (batch,), generator=g).to(torch.int32)
    return q, k, v, lens


# ----------------------------------------------------------------------------- clocks


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while a
    timed region runs."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake", 0x2: "applications_clocks_setting",
    }

    def __init__(self, device_index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.nv = pynvml
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# ----------------------------------------------------------------------------- helpers


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def measured_traffic(case: str):
    """DRAM bytes per launch of a profiled case (``--ingest-ncu`` wrote them from an ncu capture)
    with the algorithmic bytes of that same case, or None when no capture is on file."""
    try:
        with open(TRAFFIC_JSON) as f:
            return json.load(f).get(case)
    except Exception:
        return None


def median(xs):
    s = sorted(xs)
    return s[len(s) // 2]


def time_steps(fn, steps):
    """Average device time per call (ms) of ``steps`` back-to-back calls, CUDA events on
    the launching (current) stream, synchronised on both sides."""
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def time_each(fn, iters):
    """Device time (ms) of each of ``iters`` calls, one event pair per call, no flush."""
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return times


def time_steps_flushed(fn, steps, flush_buf):
    """Median per-call device time with L2 flushed (a write larger than L2) before every call."""
    times = []
    for _ in range(steps):
        flush_buf.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return median(times)


def reduce_scalar(dist, world, dev, x, op):
    if world == 1:
        return float(x)
    t = torch.tensor([float(x)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=op)
    return t.item()


# ----------------------------------------------------------------------------- CPU oracle legs


def c3_slices(n_slices):
    """``n_slices`` (batch, kv head) units of configuration 3 spread over the four batches."""
    order = [(b, hk) for hk in (0, 4, 2, 6, 1, 5, 3, 7) for b in range(4)]
    return order[:n_slices]


def cpu_prefill_sample(q, k, v, lens, scale, slices, threads):
    """Time the CPU oracle on (batch x kv-group) slices of configuration 3, driven as upstream
    drives its math path (GQA by repeat_interleave, padding as an additive bias).  Returns
    (TFLOP/s, seconds, flops)."""
    from oracle import sdpa_oracle as O

    torch.set_num_threads(threads)
    flops, t = 0.0, 0.0
    for b, hk in slices:
        qs = q[b : b + 1, hk * 4 : hk * 4 + 4]
        ks, vs = k[b : b + 1, hk : hk + 1], v[b : b + 1, hk : hk + 1]
        t0 = time.perf_counter()
        O.sdpa_forward(qs, ks, vs, is_causal=True, scale=scale, kv_lens=lens[b : b + 1])
        t += time.perf_counter() - t0
        flops += c3_flops(lens[b : b + 1], hq=4)
    return flops / t / 1e12, t, flops


def cpu_decode_sample(q, k, v, lens, scale, seqs, threads):
    """CPU oracle on whole sequences of the decode configuration, each sliced to its length as
    a caller of the math path would pass it.  q/k/v on the host.  Returns (GB/s, seconds, bytes)."""
    from oracle import sdpa_oracle as O

    torch.set_num_threads(threads)
    t, nbytes = 0.0, 0
    for b in seqs:
        n = int(lens[b])
        qs, ks, vs = q[b : b + 1], k[b : b + 1, :, :n], v[b : b + 1, :, :n]
        t0 = time.perf_counter()
        O.sdpa_forward(qs, ks, vs, scale=scale)
        t += time.perf_counter() - t0
        nbytes += 2 * 8 * n * 128 * 2 + 2 * 32 * 128 * 2 + 32 * 4
    return nbytes / t / 1e9, t, nbytes


# ----------------------------------------------------------------------------- reference arm


def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    q, k, v, lens = c3_inputs(2)
    scale = 1.0 / math.sqrt(128)
    slices = c3_slices(8)
    for _ in range(min(args.warmup, 1)):
        cpu_prefill_sample(q, k, v, lens, scale, slices[:2], threads)
    t_total, f_total = 0.0, 0.0
    for _ in range(args.steps):
        _, t, f = cpu_prefill_sample(q, k, v, lens, scale, slices, threads)
        t_total += t
        f_total += f
    val = f_total / t_total / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(CONFIG_C3),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": f"{len(slices)} of the 32 (batch x kv-group) slices [1,4,4096,128] per step, two "
                                   "from each of the four batches (rate-normalised to TFLOP/s); CPU oracle = "
                                   "restatement of upstream _sdpa_math.compute_attention driven with "
                                   "repeat_interleave GQA and an additive padding bias"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- profiler cases


def run_profile_case(args):
    """A bare loop over one kernel for profiler captures: no copies, no CPU leg.
    ``prefill`` is configuration 3 as timed by the bench; ``decode`` is configuration 4
    cut to 16 sequences (0.5 GB of cache, still larger than L2)."""
    import torch_neuronx_b200 as T

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    scale = 1.0 / math.sqrt(128)
    algorithmic = None
    if args.profile == "prefill":
        q, k, v, lens = c3_inputs(2, device=dev)
        out = T.alloc_like_query(q, q.shape)
        lse = torch.empty(4, 32, 4096, dtype=torch.float32, device=dev)
        algorithmic = 2 * q.numel() * 2 + 2 * 8 * 128 * 2 * int(lens.sum()) + lse.numel() * 4
        fn = lambda: T.sdpa_forward(q, k, v, is_causal=True, scale=scale, kv_lens=lens, out=out, lse=lse)  # noqa: E731
    elif args.profile == "gpt2":
        q, k, v = c2_inputs(dev)
        out = torch.empty_like(q)
        lse = torch.empty(8, 12, 1024, dtype=torch.float32, device=dev)
        algorithmic = 4 * q.numel() * 2 + lse.numel() * 4
        fn = lambda: T.sdpa_forward(q, k, v, is_causal=True, scale=0.125, out=out, lse=lse)  # noqa: E731
    elif args.profile == "wide":
        # multi-head-latent-attention shape: q/k head dim 192, v head dim 128 (335 MB of operands)
        g = torch.Generator(device=dev).manual_seed(5)
        q = torch.randn(4, 32, 4096, 192, generator=g, device=dev, dtype=torch.bfloat16)
        k = torch.randn(4, 32, 4096, 192, generator=g, device=dev, dtype=torch.bfloat16)
        v = torch.randn(4, 32, 4096, 128, generator=g, device=dev, dtype=torch.bfloat16)
        out = torch.empty(4, 32, 4096, 128, device=dev, dtype=torch.bfloat16)
        lse = torch.empty(4, 32, 4096, dtype=torch.float32, device=dev)
        fn = lambda: T.sdpa_forward(q, k, v, is_causal=True, out=out, lse=lse)  # noqa: E731
    elif args.profile == "bias":
        # an additive bias shared by batch and heads (34 MB) on a 2 x 32/8 x 4096^2 problem (168 MB of operands)
        g = torch.Generator(device=dev).manual_seed(6)
        q = torch.randn(2, 32, 4096, 128, generator=g, device=dev, dtype=torch.bfloat16)
        k = torch.randn(2, 8, 4096, 128, generator=g, device=dev, dtype=torch.bfloat16)
        v = torch.randn(2, 8, 4096, 128, generator=g, device=dev, dtype=torch.bfloat16)
        bias = torch.randn(4096, 4096, generator=g, device=dev, dtype=torch.bfloat16)
        out = torch.empty_like(q)
        lse = torch.empty(2, 32, 4096, dtype=torch.float32, device=dev)
        fn = lambda: T.sdpa_forward(q, k, v, attn_bias=bias, scale=scale, out=out, lse=lse)  # noqa: E731
    elif args.profile == "bwd":
        # the headline batch cut to one sequence (84 MB of operands, still around L2 size) keeps captures short
        q, k, v, lens = c3_inputs(2, device=dev)
        q, k, v, lens = q[:1].contiguous(), k[:1].contiguous(), v[:1].contiguous(), lens[:1].contiguous()
        out, lse = T.sdpa_forward(q, k, v, is_causal=True, scale=scale, kv_lens=lens)
        go = torch.randn(q.shape, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).to(dev)
        gq, gk, gv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        fn = lambda: T.sdpa_backward(go, q, k, v, out, lse, is_causal=True, scale=scale, kv_lens=lens,  # noqa: E731
                                     grad_q=gq, grad_k=gk, grad_v=gv)
    else:
        q, k, v, lens = c4_inputs(dev, batch=16)
        algorithmic = 2 * 8 * 128 * 2 * int(lens.sum()) + 2 * q.numel() * 2 + 16 * 32 * 4
        lens = lens.to(dev)
        out = torch.empty_like(q)
        lse = torch.empty(16, 32, 1, dtype=torch.float32, device=dev)
        fn = lambda: T.sdpa_forward(q, k, v, scale=scale, kv_lens=lens, out=out, lse=lse)  # noqa: E731
    for _ in range(args.warmup):
        fn()
    ms = time_steps(fn, args.steps)
    T.check_device_status()
    print(json.dumps({"profile_case": args.profile, "ms_per_step": ms, "plan": dict(T.ops.last_plan),
                      "algorithmic_bytes_per_launch": algorithmic}), flush=True)


def ingest_ncu(args):
    """Read ``ncu -i <report> --page raw --csv`` output (a file) of a ``--profile`` capture and record
    the DRAM bytes per launch of the kernel whose name contains ``--kernel`` under the case's key of
    ``profiles/traffic.json``.  ``--algorithmic-bytes`` is the figure the same ``--profile`` run printed."""
    with open(args.ingest_ncu, newline="") as f:
        rows = list(csv.reader(f))
    names, units, data = rows[0], rows[1], rows[2:]
    col = {n: i for i, n in enumerate(names)}
    scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    hits = [r for r in data if args.kernel in r[col["Kernel Name"]]]
    if not hits:
        raise SystemExit(f"no launch of a kernel named *{args.kernel}* in {args.ingest_ncu}")

    def metric(row, name):
        i = col[name]
        return float(row[i].replace(",", "")) * scale.get(units[i], 1.0)

    rd = sum(metric(r, "dram__bytes_read.sum") for r in hits) / len(hits)
    wr = sum(metric(r, "dram__bytes_write.sum") for r in hits) / len(hits)
    us = sum(float(r[col["gpu__time_duration.sum"]].replace(",", "")) for r in hits) / len(hits)
    try:
        with open(TRAFFIC_JSON) as f:
            table = json.load(f)
    except Exception:
        table = {}
    table[args.profile] = {
        "kernel": hits[0][col["Kernel Name"]][:120], "launches_averaged": len(hits), "dram_read_bytes": rd,
        "dram_write_bytes": wr, "dram_bytes_per_launch": rd + wr, "algorithmic_bytes_per_launch": args.algorithmic_bytes,
        "gpu_time_us_under_ncu": us, "command": f"python bench.py --profile {args.profile} --steps 3 --warmup 2",
    }
    with open(TRAFFIC_JSON, "w") as f:
        json.dump(table, f, indent=1, sort_keys=True)
        f.write("\n")
    print(json.dumps(table[args.profile]))


# ----------------------------------------------------------------------------- our arm


def run_ours(args, rank, local_rank, world):
    import torch_neuronx_b200 as T
    import torch.distributed as dist

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        # the ring's exchange kernels on a high-priority stream: posted beside an attention grid that fills
        # every SM, they otherwise only get placed when that grid has no CTAs left (0.4-0.8 ms exposed per
        # step at four ranks, none with the priority)
        os.environ.setdefault("TORCH_NCCL_HIGH_PRIORITY", "1")
        dist.init_process_group("nccl", device_id=dev)
    peaks = measured_peaks()
    scale = 1.0 / math.sqrt(128)
    failures = []

    # ---------------- headline: configuration 3, inputs resident in HBM ----------------
    # every rank works on its own copy of the same seeded batch: identical work per GPU
    q, k, v, lens = c3_inputs(2, device=dev)
    lens_host = lens.cpu()
    flops = c3_flops(lens_host)
    out = T.alloc_like_query(q, q.shape)
    lse = torch.empty(4, 32, 4096, dtype=torch.float32, device=dev)

    def step():
        T.sdpa_forward(q, k, v, is_causal=True, scale=scale, kv_lens=lens, out=out, lse=lse)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    T.check_device_status()
    path = T.ops.last_plan.get("path")
    T.reset_launch_counts()
    n_blocks = 5
    blocks = []
    with ClockSampler(local_rank) as clk:
        for _ in range(n_blocks):
            if world > 1:
                dist.barrier()
            blocks.append(time_steps(step, args.steps))
    launches = sum(T.launch_counts().values())
    # max over ranks per block, then the median block
    if world > 1:
        bt = torch.tensor(blocks, dtype=torch.float64, device=dev)
        dist.all_reduce(bt, op=dist.ReduceOp.MAX)
        blocks_max = bt.tolist()
    else:
        blocks_max = list(blocks)
    ms_max = median(blocks_max)
    ms = median(blocks)
    flops_total = reduce_scalar(dist, world, dev, flops, dist.ReduceOp.SUM)
    value = flops_total / (ms_max * 1e-3) / 1e12
    achieved = flops / (ms * 1e-3) / 1e12
    clocks = clk.summary()
    # one more block that runs for at least a second: the power-limited rate, with its own clock record
    n_sus = int(math.ceil(1100.0 / ms))
    if world > 1:
        dist.barrier()
    with ClockSampler(local_rank) as sclk:
        sus_ms = time_steps(step, n_sus)
    sus_ms_max = reduce_scalar(dist, world, dev, sus_ms, dist.ReduceOp.MAX)
    sustained = {"value": flops_total / (sus_ms_max * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": sus_ms_max,
                 "steps": n_sus, "seconds": sus_ms * n_sus * 1e-3, "clocks": sclk.summary(),
                 "frac_of_sustained_peak": flops / (sus_ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"]}
    # Peak to compare the headline blocks with: the burst cuBLAS figure (each block is a few ms), unless
    # the blocks themselves were power limited
    power_limited = "sw_power_cap" in clocks["reasons"] and ms * args.steps * n_blocks > 1000.0
    peak_kind = "bf16_tflops_sustained" if power_limited else "bf16_tflops"
    traffic = measured_traffic("prefill")
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks[peak_kind], "unit": "TFLOP/s",
                "frac": achieved / peaks[peak_kind],
                "traffic": traffic["dram_bytes_per_launch"] if traffic else None,
                "traffic_source": "profiles/traffic.json (ncu dram__bytes_read.sum + dram__bytes_write.sum of "
                                  "`bench.py --profile prefill`)" if traffic else None,
                "algorithmic_bytes": 2 * q.numel() * 2 + 2 * 8 * 128 * 2 * int(lens_host.sum()) + lse.numel() * 4,
                "kernel": f"{path} (bf16, D=128)",
                "peak_kind": f"{peak_kind} of {peaks['source']}", "flops_per_launch": flops,
                "frac_of_burst_peak": achieved / peaks["bf16_tflops"],
                "frac_of_sustained_peak": achieved / peaks["bf16_tflops_sustained"]}

    # ---------------- e2e: public op, pinned host buffers, copies in the timed region ---
    # Every step copies its q, k, v, kv_lens from pinned host memory, runs the public op and
    # copies the output back to pinned host memory.  Copies and compute of consecutive steps
    # overlap (separate streams, two device buffer sets), as a serving loop would do it; the
    # timed region still contains every byte of every step.
    qh, kh, vh, lh = c3_inputs(2, pinned=True)
    oh = [torch.empty(4, 32, 4096, 128, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    main = torch.cuda.current_stream(dev)
    dbuf = [[torch.empty_like(t, device=dev) for t in (qh, kh, vh, lh)] for _ in range(2)]
    obuf = [torch.empty_like(out), torch.empty_like(out)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    step_no = [0]

    def e2e_step(with_kernel=True):
        i = step_no[0] & 1
        step_no[0] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_done[i])           # the kernel that last read this buffer set is finished
            for dst, src in zip(dbuf[i], (qh, kh, vh, lh)):
                dst.copy_(src, non_blocking=True)
            ev_in[i].record(s_in)
        main.wait_event(ev_in[i])
        main.wait_event(ev_out[i])                # the previous output of this slot has left the device
        qd, kd, vd, ld = dbuf[i]
        if with_kernel:
            obuf[i] = T.scaled_dot_product_attention(qd, kd, vd, is_causal=True, scale=scale, enable_gqa=True,
                                                     kv_lens=ld)
        ev_done[i].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[i])
            oh[i].copy_(obuf[i], non_blocking=True)
            ev_out[i].record(s_out)

    def e2e_drain():
        main.wait_stream(s_in)
        main.wait_stream(s_out)

    e2e_steps = max(4, min(args.steps, 20))

    def e2e_all(with_kernel):
        for _ in range(e2e_steps):
            e2e_step(with_kernel)
        e2e_drain()

    results = {}
    for name, with_kernel in (("ceiling", False), ("e2e", True)):
        for _ in range(3):
            e2e_step(with_kernel)
        e2e_drain()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t_ms = time_steps(lambda: e2e_all(with_kernel), 1) / e2e_steps  # noqa: B023
        results[name] = reduce_scalar(dist, world, dev, t_ms, dist.ReduceOp.MAX)
    h2d = sum(t.numel() * t.element_size() for t in (qh, kh, vh, lh))
    d2h = oh[0].numel() * oh[0].element_size()
    e2e = {"value": flops_total / (results["e2e"] * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": results["e2e"], "steps": e2e_steps,
           "overlap": "copies of step i+1 / i-1 run beside the kernel of step i (3 streams, 2 buffer sets)",
           "ceiling": {"value": flops_total / (results["ceiling"] * 1e-3) / 1e12, "unit": "TFLOP/s",
                       "ms_per_step": results["ceiling"],
                       "h2d_gbs_per_gpu": h2d / (results["ceiling"] * 1e-3) / 1e9,
                       "what": "the same pinned-host copies in and out on the same streams with no kernel between "
                               "them: what the host link alone allows at this number of GPUs"}}
    del qh, kh, vh, oh, dbuf, obuf

    flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev)
    extra = {}
    threads = os.cpu_count() or 1
    run_cpu = rank == 0 and world == 1 and not args.no_cpu
    if rank == 0 and not args.no_extra:
        n_t = max(5, min(args.steps, 20))
        # ---------------- decode: configuration 4, HBM bound ----------------
        dq, dk, dv, dl = c4_inputs(dev)
        dld = dl.to(dev)
        dout = torch.empty_like(dq)
        dlse = torch.empty(64, 32, 1, dtype=torch.float32, device=dev)

        def dstep():
            T.sdpa_forward(dq, dk, dv, scale=scale, kv_lens=dld, out=dout, lse=dlse)

        for _ in range(3):
            dstep()
        torch.cuda.synchronize()
        T.check_device_status()
        dpath = T.ops.last_plan.get("path")
        dplan = dict(T.ops.last_plan)
        dms = time_steps_flushed(dstep, n_t, flush)
        kv_bytes = 2 * 8 * 128 * 2 * int(dl.sum().item())          # K and V, Hkv heads, valid rows only
        io_bytes = kv_bytes + 2 * dq.numel() * 2 + dlse.numel() * 4  # + q, out, lse
        gbs = io_bytes / (dms * 1e-3) / 1e9
        dtraffic = measured_traffic("decode")
        ratio = (dtraffic["dram_bytes_per_launch"] / dtraffic["algorithmic_bytes_per_launch"]) if dtraffic else None
        extra["decode"] = {
            "workload": "llama3-8b-shaped GQA decode bf16 q[64,32,1,128] cache[64,8,L<=8192,128], L~U[512,8192] "
                        "(configuration 4)",
            "value": gbs, "unit": "GB/s", "ms": dms, "path": dpath, "plan": dplan,
            "l2": "flushed before every timed call",
            # traffic: the ncu capture is of the 16-sequence cut (`--profile decode`); its ratio of DRAM bytes
            # to algorithmic bytes is scaled to this launch by the launch's algorithmic bytes
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": ratio * io_bytes if ratio else None,
                         "traffic_source": "profiles/traffic.json, 16-sequence capture scaled by algorithmic bytes"
                         if ratio else None,
                         "bytes_per_launch": io_bytes, "peak_kind": f"hbm_gbs of {peaks['source']}"},
        }
        # the same call replayed from a CUDA graph (how a serving loop issues its decode steps)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            dstep()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            dstep()
        gms = time_steps_flushed(graph.replay, n_t, flush)
        extra["decode"]["cuda_graph_replay"] = {"ms": gms, "value": io_bytes / (gms * 1e-3) / 1e9, "unit": "GB/s"}
        if run_cpu:
            # the reference's CPU path on the same cache: whole sequences sliced to their lengths (a bounded sample)
            hq_, hk_, hv_ = dq.cpu(), dk[:8].cpu(), dv[:8].cpu()
            cpu_decode_sample(hq_, hk_, hv_, dl, scale, [0], threads)
            c_gbs, c_t, _ = cpu_decode_sample(hq_, hk_, hv_, dl, scale, list(range(8)), threads)
            extra["decode"]["cpu_baseline"] = {"value": c_gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                                               "sample": f"the first 8 of the 64 sequences, each sliced to its "
                                                         f"length, {c_t:.1f} s of CPU oracle time"}
            del hq_, hk_, hv_
        del graph, dk, dv
        # ---------------- GPT-2-small-shaped prefill: configuration 2 ----------------
        gq, gk, gv = c2_inputs(dev)
        gout = torch.empty_like(gq)
        glse = torch.empty(8, 12, 1024, dtype=torch.float32, device=dev)

        def gstep():
            T.sdpa_forward(gq, gk, gv, is_causal=True, scale=0.125, out=gout, lse=glse)

        for _ in range(3):
            gstep()
        gms = time_steps_flushed(gstep, n_t, flush)
        gtf = C2_FLOPS / (gms * 1e-3) / 1e12
        gtraffic = measured_traffic("gpt2")
        extra["gpt2_prefill"] = {
            "workload": "gpt2-small-shaped prefill bf16 [8,12,1024,64] causal (configuration 2)",
            "value": gtf, "unit": "TFLOP/s", "ms": gms, "path": T.ops.last_plan.get("path"),
            "l2": "flushed before every timed call",
            "roofline": {"bound": "tensor", "achieved": gtf, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": gtf / peaks["bf16_tflops"],
                         "traffic": gtraffic["dram_bytes_per_launch"] if gtraffic else None,
                         "peak_kind": f"bf16_tflops of {peaks['source']}"},
        }
        # the layout upstream's callers use: [B,S,H,D] storage seen through transpose(1,2)
        gqs, gks, gvs = (t.transpose(1, 2).contiguous().transpose(1, 2) for t in (gq, gk, gv))

        def gstep_bshd():
            T.sdpa_forward(gqs, gks, gvs, is_causal=True, scale=0.125)

        for _ in range(3):
            gstep_bshd()
        gbms = time_steps_flushed(gstep_bshd, n_t, flush)
        extra["gpt2_prefill"]["bshd_storage"] = {"ms": gbms, "value": C2_FLOPS / (gbms * 1e-3) / 1e12, "unit": "TFLOP/s",
                                                 "path": T.ops.last_plan.get("path"),
                                                 "what": "q/k/v are transpose(1,2) views of [B,S,H,D] storage, output "
                                                         "allocated by the op in the query's layout"}
        if run_cpu:
            from oracle import sdpa_oracle as O

            torch.set_num_threads(threads)
            cq, ck, cv = c2_inputs()
            O.sdpa_forward(cq, ck, cv, is_causal=True, scale=0.125)
            ts = []
            for _ in range(3):
                t0 = time.perf_counter()
                O.sdpa_forward(cq, ck, cv, is_causal=True, scale=0.125)
                ts.append(time.perf_counter() - t0)
            extra["gpt2_prefill"]["cpu_baseline"] = {"value": C2_FLOPS / median(ts) / 1e12, "unit": "TFLOP/s",
                                                     "cores": threads, "kind": "port",
                                                     "sample": f"the whole configuration, median of 3 ({median(ts):.2f} s)"}
        del gq, gk, gv, gqs, gks, gvs
        # ---------------- configuration 3 in [B,S,H,D] storage ----------------
        qs_, ks_, vs_ = (t.transpose(1, 2).contiguous().transpose(1, 2) for t in (q, k, v))
        outs_ = T.alloc_like_query(qs_, qs_.shape)

        def step_bshd():
            T.sdpa_forward(qs_, ks_, vs_, is_causal=True, scale=scale, kv_lens=lens, out=outs_, lse=lse)

        for _ in range(3):
            step_bshd()
        sms = time_steps_flushed(step_bshd, n_t, flush)
        extra["config3_bshd"] = {
            "workload": "configuration 3 with q/k/v as transpose(1,2) views of [B,S,H,D] storage (the layout of "
                        "upstream's callers and stride tests); the output takes the query's layout",
            "value": flops / (sms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": sms, "path": T.ops.last_plan.get("path"),
            "out_strides": list(outs_.stride()), "l2": "flushed before every timed call",
        }
        del qs_, ks_, vs_, outs_
        # ---------------- backward of the headline configuration (tensor-core kernels) ----------------
        bgo = torch.randn(q.shape, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).to(dev)
        bgq, bgk, bgv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        step()

        def bstep():
            T.sdpa_backward(bgo, q, k, v, out, lse, is_causal=True, scale=scale, kv_lens=lens, grad_q=bgq, grad_k=bgk,
                            grad_v=bgv)

        for _ in range(3):
            bstep()
        torch.cuda.synchronize()
        T.check_device_status()
        bms = time_steps_flushed(bstep, n_t, flush)
        bflops = 2.5 * flops                      # five tile products against the forward's two
        btf = bflops / (bms * 1e-3) / 1e12
        extra["backward_config3"] = {
            "workload": "backward of configuration 3 (bf16, causal, ragged lengths): grad_q, grad_k, grad_v",
            "value": btf, "unit": "TFLOP/s (2.5 x forward FLOPs: the 5-product count)", "ms": bms,
            "path": T.ops.last_bwd_plan.get("path"), "launches": T.ops.last_bwd_plan.get("launches"),
            "l2": "flushed before every timed call",
            "roofline": {"bound": "tensor", "achieved": btf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": btf / peaks["bf16_tflops"], "traffic": None,
                         "peak_kind": f"bf16_tflops of {peaks['source']}"},
        }
        # ---------------- forward + backward back to back (what one attention layer costs in training) ----------------
        def tstep():
            step()
            bstep()

        tms = time_steps_flushed(tstep, n_t, flush)
        extra["train_step_config3"] = {
            "workload": "forward + backward of configuration 3, one call each",
            "value": 3.5 * flops / (tms * 1e-3) / 1e12, "unit": "TFLOP/s (3.5 x forward FLOPs)", "ms": tms,
            "l2": "flushed before every timed call",
        }
        del bgo, bgq, bgk, bgv
        # ---------------- additive bias and the wide head dims on the tensor-core kernels ----------------
        gen = torch.Generator(device=dev).manual_seed(7)
        bias = torch.randn(4096, 4096, generator=gen, device=dev, dtype=torch.bfloat16)
        aout, alse = torch.empty_like(out), torch.empty_like(lse)

        def bias_step():
            T.sdpa_forward(q, k, v, attn_bias=bias, scale=scale, out=aout, lse=alse)

        for _ in range(3):
            bias_step()
        ams = time_steps_flushed(bias_step, max(5, min(args.steps, 10)), flush)
        aflops = 4.0 * 128 * 4 * 32 * 4096 * 4096
        extra["bias_prefill"] = {
            "workload": "configuration 3 tensors, non-causal, with a bf16 [4096,4096] additive bias shared by batch and heads",
            "value": aflops / (ams * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": ams, "path": T.ops.last_plan.get("path"),
            "l2": "flushed before every timed call",
        }
        del bias, aout, alse
        wq = torch.randn(4, 32, 4096, 192, generator=gen, device=dev, dtype=torch.bfloat16)
        wk = torch.randn(4, 32, 4096, 192, generator=gen, device=dev, dtype=torch.bfloat16)
        wv = torch.randn(4, 32, 4096, 128, generator=gen, device=dev, dtype=torch.bfloat16)
        wout = torch.empty(4, 32, 4096, 128, device=dev, dtype=torch.bfloat16)
        wlse = torch.empty(4, 32, 4096, dtype=torch.float32, device=dev)

        def wide_step():
            T.sdpa_forward(wq, wk, wv, is_causal=True, out=wout, lse=wlse)

        for _ in range(3):
            wide_step()
        wms = time_steps_flushed(wide_step, max(5, min(args.steps, 10)), flush)
        wflops = 2.0 * (192 + 128) * 4 * 32 * (4096 * 4097 // 2)
        extra["mla_shape_prefill"] = {
            "workload": "q/k head dim 192, v head dim 128, bf16 [4,32,4096] causal, multi-head (the shape of upstream's "
                        "multi-head-latent-attention test, at benchmark size)",
            "value": wflops / (wms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": wms, "path": T.ops.last_plan.get("path"),
            "l2": "flushed before every timed call",
        }
        del wq, wk, wv, wout, wlse
        # ---------------- fp32 parity configuration: latency only ----------------
        g = torch.Generator().manual_seed(0)
        fq, fk, fv = (torch.randn(2, 8, 512, 64, generator=g).to(dev) for _ in range(3))
        for _ in range(3):
            T.sdpa_forward(fq, fk, fv, is_causal=True, scale=0.125)
        fms = time_steps_flushed(lambda: T.sdpa_forward(fq, fk, fv, is_causal=True, scale=0.125), 5, flush)
        extra["fp32_config1"] = {"workload": "fp32 [2,8,512,64] causal (configuration 1)", "ms": fms,
                                 "path": T.ops.last_plan.get("path")}
        # ---------------- host cost of one call (no synchronisation between calls) ----------------
        extra["host_us_per_call"] = host_overhead(T, dev)

    if not args.no_extra:
        extra["partition_c3"] = run_partition_c3(T, dist, dev, rank, world, q, k, v, lens, lens_host, scale, flush, peaks)
        extra["decode_per_n"] = run_decode_partition(T, dist, dev, rank, world, scale, flush, peaks)
        del q, k, v, out, lse
        torch.cuda.empty_cache()
        ring = run_ring(T, dist, dev, rank, world, peaks, run_cpu_rows=not args.no_cpu)
        extra["ring_long_context"] = ring
        if not ring["ring_check"]["ok"]:
            failures.append("ring_check")
        if world > 1:
            extra["dtensor_check"] = run_dtensor_check(T, dist, dev, rank, world)
            if not extra["dtensor_check"]["ok"]:
                failures.append("dtensor_check")

    cpu_baseline = None
    if run_cpu:
        qc, kc, vc, lc = c3_inputs(2)
        cpu_prefill_sample(qc, kc, vc, lc, scale, c3_slices(1), threads)  # warm-up
        # grow the sample until it holds about 10 s of CPU work (at most two passes over all 32 slices)
        flops_done, secs, n_done = 0.0, 0.0, 0
        while secs < 10.0 and n_done < 64:
            sl = c3_slices(32)[n_done % 32 : n_done % 32 + 8]
            _, t_, f_ = cpu_prefill_sample(qc, kc, vc, lc, scale, sl, threads)
            flops_done, secs, n_done = flops_done + f_, secs + t_, n_done + 8
        cpu_baseline = {"value": flops_done / secs / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                        "sample": f"{n_done} (batch x kv-group) slices [1,4,4096,128] of the same workload, spread "
                                  f"over its four batches, {secs:.1f} s of CPU oracle time"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": dict(CONFIG_C3),
            "per_gpu_tflops": value / world,
            "timing": f"median of {n_blocks} blocks of {args.steps} launches (max over ranks per block)",
            "blocks_ms": blocks_max, "sustained": sustained,
            "roofline": roofline, "e2e": e2e, "cpu_baseline": cpu_baseline, "clocks": clocks,
            "gpu_launches": launches,
            "decode_roofline": extra.get("decode", {}).get("roofline"),
            "extra": extra,
        }
        if failures:
            line["failed_checks"] = failures
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if failures:
        sys.exit(3)


def host_overhead(T, dev):
    """Host time per call of the three entry levels, 1000 calls each without synchronising in between,
    on a problem so small that the GPU never pushes back."""
    g = torch.Generator().manual_seed(9)
    q, k, v = ((torch.randn(1, 2, 128, 64, generator=g)).to(torch.bfloat16).to(dev) for _ in range(3))
    out = torch.empty_like(q)
    lse = torch.empty(1, 2, 128, dtype=torch.float32, device=dev)
    calls = {
        "sdpa_forward (buffers given)": lambda: T.sdpa_forward(q, k, v, is_causal=True, out=out, lse=lse),
        "aten overrideable op": lambda: torch.ops.aten._scaled_dot_product_fused_attention_overrideable(
            q, k, v, None, 0.0, True),
        "scaled_dot_product_attention": lambda: T.scaled_dot_product_attention(q, k, v, is_causal=True),
    }
    res = {}
    with torch.no_grad():
        for name, fn in calls.items():
            for _ in range(50):
                fn()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(1000):
                fn()
            t1 = time.perf_counter()
            torch.cuda.synchronize()
            res[name] = (t1 - t0) * 1e3  # 1000 calls: seconds * 1e6 / 1000
    return res


# ----------------------------------------------------------------------------- (batch x kv head) partitions


def run_partition_c3(T, dist, dev, rank, world, q, k, v, lens, lens_host, scale, flush, peaks):
    """Configuration 3's 32 (batch x kv head) units cut over the ranks by cost: every rank computes its own
    contiguous range, nothing is exchanged.  Strong scaling of ONE configuration (the headline is weak scaling)."""
    n_units = 32
    costs = [c3_flops(lens_host[u // 8 : u // 8 + 1], hq=4) for u in range(n_units)]
    qu, ku, vu, lu, (s, e) = T.local_units(q, k, v, rank, world, kv_lens=lens, costs=costs)
    outu = torch.empty_like(qu)
    lseu = torch.empty(qu.shape[0], qu.shape[1], qu.shape[2], dtype=torch.float32, device=dev)
    my_flops = float(sum(costs[s:e]))

    def fn():
        T.sdpa_forward(qu, ku, vu, is_causal=True, scale=scale, kv_lens=lu, out=outu, lse=lseu)

    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    T.check_device_status()
    if world > 1:
        dist.barrier()
    ms = time_steps_flushed(fn, 10, flush)
    ms_max = reduce_scalar(dist, world, dev, ms, dist.ReduceOp.MAX)
    total = float(sum(costs))
    res = {
        "workload": f"configuration 3's 32 (batch x kv head) units over {world} GPUs, contiguous ranges balanced by "
                    "visible (query, key) pairs, no collective",
        "value": total / (ms_max * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": ms_max, "scaling": "strong",
        "per_gpu_tflops": total / (ms_max * 1e-3) / 1e12 / world, "units_rank0": e - s,
        "l2": "flushed before every timed call", "rank0_tflops": my_flops / (ms * 1e-3) / 1e12,
    }
    if world > 1:
        # all 32 units on one GPU in the same run: the reference point of the scaling efficiency
        qa, ka, va, la = T.as_units(q, k, v, lens)
        oa = torch.empty_like(qa)
        sa = torch.empty(32, 4, 4096, dtype=torch.float32, device=dev)
        one = lambda: T.sdpa_forward(qa, ka, va, is_causal=True, scale=scale, kv_lens=la, out=oa, lse=sa)  # noqa: E731
        for _ in range(3):
            one()
        ms1 = time_steps_flushed(one, 10, flush)
        ms1 = reduce_scalar(dist, world, dev, ms1, dist.ReduceOp.MAX)
        res["one_gpu_ms_same_run"] = ms1
        res["efficiency_vs_one_gpu"] = ms1 / (world * ms_max)
    return res


def run_decode_partition(T, dist, dev, rank, world, scale, flush, peaks):
    """Configuration 4's 512 (sequence x kv head) units cut over the ranks, balanced by cache length; every
    rank streams its own share of the cache with L2 flushed before each call."""
    q, k, v, lens = c4_inputs(dev)
    costs = [float(lens[u // 8]) for u in range(512)]
    qu, ku, vu, lu, (s, e) = T.local_units(q, k, v, rank, world, kv_lens=lens.to(dev), costs=costs)
    lu = lu.contiguous()
    outu = torch.empty_like(qu)
    lseu = torch.empty(qu.shape[0], 4, 1, dtype=torch.float32, device=dev)
    my_bytes = sum(2 * 128 * 2 * c for c in costs[s:e]) + 2 * qu.numel() * 2 + lseu.numel() * 4

    def fn():
        T.sdpa_forward(qu, ku, vu, scale=scale, kv_lens=lu, out=outu, lse=lseu)

    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    T.check_device_status()
    plan = dict(T.ops.last_plan)
    if world > 1:
        dist.barrier()
    ms = time_steps_flushed(fn, 10, flush)
    ms_max = reduce_scalar(dist, world, dev, ms, dist.ReduceOp.MAX)
    total_bytes = reduce_scalar(dist, world, dev, my_bytes, dist.ReduceOp.SUM)
    my_gbs = my_bytes / (ms * 1e-3) / 1e9
    gbs_min = reduce_scalar(dist, world, dev, my_gbs, dist.ReduceOp.MIN)
    agg = total_bytes / (ms_max * 1e-3) / 1e9
    del k, v
    return {
        "workload": f"configuration 4's 512 (sequence x kv head) units over {world} GPUs, contiguous ranges balanced "
                    "by cache length, no collective",
        "value": agg, "unit": "GB/s", "ms": ms_max, "scaling": "strong", "per_gpu_gbs": agg / world,
        "slowest_gpu_gbs": gbs_min, "units_rank0": e - s, "plan_rank0": plan,
        "l2": "flushed before every timed call",
        "roofline": {"bound": "hbm", "achieved": agg / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": agg / world / peaks["hbm_gbs"], "peak_kind": f"hbm_gbs of {peaks['source']}"},
    }


# ----------------------------------------------------------------------------- configuration 5: the ring


def _global_positions(local_idx, rank, world, n_local, layout):
    """Global sequence position of local row indices (a tensor) of this rank's shard."""
    if layout == "contiguous":
        return local_idx + rank * n_local
    c = n_local // 2
    lo = local_idx < c
    return torch.where(lo, local_idx + rank * c, local_idx - c + (2 * world - 1 - rank) * c)


def run_ring(T, dist, dev, rank, world, peaks, run_cpu_rows=True):
    """Configuration 5: one causal 131072-token sequence, bf16 q [1,64,S,128], k/v [1,8,S,128],
    sequence-sharded over the ranks (zigzag placement), K/V blocks rotated with NCCL
    send/recv while the previous block is being computed.  With one GPU the same driver runs
    as a ring of one.  The result is checked on sampled rows (see ``ring_check``)."""
    from torch_neuronx_b200 import _lib, ring as R

    S, Hq, Hkv, D = 131072, 64, 8, 128
    layout = "zigzag"
    n_local = S // world
    g = torch.Generator(device=dev).manual_seed(4000 + rank)
    q = torch.randn(1, Hq, n_local, D, generator=g, device=dev, dtype=torch.bfloat16)
    k = torch.randn(1, Hkv, n_local, D, generator=g, device=dev, dtype=torch.bfloat16)
    v = torch.randn(1, Hkv, n_local, D, generator=g, device=dev, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    timeline = []

    def step(trace=None):
        return T.ring_attention(q, k, v, is_causal=True, scale=scale, layout=layout, trace=trace)

    step()
    torch.cuda.synchronize()
    T.check_device_status()
    iters = 5
    times = []
    for _ in range(iters):
        if world > 1:
            dist.barrier()
        times.append(time_each(step, 1)[0])
    if world > 1:
        tt = torch.tensor(times, dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        times = tt.tolist()
    ms = median(times)
    flops = 4.0 * D * Hq * (S * (S + 1) // 2)
    tf = flops / (ms * 1e-3) / 1e12
    block_bytes = 2 * n_local * Hkv * D * 2
    out, lse = step(trace=timeline)
    torch.cuda.synchronize()
    steps_ms = R.trace_to_ms(timeline)

    # ---- ring backward of the same sequence: K/V blocks travel as in the forward, their fp32 gradient
    # accumulators follow one step behind
    go = torch.randn(q.shape, generator=g, device=dev, dtype=torch.bfloat16)

    def bstep():
        return T.ring_attention_backward(go, q, k, v, out, lse, is_causal=True, scale=scale, layout=layout)

    bstep()
    torch.cuda.synchronize()
    T.check_device_status()
    btimes = []
    for _ in range(3):
        if world > 1:
            dist.barrier()
        btimes.append(time_each(bstep, 1)[0])
    if world > 1:
        tt = torch.tensor(btimes, dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        btimes = tt.tolist()
    bms = median(btimes)
    btf = 2.5 * flops / (bms * 1e-3) / 1e12
    dq, dk, dv = bstep()
    torch.cuda.synchronize()

    check = ring_check(T, R, _lib, dist, dev, rank, world, layout, q, k, v, go, out, lse, dq, dk, dv, scale,
                       run_cpu_rows)
    del dq, dk, dv, go, out, lse
    torch.cuda.empty_cache()
    return {
        "workload": f"long-context causal GQA prefill bf16 q[1,64,131072,128] kv[1,8,131072,128] over {world} GPU(s) "
                    "(configuration 5), zigzag ring, K/V rotated un-expanded over NCCL send/recv",
        "value": tf, "unit": "TFLOP/s", "per_gpu_tflops": tf / world, "ms": ms, "iters": iters, "iters_ms": times,
        "ring_bytes_per_step_per_gpu": block_bytes, "ring_steps": world - 1,
        "roofline": {"bound": "tensor", "achieved": tf / world, "peak": peaks["bf16_tflops_sustained"],
                     "unit": "TFLOP/s", "frac": tf / world / peaks["bf16_tflops_sustained"],
                     "peak_kind": f"bf16_tflops_sustained of {peaks['source']}",
                     "link_time_ms_per_step": block_bytes / 770e9 * 1e3},
        "rank0_step_timeline_ms": steps_ms,
        "backward": {"value": btf, "unit": "TFLOP/s (2.5 x forward FLOPs)", "per_gpu_tflops": btf / world,
                     "ms": bms, "iters_ms": btimes, "accumulator_bytes_per_step_per_gpu": 2 * block_bytes},
        "ring_check": check,
    }


def ring_check(T, R, _lib, dist, dev, rank, world, layout, q, k, v, go, out, lse, dq, dk, dv, scale, run_cpu_rows):
    """Correctness of the full-size ring result on sampled rows (outside every timed region), after upstream's
    recipe for its context-parallel test (tests/distributed/dtensor/test_scaled_dot_product_attention.py:
    515-525 compares with full attention, :624-628 insists that the result differs from local-only attention):

    * forward: 64 query rows per rank (first / last rows of both zigzag chunks, the rows either side of the
      chunk border, seeded others) recomputed against the all-gathered K/V by the independent CUDA-core
      kernel, and a few of them by the CPU oracle;
    * negative guard: the same rows must differ (in their log-sum-exp) from attention over this rank's own
      keys only;
    * backward: grad_k / grad_v of two 64-key blocks per rank (all queries) and grad_q of two 64-row blocks
      (all keys) recomputed by the CUDA-core backward kernels from the all-gathered tensors."""
    n_local, Hq, D = q.shape[2], q.shape[1], q.shape[3]
    Hkv = k.shape[1]
    c = n_local // 2

    def gather(t, dim=2):
        if world == 1:
            return t
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous())
        return R.unshard_sequence(parts, layout, dim=dim)

    kg, vg = gather(k), gather(v)
    S = kg.shape[2]
    gen = torch.Generator().manual_seed(1234 + rank)
    fixed = [0, 1, c - 1, c, c + 1, n_local - 1, c // 2, c + c // 2]
    rnd = torch.randint(0, n_local, (64 - len(fixed),), generator=gen).tolist()
    rows = torch.tensor(sorted(set(fixed + rnd)), dtype=torch.long)
    pos = _global_positions(rows, rank, world, n_local, layout)
    n_rows = rows.numel()
    rows_d, pos_d = rows.to(dev), pos.to(dev)

    # forward rows on the CUDA-core kernel: every sampled row is a "batch" of its own with its key count
    # (fp32 copies of the operands: the reference is the fp32 result, as in the parity tests)
    q_rows = q[0][:, rows_d].permute(1, 0, 2).unsqueeze(2).contiguous()            # (rows, Hq, 1, D)
    ke, ve = kg.float().expand(n_rows, Hkv, S, D), vg.float().expand(n_rows, Hkv, S, D)   # batch stride 0
    want_o, want_l = T.sdpa_forward(q_rows.float(), ke, ve, scale=scale, kv_lens=(pos_d + 1).to(torch.int32),
                                    force_path=_lib.PATH_GENERIC)
    torch.cuda.synchronize()
    generic_path = T.ops.last_plan.get("path")
    del ke, ve
    got_o = out[0][:, rows_d].permute(1, 0, 2)                                    # (rows, Hq, D)
    got_l = lse[0][:, rows_d].permute(1, 0)
    err_o = (got_o.float() - want_o[:, :, 0].float()).abs().max().item()
    err_l = (got_l - want_l[:, :, 0]).abs().max().item()

    # negative guard: attention over this rank's own keys only (a ring of one has nothing else)
    guard = guard_out = float("inf")
    if world > 1:
        st = R.RankState(q, D, layout)
        R.ring_step(st, k, v, rank, rank, world, layout, True, scale, R._default_attn, R._default_merge)
        loc_o, loc_l = st.finish(q.dtype)
        # the log-sum-exp is the robust witness: dropping the other ranks' keys lowers it by about log(share
        # of the keys that is local), whatever the scale of the values
        guard = (loc_l[0][:, rows_d] - lse[0][:, rows_d]).abs().max().item()
        guard_out = (loc_o[0][:, rows_d].float() - out[0][:, rows_d].float()).abs().max().item()
        del st, loc_o, loc_l

    # a few rows on the CPU oracle (two kv groups each)
    err_o_cpu = err_l_cpu = None
    n_cpu = 0
    if run_cpu_rows:
        from oracle import sdpa_oracle as O

        torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
        err_o_cpu = err_l_cpu = 0.0
        pick = [0, n_rows // 2, n_rows - 1, n_rows // 3, 2 * n_rows // 3, 1, n_rows - 2, n_rows // 4][: max(2, 8 // world)]
        group = Hq // Hkv
        for i in pick:
            n_keys = int(pos[i]) + 1
            for hk in (0, Hkv - 1):
                hs = slice(hk * group, (hk + 1) * group)
                ro, rl = O.sdpa_forward(q_rows[i : i + 1, hs].cpu(), kg[:, hk : hk + 1, :n_keys].cpu(),
                                        vg[:, hk : hk + 1, :n_keys].cpu(), scale=scale, compute_dtype=torch.float32)
                err_o_cpu = max(err_o_cpu, (got_o[i, hs].cpu().float() - ro[0, :, 0]).abs().max().item())
                err_l_cpu = max(err_l_cpu, (got_l[i, hs].cpu() - rl[0, :, 0]).abs().max().item())
            n_cpu += 1

    # backward: all-gathered q, grad_out, out, lse; two key blocks and two row blocks per rank
    qg, gog, outg = gather(q), gather(go), gather(out)
    lseg = gather(lse.unsqueeze(-1)).squeeze(-1)
    bwd_err = {"dq": 0.0, "dk": 0.0, "dv": 0.0}
    bwd_bad = 0
    blocks = [(c // 3) // 64 * 64, c + ((2 * c) // 3) // 64 * 64]

    def close(got, want):
        diff = (got.float() - want.float()).abs()
        bad = int((diff > 2e-2 + 5e-2 * want.float().abs()).sum().item())
        return diff.max().item(), bad

    for j_local in blocks:
        j0 = int(_global_positions(torch.tensor([j_local]), rank, world, n_local, layout)[0])
        _, gk, gv, _ = T.sdpa_backward(gog, qg, kg[:, :, j0 : j0 + 64], vg[:, :, j0 : j0 + 64], outg, lseg,
                                       is_causal=True, scale=scale, q_offset=0, k_offset=j0,
                                       force_path=_lib.PATH_GENERIC)
        for name, got, want in (("dk", dk[:, :, j_local : j_local + 64], gk), ("dv", dv[:, :, j_local : j_local + 64], gv)):
            m, bad = close(got, want)
            bwd_err[name] = max(bwd_err[name], m)
            bwd_bad += bad
        i0 = j0   # the same global positions as a block of query rows
        gq, _, _, _ = T.sdpa_backward(go[:, :, j_local : j_local + 64], q[:, :, j_local : j_local + 64], kg, vg,
                                      out[:, :, j_local : j_local + 64], lse[:, :, j_local : j_local + 64],
                                      is_causal=True, scale=scale, q_offset=i0, k_offset=0,
                                      force_path=_lib.PATH_GENERIC)
        m, bad = close(dq[:, :, j_local : j_local + 64], gq)
        bwd_err["dq"] = max(bwd_err["dq"], m)
        bwd_bad += bad
    torch.cuda.synchronize()
    T.check_device_status()
    bwd_path = T.ops.last_bwd_plan.get("path")
    del qg, gog, outg, lseg, kg, vg

    mx = lambda x: reduce_scalar(dist, world, dev, x, dist.ReduceOp.MAX)  # noqa: E731
    res = {
        "rows_per_rank": n_rows, "checker": f"{generic_path} (CUDA-core) kernel on all-gathered K/V",
        "max_abs_out": mx(err_o), "max_abs_lse": mx(err_l),
        "guard_diff": reduce_scalar(dist, world, dev, guard, dist.ReduceOp.MIN) if world > 1 else None,
        "guard_diff_out": reduce_scalar(dist, world, dev, guard_out, dist.ReduceOp.MIN) if world > 1 else None,
        "cpu_rows_per_rank": n_cpu,
        "max_abs_out_cpu": mx(err_o_cpu) if err_o_cpu is not None else None,
        "max_abs_lse_cpu": mx(err_l_cpu) if err_l_cpu is not None else None,
        "backward": {"checker": f"{bwd_path} (CUDA-core) backward kernels", "key_blocks_per_rank": len(blocks),
                     "row_blocks_per_rank": len(blocks), "max_abs_dq": mx(bwd_err["dq"]),
                     "max_abs_dk": mx(bwd_err["dk"]), "max_abs_dv": mx(bwd_err["dv"]),
                     "elements_outside_5e-2_rel_2e-2_abs": int(mx(bwd_bad))},
        "bars": "out max-abs <= 2e-2, lse <= 1e-3, guard_diff (largest |lse - lse of local-only attention| over the "
                "sampled rows, smallest over ranks) > 0.1, gradients within 2e-2 + 5e-2 |ref|",
    }
    ok = res["max_abs_out"] <= 2e-2 and res["max_abs_lse"] <= 1e-3 and res["backward"]["elements_outside_5e-2_rel_2e-2_abs"] == 0
    ok = ok and (world == 1 or res["guard_diff"] > 0.1)
    if res["max_abs_out_cpu"] is not None:
        ok = ok and res["max_abs_out_cpu"] <= 2e-2 and res["max_abs_lse_cpu"] <= 1e-3
    res["ok"] = bool(ok)
    return res


def run_dtensor_check(T, dist, dev, rank, world):
    """A sequence-sharded DTensor forward + backward through torch's context-parallel dispatcher (the handler
    this package installs) against full attention on the CPU oracle, and a head-sharded DTensor through the
    registered placements.  Small shapes; correctness only."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import DTensor, Shard
    from torch.distributed.tensor.experimental._context_parallel import _attention as cp

    from oracle import sdpa_oracle as O
    from torch_neuronx_b200 import dtensor as D

    res = {"ok": False}
    try:
        mesh = init_device_mesh("cuda", (world,))
        if not D.install_context_parallel_handler():
            res["error"] = "context-parallel handler could not be installed"
            return res
        g = torch.Generator().manual_seed(0)
        S = 256 * world
        q = torch.randn(1, 8, S, 64, generator=g)
        k = torch.randn(1, 2, S, 64, generator=g)
        v = torch.randn(1, 2, S, 64, generator=g)
        go = torch.randn(1, 8, S, 64, generator=g)
        ref_o, ref_l = O.sdpa_forward(q, k, v, is_causal=True)
        ref_g = O.sdpa_backward(go, q, k, v, ref_o, ref_l, is_causal=True)
        worst = 0.0
        for layout in ("zigzag", "contiguous"):
            D.set_sequence_layout(layout)
            loc = [T.shard_sequence(t, rank, world, layout).contiguous().to(dev) for t in (q, k, v, go)]
            qd, kd, vd = (DTensor.from_local(t, mesh, [Shard(2)]).requires_grad_() for t in loc[:3])
            cp._enable_cp_dtensor_dispatcher()
            try:
                o = torch.ops.aten._scaled_dot_product_fused_attention_overrideable(qd, kd, vd, None, 0.0, True)[0]
                o.backward(DTensor.from_local(loc[3], mesh, [Shard(2)]))
            finally:
                cp._disable_cp_dtensor_dispatcher()
            torch.cuda.synchronize()
            T.check_device_status()
            errs = [(o.to_local().detach().cpu() - T.shard_sequence(ref_o, rank, world, layout)).abs().max().item()]
            for got, want in zip((qd.grad, kd.grad, vd.grad), ref_g[:3]):
                errs.append((got.to_local().cpu() - T.shard_sequence(want, rank, world, layout)).abs().max().item())
            res[f"sequence_sharded_{layout}_max_abs(out,dq,dk,dv)"] = errs
            worst = max(worst, errs[0] / 1e-5, max(errs[1:]) / 1e-4)
        # head-sharded DTensors need no exchange: the registered placements run the op on the local heads
        qh = torch.randn(1, 2 * world, 128, 64, generator=g)
        kh = torch.randn(1, world, 128, 64, generator=g)
        vh = torch.randn(1, world, 128, 64, generator=g)
        goh = torch.randn(1, 2 * world, 128, 64, generator=g)
        rh_o, rh_l = O.sdpa_forward(qh, kh, vh, is_causal=True)
        rh_g = O.sdpa_backward(goh, qh, kh, vh, rh_o, rh_l, is_causal=True)
        parts = [t.chunk(world, dim=1)[rank].contiguous().to(dev) for t in (qh, kh, vh, goh)]
        qd, kd, vd = (DTensor.from_local(t, mesh, [Shard(1)]).requires_grad_() for t in parts[:3])
        o = torch.ops.aten._scaled_dot_product_fused_attention_overrideable(qd, kd, vd, None, 0.0, True)[0]
        o.backward(DTensor.from_local(parts[3], mesh, [Shard(1)]))
        torch.cuda.synchronize()
        errs = [(o.to_local().detach().cpu() - rh_o.chunk(world, dim=1)[rank]).abs().max().item()]
        for got, want in zip((qd.grad, kd.grad, vd.grad), rh_g[:3]):
            errs.append((got.to_local().cpu() - want.chunk(world, dim=1)[rank]).abs().max().item())
        res["head_sharded_max_abs(out,dq,dk,dv)"] = errs
        worst = max(worst, errs[0] / 1e-5, max(errs[1:]) / 1e-4)
        worst = reduce_scalar(dist, world, dev, worst, dist.ReduceOp.MAX)
        res["worst_error_over_bar"] = worst
        res["bars"] = "fp32: out <= 1e-5, gradients <= 1e-4 (max-abs, all ranks)"
        res["ok"] = bool(worst <= 1.0)
    except Exception as exc:  # reported, and the run fails
        res["error"] = f"{type(exc).__name__}: {exc}"[:300]
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--profile", default=None, choices=["prefill", "decode", "gpt2", "bwd", "wide", "bias"],
                    help="bare kernel loop on one GPU for profiler captures")
    ap.add_argument("--ingest-ncu", default=None, metavar="CSV",
                    help="with --profile and --kernel: record the DRAM bytes per launch of a capture "
                         "(`ncu -i report --page raw --csv > CSV`) in profiles/traffic.json")
    ap.add_argument("--kernel", default="", help="substring of the kernel name for --ingest-ncu")
    ap.add_argument("--algorithmic-bytes", type=float, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="headline, e2e and CPU baseline only")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU legs")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.ingest_ncu:
        ingest_ncu(args)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.profile:
        run_profile_case(args)
        return
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
