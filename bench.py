"""Benchmark of the decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one decode call over one batch of synthetic K/V already resident in
HBM.  The metric is achieved KV-bytes/s (algorithmic bytes of the call divided by
its time); ``ms_per_step`` is the time of one call.

Workloads (BASELINE.json configs):
  exact_c2   exact contiguous GQA decode, B8 Hq16 Hkv2 D64 N65536 bf16, head-major KV   [default at N=1]
  exact_c2_bnhd  same values in the public BNHD layout
  paged_c3   paged HND page-16, ragged lengths U[16384, 65536], random page order
  seed_c4    seed-only decode, Qwen2.5-3B attention shape, 384 seed tokens of 32768
  loop_c2    one decode-loop step on the config-2 cache: RoPE + KV append, then exact decode
  o_proj_3b  the output projection that follows attention, Qwen2.5-3B shape (2048 x 2048 bf16 weights)
  cp_c5      context-parallel exact decode, B1 Hq32 Hkv8 D128 N1048576 sharded over N GPUs
             (strong scaling; state exchange fused into the decode kernel over peer memory) [default at N>1]

Under torchrun (N>1) every rank runs; timing is the max over ranks of CUDA-event
time between a barrier + synchronize on both sides.  ``--impl reference`` times the
reference's CPU PyTorch path (restated in ``oracle/torch_port.py``) on the host
cores, on a bounded sample of the same workload.

Two timings are reported for every workload.  ``value`` / ``ms_per_step`` come from the
one region of ``--steps`` calls after ``--warmup`` calls.  ``protocol`` is independent of
``--steps``: at least 20 warm-up calls, then 9 repeats of at least 200 calls each, every
repeat between its own pair of CUDA events; it gives the median, minimum and maximum
microseconds per call over the repeats (the reference times its kernels the same way,
benchmarks/profile_paged_exact_decode.py:284-309).  At N=1 the line also carries a
``secondary`` list with the other configurations (paged, seed-only, BNHD, decode loop and
the 1M-token row on one GPU - the base of the strong-scaling series), each with its own
protocol timing, roofline figures, end-to-end time, the time per call under CUDA-graph replay
(``graph_replay``: 20 calls per graph) and clock record, and an entry
``exact_c2_plain_launch``: config 2 timed in a child process without programmatic dependent
launch, i.e. with nothing of a call overlapping the call before it.
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
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
# Keep stdout to the one JSON line: libraries (NCCL's version banner, for one) write to fd 1.
# Everything written to stdout before the result goes to stderr; emit() writes the real stdout.
_REAL_STDOUT = os.dup(1)
os.dup2(2, 1)


def emit(line: dict) -> None:
    sys.stdout.flush()
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())

METRIC = "kv_bytes_per_second"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
# The reference's published number for the same metric and shape (its serving-gate artifact
# artifacts/gate0/transposed_wgmma_exact_promoted_serving_gate_h100_20260818.json): config 2 on
# one H100 (not a B200), 96.3 us per call = 2787 GB/s.
PUBLISHED_GBS = {"exact_c2": 268435456 / 96.3e-6 / 1e9}
# DRAM bytes (read + write) per launch of the dominant kernel: stored results of earlier ncu
# captures of this kernel (dram__bytes_read.sum + dram__bytes_write.sum), not measured by this run.
NCU_TRAFFIC = {
    "exact_c2": (272.3e6, "profiles/stream_decode_exact_c2.md"),
    "paged_c3": (170.9e6, "profiles/stream_decode_paged_c3.md"),
    # one eighth of the 1M-token row was captured; traffic grows in proportion to the tokens read
    "cp_c5": (8 * 540.5e6, "profiles/stream_decode_cp_shard_d128.md"),
    "cp_c5_1gpu": (8 * 540.5e6, "profiles/stream_decode_cp_shard_d128.md"),
}


def measured_hbm_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """SM clock and throttle reasons while a region runs, sampled by an ``nvidia-smi`` child process.

    The sampler is a separate process on purpose: a sampling thread inside the timed process
    (NVML queries every few ms, competing for the interpreter lock with the launch loop) was
    measured to slow lock-stepped multi-GPU steps by 15 % at 8 ranks, because a launch loop that
    hiccups on one rank stalls every rank.  ``nvidia-smi -lms`` samples every ``period_ms``; the
    lines whose time stamp falls inside [begin(), end()] are summarised.
    """

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}
    QUERY = "timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.active"

    def __init__(self, index: int, period_ms: int = 25) -> None:
        self.index = index
        self.period_ms = period_ms
        self._proc = None
        self._log = None
        self._edge_samples = []  # (time, MHz, max MHz, reason bits): NVML readings taken by this process

    def start(self) -> "ClockSampler":
        import shutil
        import subprocess
        import tempfile

        exe = shutil.which("nvidia-smi")
        if exe is not None:
            self._log = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            try:
                self._proc = subprocess.Popen(
                    [exe, "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                     "-lms", str(self.period_ms)], stdout=self._log, stderr=subprocess.DEVNULL)
            except OSError:
                self._proc = None
        return self

    def _nvml_once(self) -> None:
        import datetime

        try:
            import pynvml

            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            get = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            self._edge_samples.append((datetime.datetime.now(),
                                       int(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)),
                                       int(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)),
                                       int(get(handle))))
        except Exception:
            pass

    @staticmethod
    def mark():
        """A time stamp that delimits a window of samples (see :meth:`summary`)."""

        import datetime

        return datetime.datetime.now()

    def sample_under_load(self, run=None, calls: int = 64) -> None:
        """One direct NVML reading while ``calls`` more (untimed) calls are still running."""

        if run is not None:
            for _ in range(calls):
                run()
        self._nvml_once()
        torch.cuda.synchronize()

    def stop(self) -> None:
        if self._proc is not None:
            self._proc.terminate()  # the exact child started above
            try:
                self._proc.wait(timeout=5)
            except Exception:
                self._proc.kill()
            self._proc = None

    def summary(self, t0, t1) -> dict:
        """Median SM clock and the throttle reasons seen between the two marks."""

        import datetime

        samples, reasons, max_mhz = [], set(), None
        if self._log is not None:
            try:
                self._log.flush()
                self._log.seek(0)
                for line in self._log.read().splitlines():
                    parts = [x.strip() for x in line.split(",")]
                    if len(parts) != 4:
                        continue
                    try:
                        stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f")
                        mhz, mx, bits = int(parts[1]), int(parts[2]), int(parts[3], 16)
                    except ValueError:
                        continue
                    max_mhz = mx
                    if t0 <= stamp <= t1:
                        samples.append(mhz)
                        reasons.update(name for bit, name in self.REASONS.items() if bits & bit)
            except Exception:
                pass
        for stamp, mhz, mx, bits in self._edge_samples:
            if t0 <= stamp <= t1:
                samples.append(mhz)
                max_mhz = mx
                reasons.update(name for bit, name in self.REASONS.items() if bits & bit)
        return {
            "sm_mhz": statistics.median(samples) if samples else None,
            "sm_max_mhz": max_mhz,
            "reasons": sorted(reasons),
            "samples": len(samples),
            "sampler": f"nvidia-smi -lms {self.period_ms} (child process) + one NVML reading under load",
        }


def _randn_bf16(shape, seed, device):
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(shape, generator=g, device=device, dtype=torch.float32).bfloat16()


# --------------------------------------------------------------------------
# Workloads: each returns (run_fn, q_device, out_device, info)
# --------------------------------------------------------------------------

SCHEDULE = {"dynamic": None}  # set from --schedule: None follows STREAMATTN_B200_SCHEDULE (default static)


def traffic_per_launch(workload: str, world: int):
    """(DRAM read+write bytes of one launch of the dominant kernel, where that figure comes from)."""

    total, source = NCU_TRAFFIC.get(workload, (None, None))
    if total is None:
        return None, None
    source = f"stored ncu capture {source}"
    if workload == "cp_c5":
        return total / world, source + ", scaled by the tokens one rank reads"
    return total, source


def schedule_name(workload: str) -> str:
    from streamattn_b200 import native

    if workload not in ("exact_c2", "exact_c2_bnhd", "paged_c3"):
        return "static"
    dynamic = SCHEDULE["dynamic"] if SCHEDULE["dynamic"] is not None else native.dynamic_default()
    return "dynamic (tiles claimed from a device counter; not bit-reproducible)" if dynamic else "static"


def build_exact_c2(device, layout="BHND"):
    import streamattn_b200 as sa

    B, Hq, Hkv, D, N = 8, 16, 2, 64, 65536
    q = _randn_bf16((B, 1, Hq, D), 0, device)
    k = _randn_bf16((B, Hkv, N, D), 1, device)
    v = _randn_bf16((B, Hkv, N, D), 2, device)
    if layout == "BNHD":
        k, v = k.transpose(1, 2).contiguous(), v.transpose(1, 2).contiguous()
    plan = sa.ExactDecodePlan.build(q, k, v, kv_layout=layout, dynamic_schedule=SCHEDULE["dynamic"])
    info = dict(workload="exact_c2" if layout == "BHND" else "exact_c2_bnhd", batch=B, q_heads=Hq, kv_heads=Hkv,
                head_dim=D, kv_len=N, kv_layout=layout, kernel=plan.kernel_name, ctas=plan.num_ctas,
                bytes=2 * B * Hkv * N * D * 2, launches=plan.launches_per_run)
    return {"run": plan.run, "q": q, "out": plan.output, "info": info, "plan": plan}


def build_paged_c3(device):
    import streamattn_b200 as sa

    B, Hq, Hkv, D, page, cap = 8, 16, 2, 64, 16, 65536
    max_pages = cap // page
    pool = B * max_pages
    g = torch.Generator().manual_seed(17)
    q = _randn_bf16((B, 1, Hq, D), 3, device)
    k = _randn_bf16((pool, Hkv, page, D), 4, device)
    v = _randn_bf16((pool, Hkv, page, D), 5, device)
    table = torch.randperm(pool, generator=g).to(torch.int32).view(B, max_pages)
    lengths = torch.randint(16384, 65537, (B,), generator=g).to(torch.int32)
    for b in range(B):
        table[b, -(-int(lengths[b]) // page):] = -1
    cache = sa.PagedKVCache(key=k, value=v, page_table=table.to(device), sequence_lengths=lengths.to(device),
                            layout="HND")
    plan = sa.PagedExactDecodePlan.build(q, cache, dynamic_schedule=SCHEDULE["dynamic"])
    tokens = int(lengths.sum())
    pages = int(sum(-(-int(n) // page) for n in lengths))
    info = dict(workload="paged_c3", batch=B, q_heads=Hq, kv_heads=Hkv, head_dim=D, page_size=page, capacity=cap,
                total_tokens=tokens, kernel=plan.kernel_name, ctas=plan.num_ctas,
                bytes=2 * Hkv * D * 2 * tokens + 4 * pages, launches=plan.launches_per_run)
    return {"run": plan.run, "q": q, "out": plan.output, "info": info, "plan": plan}


def build_loop_c2(device):
    """One decode-loop step on the config-2 cache: RoPE + KV append (one launch, positions and
    lengths on the device) followed by the exact decode over the rows' current lengths."""

    import streamattn_b200 as sa

    B, Hq, Hkv, D, N = 8, 16, 2, 64, 65536
    start = N - 8192
    q_raw = _randn_bf16((B, 1, Hq, D), 0, device)
    k = _randn_bf16((B, Hkv, N, D), 1, device)
    v = _randn_bf16((B, Hkv, N, D), 2, device)
    k_new = _randn_bf16((B, Hkv, 1, D), 3, device)
    v_new = _randn_bf16((B, Hkv, 1, D), 4, device)
    g = torch.Generator(device=device).manual_seed(5)
    angles = torch.randn(B, 1, D // 2, generator=g, device=device)
    emb = torch.cat((angles, angles), dim=-1)
    cos, sin = emb.cos().bfloat16(), emb.sin().bfloat16()
    lens = torch.full((B,), start, dtype=torch.int32, device=device)
    q_rot = torch.empty_like(q_raw)
    plan = sa.ExactDecodePlan.build(q_rot, k, v, kv_layout="BHND", seq_lens=lens,
                                    dynamic_schedule=SCHEDULE["dynamic"])
    append = sa.AppendKVPlan.build(k, v, k_new, v_new, lens, kv_layout="BHND", cos=cos, sin=sin, query=q_raw,
                                   query_out=q_rot, query_layout="BNHD", lengths_out=lens)
    state = {"steps": 0}

    def run():
        if start + state["steps"] >= N:  # cache full: start the rows over (rare, outside the steady state)
            lens.fill_(start)
            state["steps"] = 0
        append.run()
        state["steps"] += 1
        return plan.run()

    mean_len = (start + N) // 2
    info = dict(workload="loop_c2", batch=B, q_heads=Hq, kv_heads=Hkv, head_dim=D, kv_capacity=N,
                kv_len="grows by one per step from %d (bytes counted at the mean length %d)" % (start, mean_len),
                kv_layout="BHND", kernel=plan.kernel_name + " after append_kv_kernel", ctas=plan.num_ctas,
                bytes=2 * B * Hkv * mean_len * D * 2, launches=plan.launches_per_run + 1)
    return {"run": run, "q": q_raw, "out": plan.output, "info": info, "plan": plan}


def build_seed_c4(device):
    import streamattn_b200 as sa
    from streamattn_b200 import native

    B, Hq, Hkv, D, N, bs = 8, 16, 2, 128, 32768, 16
    g = torch.Generator().manual_seed(0)
    q = _randn_bf16((B, 1, Hq, D), 6, device)
    k = _randn_bf16((B, N, Hkv, D), 7, device)
    v = _randn_bf16((B, N, Hkv, D), 8, device)
    middle = (torch.randperm(2032 - 4, generator=g)[:4] + 4).tolist()
    blocks = [0, 1, 2, 3, *middle, *range(2032, 2048)]
    out = torch.empty_like(q)

    def bind(q_buf, out_buf):
        return native.seed_plan(q_buf, k, v, out_buf, native.new_workspace(device, B, Hq, Hkv, D), block_size=bs,
                                blocks=blocks)

    plan = bind(q, out)
    info = dict(workload="seed_c4", batch=B, q_heads=Hq, kv_heads=Hkv, head_dim=D, kv_len=N, seed_tokens=384,
                kernel=plan.kernel_name, ctas=plan.num_ctas, bytes=2 * B * Hkv * 384 * D * 2,
                launches=plan.launches,
                l2="seed set (3 MB) stays L2-resident between back-to-back calls; cold_l2 gives the HBM case")
    return {"run": plan.run, "q": q, "out": out, "info": info, "plan": plan, "rebind": bind}


def build_o_proj_3b(device):
    """The output projection that follows attention in Qwen2.5-3B: [8, 1, 2048] x [2048, 2048]^T, bf16."""

    import streamattn_b200 as sa

    B, heads, dim, hidden = 8, 16, 128, 2048
    attn = _randn_bf16((B, 1, heads, dim), 80, device)
    weight = (_randn_bf16((hidden, heads * dim), 81, device).float() / 16.0).bfloat16()
    plan = sa.OProjPlan.build(attn.view(B, 1, heads * dim), weight)
    info = dict(workload="o_proj_3b", batch=B, in_features=heads * dim, out_features=hidden,
                kernel="sm100_o_proj_weight_stream", ctas=hidden // 8, bytes=hidden * heads * dim * 2 + 2 * B * hidden * 2,
                launches=1, l2="the 8 MB of weights stay L2-resident between back-to-back calls")
    return {"run": plan.run, "q": attn, "out": plan.output, "info": info, "plan": plan}


def build_cp_c5(device, rank, world, exchange="auto", kv_len=1048576):
    from streamattn_b200.context_parallel import ContextParallelExactDecode, shard_bounds

    Hq, Hkv, D, N = 32, 8, 128, int(kv_len)
    chunk = 65536
    lo, hi = shard_bounds(N, world, rank)
    q = _randn_bf16((1, 1, Hq, D), 100, device)
    k = torch.empty(1, Hkv, hi - lo, D, dtype=torch.bfloat16, device=device)
    v = torch.empty_like(k)
    # Values depend only on the global chunk index, not on how many GPUs share the sequence.
    for c0 in range(lo - lo % chunk, hi, chunk):
        kc = _randn_bf16((1, Hkv, chunk, D), 1000 + 2 * (c0 // chunk), device)
        vc = _randn_bf16((1, Hkv, chunk, D), 1001 + 2 * (c0 // chunk), device)
        a, b = max(lo, c0), min(hi, c0 + chunk)
        k[:, :, a - lo:b - lo] = kc[:, :, a - c0:b - c0]
        v[:, :, a - lo:b - lo] = vc[:, :, a - c0:b - c0]
        del kc, vc
    def bind(q_buf, out_buf):
        return ContextParallelExactDecode(q_buf, k, v, kv_layout="BHND", exchange=exchange, output=out_buf)

    cp = bind(q, None)
    info = dict(workload="cp_c5", batch=1, q_heads=Hq, kv_heads=Hkv, head_dim=D, kv_len=N, shard_tokens=hi - lo,
                kernel=cp.kernel_name, ctas=cp._plan.num_ctas, bytes=2 * Hkv * N * D * 2,
                exchange_bytes_per_rank=cp.exchange_bytes_per_rank, exchange=cp.exchange,
                launches=cp.launches_per_run, parallelism=f"cp{world}")
    return {"run": cp.run, "q": q, "out": cp.output, "info": info, "plan": cp, "rebind": bind}


def time_region(fn, steps, device):
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize(device)
    return start.elapsed_time(stop) * 1e-3


class Ranks:
    """Barrier and max-over-ranks for one process per GPU (no-ops in a single process)."""

    def __init__(self, device, world: int, distributed: bool) -> None:
        self.device, self.world, self.distributed = device, world, distributed

    def barrier(self) -> None:
        if self.distributed:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize(self.device)

    def max_over_ranks(self, values):
        if not self.distributed or self.world == 1:
            return list(values)
        import torch.distributed as dist

        t = torch.tensor(list(values), dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]


PROTOCOL_WARMUP = 20
PROTOCOL_ITERS = 200
PROTOCOL_REPEATS = 9


def protocol_time(fn, ranks: Ranks, *, warmup: int = PROTOCOL_WARMUP, min_iters: int = PROTOCOL_ITERS,
                  repeats: int = PROTOCOL_REPEATS, min_repeat_s: float = 0.0) -> dict:
    """Median / min / max microseconds per call over ``repeats`` regions of at least ``min_iters`` calls.

    Every region sits between its own pair of CUDA events after a barrier + synchronize, and its
    time is the maximum over the ranks.  ``min_repeat_s`` > 0 lengthens the regions of short
    kernels (more calls per region).
    """

    for _ in range(max(0, warmup - 10)):
        fn()
    ranks.barrier()
    probe = ranks.max_over_ranks([time_region(fn, 10, ranks.device) / 10])[0]  # the last 10 warm-up calls, timed
    iters = max(min_iters, int(min_repeat_s / max(probe, 1e-7)) + 1)
    times = []
    for _ in range(repeats):
        ranks.barrier()
        times.append(time_region(fn, iters, ranks.device) / iters * 1e6)
    ranks.barrier()
    times = ranks.max_over_ranks(times)
    return {"us_per_call": statistics.median(times), "min_us": min(times), "max_us": max(times),
            "repeats": repeats, "iters_per_repeat": iters, "warmup": max(warmup, 10)}


def flush_l2(device, scratch: dict) -> None:
    """Overwrite a buffer larger than the 126 MB L2 so that the next call starts from HBM."""

    if "buf" not in scratch:
        scratch["buf"] = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
    scratch["buf"].add_(1)


def cold_time(fn, device, calls: int = 40) -> dict:
    """Microseconds per call with L2 flushed (outside the timed events) before every call."""

    scratch, times = {}, []
    for i in range(calls + 3):
        flush_l2(device, scratch)
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize(device)
        if i >= 3:
            times.append(start.elapsed_time(stop) * 1e3)
    return {"us_per_call": statistics.median(times), "min_us": min(times), "max_us": max(times), "calls": calls,
            "note": "single calls, 256 MB written between calls so K/V come from HBM; event pair per call"}


def make_e2e(workload: str, case, device):
    """The end-to-end step of a workload: host query in, result in host memory, waited for.

    Returns (step, mode text, pinned host query, pinned host output).  Plans that can bind pinned
    host buffers do so (the kernel reads q and writes the result across PCIe itself: one launch
    and one wait per step); the others enqueue two async copies around ``run()``.
    """

    import streamattn_b200 as sa

    run, q_dev, out_dev, plan = case["run"], case["q"], case["out"], case["plan"]
    stream = torch.cuda.current_stream(device)  # looked up once: the step itself stays minimal
    q_host = q_dev.cpu().pin_memory()
    out_host = torch.empty(out_dev.shape, dtype=out_dev.dtype).pin_memory()
    bound = "plan bound to pinned host query/output: the kernel reads q and writes out over PCIe"
    host_run = None
    if workload in ("exact_c2", "exact_c2_bnhd", "cp_c5_1gpu"):
        host_run = sa.ExactDecodePlan.build(q_host, plan.key_cache, plan.value_cache, output=out_host,
                                            kv_layout=plan.kv_layout, dynamic_schedule=SCHEDULE["dynamic"]).run
    elif workload == "paged_c3":
        host_run = sa.PagedExactDecodePlan.build(q_host, plan.cache, output=out_host, validate_metadata=False,
                                                 dynamic_schedule=SCHEDULE["dynamic"]).run
    elif workload == "seed_c4":
        host_run = case["rebind"](q_host, out_host).run
    elif workload == "cp_c5":
        host_run = case["rebind"](q_host, out_host).run
    if host_run is not None:
        def step():
            host_run()
            stream.synchronize()

        return step, bound, q_host, out_host

    def step():  # noqa: F811
        q_dev.copy_(q_host, non_blocking=True)
        run()
        out_host.copy_(out_dev, non_blocking=True)
        stream.synchronize()

    return step, "pinned-host query copied in, output copied out (two async copies around run())", q_host, out_host


def measure_without_launch_overlap() -> dict:
    """Config 2 once more in a child process with programmatic dependent launch switched off.

    Back-to-back calls normally overlap the head of a launch (set-up, the partition of the tile
    list) with the tail of the launch before it; the switch is read once per process, hence the
    child.  The difference to the headline figure is what that overlap is worth.
    """

    env = dict(os.environ, STREAMATTN_B200_NO_PDL="1")
    cmd = [sys.executable, os.path.abspath(__file__), "--workload", "exact_c2", "--profile", "--steps", "1000",
           "--warmup", "50"]
    entry = {"workload": "exact_c2_plain_launch",
             "note": "config 2 with STREAMATTN_B200_NO_PDL=1 (plain stream serialization): nothing of a launch "
                     "overlaps the launch before it; one region of 1000 back-to-back calls in a child process"}
    try:
        out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
        lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
        entry["us_per_call"] = json.loads(lines[-1])["us_per_call"]
    except Exception as exc:  # the figure is informative: the line must not depend on it
        entry["error"] = f"{type(exc).__name__}: {exc}"[:200]
    return entry


def graph_replay_time(run, device, calls: int = 20, replays: int = 10, repeats: int = 9) -> dict:
    """Microseconds per call when ``calls`` consecutive calls are captured into one CUDA graph and
    the graph is replayed (the reference also times its decode plans under graph replay).

    Median over ``repeats`` regions of ``replays`` replays each, every region between its own pair
    of CUDA events.  The loop workload is left out by its caller: its cache grows with every call.
    """

    side = torch.cuda.Stream(device=device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        for _ in range(3):
            run()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(calls):
                run()
    torch.cuda.synchronize(device)
    for _ in range(3):
        graph.replay()
    times = []
    for _ in range(repeats):
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(replays):
            graph.replay()
        stop.record()
        torch.cuda.synchronize(device)
        times.append(start.elapsed_time(stop) * 1e3 / (replays * calls))
    return {"us_per_call": statistics.median(times), "min_us": min(times), "max_us": max(times),
            "calls_per_graph": calls, "replays_per_repeat": replays, "repeats": repeats}


def measure_case(workload: str, case, ranks: Ranks, clocks: ClockSampler, *, steps: int, warmup: int,
                 headline: bool) -> dict:
    """All figures of one workload: --steps region (headline only), protocol timing, e2e, roofline, clocks."""

    device, world = ranks.device, ranks.world
    run, info = case["run"], dict(case["info"])
    alg_bytes = info.pop("bytes")
    launches = info.pop("launches")
    per_gpu_bytes = alg_bytes / world if workload == "cp_c5" else alg_bytes
    peak, peak_kind = measured_hbm_peak()
    result = {"workload": workload}

    t_begin = clocks.mark()
    if headline:
        for _ in range(warmup):
            run()
        ranks.barrier()
        elapsed = time_region(run, steps, device)
        ranks.barrier()
        result["step_s"] = ranks.max_over_ranks([elapsed])[0] / steps
    proto = protocol_time(run, ranks)
    # Keep the same call running (untimed) for a moment so that the clock sampler, which reads
    # every 25 ms, sees the GPU under this very load; every rank runs the same number of calls.
    extra = int(min(0.15 / max(proto["us_per_call"] * 1e-6, 1e-7), 20000))
    clocks.sample_under_load(run, calls=extra)
    t_end = clocks.mark()
    result["protocol"] = proto

    e2e_step, e2e_mode, q_host, out_host = make_e2e(workload, case, device)
    e2e = protocol_time(e2e_step, ranks, warmup=10, min_iters=50, min_repeat_s=0.0)
    if workload != "loop_c2":  # the loop's cache grows between the two runs
        run()
        torch.cuda.synchronize(device)
        torch.testing.assert_close(out_host.float(), case["out"].float().cpu(), atol=2e-2, rtol=0)
    # The same call captured into a CUDA graph (not the loop, whose cache grows with every call,
    # nor the fused context-parallel plan, whose step number is a launch argument).
    graph = None
    if workload not in ("loop_c2", "cp_c5"):
        try:
            graph = graph_replay_time(run, device)
        except Exception as exc:  # informative figure: the line must not depend on it
            graph = {"error": f"{type(exc).__name__}: {exc}"[:200]}
            torch.cuda.synchronize(device)
    us = proto["us_per_call"]
    achieved = per_gpu_bytes / (us * 1e-6) / 1e9
    traffic, traffic_source = traffic_per_launch(workload, world)
    result.update({
        "us_per_call": us, "min_us": proto["min_us"], "max_us": proto["max_us"],
        "gb_per_s": alg_bytes / (us * 1e-6) / 1e9,
        "config": {**info, "schedule": schedule_name(workload),
                   "l2_hygiene": info.get("l2", "inputs larger than the 126 MB L2")},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "traffic_source": traffic_source,
                     "peak_source": f"{peak_kind} copy bandwidth", "frac_of_nominal_8tbs": achieved / 8000.0,
                     "kernel": info["kernel"], "algorithmic_bytes_per_launch": per_gpu_bytes,
                     "timed": "median of the protocol repeats"},
        "e2e": {"value": alg_bytes / (e2e["us_per_call"] * 1e-6) / 1e9, "unit": UNIT,
                "us_per_call": e2e["us_per_call"], "min_us": e2e["min_us"], "max_us": e2e["max_us"],
                "h2d_bytes_per_step": q_host.numel() * q_host.element_size(),
                "d2h_bytes_per_step": out_host.numel() * out_host.element_size(),
                "note": e2e_mode + "; the KV cache is resident device state bound to the plan"},
        "launches_per_call": launches,
        "graph_replay": graph,
        "clock_window": (t_begin, t_end),
        "device_status": case["plan"].device_status() if hasattr(case["plan"], "device_status") else 0,
    })
    if workload == "seed_c4":
        result["cold_l2"] = cold_time(run, device)
    return result


def cpu_baseline_sample(workload: str, steps: int = 3, warmup: int = 1, budget_s: float = 30.0) -> dict:
    """Reference CPU path (oracle port) on a bounded sample of the workload."""

    from oracle import torch_port

    cores = torch.get_num_threads()
    g = torch.Generator().manual_seed(0)
    if workload in ("exact_c2", "exact_c2_bnhd", "loop_c2", "cp_c5"):
        if workload == "cp_c5":
            B, Hq, Hkv, D, N, note = 1, 32, 8, 128, 65536, "65536 of 1048576 tokens of the row, fp32 on CPU"
        else:
            B, Hq, Hkv, D, N, note = 2, 16, 2, 64, 65536, "2 of 8 rows at full kv_len 65536, fp32 on CPU"
        q = torch.randn(B, 1, Hq, D, generator=g)
        k = torch.randn(B, N, Hkv, D, generator=g)
        v = torch.randn(B, N, Hkv, D, generator=g)
        fn = lambda: torch_port.dense_decode(q, k, v)
        alg = 2 * B * Hkv * N * D * 2
    elif workload == "paged_c3":
        B, Hq, Hkv, D, page, n = 1, 16, 2, 64, 16, 4096
        q = torch.randn(B, 1, Hq, D, generator=g)
        k = torch.randn(n // page, Hkv, page, D, generator=g)
        v = torch.randn(n // page, Hkv, page, D, generator=g)
        table = torch.randperm(n // page, generator=g).to(torch.int32).view(1, -1)
        lens = torch.tensor([n], dtype=torch.int32)
        fn = lambda: torch_port.paged_decode(q, k, v, table, lens, layout="HND")
        alg = 2 * Hkv * D * 2 * n
        note = "1 row of 4096 tokens (page-streaming python loop of the reference), fp32 on CPU"
        steps, warmup = 1, 0
    else:
        B, Hq, Hkv, D, N = 8, 16, 2, 128, 32768
        q = torch.randn(B, 1, Hq, D, generator=g)
        k = torch.randn(B, N, Hkv, D, generator=g)
        v = torch.randn(B, N, Hkv, D, generator=g)
        tokens = torch.cat([torch.arange(64), torch.arange(32448, 32768)])
        fn = lambda: torch_port.seed_decode(q, k, v, tokens)
        alg = 2 * B * Hkv * 384 * D * 2
        note = "full config-4 shape, 384 seed tokens, fp32 on CPU"
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    done = 0
    while done < steps:  # every requested step, unless the CPU time budget runs out first
        fn()
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = (time.perf_counter() - t0) / done
    return {"value": alg / dt / 1e9, "unit": UNIT, "cores": cores, "kind": "port", "sample": note,
            "ms_per_sample": dt * 1e3, "samples_timed": done}


def quick_time(fn, device, iters: int = 200, repeats: int = 5, warmup: int = 20) -> float:
    """Median microseconds per call over ``repeats`` event-timed regions of ``iters`` calls."""

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(device)
    return statistics.median(time_region(fn, iters, device) / iters * 1e6 for _ in range(repeats))


def measure_seed_grid(device) -> dict:
    """Seed-only decode at batch 1-8 x 128-1024 seed tokens (Qwen2.5-3B attention shape): the grid
    the latency model picks (``seed_autotune``) against a sweep of CTAs per (row, KV head) pair."""

    from streamattn_b200 import native
    from streamattn_b200.seed_autotune import SeedKernelShape, autotune_seed_kernel_mode

    Hq, Hkv, D, N, bs = 16, 2, 128, 32768, 32
    cells, worst = [], 0.0
    for B in (1, 2, 4, 8):
        q = _randn_bf16((B, 1, Hq, D), 40 + B, device)
        k = _randn_bf16((B, N, Hkv, D), 50 + B, device)
        v = _randn_bf16((B, N, Hkv, D), 60 + B, device)
        out = torch.empty_like(q)
        pairs = B * Hkv
        for S in (128, 384, 1024):
            nb = S // bs
            blocks = list(range(nb // 2)) + list(range(N // bs - (nb - nb // 2), N // bs))
            shape = SeedKernelShape(batch=B, q_heads=Hq, kv_heads=Hkv, kv_len=N, dim=D, block_size=bs,
                                    sink_blocks=nb, recent_blocks=0, middle_seed_blocks=0)
            pick = autotune_seed_kernel_mode(shape, sm_count=native.sm_count(device))
            swept = {}
            for chunks in sorted({1, 2, 3, 4, 6, 8, 12, pick.recommended_num_ctas // pairs}):
                ctas = chunks * pairs
                if chunks > shape.tiles_per_pair or ctas > 148:
                    continue
                ws = native.new_workspace(device, B, Hq, Hkv, D, ctas)
                plan = native.seed_plan(q, k, v, out, ws, block_size=bs, blocks=blocks, num_ctas=ctas)
                swept[ctas] = quick_time(plan.run, device)
            best_ctas = min(swept, key=swept.get)
            chosen_us = swept[pick.recommended_num_ctas]
            loss = chosen_us / swept[best_ctas] - 1.0
            worst = max(worst, loss)
            cells.append({"batch": B, "seed_tokens": S, "chosen_ctas": pick.recommended_num_ctas,
                          "chosen_us": chosen_us, "predicted_us": pick.predicted_us, "best_ctas": best_ctas,
                          "best_us": swept[best_ctas], "chosen_over_best": 1.0 + loss,
                          "swept_us_by_ctas": {str(c): t for c, t in swept.items()}})
        del q, k, v
    return {"workload": "seed_grid", "shape": "Hq16 Hkv2 D128 N32768 bf16, block 32, sink+recent blocks",
            "l2": "seed sets stay L2-resident between back-to-back calls", "timing": "median of 5 x 200 calls",
            "worst_chosen_over_best": 1.0 + worst, "cells": cells}


def measure_o_proj(device) -> dict:
    """The output projection that follows attention (Qwen2.5-3B: 2048 -> 2048, bf16, 8 MB of weights):
    alone, with L2 flushed, and chained behind the seed-only decode of the config-4 shape."""

    import streamattn_b200 as sa

    case = build_seed_c4(device)
    B, hidden = 8, 2048
    weight = (_randn_bf16((hidden, hidden), 70, device).float() / 16.0).bfloat16()
    proj = sa.OProjPlan.build(case["out"].view(B, 1, hidden), weight)
    late = sa.OProjPlan.build(case["out"].view(B, 1, hidden), weight, prefetch_weights=False)
    decode = case["run"]

    def chain():
        decode()
        return proj.run()

    def chain_late():
        decode()
        return late.run()

    alg = hidden * hidden * 2 + 2 * B * hidden * 2
    peak, peak_kind = measured_hbm_peak()
    alone = quick_time(proj.run, device)
    cold = cold_time(proj.run, device)
    decode_us = quick_time(decode, device)
    chain_us = quick_time(chain, device)
    chain_late_us = quick_time(chain_late, device)
    cold_gbs = alg / (cold["us_per_call"] * 1e-6) / 1e9
    # The same projection behind the decode-loop step of config 2 (append + decode; 16 heads x 64
    # = 1024 input features, 2048 outputs): three launches per step on one stream.
    del case
    torch.cuda.empty_cache()
    loop = build_loop_c2(device)
    weight_c2 = (_randn_bf16((hidden, 1024), 71, device).float() / 16.0).bfloat16()
    proj_c2 = sa.OProjPlan.build(loop["out"].view(B, 1, 1024), weight_c2)
    loop_step = loop["run"]

    def loop_chain():
        loop_step()
        return proj_c2.run()

    loop_us = quick_time(loop_step, device)
    loop_chain_us = quick_time(loop_chain, device)
    del loop
    torch.cuda.empty_cache()
    return {"workload": "o_proj_qwen3b", "batch": B, "in_features": hidden, "out_features": hidden,
            "loop_c2_us": loop_us, "loop_c2_then_o_proj_us": loop_chain_us,
            "loop_c2_o_proj_visible_us": loop_chain_us - loop_us,
            "algorithmic_bytes": alg, "us_per_call_l2_warm": alone, "cold_l2": cold,
            "roofline_cold": {"bound": "hbm", "achieved": cold_gbs, "peak": peak, "unit": "GB/s",
                              "frac": cold_gbs / peak, "peak_source": f"{peak_kind} copy bandwidth",
                              "note": "8 MB per launch: launch latency, not bandwidth, dominates"},
            "seed_decode_us": decode_us, "seed_decode_then_o_proj_us": chain_us,
            "o_proj_visible_us": chain_us - decode_us,
            "seed_decode_then_o_proj_no_weight_prefetch_us": chain_late_us,
            "timing": "median of 5 x 200 calls; chain = two launches per step on one stream"}


BUILDERS = {
    "exact_c2": lambda device: build_exact_c2(device),
    "exact_c2_bnhd": lambda device: build_exact_c2(device, "BNHD"),
    "paged_c3": build_paged_c3,
    "seed_c4": build_seed_c4,
    "loop_c2": build_loop_c2,
    "cp_c5_1gpu": lambda device: build_cp_c5_single(device),
    "o_proj_3b": build_o_proj_3b,
}
SECONDARY = ("paged_c3", "seed_c4", "exact_c2_bnhd", "loop_c2", "cp_c5_1gpu")


def cp_oracle_check(device, out_dev, kv_head: int = 0) -> float:
    """Max |difference| between the context-parallel result and the CPU oracle on one KV group.

    The oracle (C, double accumulation) is run on the same seeded values for the query heads of
    ``kv_head`` over the whole 1M-token row; it is the checker here, outside every timed region.
    """

    from oracle import cpu_oracle

    Hq, Hkv, D, N, chunk = 32, 8, 128, 1048576, 65536
    group = Hq // Hkv
    q = _randn_bf16((1, 1, Hq, D), 100, device)[:, :, kv_head * group:(kv_head + 1) * group].float().cpu()
    k = torch.empty(1, 1, N, D, dtype=torch.float32)
    v = torch.empty_like(k)
    for c0 in range(0, N, chunk):
        k[:, :, c0:c0 + chunk] = _randn_bf16((1, Hkv, chunk, D), 1000 + 2 * (c0 // chunk), device)[:, kv_head:kv_head + 1].float().cpu()
        v[:, :, c0:c0 + chunk] = _randn_bf16((1, Hkv, chunk, D), 1001 + 2 * (c0 // chunk), device)[:, kv_head:kv_head + 1].float().cpu()
    want = cpu_oracle.exact_decode(q, k, v, kv_layout="BHND")
    got = out_dev[:, :, kv_head * group:(kv_head + 1) * group].float().cpu()
    return float((got - want).abs().max())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto",
                    choices=["auto", "exact_c2", "exact_c2_bnhd", "paged_c3", "seed_c4", "loop_c2", "cp_c5",
                             "cp_c5_1gpu", "o_proj_3b"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true",
                    help="N=1: only the headline workload (the other configurations are skipped)")
    ap.add_argument("--no-oracle-check", action="store_true",
                    help="cp_c5: skip the CPU-oracle comparison of one KV group (about 10 s on rank 0)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "fused", "peer", "nccl"],
                    help="cp_c5 only: how the per-rank states meet (fused peer-store kernel or NCCL all-gather)")
    ap.add_argument("--schedule", default="default", choices=["default", "static", "dynamic"],
                    help="tile schedule of the exact/paged plans: static is bit-reproducible (the default), "
                         "dynamic claims tiles from a device counter")
    ap.add_argument("--cp-kv-len", type=int, default=1048576,
                    help="cp_c5 only: total tokens of the row (131072 on one GPU = the shard one of 8 GPUs holds; "
                         "used for small profiler captures)")
    ap.add_argument("--profile", action="store_true",
                    help="only warm-up + the timed region (for runs under ncu): no e2e, CPU or clock legs")
    args = ap.parse_args()
    SCHEDULE["dynamic"] = {"default": None, "static": False, "dynamic": True}[args.schedule]

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    workload = args.workload
    if workload == "auto":
        workload = "exact_c2" if max(world, args.gpus) == 1 else "cp_c5"
    warmup = max(3, args.warmup)

    if args.impl == "reference":
        if rank != 0:
            return
        # Every requested step is one bounded sample; a run that would exceed about two minutes of
        # CPU time stops early and says how many steps it timed.
        base = cpu_baseline_sample(workload, steps=max(1, args.steps), warmup=min(warmup, 3), budget_s=120.0)
        line = {
            "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": base["samples_timed"], "steps_requested": args.steps, "warmup": min(warmup, 3),
            "ms_per_step": base["ms_per_sample"],
            "higher_is_better": True, "scaling": "strong" if workload.startswith("cp_c5") else "weak",
            "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": workload, "sample": base["sample"]},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
        emit(line)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback)")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    clocks = ClockSampler(local_rank).start()  # child process: it comes up while the inputs are built
    distributed = world > 1
    if distributed or workload == "cp_c5":
        import torch.distributed as dist

        if not distributed:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29555")
            dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
        else:
            dist.init_process_group("nccl", device_id=device)
        distributed = True
    ranks = Ranks(device, world, distributed)

    def build(name):
        if name == "cp_c5":
            return build_cp_c5(device, rank, world, args.exchange, args.cp_kv_len)
        return BUILDERS[name](device)

    case = build(workload)

    if args.profile:
        for _ in range(warmup):
            case["run"]()
        ranks.barrier()
        step_s = ranks.max_over_ranks([time_region(case["run"], args.steps, device)])[0] / args.steps
        if rank == 0:
            emit({"profile_run": True, "workload": workload, "us_per_call": step_s * 1e6})
        clocks.stop()
        if distributed:
            dist.destroy_process_group()
        return

    head = measure_case(workload, case, ranks, clocks, steps=args.steps, warmup=warmup, headline=True)
    step_s = head.pop("step_s")
    alg_bytes = case["info"]["bytes"]
    launches = case["info"]["launches"]

    extra = {}
    if workload == "cp_c5":
        plan = case["plan"]
        # The shard kernel alone (no exchange): what the exchange + rank skew add is the difference.
        extra["cp_local_kernel_us"] = protocol_time(plan.run_local, ranks, repeats=5, min_repeat_s=0.0)["us_per_call"]
        if world > 1:
            # Every rank holds the merged result: the copies must be bit-identical.
            case["run"]()
            torch.cuda.synchronize(device)
            mine = case["out"].contiguous().view(torch.int16).to(torch.int32)
            low, high = mine.clone(), mine.clone()
            dist.all_reduce(low, op=dist.ReduceOp.MIN)
            dist.all_reduce(high, op=dist.ReduceOp.MAX)
            extra["cp_ranks_identical"] = bool(torch.equal(low, high))
            if rank == 0:
                # One-GPU time of the same 1M-token row, measured in this run on rank 0: the base of
                # the strong-scaling series.
                full = build_cp_c5_single(device)
                single = protocol_time(full["run"], Ranks(device, 1, False), repeats=5, min_iters=20,
                                       min_repeat_s=0.0)
                extra["cp_single_gpu_us"] = single["us_per_call"]
                cp_max_abs = float((full["run"]().float() - case["out"].float()).abs().max())
                assert cp_max_abs <= 2e-2, f"context-parallel result differs from the one-GPU result by {cp_max_abs}"
                extra["cp_max_abs_vs_1gpu"] = cp_max_abs
                extra["cp_speedup_vs_1gpu"] = single["us_per_call"] / head["us_per_call"]
                extra["strong_scaling_efficiency"] = single["us_per_call"] / (world * head["us_per_call"])
                extra["strong_scaling_note"] = ("cp_single_gpu_us / (n_gpus * us_per_call): the same 1M-token row on "
                                                "one GPU, timed on rank 0 in this run, against the protocol median "
                                                "of the sharded step")
                del full
                torch.cuda.empty_cache()
        if rank == 0 and not args.no_oracle_check and args.cp_kv_len == 1048576:
            diff = cp_oracle_check(device, case["out"])
            assert diff <= 2e-2, f"context-parallel result differs from the CPU oracle by {diff}"
            extra["cp_max_abs_vs_oracle"] = diff
            extra["cp_oracle_heads"] = "query heads 0-3 (KV head 0), all 1,048,576 tokens, C oracle in double"
        ranks.barrier()

    secondary = []
    if world == 1 and workload == "exact_c2" and not args.no_secondary:
        del case
        torch.cuda.empty_cache()
        for name in SECONDARY:
            other = build(name)
            entry = measure_case(name, other, ranks, clocks, steps=args.steps, warmup=warmup, headline=False)
            secondary.append(entry)
            del other
            torch.cuda.empty_cache()
    extras = []
    if world == 1 and workload == "exact_c2" and not args.no_secondary:
        extras = [measure_seed_grid(device), measure_o_proj(device)]
        torch.cuda.empty_cache()
        extras.append(measure_without_launch_overlap())
    clocks.stop()
    for entry in [head, *secondary]:
        entry["clocks"] = clocks.summary(*entry.pop("clock_window"))
    secondary.extend(extras)

    if rank == 0:
        # Whole-job figure: the sharded row is one job for all ranks; every other workload is
        # batch-parallel - each rank serves its own rows, no collective - so the ranks' bytes add up.
        job_bytes = alg_bytes if workload.startswith("cp_c5") else alg_bytes * world
        value = job_bytes / step_s / 1e9
        roofline = dict(head["roofline"])
        # The line's roofline follows the --steps region, like ``value``; the protocol median is beside it.
        per_gpu_bytes = roofline["algorithmic_bytes_per_launch"]
        roofline["achieved"] = per_gpu_bytes / step_s / 1e9
        roofline["frac"] = roofline["achieved"] / roofline["peak"]
        roofline["frac_of_nominal_8tbs"] = roofline["achieved"] / 8000.0
        roofline["timed"] = "the --steps region; protocol.roofline_frac is the median-of-repeats figure"
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": step_s * 1e3, "us_per_call": step_s * 1e6,
            "higher_is_better": True, "scaling": "strong" if workload.startswith("cp_c5") else "weak",
            "vs_baseline": alg_bytes / step_s / 1e9 / PUBLISHED_GBS[workload] if workload in PUBLISHED_GBS else None,
            "dtype": "bf16", "data": "synthetic",
            "config": {**head["config"],
                       **({"vs_baseline_is": "the reference's published 96.3 us on one H100 for this shape"}
                          if workload in PUBLISHED_GBS else {}),
                       "timing": "CUDA events around K back-to-back calls, max over ranks"},
            "roofline": roofline,
            "protocol": {**head["protocol"], "gb_per_s": head["gb_per_s"],
                         "roofline_frac": head["roofline"]["frac"],
                         "how": "median of 9 repeats, each >= 200 calls between one pair of CUDA events, after "
                                ">= 20 warm-up calls; max over ranks per repeat"},
            "e2e": head["e2e"],
            "graph_replay": head.get("graph_replay"),
            "gpu_launches": args.steps * launches,
            "clocks": head["clocks"],
            "device_status": head["device_status"],
            **extra,
        }
        if secondary:
            line["secondary"] = secondary
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline_sample("cp_c5" if workload == "cp_c5_1gpu" else workload)
        emit(line)
    if distributed:
        dist.destroy_process_group()


def build_cp_c5_single(device):
    """The whole 1M-token config-5 row on one GPU (one launch, no exchange): the strong-scaling base."""

    import streamattn_b200 as sa

    Hq, Hkv, D, N = 32, 8, 128, 1048576
    q = _randn_bf16((1, 1, Hq, D), 100, device)
    k = torch.empty(1, Hkv, N, D, dtype=torch.bfloat16, device=device)
    v = torch.empty_like(k)
    chunk = 65536
    for c0 in range(0, N, chunk):
        k[:, :, c0:c0 + chunk] = _randn_bf16((1, Hkv, chunk, D), 1000 + 2 * (c0 // chunk), device)
        v[:, :, c0:c0 + chunk] = _randn_bf16((1, Hkv, chunk, D), 1001 + 2 * (c0 // chunk), device)
    plan = sa.ExactDecodePlan.build(q, k, v, kv_layout="BHND")
    info = dict(workload="cp_c5_1gpu", batch=1, q_heads=Hq, kv_heads=Hkv, head_dim=D, kv_len=N, kv_layout="BHND",
                kernel=plan.kernel_name, ctas=plan.num_ctas, bytes=2 * Hkv * N * D * 2,
                launches=plan.launches_per_run)
    return {"run": plan.run, "q": q, "out": plan.output, "info": info, "plan": plan}


if __name__ == "__main__":
    main()
