"""Benchmark of the paged-KV attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  Headline: paged bf16 GQA decode at serving scale (batch
128, 64 query heads, 8 KV heads, head_dim 128, 64-token pages, cached lengths
uniform in [1024, 32768], fused one-token append, causal), reported as KV bytes
read per second (the reference benchmark's kv_bytes_read accounting).  A step
is one decode call over the whole batch.

Timing protocol (after benchmarks/common/timing.py:33-74 of the reference
project): W warm-up steps, then `rounds` rounds; a round is the K steps repeated
back to back until it lasts at least --min-round-s, bracketed by a barrier and
a device synchronise on both sides and timed with CUDA events on the launch
stream; the time of a round is the maximum over ranks; ms_per_step is the
median over rounds, with the spread beside it.

* value: device-resident inputs.
* e2e: the same step through flywheel_tpu.flash_attn_with_kvcache with the
  per-step inputs (q, new k/v, lengths, block table) in pinned host memory and
  the output read back to the host inside the timed region; the KV cache stays
  resident on the device, as it does in serving.
* roofline: algorithmic KV bytes per launch / this rank's measured time per
  launch, against the measured HBM copy bandwidth in MEASURED_PEAKS.json.
* prefill, c1, c3, long_context, strong, mixed: the other benchmark
  configurations (chunked prefill; contiguous decode; fp8 verify-window decode;
  one 128K-token request split over the GPUs with its (o, lse) exchange; one
  decode batch split over the GPUs by request and by KV head; a step mixing
  decode rows and prefill chunks), each with its own figures.
* cpu_baseline: the C + OpenMP restatement of the reference's test oracle
  (oracle/paged_decode_ref.c) on the same batch, on all host cores.
* --impl reference: that CPU restatement as its own arm (the reference itself
  needs JAX, which this image lacks); a step is the first 32 requests.

With N > 1 (torchrun) every rank runs the same batch shape with the same
lengths (requests shard with no communication); value is the bytes of all ranks
divided by the slowest rank's time.

Other workloads, one JSON line each (device-resident inputs):
    --config c1 | c3                     contiguous bf16 decode; paged fp8 verify window
    --config serve-d256-gqa | serve-d256-mha | gate-decode | gate-verify
                                         the reference's serving / perf-gate decode shapes
    --config dense-causal-8k | dense-causal-32k      flash_attn_func, causal
    --config serve-d256-prefill-gqa | -mha           16K sequence in 1K chunks, head_dim 256
    --prefill-only [--prefill-pool e4m3] [--prefill-head-dim 256] [--sustained-s S]
                                         the chunked-prefill workload alone
    --long-context [--exchange p2p|nccl] one 128K-token request split over the GPUs
"""

from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import pathlib
import sys
import threading
import time

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "flywheel-tpu_b200"))
sys.path.insert(0, str(ROOT))

import bench_workloads as workloads  # noqa: E402

BATCH, HQ, HK, D, PAGE = 128, 64, 8, 128, 64
LEN_LO, LEN_HI = 1024, 32768
FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS = 6650.0, 1590.0


def measured_peaks():
    """(HBM GB/s, bf16 burst TFLOP/s, bf16 sustained TFLOP/s, "measured" | "fallback")."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        burst = float(data.get("bf16_tflops", 0))
        return float(data["hbm_gbs"]), burst, float(data.get("bf16_tflops_sustained", burst)), "measured"
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, 1400.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the
    timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self.stop_flag = threading.Event()

    def run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
            names = {
                getattr(pynvml, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
                getattr(pynvml, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
                getattr(pynvml, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                getattr(pynvml, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
            }
            while not self.stop_flag.is_set():
                self.samples.append(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                mask = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
                time.sleep(0.004)
        except Exception as exc:  # pylint: disable=broad-except
            self.reasons.add(f"nvml_unavailable:{type(exc).__name__}")

    def summary(self):
        self.stop_flag.set()
        self.join(timeout=2)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def physical_gpu_index(local_index):
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible:
        try:
            return int(visible.split(",")[local_index])
        except (ValueError, IndexError):
            return local_index
    return local_index


class Ranks:
    """The process group as the benchmark sees it: barrier, max / sum over ranks."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise RuntimeError("bench.py needs a CUDA device; there is no CPU path.")
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        self.torch, self.dist = torch, dist
        if self.world > 1:
            # the long-context exchange below uses plain peer stores; NVLS is left out of NCCL too
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            dist.init_process_group("nccl", device_id=self.device)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def _reduce(self, values, op):
        if self.world == 1:
            return [float(v) for v in values]
        t = self.torch.tensor([float(v) for v in values], dtype=self.torch.float64, device=self.device)
        self.dist.all_reduce(t, op=op)
        return t.tolist()

    def max(self, values):
        return self._reduce(values, self.dist.ReduceOp.MAX)

    def sum(self, values):
        return self._reduce(values, self.dist.ReduceOp.SUM)

    def close(self):
        if self.dist.is_initialized():
            self.dist.destroy_process_group()


def timed_rounds(enqueue_pass, steps, ranks, *, rounds, min_round_s, before_round=None):
    """Times `enqueue_pass` (which enqueues `steps` steps on the current stream).

    One calibration pass sizes a round: the pass is repeated `reps` times back to
    back so that a round lasts at least min_round_s (the same reps on every rank:
    it comes from the slowest rank's calibration).  Each round sits between a
    barrier + device synchronise on both sides and is timed with CUDA events on
    the launch stream; its time is the maximum over ranks.  Returns the median
    over rounds of ms per step, the spread, and this rank's own median."""
    torch = ranks.torch
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def one(reps):
        if before_round is not None:
            before_round()
        ranks.barrier()
        start.record()
        for _ in range(reps):
            enqueue_pass()
        end.record()
        ranks.barrier()
        return start.elapsed_time(end)

    calibration = ranks.max([one(1)])[0]
    reps = max(1, math.ceil(min_round_s * 1e3 / max(calibration, 1e-3)))
    own = [one(reps) / (reps * steps) for _ in range(rounds)]
    # the all-reduce runs after the timed rounds: no collective sits between two of them
    job = ranks.max(own)
    return {"ms_per_step": float(np.median(job)), "ms_min": float(min(job)), "ms_max": float(max(job)),
            "own_ms_per_step": float(np.median(own)), "rounds": rounds, "steps_per_round": reps * steps,
            "round_s": float(np.median(job)) * reps * steps / 1e3}


def round_summary(t):
    return {"count": t["rounds"], "steps_per_round": t["steps_per_round"], "round_s": round(t["round_s"], 4),
            "ms_per_step_median": t["ms_per_step"], "ms_per_step_min": t["ms_min"], "ms_per_step_max": t["ms_max"],
            "spread": (t["ms_max"] - t["ms_min"]) / t["ms_per_step"] if t["ms_per_step"] else None}


# ---------------------------------------------------------------- headline: paged bf16 decode
def decode_lengths():
    """The batch's cached lengths and block table: the same on every rank, so the
    ranks stream the same number of bytes and the N-GPU figure measures the code,
    not the draw."""
    rng = np.random.default_rng(0)
    lens = rng.integers(LEN_LO, LEN_HI + 1, BATCH).astype(np.int32)
    table, pool_pages = workloads.paged_table(rng, lens, 1, PAGE, slack=0.10)
    return lens, table, pool_pages


def fill_normal(pool, gen, rows_per_chunk=4096):
    import torch
    for lo in range(0, pool.shape[0], rows_per_chunk):
        hi = min(pool.shape[0], lo + rows_per_chunk)
        block = torch.randn((hi - lo, *pool.shape[1:]), generator=gen, device=pool.device, dtype=torch.float32)
        pool[lo:hi] = block.to(pool.dtype)


def build_workload(value_seed, device, *, requests=None, kv_heads=slice(0, HK)):
    """The serving-scale decode workload on `device`: device tensors plus pinned
    host copies of the per-step inputs.  `requests` keeps a subset of the batch
    (request sharding: the rank gets its own pool holding only their pages);
    `kv_heads` keeps a slice of the KV heads and the query heads that share them
    (KV-head sharding: same table, narrower pool)."""
    import torch
    lens, table, pool_pages = decode_lengths()
    if requests is not None:
        lens = lens[requests]
        rng = np.random.default_rng(1)
        table, pool_pages = workloads.paged_table(rng, lens, 1, PAGE, slack=0.10)
    hk = kv_heads.stop - kv_heads.start
    hq = hk * (HQ // HK)
    batch = len(lens)
    gen = torch.Generator(device=device)
    gen.manual_seed(value_seed)
    pool = torch.empty((pool_pages, PAGE, 2 * hk, D), dtype=torch.bfloat16, device=device)
    fill_normal(pool, gen)
    host = {
        "q": torch.randn((batch, 1, hq, D), dtype=torch.float32).to(torch.bfloat16).pin_memory(),
        "k": torch.randn((batch, 1, hk, D), dtype=torch.float32).to(torch.bfloat16).pin_memory(),
        "v": torch.randn((batch, 1, hk, D), dtype=torch.float32).to(torch.bfloat16).pin_memory(),
        "lens": torch.from_numpy(lens).pin_memory(),
        "table": torch.from_numpy(table).pin_memory(),
    }
    dev = {name: t.to(device) for name, t in host.items()}
    return {"pool": pool, "host": host, "dev": dev, "lens": lens, "table": table, "batch": batch, "hq": hq,
            "hk": hk, "kv_bytes": workloads.decode_kv_bytes(lens, 1, hk, D, 2), "pool_pages": pool_pages}


def make_decode_call(work, device):
    """A closure that enqueues one decode step through the C ABI on device
    buffers (no host traffic), and the output tensor it fills."""
    import torch
    from flywheel_tpu.softmax_attention import _native
    dev = work["dev"]
    out = torch.empty_like(dev["q"])
    args = _native.FwDecodeArgs(
        q=dev["q"].data_ptr(), out=out.data_ptr(), kv_cache=work["pool"].data_ptr(),
        k_new=dev["k"].data_ptr(), v_new=dev["v"].data_ptr(),
        cache_seqlens=dev["lens"].data_ptr(), block_table=dev["table"].data_ptr(),
        num_pages=work["pool"].shape[0], page_size=PAGE, pages_per_seq=dev["table"].shape[1],
        batch=work["batch"], seqlen_q=1, nheads=work["hq"], nheads_k=work["hk"], head_dim=D, kv_dtype=0,
        causal=1, window_left=-1, softmax_scale=D ** -0.5, softcap=0.0, num_ctas=0)
    return bind_decode(args, device), out


def bind_decode(args, device):
    """Gives `args` a zeroed workspace and returns (enqueue, read status)."""
    import torch
    from flywheel_tpu.softmax_attention import _native
    lib = _native.library()
    nbytes = lib.fw_decode_workspace_bytes(ctypes.byref(args))
    if nbytes == 0:
        raise RuntimeError(_native.last_error())
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device=device)
    args.workspace, args.workspace_bytes = scratch.data_ptr(), nbytes
    stream = torch.cuda.current_stream(device).cuda_stream

    def call():
        _native.check(lib.fw_decode_kvcache(ctypes.byref(args), stream))

    def status():
        return _native.read_status(scratch, device)

    return call, status


def hbm_roofline(nbytes, ms, kernel, traffic=None):
    hbm_peak, _, _, kind = measured_peaks()
    achieved = nbytes / (ms * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
            "traffic": traffic, "peak_kind": f"of {kind}", "kernel": kernel,
            "algorithmic_bytes_per_launch": nbytes, "frac_of_nominal_8TBs": achieved / 8000.0}


# ---------------------------------------------------------------- chunked prefill (config 4)
PF_BATCH, PF_HQ, PF_HK = 16, 32, 8


def build_prefill_workload(seed, device, *, head_dim=128, pool_dtype="bf16"):
    """Chunked prefill over a paged cache: 16 requests, cached prefix U[0,16384]
    in 64-token pages (random block table), new chunk U[512,2048] already written
    to the pool (seqused_k = prefix + chunk), 32 q heads, 8 kv heads, causal,
    head-major q.  pool_dtype "e4m3" re-types the pool (per-tensor descale 5.5 / 448)."""
    import torch
    rng = np.random.default_rng(1000 + seed)
    prefix = rng.integers(0, 16384 + 1, PF_BATCH).astype(np.int32)
    chunk = rng.integers(512, 2048 + 1, PF_BATCH).astype(np.int32)
    seqused = (prefix + chunk).astype(np.int32)
    table, pool_pages = workloads.paged_table(rng, seqused, 0, PAGE, slack=0.10)
    gen = torch.Generator(device=device)
    gen.manual_seed(1000 + seed)
    pool = torch.randn((pool_pages, PAGE, 2 * PF_HK, head_dim), generator=gen, device=device,
                       dtype=torch.float32).to(torch.bfloat16)
    descale = None
    if pool_dtype == "e4m3":
        pool = (pool.float() * (448.0 / 5.5)).clamp(-448, 448).to(torch.float8_e4m3fn)
        descale = torch.tensor([5.5 / 448.0], dtype=torch.float32, device=device)
    cu = np.concatenate(([0], np.cumsum(chunk))).astype(np.int32)
    total_q = int(cu[-1])
    q_host = torch.randn((PF_HQ, total_q, head_dim), dtype=torch.float32).to(torch.bfloat16).pin_memory()
    return {"pool": pool, "descale": descale, "q_host": q_host, "q": q_host.to(device), "cu": cu, "seqused": seqused,
            "table": table, "prefix": prefix, "chunk": chunk, "total_q": total_q, "head_dim": head_dim,
            "flops": workloads.prefill_flops(prefix, chunk, PF_HQ, head_dim),
            "cu_dev": torch.from_numpy(cu).to(device), "seqused_dev": torch.from_numpy(seqused).to(device),
            "table_dev": torch.from_numpy(table).to(device)}


def make_prefill_call(work, device, route="auto"):
    import torch
    from flywheel_tpu.softmax_attention import _native
    out = torch.empty_like(work["q"])
    d = work["head_dim"]
    args = _native.FwPrefillArgs(
        q=work["q"].data_ptr(), out=out.data_ptr(), kv_cache=work["pool"].data_ptr(),
        cu_seqlens_q=work["cu_dev"].data_ptr(), seqused_k=work["seqused_dev"].data_ptr(),
        block_table=work["table_dev"].data_ptr(), num_pages=work["pool"].shape[0], page_size=PAGE,
        pages_per_seq=work["table_dev"].shape[1], batch=PF_BATCH, total_q=work["total_q"],
        max_seqlen_q=int(work["chunk"].max()), nheads=PF_HQ, nheads_k=PF_HK, head_dim=d,
        kv_dtype=0 if work["descale"] is None else 1,
        causal=1, window_left=-1, softmax_scale=d ** -0.5, softcap=0.0, token_major=0,
        route=_native.ROUTE_CODE[route])
    if work["descale"] is not None:
        args.k_descale = args.v_descale = work["descale"].data_ptr()
    lib = _native.library()
    nbytes = lib.fw_prefill_workspace_bytes(ctypes.byref(args))
    if nbytes == 0:
        raise RuntimeError(_native.last_error())
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device=device)
    args.workspace, args.workspace_bytes = scratch.data_ptr(), nbytes
    stream = torch.cuda.current_stream(device).cuda_stream

    def call():
        _native.check(lib.fw_prefill_paged(ctypes.byref(args), stream))

    return call, out, scratch


def bench_prefill(ns, ranks):
    """Times the chunked-prefill workload: burst (rounds of >= min_round_s) and,
    with --sustained-s, one back-to-back run of that many seconds to set beside
    the sustained bf16 peak."""
    import torch
    from flywheel_tpu import flash_attn_varlen_func
    from flywheel_tpu.softmax_attention import _native
    device = ranks.device
    work = build_prefill_workload(0, device, head_dim=ns.prefill_head_dim, pool_dtype=ns.prefill_pool)
    call, out, scratch = make_prefill_call(work, device)
    steps = max(5, min(ns.steps, 30))
    for _ in range(ns.warmup):
        call()

    def one_pass():
        for _ in range(steps):
            call()

    timing = timed_rounds(one_pass, steps, ranks, rounds=ns.rounds, min_round_s=ns.min_round_s)
    sustained = None
    if ns.sustained_s > 0:
        sustained = timed_rounds(one_pass, steps, ranks, rounds=1, min_round_s=ns.sustained_s)
    status = _native.read_status(scratch, device)
    if status != 0:
        words = scratch[:16].view(torch.int32).cpu().tolist()
        raise RuntimeError(f"prefill kernel reported device status {status} (words {words})")
    e2e_ms = None
    if not ns.skip_e2e:
        def e2e_pass():
            for _ in range(3):
                flash_attn_varlen_func(       # host q in, host out back (the API copies it)
                    work["q_host"], work["pool"], None, work["cu"], None, int(work["chunk"].max()),
                    int(work["seqused"].max()), causal=True, block_table=work["table"],
                    seqused_k=work["seqused"], k_descale=work["descale"], v_descale=work["descale"],
                    nheads_k=PF_HK)

        e2e_pass()
        e2e_ms = timed_rounds(e2e_pass, 3, ranks, rounds=3, min_round_s=0.0)["ms_per_step"]
    check = None
    if ranks.rank == 0 and not ns.skip_cpu_baseline and work["descale"] is None:
        # spot-check the shortest request against the CPU oracle
        from flywheel_tpu.softmax_attention import _arrays
        from oracle import paged_attention as oracle
        r = int(np.argmin(work["seqused"]))
        pages = work["table"][r, : -(-int(work["seqused"][r]) // PAGE)]
        sub_pool = _arrays.to_host_numpy(work["pool"][torch.from_numpy(pages).to(device).long()])
        lo, hi = int(work["cu"][r]), int(work["cu"][r + 1])
        q_rows = _arrays.to_host_numpy(work["q_host"][:, lo:hi]).transpose(1, 0, 2)
        t0 = time.perf_counter()
        want, _ = oracle.ragged_paged_attention(
            q_rows, sub_pool, np.array([0, hi - lo]), work["seqused"][r:r + 1],
            np.arange(len(pages), dtype=np.int32)[None], nheads_k=PF_HK, causal=True)
        cpu_s = time.perf_counter() - t0
        got = out[:, lo:hi].float().cpu().numpy().transpose(1, 0, 2)
        flops_r = (4 * int(work["chunk"][r]) * (int(work["prefix"][r]) + (int(work["chunk"][r]) + 1) / 2) * PF_HQ
                   * work["head_dim"])
        check = {"max_abs_err_vs_cpu": float(np.abs(got - want).max()),
                 "cpu_tflops": flops_r / cpu_s / 1e12, "cpu_sample": f"request {r} of {PF_BATCH}, {cpu_s:.2f} s"}
    _, burst_peak, sustained_peak, kind = measured_peaks()
    flops = float(work["flops"])
    per_gpu = flops / (timing["ms_per_step"] * 1e-3) / 1e12
    result = {
        "metric": "chunked_prefill_tflops", "value": per_gpu * ranks.world, "unit": "TFLOP/s", "per_gpu": per_gpu,
        "ms_per_step": timing["ms_per_step"], "rounds": round_summary(timing),
        "config": {"workload": "chunked prefill over a paged cache, 16 requests, prefix U[0,16384], chunk "
                               f"U[512,2048], 32 q heads, 8 kv heads, head_dim {work['head_dim']}, page 64, causal, "
                               f"head-major q, {ns.prefill_pool} pool", "total_q": work["total_q"],
                   "sharding": "one independent copy of the workload per GPU"},
        "e2e": {"value": flops * ranks.world / (e2e_ms * 1e-3) / 1e12 if e2e_ms else None, "unit": "TFLOP/s",
                "h2d_bytes_per_step": work["q_host"].numel() * 2, "d2h_bytes_per_step": work["q_host"].numel() * 2,
                "ms_per_step": e2e_ms},
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": burst_peak, "unit": "TFLOP/s",
                     "frac": per_gpu / burst_peak, "peak_kind": f"of {kind} (bf16 burst)",
                     "frac_of_nominal_2250": per_gpu / 2250.0, "algorithmic_flops_per_launch": flops,
                     "kernel": "fw::prefill_tcgen05_kernel (+ prefill_plan_kernel)"},
        "check": check,
    }
    if sustained is not None:
        tf = flops / (sustained["ms_per_step"] * 1e-3) / 1e12
        result["sustained"] = {"seconds": sustained["round_s"], "ms_per_step": sustained["ms_per_step"],
                               "per_gpu": tf, "peak": sustained_peak, "frac": tf / sustained_peak,
                               "peak_kind": f"of {kind} (bf16 sustained)"}
    return result


# ---------------------------------------------------------------- long context (config 5)
def bench_long_context(ns, ranks, exchange):
    """Single-request long-context decode: one 128K-token paged bf16 cache (page
    64, random block table), 64 q heads, 8 kv heads, 256 decode steps with the
    fused append, the pages dealt round-robin over the ranks; per step every rank
    decodes its pages, then the (o, lse) states are exchanged and merged: p2p
    (peer stores over NVLink + flags, fused with the merge) or nccl (all-gather +
    merge).  A pass is the 256 steps from 131072 cached tokens on."""
    import torch
    from flywheel_tpu.softmax_attention import _native, distributed as d
    device, world, rank = ranks.device, ranks.world, ranks.rank
    context, steps = 131072, 256
    total_pages = (context + steps) // PAGE + 1
    local_pages = len(d.owned_pages(total_pages, world, rank))
    rng = np.random.default_rng(2000 + rank)
    perm = rng.permutation(local_pages + 4)[:local_pages].astype(np.int32)
    gen = torch.Generator(device=device)
    gen.manual_seed(2000 + rank)
    pool = torch.empty((local_pages + 4, PAGE, 2 * HK, D), dtype=torch.bfloat16, device=device)
    fill_normal(pool, gen, rows_per_chunk=512)
    table = torch.from_numpy(perm[None]).to(device)
    decoder = d.ShardedDecoder(pool=pool, table=table, nheads=HQ, nheads_k=HK, exchange=exchange)
    q = torch.randn((1, 1, HQ, D), device=device).to(torch.bfloat16)
    k = torch.randn((1, 1, HK, D), device=device).to(torch.bfloat16)
    v = torch.randn((1, 1, HK, D), device=device).to(torch.bfloat16)
    graph = decoder.capture(q, k, v, context)

    def one_pass():
        decoder.set_length(context)
        for _ in range(steps):
            graph.replay()

    for _ in range(2):
        one_pass()
    timing = timed_rounds(one_pass, steps, ranks, rounds=ns.rounds, min_round_s=min(ns.min_round_s, 0.25))
    status = _native.read_status(decoder.scratch, device)
    decoder.close()
    if status != 0:
        raise RuntimeError(f"a kernel of the long-context step reported device status {status}")
    kv_bytes = sum((context + step + 1) * 2 * HK * D * 2 for step in range(steps)) / steps
    ms = timing["ms_per_step"]
    hbm_peak, _, _, kind = measured_peaks()
    value = kv_bytes / (ms * 1e-3) / 1e9
    return {"ms_per_step": ms, "us_per_step": ms * 1e3, "value": value, "unit": "GB/s", "per_gpu": value / world,
            "rounds": round_summary(timing),
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": hbm_peak, "unit": "GB/s",
                         "frac": value / world / hbm_peak, "peak_kind": f"of {kind}",
                         "algorithmic_bytes_per_launch": kv_bytes / world,
                         "note": "latency-bound: a rank's share is tens of microseconds of HBM time"}}


def check_long_context(ranks, exchange):
    """One sharded decode step of a small request (pages dealt round-robin over
    the ranks, eager launches) against the CPU oracle's attend_rows on rank 0."""
    import ml_dtypes
    import torch
    from flywheel_tpu.softmax_attention import distributed as d
    device, world, rank = ranks.device, ranks.world, ranks.rank
    bf16 = np.dtype(ml_dtypes.bfloat16)
    rng = np.random.default_rng(77)                     # the same draws on every rank
    heads, kv_heads, total_pages, length = HQ, HK, 40, 2000 + 37
    draw = lambda shape: rng.standard_normal(shape, dtype=np.float32).astype(bf16)
    keys, values = draw((total_pages * PAGE, kv_heads, D)), draw((total_pages * PAGE, kv_heads, D))
    q, k, v = draw((1, 1, heads, D)), draw((1, 1, kv_heads, D)), draw((1, 1, kv_heads, D))
    owned = np.asarray(d.owned_pages(total_pages, world, rank))
    perm = np.random.default_rng(90 + rank).permutation(len(owned) + 2)[:len(owned)]
    merged = np.stack([keys, values], axis=2).reshape(total_pages, PAGE, 2 * kv_heads, D)  # [k0, v0, k1, v1, ...]
    pool = np.zeros((len(owned) + 2, PAGE, 2 * kv_heads, D), bf16)
    pool[perm] = merged[owned]
    to_t = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(device).view(torch.bfloat16)
    decoder = d.ShardedDecoder(pool=to_t(pool), table=torch.from_numpy(perm.astype(np.int32)[None]).to(device),
                               nheads=heads, nheads_k=kv_heads, exchange=exchange)
    out, _ = decoder.step(to_t(q), to_t(k), to_t(v), length)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()[0]
    decoder.close()
    if rank != 0:
        return None
    from oracle import paged_attention as oracle       # the checker, on rank 0 only
    keys[length], values[length] = k[0, 0], v[0, 0]
    want, _ = oracle.attend_rows(q[0].astype(np.float32), keys[:length + 1].astype(np.float32),
                                 values[:length + 1].astype(np.float32), total=length + 1, causal=True,
                                 window_left=None, softcap=0.0, scale=D ** -0.5, sinks=None)
    return {"max_abs_err": float(np.abs(got - want).max()), "tolerance": 2e-2,
            "case": f"1 request, {length} cached tokens + 1 appended, pages round-robin over {world} rank(s), "
                    f"{exchange} exchange, against oracle.attend_rows"}


def long_context_key(ns, ranks):
    result = {"metric": "long_context_decode_kv_read_bandwidth", "scaling": "strong", "n_gpus": ranks.world,
              "config": {"workload": "1 request, 128K-token paged bf16 cache, page 64, 64 q heads, 8 kv heads, 256 "
                                     "decode steps with fused append, pages dealt round-robin over the GPUs, "
                                     "(o, lse) states exchanged and merged per step; one CUDA graph replayed per "
                                     "step", "nvls": os.environ.get("NCCL_NVLS_ENABLE", "default")}}
    exchanges = ["p2p", "nccl"] if ranks.world > 1 else ["p2p"]
    for exchange in exchanges:
        entry = bench_long_context(ns, ranks, exchange)
        entry["how"] = ("no exchange: one rank holds every page" if ranks.world == 1 else
                        "peer stores of (o, lse) over NVLink + flags, fused with the merge" if exchange == "p2p"
                        else "NCCL all-gather of (o, lse) + merge")
        entry["check"] = check_long_context(ranks, exchange)
        result[exchange if ranks.world > 1 else "single"] = entry
    main = result["p2p" if ranks.world > 1 else "single"]
    result.update({"value": main["value"], "unit": "GB/s", "ms_per_step": main["ms_per_step"],
                   "us_per_step": main["us_per_step"], "check": main["check"]})
    return result


# ---------------------------------------------------------------- strong scaling of one decode batch
def strong_scaling_key(ns, ranks, full_batch_ms):
    """One 128-request batch split over the ranks, no communication on the data
    path: by request (distributed.request_shard: longest first to the least
    loaded GPU) and by KV head (distributed.kv_head_shard).  value = the whole
    batch's KV bytes / the slowest rank's time."""
    from flywheel_tpu.softmax_attention import distributed as d
    lens, _, _ = decode_lengths()
    total_bytes = workloads.decode_kv_bytes(lens, 1, HK, D, 2)
    result = {"scaling": "strong", "n_gpus": ranks.world, "full_batch_ms_on_one_gpu": full_batch_ms}
    shards = {"request_shard": dict(requests=np.asarray(d.request_shard(lens, ranks.world, ranks.rank)))}
    if HK % ranks.world == 0:
        shards["kv_head_shard"] = dict(kv_heads=d.kv_head_shard(HQ, HK, ranks.world, ranks.rank)[1])
    for name, how in shards.items():
        work = build_workload(100 + ranks.rank, ranks.device, **how)
        (call, status), _ = make_decode_call(work, ranks.device)
        for _ in range(ns.warmup):
            call()

        def one_pass():
            for _ in range(ns.steps):
                call()

        timing = timed_rounds(one_pass, ns.steps, ranks, rounds=3, min_round_s=min(ns.min_round_s, 0.2))
        if status() != 0:
            raise RuntimeError("decode kernel reported a device status")
        shares = ranks.sum([work["kv_bytes"]])[0]
        ms = timing["ms_per_step"]
        result[name] = {"value": total_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms,
                        "speedup_vs_one_gpu": full_batch_ms / ms, "efficiency": full_batch_ms / ms / ranks.world,
                        "rank0_requests": work["batch"], "rank0_kv_heads": work["hk"],
                        "bytes_check": shares / total_bytes, "rounds": round_summary(timing)}
        del work, call
        ranks.torch.cuda.empty_cache()
    return result


# ---------------------------------------------------------------- a mixed step (decode rows + prefill chunks)
def bench_mixed(ns, ranks):
    """One serving step that mixes 96 one-token decode requests (cached lengths
    U[1024,32768]) with 8 prefill chunks (prefix U[0,16384], chunk U[512,2048])
    over one paged bf16 pool, 32 q heads, 8 kv heads, page 64: the page write of
    all scheduled tokens plus attention.  Timed twice on device-resident inputs:
    through paged_extend (decode kernel for the one-token rows, tensor-core
    prefill for the chunks, one launch sequence) and through the packed
    flash_attn_with_kvcache call, where every request, one-token ones included,
    takes tensor-core query tiles."""
    import torch
    from flywheel_tpu import flash_attn_with_kvcache
    from flywheel_tpu.softmax_attention.extend import paged_extend
    device = ranks.device
    rng = np.random.default_rng(3000)
    n_decode, n_prefill, hq, hk = 96, 8, 32, 8
    before = np.concatenate([rng.integers(LEN_LO, LEN_HI + 1, n_decode), rng.integers(0, 16384 + 1, n_prefill)])
    new = np.concatenate([np.ones(n_decode, np.int64), rng.integers(512, 2048 + 1, n_prefill)])
    before, new = before.astype(np.int32), new.astype(np.int32)
    after = before + new
    cu = np.concatenate(([0], np.cumsum(new))).astype(np.int32)
    total = int(cu[-1])
    table, pool_pages = workloads.paged_table(rng, after, 0, PAGE, slack=0.10)
    columns = []
    for r in range(len(before)):
        pos, row = int(before[r]), int(cu[r])
        while pos < after[r]:
            run = min(int(after[r]) - pos, PAGE - pos % PAGE)
            columns.append((int(table[r, pos // PAGE]) * PAGE + pos % PAGE, row, run))
            pos, row = pos + run, row + run
    slices = torch.from_numpy(np.ascontiguousarray(np.array(columns, np.int32).T)).to(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(3000)
    pool = torch.empty((pool_pages, PAGE, 2 * hk, D), dtype=torch.bfloat16, device=device)
    fill_normal(pool, gen)
    q = torch.randn((total, hq, D), device=device).to(torch.bfloat16)
    k = torch.randn((total, hk, D), device=device).to(torch.bfloat16)
    v = torch.randn((total, hk, D), device=device).to(torch.bfloat16)
    dev = lambda a: torch.from_numpy(a).to(device)
    after_t, before_t, cu_t, table_t = dev(after), dev(before), dev(cu), dev(table)
    count = torch.tensor([len(columns)], dtype=torch.int32, device=device)
    n_dec = torch.tensor([n_decode], dtype=torch.int32, device=device)
    n_act = torch.tensor([n_decode + n_prefill], dtype=torch.int32, device=device)

    def mixed_pass():
        for _ in range(5):
            paged_extend(q, k, v, pool, after_t, table_t, cu_t, slices, count, n_dec, n_act)

    def packed_pass():
        for _ in range(5):
            flash_attn_with_kvcache(q, pool, None, k, v, cache_seqlens=before_t, block_table=table_t,
                                    cu_seqlens_q=cu_t, max_seqlen_q=int(new.max()), causal=True)

    out_mixed, _ = paged_extend(q, k, v, pool, after_t, table_t, cu_t, slices, count, n_dec, n_act)
    out_packed = flash_attn_with_kvcache(q, pool, None, k, v, cache_seqlens=before_t, block_table=table_t,
                                         cu_seqlens_q=cu_t, max_seqlen_q=int(new.max()), causal=True)[0]
    agree = float((out_mixed.float() - out_packed.float()).abs().max())
    mixed = timed_rounds(mixed_pass, 5, ranks, rounds=3, min_round_s=min(ns.min_round_s, 0.2))
    packed = timed_rounds(packed_pass, 5, ranks, rounds=3, min_round_s=min(ns.min_round_s, 0.2))
    kv_bytes = workloads.decode_kv_bytes(before[:n_decode], 1, hk, D, 2)
    flops = workloads.prefill_flops(before[n_decode:], new[n_decode:], hq, D)
    return {"metric": "mixed_step_ms", "unit": "ms", "higher_is_better": False,
            "config": {"workload": f"{n_decode} decode requests U[1024,32768] + {n_prefill} prefill chunks (prefix "
                                   "U[0,16384], chunk U[512,2048]), 32 q heads, 8 kv heads, head_dim 128, page 64, "
                                   "bf16; page write of the scheduled tokens included", "tokens": total},
            "value": mixed["ms_per_step"], "ms_per_step": mixed["ms_per_step"],
            "decode_kv_bytes": kv_bytes, "prefill_flops": flops,
            "packed_route_ms_per_step": packed["ms_per_step"],
            "speedup_over_packed_route": packed["ms_per_step"] / mixed["ms_per_step"],
            "max_abs_diff_between_routes": agree, "rounds": round_summary(mixed)}


# ---------------------------------------------------------------- secondary decode configurations
# The reference's own serving and perf-gate decode shapes (page 128), beside
# which its TPU tables sit: docs/v7x.md:129-150 and scripts/perf_gate.py:80-107
# of the reference.  Paged bf16, single-token decode unless q_len says otherwise.
SECONDARY_SHAPES = {
    "serve-d256-gqa": dict(batch=128, hq=32, hk=4, d=256, page=128, q_len=1, lens=(15360, 15360)),
    "serve-d256-gqa-b32": dict(batch=32, hq=32, hk=4, d=256, page=128, q_len=1, lens=(15360, 15360)),
    "serve-d256-gqa-b256": dict(batch=256, hq=32, hk=4, d=256, page=128, q_len=1, lens=(15360, 15360)),
    "serve-d256-mha": dict(batch=32, hq=32, hk=32, d=256, page=128, q_len=1, lens=(15360, 15360)),
    "serve-d256-mha-b128": dict(batch=128, hq=32, hk=32, d=256, page=128, q_len=1, lens=(15360, 15360)),
    "gate-decode": dict(batch=64, hq=32, hk=8, d=128, page=128, q_len=1, lens=(6144, 10239)),
    "gate-verify": dict(batch=32, hq=32, hk=8, d=128, page=128, q_len=4, lens=(6144, 10239)),
    # the verify window of configuration 3 (32 query rows per KV head) on a bf16 pool, no softcap or window
    "verify-bf16-gqa8": dict(batch=128, hq=64, hk=8, d=128, page=64, q_len=4, lens=(1024, 32768)),
}
CONFIG_TEXT = {
    "c1": "contiguous bf16 GQA decode, batch 8, 32 q heads, 8 kv heads, head_dim 128, caches (8, 2048, 8, 128), "
          "cached lengths U[128,2047], fused one-token append, causal",
    "c3": "paged fp8 e4m3 decode with per-tensor descales, batch 128, 64 q heads, 8 kv heads, head_dim 128, page "
          "64, cached lengths U[1024,32768], sliding window 4096, softcap 50, one sink per head, 4-token verify "
          "window with fused append",
}


def bench_config(ns, name, ranks):
    """Secondary decode configurations (device-resident): c1 = contiguous bf16
    GQA decode; c3 = paged fp8 e4m3 verify-window decode; and the reference's
    serving / perf-gate shapes."""
    import torch
    from flywheel_tpu.softmax_attention import _native
    device = ranks.device
    rng = np.random.default_rng(0)
    e2e = None
    if name == "c1":
        batch, hq, hk, cap = 8, 32, 8, 2048
        lens = rng.integers(128, 2048, batch).astype(np.int32)
        kc = torch.randn((batch, cap, hk, D), device=device).to(torch.bfloat16)
        vc = torch.randn((batch, cap, hk, D), device=device).to(torch.bfloat16)
        q = torch.randn((batch, 1, hq, D), device=device).to(torch.bfloat16)
        k = torch.randn((batch, 1, hk, D), device=device).to(torch.bfloat16)
        v = torch.randn((batch, 1, hk, D), device=device).to(torch.bfloat16)
        lens_t = torch.from_numpy(lens).to(device)
        out = torch.empty_like(q)
        args = _native.FwDecodeArgs(
            q=q.data_ptr(), out=out.data_ptr(), kv_cache=kc.data_ptr(), v_cache=vc.data_ptr(),
            k_new=k.data_ptr(), v_new=v.data_ptr(), cache_seqlens=lens_t.data_ptr(), num_pages=batch,
            page_size=cap, pages_per_seq=1, batch=batch, seqlen_q=1, nheads=hq, nheads_k=hk, head_dim=D,
            kv_dtype=0, causal=1, window_left=-1, softmax_scale=D ** -0.5, softcap=0.0)
        kv_bytes = workloads.decode_kv_bytes(lens, 1, hk, D, 2)
        keep = (kc, vc, q, k, v, lens_t, out)
        kernel = "fw::decode_kernel<bf16> (+ combine_kernel)"
        # the same step end to end: q, new k / v and the lengths in pinned host memory, the caches
        # resident, the output read back; at this size the host side is most of the step
        from flywheel_tpu import flash_attn_with_kvcache
        pinned = [t.cpu().pin_memory() for t in (q, k, v, lens_t)]

        def e2e_pass():
            for _ in range(20):
                flash_attn_with_kvcache(pinned[0], kc, vc, pinned[1], pinned[2], cache_seqlens=pinned[3],
                                        causal=True)

        e2e_pass()
        e2e_ms = timed_rounds(e2e_pass, 20, ranks, rounds=3, min_round_s=0.05)["own_ms_per_step"]
        e2e = {"value": kv_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in pinned),
               "d2h_bytes_per_step": q.numel() * 2,
               "note": "through flywheel_tpu.flash_attn_with_kvcache; L2 not flushed between these steps"}
    elif name in SECONDARY_SHAPES:
        spec = SECONDARY_SHAPES[name]
        batch, hq, hk, d, page, q_len = (spec[key] for key in ("batch", "hq", "hk", "d", "page", "q_len"))
        lo, hi = spec["lens"]
        lens = rng.integers(lo, hi + 1, batch).astype(np.int32)
        table, pool_pages = workloads.paged_table(rng, lens, q_len, page, slack=0.10)
        pool = torch.empty((pool_pages, page, 2 * hk, d), dtype=torch.bfloat16, device=device)
        rows = max(1, (256 << 20) // (page * 2 * hk * d * 2))
        for first in range(0, pool_pages, rows):
            pool[first:first + rows].normal_()
        q = torch.randn((batch, q_len, hq, d), device=device).to(torch.bfloat16)
        k = torch.randn((batch, q_len, hk, d), device=device).to(torch.bfloat16)
        v = torch.randn((batch, q_len, hk, d), device=device).to(torch.bfloat16)
        lens_t, table_t = torch.from_numpy(lens).to(device), torch.from_numpy(table).to(device)
        out = torch.empty_like(q)
        args = _native.FwDecodeArgs(
            q=q.data_ptr(), out=out.data_ptr(), kv_cache=pool.data_ptr(), k_new=k.data_ptr(),
            v_new=v.data_ptr(), cache_seqlens=lens_t.data_ptr(), block_table=table_t.data_ptr(),
            num_pages=pool_pages, page_size=page, pages_per_seq=table.shape[1], batch=batch, seqlen_q=q_len,
            nheads=hq, nheads_k=hk, head_dim=d, kv_dtype=0, causal=1, window_left=-1,
            softmax_scale=d ** -0.5, softcap=0.0)
        kv_bytes = workloads.decode_kv_bytes(lens, q_len, hk, d, 2)
        keep = (pool, q, k, v, lens_t, table_t, out)
        kernel = "fw::decode_kernel<bf16> (+ combine_kernel)"
    else:  # c3
        batch, hq, hk, q_len, window = 128, 64, 8, 4, 4095
        lens = rng.integers(LEN_LO, LEN_HI + 1, batch).astype(np.int32)
        table, pool_pages = workloads.paged_table(rng, lens, q_len, PAGE, slack=0.10)
        pool = torch.empty((pool_pages, PAGE, 2 * hk, D), dtype=torch.float8_e4m3fn, device=device)
        for lo in range(0, pool_pages, 8192):
            hi = min(pool_pages, lo + 8192)
            block = torch.randn((hi - lo, PAGE, 2 * hk, D), device=device)
            pool[lo:hi] = (block * (448.0 / 5.5)).clamp(-448, 448).to(torch.float8_e4m3fn)
        descale = torch.tensor([5.5 / 448.0], dtype=torch.float32, device=device)
        q = torch.randn((batch, q_len, hq, D), device=device).to(torch.bfloat16)
        k = (torch.randn((batch, q_len, hk, D), device=device) * (448.0 / 5.5)).to(torch.float8_e4m3fn)
        v = (torch.randn((batch, q_len, hk, D), device=device) * (448.0 / 5.5)).to(torch.float8_e4m3fn)
        sinks = torch.randn(hq, device=device)
        lens_t, table_t = torch.from_numpy(lens).to(device), torch.from_numpy(table).to(device)
        out = torch.empty_like(q)
        args = _native.FwDecodeArgs(
            q=q.data_ptr(), out=out.data_ptr(), kv_cache=pool.data_ptr(), k_new=k.data_ptr(),
            v_new=v.data_ptr(), cache_seqlens=lens_t.data_ptr(), block_table=table_t.data_ptr(),
            k_descale=descale.data_ptr(), v_descale=descale.data_ptr(), sinks=sinks.data_ptr(),
            num_pages=pool_pages, page_size=PAGE, pages_per_seq=table.shape[1], batch=batch, seqlen_q=q_len,
            nheads=hq, nheads_k=hk, head_dim=D, kv_dtype=1, causal=1, window_left=window,
            softmax_scale=D ** -0.5, softcap=50.0)
        kv_bytes = workloads.decode_kv_bytes(lens, q_len, hk, D, 1, window_left=window)
        keep = (pool, descale, q, k, v, sinks, lens_t, table_t, out)
        kernel = "fw::decode_kernel<e4m3> (+ combine_kernel)"
    call, status = bind_decode(args, device)
    for _ in range(ns.warmup):
        call()
    if kv_bytes < (512 << 20):
        # A step moves less than L2 holds (c1: 36 MB): flush L2 between steps so the
        # caches are read from HBM like in serving, and time every step by itself.
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
        steps, times = max(ns.steps, 100), []
        for _ in range(steps):
            flush.zero_()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            call()
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end))
        ms, l2 = float(np.median(times)), "L2 flushed between steps; every step timed by itself"
        rounds = {"count": steps, "steps_per_round": 1, "ms_per_step_median": ms,
                  "ms_per_step_min": float(min(times)), "ms_per_step_max": float(max(times))}
    else:
        def one_pass():
            for _ in range(ns.steps):
                call()

        timing = timed_rounds(one_pass, ns.steps, ranks, rounds=ns.rounds, min_round_s=min(ns.min_round_s, 0.25))
        ms, l2, rounds = timing["own_ms_per_step"], "inputs exceed L2", round_summary(timing)
    if status() != 0:
        raise RuntimeError("decode kernel reported a device status")
    del keep
    torch.cuda.empty_cache()
    result = {"metric": "decode_kv_read_bandwidth",
              "config": {"workload": CONFIG_TEXT.get(name, name), "name": name, "l2": l2},
              "value": kv_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms, "rounds": rounds,
              "gpu_launches_per_step": 2, "roofline": hbm_roofline(kv_bytes, ms, kernel)}
    if e2e is not None:
        result["e2e"] = e2e
    return result


# Dense causal prefill shapes for flash_attn_func (the reference's dense-prefill
# table uses 32:8 heads, head_dim 128; docs/v7x.md:54 of the reference).
DENSE_SHAPES = {
    "dense-causal-8k": dict(batch=4, hq=32, hk=8, seqlen=8192),
    "dense-causal-32k": dict(batch=1, hq=32, hk=8, seqlen=32768),
}


def bench_dense(ns, name, device):
    """flash_attn_func (head-major, causal) through the public API on device
    tensors: TFLOP/s = 4 * visible pairs * heads * head_dim / time."""
    import torch
    from flywheel_tpu import flash_attn_func
    spec = DENSE_SHAPES[name]
    batch, hq, hk, seqlen = (spec[key] for key in ("batch", "hq", "hk", "seqlen"))
    q = torch.randn((batch, hq, seqlen, D), device=device).to(torch.bfloat16)
    k = torch.randn((batch, hk, seqlen, D), device=device).to(torch.bfloat16)
    v = torch.randn((batch, hk, seqlen, D), device=device).to(torch.bfloat16)
    flops = 4.0 * batch * (seqlen * (seqlen + 1) / 2) * hq * D
    steps = max(ns.steps, 10)
    times = []
    for i in range(ns.warmup + steps):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        flash_attn_func(q, k, v, causal=True)
        end.record()
        torch.cuda.synchronize()
        if i >= ns.warmup:
            times.append(start.elapsed_time(end))
    ms = float(np.median(times))
    _, tensor_peak, _, kind = measured_peaks()
    tflops = flops / (ms * 1e-3) / 1e12
    return {"metric": "dense_causal_prefill_tflops", "config": {"workload": name, **spec, "head_dim": D,
            "l2": "inputs exceed L2" if 3 * q.numel() * 2 > (126 << 20) else "inputs fit L2 (compute-bound)"},
            "value": tflops, "unit": "TFLOP/s", "ms_per_step": ms, "steps": steps,
            "algorithmic_flops_per_launch": flops,
            "roofline": {"bound": "tensor", "achieved": tflops, "peak": tensor_peak,
                         "frac": tflops / tensor_peak if tensor_peak else None, "peak_kind": f"of {kind}"}}


SERVING_PREFILL = {"serve-d256-prefill-gqa": dict(hk=4), "serve-d256-prefill-mha": dict(hk=32)}


def bench_serving_prefill(ns, name, device):
    """The reference's serving prefill scenario (docs/v7x.md:129-150 of the
    reference): one 16K-token sequence prefilled in 1K chunks through
    flash_attn_with_kvcache (append + attend, 16 calls), 32 q heads, head_dim
    256, page 128 shuffled.  TFLOP/s over the 16 calls together."""
    import torch
    from flywheel_tpu import flash_attn_with_kvcache
    hk = SERVING_PREFILL[name]["hk"]
    hq, d, page, total, chunk = 32, 256, 128, 16384, 1024
    pages = total // page
    gen = torch.Generator(device=device)
    gen.manual_seed(7)
    pool = torch.zeros((pages + 8, page, 2 * hk, d), dtype=torch.bfloat16, device=device)
    table = torch.randperm(pages + 8, generator=gen, device=device)[:pages].to(torch.int32)[None].contiguous()
    q = torch.randn((1, chunk, hq, d), device=device).to(torch.bfloat16)
    k = torch.randn((1, chunk, hk, d), device=device).to(torch.bfloat16)
    v = torch.randn((1, chunk, hk, d), device=device).to(torch.bfloat16)
    lens = [torch.tensor([i * chunk], dtype=torch.int32, device=device) for i in range(total // chunk)]

    def sequence():
        for cached in lens:
            flash_attn_with_kvcache(q, pool, None, k, v, cache_seqlens=cached, block_table=table, causal=True)

    flops = 4.0 * (total * (total + 1) / 2) * hq * d
    steps = max(3, min(ns.steps, 10))
    for _ in range(2):
        sequence()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        sequence()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    _, tensor_peak, _, kind = measured_peaks()
    tflops = flops / (ms * 1e-3) / 1e12
    return {"metric": "serving_chunked_prefill_tflops", "config": {"workload": name, "nheads": hq, "nheads_k": hk,
            "head_dim": d, "page_size": page, "sequence": total, "chunk": chunk,
            "calls": "16 x flash_attn_with_kvcache (ragged append + chunked prefill)"},
            "value": tflops, "unit": "TFLOP/s", "ms_per_sequence": ms, "steps": steps,
            "algorithmic_flops_per_sequence": flops,
            "roofline": {"bound": "tensor", "achieved": tflops, "peak": tensor_peak,
                         "frac": tflops / tensor_peak if tensor_peak else None, "peak_kind": f"of {kind}"}}


# ---------------------------------------------------------------- CPU baseline and the reference arm
def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:  # pragma: no cover
        return os.cpu_count() or 1


def cpu_baseline(work, repeats=3):
    """Times the C/OpenMP restatement of the reference's test oracle
    (oracle/paged_decode_ref.c) on the whole decode batch, on all host cores."""
    from flywheel_tpu.softmax_attention import _arrays
    from oracle import c_port
    lens, table, threads = work["lens"], work["table"], host_threads()
    pool = _arrays.to_host_numpy(work["pool"])
    host = work["host"]
    q, k, v = (_arrays.to_host_numpy(host[name]) for name in ("q", "k", "v"))
    c_port.paged_decode(q[:2], pool, k[:2], v[:2], lens[:2], table[:2], nheads_k=HK, in_place=True,
                        threads=threads)  # page in
    times = []
    for _ in range(repeats):
        start = time.perf_counter()
        out, _, _ = c_port.paged_decode(q, pool, k, v, lens, table, nheads_k=HK, causal=True, in_place=True,
                                        threads=threads)
        times.append(time.perf_counter() - start)
    seconds = float(np.median(times))
    nbytes = work["kv_bytes"]
    return {"value": nbytes / seconds / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"all {len(lens)} requests ({nbytes / 1e9:.2f} GB of KV), median of {repeats} passes of "
                      f"{seconds:.2f} s, C + OpenMP restatement of the reference's test oracle"}, out, len(lens)


def run_reference_arm(ns):
    """The reference's CPU path stands in as the C + OpenMP restatement of its
    own test oracle (the reference itself needs JAX, absent from this image),
    on all host cores - the thread count is set by this program, not taken from
    the launcher's environment; a step is the first 32 requests of the decode
    batch over a pool of its own (values tiled from 256 random pages: they do not
    change the timing)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import ml_dtypes
    from oracle import c_port
    bf16 = np.dtype(ml_dtypes.bfloat16)
    rng = np.random.default_rng(0)
    lens = rng.integers(LEN_LO, LEN_HI + 1, BATCH).astype(np.int32)
    sample, threads = min(32, BATCH), host_threads()
    table, pool_pages = workloads.paged_table(rng, lens[:sample], 1, PAGE, slack=0.10)
    draw = lambda shape: rng.standard_normal(shape, dtype=np.float32).astype(bf16)
    block = draw((256, PAGE, 2 * HK, D))
    pool = np.ascontiguousarray(np.tile(block, (-(-pool_pages // 256), 1, 1, 1))[:pool_pages])
    q, k, v = draw((sample, 1, HQ, D)), draw((sample, 1, HK, D)), draw((sample, 1, HK, D))
    nbytes = workloads.decode_kv_bytes(lens[:sample], 1, HK, D, 2)
    times = []
    for step in range(ns.warmup + ns.steps):
        start = time.perf_counter()
        c_port.paged_decode(q, pool, k, v, lens[:sample], table, nheads_k=HK, causal=True, in_place=True,
                            threads=threads)
        if step >= ns.warmup:
            times.append(time.perf_counter() - start)
    ms = 1e3 * float(np.mean(times))
    value = nbytes / (ms * 1e-3) / 1e9
    sample_text = (f"first {sample} of {BATCH} requests per step ({nbytes / 1e9:.2f} GB of KV) over a pool of their "
                   f"own pages; C + OpenMP restatement of the reference's test oracle on {threads} host threads")
    config = workload_config()
    config["reference_sample"] = sample_text
    print(json.dumps({
        "impl": "reference", "metric": "paged_decode_kv_read_bandwidth", "value": value, "unit": "GB/s",
        "n_gpus": ns.gpus, "steps": ns.steps, "warmup": ns.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": config,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": sample_text},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config():
    return {"workload": "paged bf16 GQA decode, batch 128, 64 q heads, 8 kv heads, head_dim 128, "
                        "page 64, cached lengths U[1024,32768], pool = pages in use + 10%, random block "
                        "table, fused one-token append, causal",
            "l2": "inputs (about 9 GB of KV per step) far exceed the 126 MB L2",
            "sharding": "one copy of the batch per GPU, the same lengths on every GPU (request sharding, no "
                        "collective on the data path)"}


# ---------------------------------------------------------------- main
def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--rounds", type=int, default=5, help="timed rounds per measurement (median reported)")
    parser.add_argument("--min-round-s", type=float, default=0.5, help="shortest round, in seconds")
    parser.add_argument("--sustained-s", type=float, default=2.0,
                        help="length of the back-to-back prefill run set beside the sustained bf16 peak (0 = off)")
    parser.add_argument("--skip-cpu-baseline", action="store_true")
    parser.add_argument("--skip-e2e", action="store_true")
    parser.add_argument("--skip-prefill", action="store_true")
    parser.add_argument("--skip-extra", action="store_true", help="leave out c1, c3, long_context and strong")
    parser.add_argument("--config", choices=["c1", "c3", *SECONDARY_SHAPES, *DENSE_SHAPES, *SERVING_PREFILL],
                        default=None, help="run one secondary configuration instead of the headline")
    parser.add_argument("--long-context", action="store_true",
                        help="run only the single-request 128K-token decode split over the GPUs")
    parser.add_argument("--exchange", choices=["p2p", "nccl"], default="p2p")
    parser.add_argument("--prefill-only", action="store_true",
                        help="run only the chunked-prefill workload (profiler captures)")
    parser.add_argument("--prefill-pool", choices=["bf16", "e4m3"], default="bf16")
    parser.add_argument("--prefill-head-dim", type=int, choices=[128, 256], default=128)
    parser.add_argument("--batch", type=int, default=128,
                        help="requests per step; smaller than 128 only for profiler captures")
    ns = parser.parse_args()
    globals()["BATCH"] = ns.batch
    ns.warmup = max(ns.warmup, 3) if ns.impl == "ours" else ns.warmup
    if ns.impl == "reference":
        run_reference_arm(ns)
        return

    ranks = Ranks()
    torch, device, world, rank = ranks.torch, ranks.device, ranks.world, ranks.rank
    try:
        if ns.config in DENSE_SHAPES:
            print(json.dumps(bench_dense(ns, ns.config, device)))
        elif ns.config in SERVING_PREFILL:
            print(json.dumps(bench_serving_prefill(ns, ns.config, device)))
        elif ns.config:
            print(json.dumps(bench_config(ns, ns.config, ranks)))
        elif ns.long_context:
            entry = bench_long_context(ns, ranks, ns.exchange)
            entry["check"] = check_long_context(ranks, ns.exchange)
            if rank == 0:
                print(json.dumps({"metric": "long_context_decode_kv_read_bandwidth", "n_gpus": world,
                                  "exchange": ns.exchange, **entry}))
        elif ns.prefill_only:
            result = bench_prefill(ns, ranks)
            if rank == 0:
                print(json.dumps(result), flush=True)
        else:
            headline(ns, ranks)
    finally:
        ranks.close()


def headline(ns, ranks):
    from flywheel_tpu import flash_attn_with_kvcache
    torch, device, world, rank = ranks.torch, ranks.device, ranks.world, ranks.rank
    work = build_workload(value_seed=rank, device=device)
    (call, status), out = make_decode_call(work, device)

    def one_pass():
        for _ in range(ns.steps):
            call()

    # ---- device-resident arm
    for _ in range(ns.warmup):
        call()
    sampler = ClockSampler(physical_gpu_index(ranks.local_rank))
    sampler.start()
    timing = timed_rounds(one_pass, ns.steps, ranks, rounds=ns.rounds, min_round_s=ns.min_round_s)
    clocks = sampler.summary()
    if status() != 0:
        raise RuntimeError("decode kernel reported a device status")

    # ---- end-to-end arm: host inputs in, host output back, every step
    host = work["host"]

    def e2e_pass():
        for _ in range(ns.steps):
            flash_attn_with_kvcache(   # returns a host tensor: the API copied it device -> host and synchronised
                host["q"], work["pool"], None, host["k"], host["v"], cache_seqlens=host["lens"],
                block_table=host["table"], causal=True)

    e2e = None
    if not ns.skip_e2e:
        e2e_pass()
        e2e = timed_rounds(e2e_pass, ns.steps, ranks, rounds=ns.rounds, min_round_s=ns.min_round_s)
    h2d = sum(host[name].numel() * host[name].element_size() for name in ("q", "k", "v", "lens", "table"))
    d2h = host["q"].numel() * host["q"].element_size()
    job_bytes = ranks.sum([float(work["kv_bytes"])])[0]

    line = None
    if rank == 0:
        ms = timing["ms_per_step"]
        value = job_bytes / (ms * 1e-3) / 1e9
        # reads 1.0011 x algorithmic in the small-case ncu capture (profiles/decode_bf16_paged_c2.md);
        # writes = the per-CTA partial states
        traffic = work["kv_bytes"] * 1.0011 + (BATCH + 148) * HQ * (D + 2) * 4
        line = {
            "metric": "paged_decode_kv_read_bandwidth", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": ns.steps, "warmup": ns.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(), "per_gpu": value / world, "clocks": clocks,
            "rounds": round_summary(timing),
            "timed_region_s": timing["round_s"] * timing["rounds"],
            "gpu_launches": 2 * timing["steps_per_round"] * timing["rounds"],
            "gpu_launches_per_step": 2,
            "e2e": {"value": job_bytes / (e2e["ms_per_step"] * 1e-3) / 1e9 if e2e else None, "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e["ms_per_step"] if e2e else None,
                    "rounds": round_summary(e2e) if e2e else None},
            # this rank's bytes over this rank's own time per launch pair (decode + combine)
            "roofline": hbm_roofline(work["kv_bytes"], timing["own_ms_per_step"],
                                     "fw::decode_kernel<bf16> (+ combine_kernel, <1% of the launch pair)", traffic),
        }
    full_batch_ms = timing["ms_per_step"]
    cpu = None
    if rank == 0 and world == 1 and not ns.skip_cpu_baseline:
        base, cpu_out, count = cpu_baseline(work)
        cpu = (base, float(np.abs(out[:count].float().cpu().numpy() - cpu_out).max()))
    del work, call, out
    torch.cuda.empty_cache()

    def guarded(measure):
        """A secondary measurement that fails must not take the headline line with it."""
        try:
            return measure()
        except Exception as exc:  # pylint: disable=broad-except
            torch.cuda.empty_cache()
            return {"error": f"{type(exc).__name__}: {exc}"[:300]}

    prefill = None if ns.skip_prefill else guarded(lambda: bench_prefill(ns, ranks))
    extra = {}
    if not ns.skip_extra:
        if world == 1:
            extra["c1"] = guarded(lambda: bench_config(ns, "c1", ranks))
            extra["c3"] = guarded(lambda: bench_config(ns, "c3", ranks))
            extra["mixed"] = guarded(lambda: bench_mixed(ns, ranks))
        else:
            # every rank has just timed the full batch by itself: that is the one-GPU time
            extra["strong"] = guarded(lambda: strong_scaling_key(ns, ranks, full_batch_ms))
        extra["long_context"] = guarded(lambda: long_context_key(ns, ranks))
    if rank == 0:
        if prefill is not None:
            line["prefill"] = prefill
        line.update(extra)
        if cpu is not None:
            line["cpu_baseline"], line["sample_max_abs_err_vs_cpu"] = cpu
        print(json.dumps(line))


if __name__ == "__main__":
    main()
