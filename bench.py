"""Benchmark of the paged-KV attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  Headline: paged bf16 GQA decode at serving scale (batch
128, 64 query heads, 8 KV heads, head_dim 128, 64-token pages, cached lengths
uniform in [1024, 32768], fused one-token append, causal), reported as KV bytes
read per second (the reference benchmark's kv_bytes_read accounting).  A step
is one decode call over the whole batch.

* value: device-resident inputs, timed with CUDA events on the launch stream.
* e2e: the same step through flywheel_tpu.flash_attn_with_kvcache with the
  per-step inputs (q, new k/v, lengths, block table) in pinned host memory and
  the output read back to the host inside the timed region; the KV cache stays
  resident on the device, as it does in serving.
* roofline: algorithmic KV bytes per launch / measured launch time, against
  the measured HBM copy bandwidth in MEASURED_PEAKS.json.
* cpu_baseline: the C + OpenMP restatement of the reference's test oracle
  (oracle/paged_decode_ref.c) on the same batch, on all host cores.
* --impl reference: that CPU restatement as its own arm (the reference itself
  needs JAX, which this image lacks); a step is the first 32 requests.

With N > 1 (torchrun) every rank runs its own copy of the workload with its own
seed (requests shard with no communication); value is the sum of bytes over
ranks divided by the slowest rank's time.

Other workloads, one JSON line each (device-resident inputs):
    --config c1 | c3                     contiguous bf16 decode; paged fp8 verify window
    --config serve-d256-gqa | serve-d256-mha | gate-decode | gate-verify
                                         the reference's serving / perf-gate decode shapes
    --config dense-causal-8k | dense-causal-32k      flash_attn_func, causal
    --config serve-d256-prefill-gqa | -mha           16K sequence in 1K chunks, head_dim 256
    --prefill-only [FW_PREFILL_POOL=e4m3] [FW_PREFILL_HEAD_DIM=256]   the chunked-prefill workload alone
    --long-context [FLYWHEEL_EXCHANGE=p2p|nccl]      one 128K-token request split over the GPUs
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import pathlib
import sys
import threading
import time

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "flywheel-tpu_b200"))
sys.path.insert(0, str(ROOT))

BATCH, HQ, HK, D, PAGE = 128, 64, 8, 128, 64
LEN_LO, LEN_HI = 1024, 32768
FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), float(data.get("bf16_tflops", 0)), "measured"
    return FALLBACK_HBM_GBS, 1590.0, "fallback"


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


def build_workload(seed, device):
    """The serving-scale decode workload on `device`: returns a dict of device
    tensors plus the host copies of the per-step inputs."""
    import torch
    from flywheel_tpu.testing import workloads
    rng = np.random.default_rng(seed)
    lens = rng.integers(LEN_LO, LEN_HI + 1, BATCH).astype(np.int32)
    table, pool_pages = workloads.paged_table(rng, lens, 1, PAGE, slack=0.10)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    pool = torch.empty((pool_pages, PAGE, 2 * HK, D), dtype=torch.bfloat16, device=device)
    chunk = 4096
    for lo in range(0, pool_pages, chunk):
        hi = min(pool_pages, lo + chunk)
        pool[lo:hi] = torch.randn((hi - lo, PAGE, 2 * HK, D), generator=gen, device=device,
                                  dtype=torch.float32).to(torch.bfloat16)
    host = {
        "q": torch.randn((BATCH, 1, HQ, D), dtype=torch.float32).to(torch.bfloat16).pin_memory(),
        "k": torch.randn((BATCH, 1, HK, D), dtype=torch.float32).to(torch.bfloat16).pin_memory(),
        "v": torch.randn((BATCH, 1, HK, D), dtype=torch.float32).to(torch.bfloat16).pin_memory(),
        "lens": torch.from_numpy(lens).pin_memory(),
        "table": torch.from_numpy(table).pin_memory(),
    }
    dev = {name: t.to(device) for name, t in host.items()}
    kv_bytes = workloads.decode_kv_bytes(lens, 1, HK, D, 2)
    return {"pool": pool, "host": host, "dev": dev, "lens": lens, "table": table,
            "kv_bytes": kv_bytes, "pool_pages": pool_pages}


PF_BATCH, PF_HQ, PF_HK = 16, 32, 8
PF_D = int(os.environ.get("FW_PREFILL_HEAD_DIM", "128"))  # 256 for the head_dim 256 variant of the workload


def build_prefill_workload(seed, device):
    """Chunked prefill over a paged bf16 cache: 16 requests, cached prefix
    U[0,16384] in 64-token pages (random block table), new chunk U[512,2048]
    already written to the pool (seqused_k = prefix + chunk), 32 q heads, 8 kv
    heads, head_dim 128, causal, head-major q."""
    import torch
    from flywheel_tpu.testing import workloads
    rng = np.random.default_rng(1000 + seed)
    prefix = rng.integers(0, 16384 + 1, PF_BATCH).astype(np.int32)
    chunk = rng.integers(512, 2048 + 1, PF_BATCH).astype(np.int32)
    seqused = (prefix + chunk).astype(np.int32)
    table, pool_pages = workloads.paged_table(rng, seqused, 0, PAGE, slack=0.10)
    gen = torch.Generator(device=device)
    gen.manual_seed(1000 + seed)
    pool = torch.randn((pool_pages, PAGE, 2 * PF_HK, PF_D), generator=gen, device=device,
                       dtype=torch.float32).to(torch.bfloat16)
    # FW_PREFILL_POOL=e4m3 re-types the pool for the fp8 variant of the workload
    # (same shapes; per-tensor descale 5.5 / 448).
    descale = None
    if os.environ.get("FW_PREFILL_POOL", "bf16") == "e4m3":
        pool = (pool.float() * (448.0 / 5.5)).clamp(-448, 448).to(torch.float8_e4m3fn)
        descale = torch.tensor([5.5 / 448.0], dtype=torch.float32, device=device)
    cu = np.concatenate(([0], np.cumsum(chunk))).astype(np.int32)
    total_q = int(cu[-1])
    q_host = torch.randn((PF_HQ, total_q, PF_D), dtype=torch.float32).to(torch.bfloat16).pin_memory()
    return {"pool": pool, "descale": descale, "q_host": q_host, "q": q_host.to(device), "cu": cu, "seqused": seqused,
            "table": table, "prefix": prefix, "chunk": chunk, "total_q": total_q,
            "flops": workloads.prefill_flops(prefix, chunk, PF_HQ, PF_D),
            "cu_dev": torch.from_numpy(cu).to(device), "seqused_dev": torch.from_numpy(seqused).to(device),
            "table_dev": torch.from_numpy(table).to(device)}


def make_prefill_call(work, device):
    import torch
    from flywheel_tpu.softmax_attention import _native
    out = torch.empty_like(work["q"])
    args = _native.FwPrefillArgs(
        q=work["q"].data_ptr(), out=out.data_ptr(), kv_cache=work["pool"].data_ptr(),
        cu_seqlens_q=work["cu_dev"].data_ptr(), seqused_k=work["seqused_dev"].data_ptr(),
        block_table=work["table_dev"].data_ptr(), num_pages=work["pool"].shape[0], page_size=PAGE,
        pages_per_seq=work["table_dev"].shape[1], batch=PF_BATCH, total_q=work["total_q"],
        max_seqlen_q=int(work["chunk"].max()), nheads=PF_HQ, nheads_k=PF_HK, head_dim=PF_D,
        kv_dtype=0 if work["descale"] is None else 1,
        causal=1, window_left=-1, softmax_scale=PF_D ** -0.5, softcap=0.0, token_major=0)
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


def bench_prefill(ns, device, rank, world, barrier):
    """Times the chunked-prefill workload; returns the per-rank numbers."""
    import torch
    from flywheel_tpu import flash_attn_varlen_func
    from flywheel_tpu.softmax_attention import _native
    work = build_prefill_workload(rank, device)
    call, out, scratch = make_prefill_call(work, device)
    steps = max(5, min(ns.steps, 30))
    for _ in range(ns.warmup):
        call()
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        call()
    end.record()
    barrier()
    ms = start.elapsed_time(end) / steps
    status_words = scratch[:16].view(torch.int32).cpu().tolist()
    status = _native.read_status(scratch, device)
    if status != 0:
        raise RuntimeError(f"prefill kernel reported device status {status} (words {status_words})")
    e2e_ms = None
    if not ns.skip_e2e:
        def e2e_step():
            result = flash_attn_varlen_func(
                work["q_host"], work["pool"], None, work["cu"], None, int(work["chunk"].max()),
                int(work["seqused"].max()), causal=True, block_table=work["table"],
                seqused_k=work["seqused"])
            return result          # a host tensor: the API copied it back

        for _ in range(2):
            e2e_step()
        barrier()
        start.record()
        for _ in range(5):
            e2e_step()
        end.record()
        barrier()
        e2e_ms = start.elapsed_time(end) / 5
    check = None
    if rank == 0 and not ns.skip_cpu_baseline:
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
        flops_r = 4 * int(work["chunk"][r]) * (int(work["prefix"][r]) + (int(work["chunk"][r]) + 1) / 2) * PF_HQ * PF_D
        check = {"max_abs_err_vs_cpu": float(np.abs(got - want).max()),
                 "cpu_tflops": flops_r / cpu_s / 1e12, "cpu_sample": f"request {r} of {PF_BATCH}, {cpu_s:.2f} s"}
    return {"ms": ms, "flops": work["flops"], "e2e_ms": e2e_ms, "total_q": work["total_q"],
            "h2d": work["q_host"].numel() * 2, "check": check}


def bench_long_context(ns, device, rank, world, barrier):
    """Single-request long-context decode: one 128K-token paged bf16 cache (page
    64, random block table), 64 q heads, 8 kv heads, 256 decode steps with the
    fused append, the pages split evenly over the ranks; per step every rank
    decodes its pages, then the (o, lse) states are exchanged and merged:
    FLYWHEEL_EXCHANGE=p2p (default; peer stores over NVLink + flags, fused with
    the merge) or nccl (all-gather + merge)."""
    import torch
    import torch.distributed as dist
    from flywheel_tpu.softmax_attention import distributed as d
    context, steps = 131072, 256
    total_pages = (context + steps) // PAGE + 1
    first, last = d.page_range(total_pages, world, rank)
    local_pages = last - first
    rng = np.random.default_rng(2000 + rank)
    perm = rng.permutation(local_pages + 4)[:local_pages].astype(np.int32)
    gen = torch.Generator(device=device)
    gen.manual_seed(2000 + rank)
    pool = torch.randn((local_pages + 4, PAGE, 2 * HK, D), generator=gen, device=device,
                       dtype=torch.float32).to(torch.bfloat16)
    table = torch.from_numpy(perm[None]).to(device)
    if world == 1 and not dist.is_initialized():
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29555", rank=0, world_size=1,
                                device_id=device)
    exchange = os.environ.get("FLYWHEEL_EXCHANGE", "p2p")
    decoder = d.ShardedDecoder(pool=pool, table=table, total_pages=total_pages, nheads=HQ, nheads_k=HK,
                               exchange=exchange)
    q = torch.randn((1, 1, HQ, D), device=device).to(torch.bfloat16)
    k = torch.randn((1, 1, HK, D), device=device).to(torch.bfloat16)
    v = torch.randn((1, 1, HK, D), device=device).to(torch.bfloat16)
    graph = decoder.capture(q, k, v, context, steps + 8)
    for step in range(8):
        graph.replay()
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for step in range(steps):
        graph.replay()
    end.record()
    barrier()
    ms = torch.tensor([start.elapsed_time(end) / steps], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    kv_bytes = sum((context + step + 1) * 2 * HK * D * 2 for step in range(steps)) / steps
    if _native_status(decoder, device) != 0:
        raise RuntimeError("a kernel of the long-context step reported a device status")
    decoder.close()
    how = ("peer stores of (o, lse) over NVLink + flags, fused with the merge" if exchange == "p2p"
           else "NCCL all-gather of (o, lse) + merge")
    return {"metric": "long_context_decode_kv_read_bandwidth", "value": kv_bytes / (float(ms) * 1e-3) / 1e9,
            "unit": "GB/s", "ms_per_step": float(ms), "n_gpus": world, "steps": steps, "scaling": "strong",
            "config": {"workload": "1 request, 128K-token paged bf16 cache, page 64, 64 q heads, 8 kv heads, "
                                   "256 decode steps with fused append, pages split evenly over the GPUs, "
                                   + how + " per step", "exchange": exchange},
            "per_step": "decode kernel + combine + exchange + merge, replayed as one CUDA graph"}


def _native_status(decoder, device):
    from flywheel_tpu.softmax_attention import _native
    return _native.read_status(decoder.scratch, device)


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
}


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
    _, tensor_peak, kind = measured_peaks()
    tflops = flops / (ms * 1e-3) / 1e12
    return {"metric": "dense_causal_prefill_tflops", "config": {"workload": name, **spec, "head_dim": D,
            "l2": "inputs exceed L2" if 3 * q.numel() * 2 > (126 << 20) else "inputs fit L2 (compute-bound)"},
            "value": tflops, "unit": "TFLOP/s", "ms_per_step": ms, "steps": steps,
            "algorithmic_flops_per_launch": flops,
            "roofline": {"bound": "tensor", "achieved": tflops, "peak": tensor_peak,
                         "frac": tflops / tensor_peak if tensor_peak else None, "peak_kind": f"of {kind}"}}


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
    _, tensor_peak, kind = measured_peaks()
    tflops = flops / (ms * 1e-3) / 1e12
    return {"metric": "serving_chunked_prefill_tflops", "config": {"workload": name, "nheads": hq, "nheads_k": hk,
            "head_dim": d, "page_size": page, "sequence": total, "chunk": chunk,
            "calls": "16 x flash_attn_with_kvcache (ragged append + chunked prefill)"},
            "value": tflops, "unit": "TFLOP/s", "ms_per_sequence": ms, "steps": steps,
            "algorithmic_flops_per_sequence": flops,
            "roofline": {"bound": "tensor", "achieved": tflops, "peak": tensor_peak,
                         "frac": tflops / tensor_peak if tensor_peak else None, "peak_kind": f"of {kind}"}}


SERVING_PREFILL = {"serve-d256-prefill-gqa": dict(hk=4), "serve-d256-prefill-mha": dict(hk=32)}


def bench_config(ns, name, device):
    """Secondary decode configurations (one JSON line each, device-resident):
    c1 = contiguous bf16 GQA decode (batch 8, 32:8 heads, capacity 2048, lengths
    U[128,2047], fused append); c3 = paged fp8 e4m3 decode with per-tensor
    descales, sliding window 4096, softcap 50, sinks, 4-token verify window."""
    import torch
    from flywheel_tpu.softmax_attention import _native
    from flywheel_tpu.testing import workloads
    rng = np.random.default_rng(0)
    lib = _native.library()
    if name == "c1":
        batch, hq, hk, cap, q_len = 8, 32, 8, 2048, 1
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
    else:
        batch, hq, hk, q_len, window = 128, 64, 8, 4, 4095
        # experiment knobs for profiling sessions; the defaults are the configuration
        q_len = int(os.environ.get("FW_C3_QLEN", q_len))
        window = int(os.environ.get("FW_C3_WINDOW", window))
        softcap_value = float(os.environ.get("FW_C3_SOFTCAP", 50.0))
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
            softmax_scale=D ** -0.5, softcap=softcap_value)
        kv_bytes = workloads.decode_kv_bytes(lens, q_len, hk, D, 1, window_left=window if window >= 0 else None)
        keep = (pool, descale, q, k, v, sinks, lens_t, table_t, out)
    nbytes = lib.fw_decode_workspace_bytes(ctypes.byref(args))
    if nbytes == 0:
        raise RuntimeError(_native.last_error())
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device=device)
    args.workspace, args.workspace_bytes = scratch.data_ptr(), nbytes
    stream = torch.cuda.current_stream(device).cuda_stream
    # c1 moves 36 MB per step: rotate nothing, but flush L2 between steps so the
    # caches are read from HBM like in serving.
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device) if kv_bytes < (512 << 20) else None
    steps = max(ns.steps, 20)
    times = []
    for i in range(ns.warmup + steps):
        if flush is not None:
            flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        _native.check(lib.fw_decode_kvcache(ctypes.byref(args), stream))
        end.record()
        torch.cuda.synchronize()
        if i >= ns.warmup:
            times.append(start.elapsed_time(end))
    if _native.read_status(scratch, device) != 0:
        raise RuntimeError("decode kernel reported a device status")
    ms = float(np.median(times))
    hbm_peak, _, kind = measured_peaks()
    del keep
    return {"metric": "decode_kv_read_bandwidth", "config": {"workload": name,
            "l2": "L2 flushed between steps" if flush is not None else "inputs exceed L2"},
            "value": kv_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms, "steps": steps,
            "algorithmic_bytes_per_launch": kv_bytes,
            "roofline": {"bound": "hbm", "achieved": kv_bytes / (ms * 1e-3) / 1e9, "peak": hbm_peak,
                         "frac": kv_bytes / (ms * 1e-3) / 1e9 / hbm_peak, "peak_kind": f"of {kind}"}}


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
        batch=BATCH, seqlen_q=1, nheads=HQ, nheads_k=HK, head_dim=D, kv_dtype=0, causal=1,
        window_left=-1, softmax_scale=D ** -0.5, softcap=0.0, num_ctas=0)
    lib = _native.library()
    nbytes = lib.fw_decode_workspace_bytes(ctypes.byref(args))
    if nbytes == 0:
        raise RuntimeError(_native.last_error())
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device=device)
    args.workspace, args.workspace_bytes = scratch.data_ptr(), nbytes
    stream = torch.cuda.current_stream(device).cuda_stream

    def call():
        _native.check(lib.fw_decode_kvcache(ctypes.byref(args), stream))

    return call, out, scratch


def cpu_baseline(work, repeats=3):
    """Times the C/OpenMP restatement of the reference's test oracle
    (oracle/paged_decode_ref.c) on the whole decode batch, on all host cores."""
    from flywheel_tpu.softmax_attention import _arrays
    from oracle import c_port
    lens, table = work["lens"], work["table"]
    pool = _arrays.to_host_numpy(work["pool"])
    host = work["host"]
    q, k, v = (_arrays.to_host_numpy(host[name]) for name in ("q", "k", "v"))
    c_port.paged_decode(q[:2], pool, k[:2], v[:2], lens[:2], table[:2], nheads_k=HK, in_place=True)  # page in
    times = []
    for _ in range(repeats):
        start = time.perf_counter()
        out, _, _ = c_port.paged_decode(q, pool, k, v, lens, table, nheads_k=HK, causal=True, in_place=True)
        times.append(time.perf_counter() - start)
    seconds = float(np.median(times))
    nbytes = work["kv_bytes"]
    return {"value": nbytes / seconds / 1e9, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"all {len(lens)} requests ({nbytes / 1e9:.2f} GB of KV), median of {repeats} passes of "
                      f"{seconds:.2f} s, C + OpenMP restatement of the reference's test oracle"}, out, len(lens)


def run_reference_arm(ns):
    """The reference's CPU path stands in as the C + OpenMP restatement of its
    own test oracle (the reference itself needs JAX, absent from this image),
    on all host cores; a step is the first 32 requests of the decode batch."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import ml_dtypes
    from flywheel_tpu.testing import workloads
    from oracle import c_port
    bf16 = np.dtype(ml_dtypes.bfloat16)
    rng = np.random.default_rng(0)
    lens = rng.integers(LEN_LO, LEN_HI + 1, BATCH).astype(np.int32)
    sample = min(32, BATCH)
    table, pool_pages = workloads.paged_table(rng, lens[:sample], 1, PAGE, slack=0.10)
    draw = lambda shape: rng.standard_normal(shape, dtype=np.float32).astype(bf16)
    # values do not change the timing: one random block of pages, repeated
    block = draw((256, PAGE, 2 * HK, D))
    pool = np.ascontiguousarray(np.tile(block, (-(-pool_pages // 256), 1, 1, 1))[:pool_pages])
    q, k, v = draw((sample, 1, HQ, D)), draw((sample, 1, HK, D)), draw((sample, 1, HK, D))
    nbytes = workloads.decode_kv_bytes(lens[:sample], 1, HK, D, 2)
    times = []
    for step in range(ns.warmup + ns.steps):
        start = time.perf_counter()
        c_port.paged_decode(q, pool, k, v, lens[:sample], table, nheads_k=HK, causal=True, in_place=True)
        if step >= ns.warmup:
            times.append(time.perf_counter() - start)
    ms = 1e3 * float(np.mean(times))
    value = nbytes / (ms * 1e-3) / 1e9
    sample_text = (f"first {sample} of {BATCH} requests per step ({nbytes / 1e9:.2f} GB of KV); C + OpenMP "
                   "restatement of the reference's test oracle on all host cores")
    print(json.dumps({
        "impl": "reference", "metric": "paged_decode_kv_read_bandwidth", "value": value, "unit": "GB/s",
        "n_gpus": ns.gpus, "steps": ns.steps, "warmup": ns.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
                         "sample": sample_text},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config():
    return {"workload": "paged bf16 GQA decode, batch 128, 64 q heads, 8 kv heads, head_dim 128, "
                        "page 64, cached lengths U[1024,32768], pool = pages in use + 10%, random block "
                        "table, fused one-token append, causal",
            "l2": "inputs (about 9 GB of KV per step) far exceed the 126 MB L2",
            "sharding": "one independent copy of the workload per GPU (request sharding, no collective)"}


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--skip-cpu-baseline", action="store_true")
    parser.add_argument("--skip-e2e", action="store_true")
    parser.add_argument("--skip-prefill", action="store_true")
    parser.add_argument("--config", choices=["c1", "c3", *SECONDARY_SHAPES, *DENSE_SHAPES, *SERVING_PREFILL], default=None,
                        help="run one secondary decode configuration instead of the headline")
    parser.add_argument("--long-context", action="store_true",
                        help="run the single-request 128K-token decode split over the GPUs")
    parser.add_argument("--prefill-only", action="store_true",
                        help="run only the chunked-prefill workload (profiler captures)")
    parser.add_argument("--batch", type=int, default=128,
                        help="requests per step; smaller than 128 only for profiler captures")
    ns = parser.parse_args()
    globals()["BATCH"] = ns.batch
    ns.warmup = max(ns.warmup, 3) if ns.impl == "ours" else ns.warmup
    if ns.impl == "reference":
        run_reference_arm(ns)
        return

    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path.")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if ns.config in DENSE_SHAPES:
        print(json.dumps(bench_dense(ns, ns.config, device)))
        return
    if ns.config in SERVING_PREFILL:
        print(json.dumps(bench_serving_prefill(ns, ns.config, device)))
        return
    if ns.config:
        print(json.dumps(bench_config(ns, ns.config, device)))
        return
    if ns.long_context:
        result = bench_long_context(ns, device, rank, world, barrier)
        if rank == 0:
            print(json.dumps(result))
        if dist.is_initialized():
            dist.destroy_process_group()
        return
    if ns.prefill_only:
        pf = bench_prefill(ns, device, rank, world, barrier)
        ms = torch.tensor([pf["ms"]], dtype=torch.float64, device=device)
        flops = torch.tensor([float(pf["flops"])], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.all_reduce(flops, op=dist.ReduceOp.SUM)
        if rank == 0:
            print(json.dumps({"metric": "chunked_prefill_tflops", "value": float(flops) / (float(ms) * 1e-3) / 1e12,
                              "unit": "TFLOP/s", "ms_per_step": float(ms), "n_gpus": world}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    from flywheel_tpu import flash_attn_with_kvcache
    work = build_workload(seed=rank, device=device)
    call, out, scratch = make_decode_call(work, device)

    # ---- device-resident arm
    for _ in range(ns.warmup):
        call()
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(ns.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(ns.steps)]
    whole_start, whole_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    whole_start.record()
    for i in range(ns.steps):
        starts[i].record()
        call()
        ends[i].record()
    whole_end.record()
    barrier()
    clocks = sampler.summary()
    total_ms = whole_start.elapsed_time(whole_end)
    launch_ms = float(np.mean([s.elapsed_time(e) for s, e in zip(starts, ends)]))
    from flywheel_tpu.softmax_attention import _native
    status = _native.read_status(scratch, device)
    if status != 0:
        raise RuntimeError(f"decode kernel reported device status {status}")

    # ---- end-to-end arm: host inputs in, host output back, every step
    host = work["host"]

    def e2e_step():
        result, _ = flash_attn_with_kvcache(
            host["q"], work["pool"], None, host["k"], host["v"], cache_seqlens=host["lens"],
            block_table=host["table"], causal=True)
        return result               # a host tensor: the API copied it device -> host and synchronised

    e2e_start, e2e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if ns.skip_e2e:
        e2e_start.record()
        e2e_end.record()
        barrier()
        e2e_ms = 0.0
    else:
        for _ in range(ns.warmup):
            e2e_step()
        barrier()
        e2e_start.record()
        for _ in range(ns.steps):
            e2e_step()
        e2e_end.record()
        barrier()
        e2e_ms = e2e_start.elapsed_time(e2e_end)
    h2d = sum(host[name].numel() * host[name].element_size() for name in ("q", "k", "v", "lens", "table"))
    d2h = host["q"].numel() * host["q"].element_size()

    times = torch.tensor([total_ms, e2e_ms, launch_ms], dtype=torch.float64, device=device)
    nbytes = torch.tensor([float(work["kv_bytes"])], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(nbytes, op=dist.ReduceOp.SUM)
    total_ms, e2e_ms, launch_ms = (float(x) for x in times.tolist())
    job_bytes = float(nbytes.item())

    prefill = None if ns.skip_prefill else bench_prefill(ns, device, rank, world, barrier)
    if prefill is not None:
        pf = torch.tensor([prefill["ms"], prefill["e2e_ms"] or 0.0], dtype=torch.float64, device=device)
        pf_flops = torch.tensor([float(prefill["flops"])], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(pf, op=dist.ReduceOp.MAX)
            dist.all_reduce(pf_flops, op=dist.ReduceOp.SUM)
        prefill["ms"], prefill["e2e_ms"] = float(pf[0]), float(pf[1]) or None
        prefill["job_flops"] = float(pf_flops.item())

    if rank == 0:
        hbm_peak, _, peak_kind = measured_peaks()
        value = job_bytes * ns.steps / (total_ms * 1e-3) / 1e9
        achieved = work["kv_bytes"] / (launch_ms * 1e-3) / 1e9
        line = {
            "metric": "paged_decode_kv_read_bandwidth", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": ns.steps, "warmup": ns.warmup, "ms_per_step": total_ms / ns.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(), "per_gpu": value / world,
            "clocks": clocks, "gpu_launches": 2 * ns.steps,
            "e2e": {"value": job_bytes * ns.steps / (e2e_ms * 1e-3) / 1e9 if e2e_ms > 0 else None, "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / ns.steps},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak,
                         # dram read+write per launch, scaled from the small-case ncu capture in
                         # profiles/decode_bf16_paged_c2.md (reads 1.0011 x algorithmic, writes =
                         # the per-CTA partial states)
                         "traffic": work["kv_bytes"] * 1.0011 + (BATCH + 148) * HQ * (D + 2) * 4, "peak_kind": f"of {peak_kind}",
                         "kernel": "fw::decode_kernel<bf16> (+ combine_kernel, <1% of the launch pair)",
                         "algorithmic_bytes_per_launch": work["kv_bytes"],
                         "frac_of_nominal_8TBs": achieved / 8000.0},
        }
        if prefill is not None:
            _, tf_peak, _ = measured_peaks()
            tflops = prefill["job_flops"] / (prefill["ms"] * 1e-3) / 1e12
            per_gpu = tflops / world
            line["prefill"] = {
                "metric": "chunked_prefill_tflops", "value": tflops, "unit": "TFLOP/s", "per_gpu": per_gpu,
                "ms_per_step": prefill["ms"],
                "config": {"workload": "chunked prefill over a paged bf16 cache, 16 requests, prefix U[0,16384], "
                                       "chunk U[512,2048], 32 q heads, 8 kv heads, head_dim 128, page 64, "
                                       "causal, head-major q", "total_q": prefill["total_q"]},
                "e2e": {"value": prefill["job_flops"] / (prefill["e2e_ms"] * 1e-3) / 1e12 if prefill["e2e_ms"]
                        else None, "unit": "TFLOP/s", "h2d_bytes_per_step": prefill["h2d"],
                        "d2h_bytes_per_step": prefill["h2d"], "ms_per_step": prefill["e2e_ms"]},
                "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": tf_peak, "unit": "TFLOP/s",
                             "frac": per_gpu / tf_peak, "peak_kind": f"of {peak_kind} (bf16 burst)",
                             "frac_of_nominal_2250": per_gpu / 2250.0,
                             "algorithmic_flops_per_launch": prefill["flops"]},
                "check": prefill["check"],
            }
        if world == 1 and not ns.skip_cpu_baseline:
            base, cpu_out, count = cpu_baseline(work)
            line["cpu_baseline"] = base
            got = out[:count].float().cpu().numpy()
            line["sample_max_abs_err_vs_cpu"] = float(np.abs(got - cpu_out).max())
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
