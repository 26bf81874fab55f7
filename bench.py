#!/usr/bin/env python
"""Benchmark of the paged GQA split-KV decode attention path.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload c2|c3|c1|c4|c5p]

One step = one attention call (the split-KV map kernel and the LSE reduce kernel) over one batch of synthetic
paged decode requests.
Default workload: batch 64, q_len 1, Hq 64 / Hkv 8 / head_dim 128, bf16, context lengths uniform in
[1024, 8192] (seed 1), 16-token pages in a 40,000-page pool with random block tables, split-KV partitions
of 512 tokens. Metric: KV-read GB/s = algorithmic KV bytes (every visible K and V row once) / time.
With N > 1 every rank runs its own batch of independent requests (no collective on the data path; weak
scaling) and the value is the sum of all ranks' KV bytes over the slowest rank's time.
The line also carries ``parity`` (the bench's own output against the CPU oracle on the same stored inputs) and,
for the default workload, ``split_kv``: one long sequence of 131,072 / 524,288 / 1,048,576 tokens whose pages are
split over the same N ranks (local map, one NCCL all-gather of a 16.5 KB record per rank, LSE merge), with the
step, the local kernels, the exchange and the efficiency against one GPU.
Other workloads are exploration cases: c3 speculative verify, c1 the small fp16 case, c4 one long sequence
whose pages are split over the ranks (one all-gather per step; strong scaling), c5p chunked prefill (TFLOP/s).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (batch, q_len, Hq, Hkv, D, dtype, context range, seed, partition)
    "c2": dict(batch=64, q_len=1, hq=64, hkv=8, d=128, dtype="bf16", lo=1024, hi=8192, seed=1, partition=512,
               pool_pages=40000, label="paged decode B64 Hq64/Hkv8/D128 bf16 ctx U[1024,8192] P16 part512"),
    "c3": dict(batch=32, q_len=4, hq=24, hkv=4, d=256, dtype="bf16", lo=4096, hi=32768, seed=2, partition=0,
               pool_pages=0, label="verify B32 q4 Hq24/Hkv4/D256 bf16 prefix U[4096,32768] P16"),
    "c4": dict(batch=1, q_len=1, hq=16, hkv=2, d=256, dtype="bf16", lo=0, hi=0, seed=3, partition=0, pool_pages=0,
               contexts=[1048576], label="one sequence, decode, Hq16/Hkv2/D256 bf16 P16, pages split in token order"),
    # prefill half of configuration 5: eight causal 2,048-token chunks appended to prefixes U[0, 30720]
    "c5p": dict(batch=8, q_len=2048, hq=64, hkv=8, d=128, dtype="bf16", lo=2048, hi=32768, seed=4, partition=0,
                pool_pages=0, label="chunked prefill B8 chunk 2048 Hq64/Hkv8/D128 bf16 prefix U[0,30720] P16"),
    # configuration 5: eight causal 2,048-token prefill chunks on prefixes U[0, 30720] plus 56 decode requests with
    # contexts U[1024, 8192], one call
    "c5": dict(batch=64, q_len=0, hq=64, hkv=8, d=128, dtype="bf16", lo=0, hi=0, seed=4, partition=0, pool_pages=0,
               label="8 prefill chunks of 2048 on prefixes U[0,30720] + 56 decode ctx U[1024,8192], one call, "
                     "Hq64/Hkv8/D128 bf16 P16"),
    "c1": dict(batch=4, q_len=1, hq=16, hkv=2, d=256, dtype="f16", lo=0, hi=0, seed=0, partition=0, pool_pages=0,
               contexts=[128, 517, 1024, 2048], label="decode B4 Hq16/Hkv2/D256 fp16 ctx {128,517,1024,2048} P16"),
}
PAGE = 16
SPLIT_CONTEXTS = (131072, 524288, 1048576)  # one long sequence split over the ranks (configuration 4)


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# dram__bytes_read.sum + dram__bytes_write.sum of one map-kernel launch over its algorithmic K/V bytes, from
# profiler captures of the decode workload at a reduced batch (315.70 MB moved for 309.67 MB of 16-bit pages;
# 307.75 MB for 301.35 MB of FP8 pages); traffic grows with the tokens processed, so the ratio carries to the
# full batch.
MAP_TRAFFIC_PER_KV_BYTE = 315.70 / 309.67
MAP_TRAFFIC_PER_FP8_KV_BYTE = 307.75 / 301.35


def map_kernel_name(spec):
    """Which kernel the library picks for the workload's map tasks (rows per task = Q tokens x heads per group):
    the token-major kernel for FP8 pages and for 17-32-row tasks, the row-major warp-level kernel otherwise."""
    rows = spec.get("q_len", 1) * (spec["hq"] // spec["hkv"])
    widest = 32 if spec["d"] == 128 else 24
    if spec.get("kv_elem", 2) == 1 and rows <= widest:
        return "sdpa_tm_kernel"
    if 16 < rows <= widest:
        return "sdpa_tm_kernel"
    return "sdpa_map_kernel"


def traffic_estimate(spec, kv_bytes):
    """Bytes one map-kernel launch moves to and from DRAM, scaled from the profiler captures; only for the decode
    workload that was captured (None elsewhere)."""
    if spec.get("q_len") == 1 and spec["d"] == 128 and spec["hkv"] == 8 and spec.get("partition") == 512:
        ratio = MAP_TRAFFIC_PER_KV_BYTE if spec.get("kv_elem", 2) == 2 else MAP_TRAFFIC_PER_FP8_KV_BYTE
        return int(kv_bytes * ratio)
    return None


def attention_flops(spec, contexts):
    """4 * Hq * D flops per (query token, visible KV token) pair of one rank's batch (QK^T and PV)."""
    q = spec["q_len"]
    pairs = sum(q * (c - q) + q * (q + 1) // 2 for c in contexts)
    return 4.0 * spec["hq"] * spec["d"] * pairs


def contexts_for(spec, rank, world=1):
    """Context lengths of the requests rank ``rank`` of ``world`` owns. One GPU: the workload's batch. Several: the
    job's requests (``batch`` per GPU, every GPU's share drawn with its own seed) are binned over the ranks
    longest-first by context length (`split_kv.assign_requests`), so that every rank streams about the same bytes;
    no rank needs another rank's data, there is no collective on the data path."""
    if "contexts" in spec:
        return list(spec["contexts"])

    def draw(r):
        rng = np.random.default_rng(spec["seed"] + 1000 * r)
        return rng.integers(spec["lo"], spec["hi"] + 1, size=spec["batch"]).tolist()

    if world <= 1:
        return draw(rank)
    from khalamari_b200.split_kv import assign_requests
    job = [ctx for r in range(world) for ctx in draw(r)]
    return [job[i] for i in assign_requests(job, world)[rank]]


def workload_config(spec, contexts, world):
    """The ``config`` object of the JSON line: the same for this library's arm and the reference arm."""
    kv_bytes = sum(contexts) * 2 * spec["hkv"] * spec["d"] * spec.get("kv_elem", 2)
    return {"workload": spec["label"], "batch_per_gpu": len(contexts), "q_len": spec["q_len"],
            "kv_tokens_per_gpu": int(sum(contexts)),
            "l2": "inputs (KV pages read per step) larger than L2; no flush" if kv_bytes > 126e6
            else "KV pages read per step fit L2: not an HBM measurement",
            "parallelism": f"dp{world} by request"}


class ClockSampler:
    """Samples SM clocks and clock-event (throttle) reasons of one GPU through NVML while the bench runs.
    Reading only; nothing is set. Falls back to nvidia-smi when the NVML binding is missing."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, uuid: str | None, index: int):
        self.uuid = uuid
        self.index = index
        self.samples = []  # (time, sm_mhz, reasons bitmask)
        self.max_mhz = None
        self.stop = threading.Event()
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            if uuid:
                try:
                    self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
                except Exception:
                    self.handle = None
            if self.handle is None:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nvml = None

    def _sample(self):
        now = time.perf_counter()
        if self.nvml is not None:
            try:
                mhz = int(self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM))
                try:
                    mask = int(self.nvml.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    mask = int(self.nvml.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((now, mhz, mask))
            except Exception:
                pass
            return
        try:
            out = subprocess.run(
                ["nvidia-smi", f"--id={self.index}",
                 "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
                 "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                 "clocks_event_reasons.sw_power_cap", "--format=csv,noheader,nounits"],
                capture_output=True, text=True, timeout=10).stdout
            parts = [p.strip() for p in out.strip().split(",")]
            if len(parts) >= 6:
                mask = 0
                for bit, text in zip((0x8, 0x40, 0x20, 0x4), parts[2:6]):
                    if text.lower().startswith("active"):
                        mask |= bit
                self.max_mhz = int(float(parts[1]))
                self.samples.append((now, int(float(parts[0])), mask))
        except Exception:
            pass

    def _run(self):
        while not self.stop.is_set():
            self._sample()
            self.stop.wait(0.01 if self.nvml is not None else 0.2)

    def __enter__(self):
        self.thread.start()
        return self

    def __exit__(self, *exc):
        self.stop.set()
        self.thread.join(timeout=15)

    def summary(self, begin: float, end: float):
        """Median SM clock and the reasons seen between two perf_counter() stamps (the timed region); when
        that window is shorter than three samples, the window is widened to all samples taken under load."""
        window = [s for s in self.samples if begin <= s[0] <= end]
        label = "timed region"
        if len(window) < 3:
            window = self.samples
            label = "ramp + timed region + end-to-end loop"
        if not window:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unsampled"]}
        mhz = sorted(s[1] for s in window)
        mask = 0
        for s in window:
            mask |= s[2]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz,
                "reasons": [name for bit, name in self.REASONS.items() if mask & bit], "samples": len(window),
                "window": label}


def build_device_case(device, spec, contexts, torch, seed):
    """Synthetic inputs created on the device: N(0,1) Q/K/V in the storage dtype, a shared page pool and
    per-request block tables that are random permutations of pool pages. Only pages a request owns are
    filled; the rest of the pool keeps its allocation bytes."""
    from khalamari_b200.device import Buffer
    dt = torch.bfloat16 if spec["dtype"] == "bf16" else torch.float16
    hq, hkv, d = spec["hq"], spec["hkv"], spec["d"]
    page_elems = 2 * hkv * PAGE * d
    pages_per_req = [-(-c // PAGE) for c in contexts]
    pool_pages = spec["pool_pages"] or (sum(pages_per_req) + 16)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    fp8 = spec.get("kv_elem", 2) == 1  # pages of FP8 E4M3FN codes (the reference's cache format)
    pool = torch.empty(pool_pages * page_elems, dtype=torch.uint8 if fp8 else dt, device="cuda")
    chunk = 1 << 26
    for begin in range(0, pool.numel(), chunk):
        end = min(begin + chunk, pool.numel())
        values = torch.randn(end - begin, generator=gen, device="cuda", dtype=torch.float32)
        pool[begin:end] = values.to(torch.float8_e4m3fn).view(torch.uint8) if fp8 else values.to(dt)
    num_blocks = max(pages_per_req)
    rng = np.random.default_rng(seed)
    perm = rng.permutation(pool_pages).astype(np.uint32)
    table = np.zeros((len(contexts), num_blocks), dtype=np.uint32)
    cursor = 0
    for r, n in enumerate(pages_per_req):
        table[r, :n] = perm[cursor:cursor + n]
        cursor += n
    q_lens = spec.get("q_lens") or [spec["q_len"]] * len(contexts)
    total_q = sum(q_lens)
    q = torch.randn(total_q * hq * d, generator=gen, device="cuda", dtype=torch.float32).to(dt)
    out = torch.zeros_like(q)
    wrap = lambda t: Buffer.wrap(device, t.data_ptr(), t.numel() * t.element_size())
    return dict(pool=pool, q=q, out=out, table=table, d_pool=wrap(pool), d_q=wrap(q), d_out=wrap(out),
                d_table=Buffer.from_slice(device, table.reshape(-1)), num_blocks=num_blocks)


# ---- parity of the bench's own output against the CPU oracle (rank 0, outside every timed region) ----------
def _storage_to_f32(bits_u8, spec, fp8):
    import oracle
    if fp8:
        lut = oracle.bf16_bits_to_f32(oracle.fp8_to_bf16_bits(np.arange(256, dtype=np.uint8)))
        return lut[bits_u8]
    bits = np.ascontiguousarray(bits_u8).view(np.uint16)
    if spec["dtype"] == "bf16":
        return oracle.bf16_bits_to_f32(bits)
    return bits.view(np.float16).astype(np.float32)


def oracle_parity(spec, contexts, q_lens, case, out_f32, sample_tokens=None):
    """Copies the device-resident Q, page pool and block tables back, gathers every request's K/V rows through the
    oracle's paged gather (the reference's address function), runs the CPU oracle on those values and compares the
    output the bench produced. ``sample_tokens``: per request, the new-token indices to check (None: all of them).
    Returns the ``parity`` object of the JSON line and the seconds the oracle pass took."""
    import torch

    import oracle
    hq, hkv, d = spec["hq"], spec["hkv"], spec["d"]
    fp8 = spec.get("kv_elem", 2) == 1
    elem = 1 if fp8 else 2
    pool = case["pool"].view(torch.uint8).cpu().numpy()
    q_all = _storage_to_f32(case["q"].view(torch.uint8).cpu().numpy(), spec, False).reshape(-1, hq, d)
    layout = oracle.PageTableLayout(len(contexts), 1, case["num_blocks"], 1)
    table = case["table"].reshape(-1)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int64)
    q_rows, ks, vs, histories, flat = [], [], [], [], []
    for r, ctx in enumerate(contexts):
        tokens = range(q_lens[r]) if sample_tokens is None else sample_tokens[r]
        if not len(tokens):
            continue
        k_u8, v_u8 = oracle.gather_paged(pool, table, layout, r, 0, PAGE, hkv, d, elem, ctx)
        k = _storage_to_f32(k_u8, spec, fp8).reshape(ctx, hkv, d)
        v = _storage_to_f32(v_u8, spec, fp8).reshape(ctx, hkv, d)
        if sample_tokens is None:
            q_rows.append(q_all[cu[r]:cu[r + 1]])
            ks.append(k)
            vs.append(v)
            histories.append((ctx - q_lens[r], q_lens[r]))
            flat.extend(range(int(cu[r]), int(cu[r + 1])))
        else:
            for t in tokens:
                visible = ctx - q_lens[r] + t + 1
                q_rows.append(q_all[cu[r] + t:cu[r] + t + 1])
                ks.append(k[:visible])
                vs.append(v[:visible])
                histories.append((visible - 1, 1))
                flat.append(int(cu[r]) + t)
    cu_oracle = np.concatenate([[0], np.cumsum([n for _, n in histories])])
    scale = spec.get("scale") or 1.0 / float(np.sqrt(d))
    t0 = time.perf_counter()
    expected = oracle.projected_gqa(cu_oracle, [h for h, _ in histories], np.concatenate(q_rows), ks, vs, d, hq, hkv,
                                    scale, host_threads())
    seconds = time.perf_counter() - t0
    actual = out_f32.reshape(-1, hq, d)[flat]
    err = np.abs(actual - expected)
    ok = (err <= 2e-3) | (err <= 1e-2 * np.abs(expected))
    beyond = err > 2e-3
    return {"max_abs": float(err.max()), "max_rel": float((err / np.maximum(np.abs(expected), 1e-30))[beyond].max())
            if beyond.any() else 0.0, "rows_checked": int(len(flat) * hq), "rows_total": int(cu[-1] * hq),
            "rule": "per element |a-b| <= 2e-3 or |a-b| <= 1e-2*|b|, against the CPU oracle on the same stored "
                    "Q/K/V, gathered from the bench's own page pool",
            "pass": bool(ok.all()) and bool(np.isfinite(actual).all())}, seconds


def output_f32(tensor, spec, torch):
    return tensor.float().cpu().numpy()


def init_ranks(torch):
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def run_ours(args):
    import torch
    import torch.distributed as dist

    from khalamari_b200.device import Device, Dtype, PinnedArray, Stream
    from khalamari_b200.gqa import GQAAttention, GQACore, HostPipeline
    from khalamari_b200.request_page_table import GQAPageTableLayout
    from khalamari_b200.selector import SelectorPolicy

    rank, world, local = init_ranks(torch)
    spec = dict(WORKLOADS[args.workload])
    if args.batch:
        spec["batch"] = args.batch
        spec["label"] += f" [batch {args.batch}]"
    if args.pool_pages:
        spec["pool_pages"] = args.pool_pages
    if args.partition >= 0:
        spec["partition"] = args.partition
        spec["label"] += f" [partition {args.partition or 'selector'}]"
    if args.uniform_context:
        spec["contexts"] = [args.uniform_context] * spec["batch"]
        spec["label"] += f" [uniform context {args.uniform_context}]"
    if args.q_len:
        spec["q_len"] = args.q_len
        spec["label"] += f" [q_len {args.q_len}]"
    if args.kv_dtype == "fp8":
        spec["kv_elem"] = 1
        spec["label"] += " [K/V pages of FP8 E4M3FN]"
    kv_elem = spec.get("kv_elem", 2)
    contexts = contexts_for(spec, rank, world)
    q_len = spec["q_len"]
    q_lens = [q_len] * len(contexts)
    device = Device(local)
    case = build_device_case(device, spec, contexts, torch, spec["seed"] + 1000 * rank)
    torch_stream = torch.cuda.current_stream()
    stream = Stream(device, torch_stream.cuda_stream)
    io_dtype = Dtype.Bfloat16 if spec["dtype"] == "bf16" else Dtype.Float16
    layout = GQAPageTableLayout(len(contexts), 1, case["num_blocks"], 1)
    scale = spec.get("scale") or 1.0 / float(np.sqrt(spec["d"]))
    attention = GQAAttention(device, GQACore(spec["d"], spec["hq"], spec["hkv"], scale), io_dtype,
                             2 * spec["hkv"] * PAGE * spec["d"] * kv_elem, layout, len(contexts) * q_len,
                             SelectorPolicy.B200, kv_dtype=Dtype.Fp8E4M3FN if kv_elem == 1 else None)
    req_slots = list(range(len(contexts)))
    token_indices = [c - q_len for c in contexts]
    cu_tokens = [i * q_len for i in range(len(contexts) + 1)]
    selection = None
    if spec["partition"]:
        variant = next(v for v in attention.selector.variants() if v.kind == 0 and v.thread_block.max_q_tokens == 1)
        selection = attention.select_partitioned(variant, spec["partition"], False, token_indices, cu_tokens)
    attention.fused = args.fused
    attention.prepare(req_slots, token_indices, cu_tokens, selection=selection)
    shape = attention.metadata.replay_shape()
    kv_bytes = sum(contexts) * 2 * spec["hkv"] * spec["d"] * kv_elem  # q_len new tokens are already in the cache

    def step(after_map=None):
        return attention.record_sdpa(stream, case["d_q"], case["d_pool"], case["d_table"], case["d_out"], 0, after_map)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    device.check(stream)
    props = torch.cuda.get_device_properties(local)
    sampler = ClockSampler(str(getattr(props, "uuid", "")) or None, local)

    def barrier():
        if world > 1:
            dist.barrier()

    # per step: start, end of the map kernel, end of the step (after the reduce kernel)
    events = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    launches = 0
    sampler.__enter__()
    # untimed ramp: keep the GPU under this load for about half a second so that clocks settle and the
    # sampler sees them before the (short) timed region starts
    ramp_end = time.perf_counter() + args.ramp_ms * 1e-3
    while time.perf_counter() < ramp_end:
        for _ in range(20):
            step()
        torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(args.steps):
        events[i][0].record(torch_stream)
        launches += step()
        events[i][2].record(torch_stream)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    barrier()
    timed_window = (t0, t1)
    device.check(stream)
    step_ms = [events[i][0].elapsed_time(events[i][2]) for i in range(args.steps)]
    total_ms = events[0][0].elapsed_time(events[-1][2])
    ms_per_step = total_ms / args.steps
    if args.fused or attention.metadata.direct_output():
        map_ms = step_ms  # the step is one kernel launch
    else:
        # The map kernel's own duration: the same K steps once more, with an event between the two launches. (In the
        # steps above nothing sits between them, so the reducer's launch overlaps the map kernel's tail, as it does
        # for a caller; an event record there would undo that.)
        split_events = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(args.steps)]
        for i in range(args.steps):
            split_events[i][0].record(torch_stream)
            step(lambda i=i: split_events[i][1].record(torch_stream))
        torch.cuda.synchronize()
        map_ms = [split_events[i][0].elapsed_time(split_events[i][1]) for i in range(args.steps)]
    device_out = case["out"].clone()

    # ---- end to end through the component seam with host buffers -------------------------------------
    # Every step: Q from page-locked host memory to the device, the batch planned on the host (selector and
    # metadata: nothing precomputed), the metadata block to the device, map + reduce, the output back to host
    # memory. Two steps are in flight: a step's output copy runs beside the next step's kernels.
    elems = len(contexts) * q_len * spec["hq"] * spec["d"]
    q_host = PinnedArray(elems, np.uint16)
    out_hosts = [PinnedArray(elems, np.uint16) for _ in range(2)]
    q_host.array[:] = case["q"].view(torch.int16).cpu().numpy().view(np.uint16)
    pipeline = HostPipeline(attention, stream)
    partition = spec["partition"] or None

    def submit(i):
        return pipeline.submit(q_host, out_hosts[i % 2], case["d_pool"], case["d_table"], req_slots, token_indices,
                               cu_tokens, 0, partition)

    for i in range(4):
        submit(i)
    pipeline.drain()
    barrier()
    torch.cuda.synchronize()
    e2e_steps = args.steps
    h2d = d2h = 0
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        _, _, h2d, d2h = submit(i)
    pipeline.drain()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    # one step alone, nothing else in flight: the latency a single caller sees
    t0 = time.perf_counter()
    ticket = submit(e2e_steps)[0]
    pipeline.wait(ticket)
    e2e_latency_s = time.perf_counter() - t0
    last = out_hosts[e2e_steps % 2].array
    checksum = float(np.abs(last.view(np.int16).astype(np.float32)).sum())
    e2e_matches = bool(np.array_equal(last, device_out.view(torch.int16).cpu().numpy().view(np.uint16).reshape(-1)))
    device.check(stream)
    sampler.__exit__(None, None, None)
    clock_summary = sampler.summary(*timed_window)

    # ---- max over ranks ----------------------------------------------------------------------------
    stats = torch.tensor([ms_per_step, e2e_s * 1e3, float(np.mean(map_ms)), e2e_latency_s * 1e3], device="cuda",
                         dtype=torch.float64)
    totals = torch.tensor([float(kv_bytes), float(len(contexts) * q_len)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(totals, op=dist.ReduceOp.SUM)
    ms_per_step, e2e_ms, map_ms_mean, e2e_latency_ms = stats.tolist()
    total_kv_bytes, total_tokens = totals.tolist()

    result = None
    if rank == 0:
        peak, peak_kind = load_peaks()
        value = total_kv_bytes / (ms_per_step * 1e-3) / 1e9
        achieved = kv_bytes / (map_ms_mean * 1e-3) / 1e9  # rank 0's map kernel against one GPU's peak
        result = {
            "metric": "GQA decode KV-read GB/s", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if spec["dtype"] == "bf16" else "f16",
            "data": "synthetic",
            "config": workload_config(spec, contexts, world),
            "map_tasks": shape.num_sdpa_map_task_templates * spec["hkv"],
            "tokens_per_s": round(total_tokens / (ms_per_step * 1e-3), 1),
            "tflops": round(attention_flops(spec, contexts) / (ms_per_step * 1e-3) / 1e12, 2),
            "hbm_frac": round(value / world / peak, 4),
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "traffic": traffic_estimate(spec, kv_bytes), "peak_source": f"of {peak_kind}",
                         "kernel": map_kernel_name(spec), "kernel_ms": round(map_ms_mean, 5),
                         "kernel_ms_from": "a second pass of the same steps with an event between the map and the "
                                           "reduce launch"},
            "e2e": {"value": round(total_kv_bytes / (e2e_ms * 1e-3) / 1e9, 2), "unit": "GB/s",
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "ms_per_step": round(e2e_ms, 5),
                    "tokens_per_s": round(total_tokens / (e2e_ms * 1e-3), 1),
                    "steps_in_flight": HostPipeline.SLOTS, "single_step_latency_ms": round(e2e_latency_ms, 5),
                    "selector_in_timed_region": True, "output_equals_device_path": e2e_matches},
            "gpu_launches": launches,
            "clocks": clock_summary,
            "step_ms_min_median_max": [round(min(step_ms), 5), round(sorted(step_ms)[len(step_ms) // 2], 5),
                                       round(max(step_ms), 5)],
            "output_checksum": checksum,
        }
        if not args.no_parity:
            sample = None
            if q_len > 64:  # prefill chunks: first, middle and last new token of every sequence
                sample = [[0, q_len // 2, q_len - 1] for _ in contexts]
            parity, oracle_s = oracle_parity(spec, contexts, q_lens, case, output_f32(device_out, spec, torch), sample)
            result["parity"] = parity
            if world == 1 and sample is None and not args.no_cpu_baseline:
                # the oracle pass of the parity check IS the CPU restatement on this very batch
                result["cpu_baseline"] = {
                    "value": round(kv_bytes / oracle_s / 1e9, 4), "unit": "GB/s", "cores": host_threads(),
                    "kind": "port", "tokens_per_s": round(len(contexts) * q_len / oracle_s, 2),
                    "sample": f"all {len(contexts)} requests of the bench batch (the stored Q/K/V of the GPU run), "
                              f"one pass, {oracle_s:.2f} s"}
        if world == 1 and "cpu_baseline" not in result and not args.no_cpu_baseline:
            result["cpu_baseline"] = cpu_baseline(spec, contexts, sample_requests=len(contexts))
    del pipeline
    return result, dict(device=device, stream=stream, torch_stream=torch_stream)


def run_mixed(args):
    """Workload c5: prefill chunks and decode requests in ONE call (MixedBatchAttention: the decode requests through
    the SlicedKv kernels, the prefill chunks through the tensor-memory kernel, recorded back to back). Reports the
    whole call, each part (events between the parts), and the same batch through a single selection."""
    import torch

    from khalamari_b200.device import Device, Dtype, Stream
    from khalamari_b200.gqa import GQACore, MixedBatchAttention
    from khalamari_b200.request_page_table import GQAPageTableLayout

    rank, world, local = init_ranks(torch)
    spec = dict(WORKLOADS["c5"])
    chunk = args.chunk or 2048
    rng = np.random.default_rng(spec["seed"] + 1000 * rank)
    prefixes = rng.integers(0, 30720 + 1, size=8).tolist()
    decode_contexts = rng.integers(1024, 8192 + 1, size=56).tolist()
    contexts = [p + chunk for p in prefixes] + decode_contexts
    q_lens = [chunk] * 8 + [1] * 56
    spec["q_lens"] = q_lens
    hq, hkv, d = spec["hq"], spec["hkv"], spec["d"]
    device = Device(local)
    case = build_device_case(device, spec, contexts, torch, spec["seed"] + 1000 * rank)
    torch_stream = torch.cuda.current_stream()
    stream = Stream(device, torch_stream.cuda_stream)
    layout = GQAPageTableLayout(len(contexts), 1, case["num_blocks"], 1)
    total_tokens = sum(q_lens)
    scale = 1.0 / float(np.sqrt(d))
    mixed = MixedBatchAttention(device, GQACore(d, hq, hkv, scale), Dtype.Bfloat16, 2 * hkv * PAGE * d * 2, layout,
                                total_tokens, max_decode_tokens=64)
    req_slots = list(range(len(contexts)))
    token_indices = [c - q for c, q in zip(contexts, q_lens)]
    cu_tokens = np.concatenate([[0], np.cumsum(q_lens)]).tolist()

    def timed(record, count, marks):
        for _ in range(max(args.warmup, 3)):
            record(None)
        torch.cuda.synchronize()
        events = [[torch.cuda.Event(enable_timing=True) for _ in range(marks + 1)] for _ in range(count)]
        launches = 0
        for i in range(count):
            events[i][0].record(torch_stream)
            seen = [0]

            def between(i=i, seen=seen):
                seen[0] += 1
                events[i][seen[0]].record(torch_stream)

            launches += record(between)
        torch.cuda.synchronize()
        device.check(stream)
        per_mark = [float(np.mean([e[k].elapsed_time(e[k + 1]) for e in events])) for k in range(marks)]
        return events[0][0].elapsed_time(events[-1][marks]) / count, per_mark, launches

    steps = min(args.steps, 10)
    mixed.prepare(req_slots, token_indices, cu_tokens)
    names = ["decode" if part is mixed._parts.get("decode") else "prefill" for part, _, _ in mixed.plan]
    props = torch.cuda.get_device_properties(local)
    sampler = ClockSampler(str(getattr(props, "uuid", "")) or None, local)
    sampler.__enter__()
    t0 = time.perf_counter()
    split_ms, part_ms, launches = timed(
        lambda between: mixed.record_sdpa(stream, case["d_q"], case["d_pool"], case["d_table"], case["d_out"], 0, between),
        steps, len(mixed.plan))
    t1 = time.perf_counter()
    sampler.__exit__(None, None, None)
    out_split = case["out"].clone()
    # the same batch through one selection (the reference's form: the decode rows ride the prefill tiles)
    whole = mixed._part("whole", total_tokens)
    whole.prepare(req_slots, token_indices, cu_tokens, total_tokens)
    case["out"].zero_()
    single_ms, _, _ = timed(
        lambda between: (whole.record_sdpa(stream, case["d_q"], case["d_pool"], case["d_table"], case["d_out"], 0),
                         between() if between else None)[0], steps, 1)
    agree = float((out_split.float() - case["out"].float()).abs().max().item())
    if rank != 0:
        return None
    prefill_pairs = sum(chunk * p + chunk * (chunk + 1) // 2 for p in prefixes)
    prefill_flops = 4.0 * hq * d * prefill_pairs
    decode_bytes = sum(decode_contexts) * 2 * hkv * d * 2
    prefill_min_bytes = sum(p + chunk for p in prefixes) * 2 * hkv * d * 2
    by_name = dict(zip(names, part_ms))
    peak, peak_kind = load_peaks()
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    tensor_peak = float(peaks.get("bf16_tflops", 1590.0))
    result = {
        "metric": "GQA decode KV-read GB/s", "value": round((decode_bytes + prefill_min_bytes) / (split_ms * 1e-3) / 1e9, 2),
        "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": round(split_ms, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": spec["label"], "batch_per_gpu": len(contexts), "new_tokens": total_tokens,
                   "kv_tokens_per_gpu": int(sum(contexts)), "l2": "inputs larger than L2; no flush",
                   "parallelism": f"dp{world} by request"},
        "tflops": round((prefill_flops + 4.0 * hq * d * sum(decode_contexts)) / (split_ms * 1e-3) / 1e12, 2),
        "tokens_per_s": round(total_tokens / (split_ms * 1e-3), 1),
        "mix": {"form": "two selections recorded back to back (decode: SlicedKv map + reduce; prefill: tensor-memory "
                        "tiles, direct or map + reduce)",
                "prefill_ms": round(by_name.get("prefill", 0.0), 5), "decode_ms": round(by_name.get("decode", 0.0), 5),
                "prefill_tflops": round(prefill_flops / (by_name["prefill"] * 1e-3) / 1e12, 2) if by_name.get("prefill") else None,
                "decode_kv_gbs": round(decode_bytes / (by_name["decode"] * 1e-3) / 1e9, 1) if by_name.get("decode") else None,
                "single_selection_ms": round(single_ms, 5),
                "max_abs_difference_between_the_two_forms": agree},
        "roofline": {"bound": "tensor", "achieved": round(prefill_flops / (by_name.get("prefill", split_ms) * 1e-3) / 1e12, 2),
                     "peak": tensor_peak, "unit": "TFLOP/s",
                     "frac": round(prefill_flops / (by_name.get("prefill", split_ms) * 1e-3) / 1e12 / tensor_peak, 4),
                     "traffic": None, "peak_source": "of measured (burst)" if peaks else "of fallback",
                     "kernel": "sdpa_tc_kernel (prefill part)", "kernel_ms": round(by_name.get("prefill", split_ms), 5)},
        "gpu_launches": launches, "clocks": sampler.summary(t0, t1),
    }
    if not args.no_parity:
        sample = [[0, chunk // 2, chunk - 1] for _ in range(8)] + [[0] for _ in range(56)]
        parity, _ = oracle_parity(spec, contexts, q_lens, case, out_split.float().cpu().numpy(), sample)
        result["parity"] = parity
    return result


def measure_split_sequence(args, torch, context, rank, world, local, device, stream, torch_stream, steps,
                           partition=None, check_parity=True):
    """ONE long sequence whose pages are split in token order over the ranks. A step is: local split-KV map, local
    merge into this rank's record, all-gather of the records (NCCL), merge of the gathered records on every rank.
    Measures the step, the local part alone (map + local merge) and, on rank 0, the same sequence on one GPU (the
    denominator of the scaling efficiency). Returns a dict on rank 0."""
    import torch.distributed as dist

    from khalamari_b200 import split_kv
    from khalamari_b200.device import Dtype
    from khalamari_b200.gqa import GQAAttention, GQACore
    from khalamari_b200.request_page_table import GQAPageTableLayout
    from khalamari_b200.selector import SelectorPolicy

    spec = dict(WORKLOADS["c4"])
    hq, hkv, d = spec["hq"], spec["hkv"], spec["d"]
    scale = 1.0 / 16.0

    def build(local_len, seed, ranks):
        case = build_device_case(device, spec, [max(local_len, 1)], torch, seed)
        layout = GQAPageTableLayout(1, 1, case["num_blocks"], 1)
        attention = GQAAttention(device, GQACore(d, hq, hkv, scale), Dtype.Bfloat16, 2 * hkv * PAGE * d * 2, layout, 1,
                                 SelectorPolicy.B200)
        decode = split_kv.SplitKvDecode(device, attention, ranks)
        decode.prepare(0, local_len, partition)
        return case, attention, decode

    def timed(fn, count, all_ranks):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1 and all_ranks:
            dist.barrier()
        torch.cuda.synchronize()
        first = torch.cuda.Event(enable_timing=True)
        last = torch.cuda.Event(enable_timing=True)
        first.record(torch_stream)
        n = 0
        for _ in range(count):
            n += fn() or 0
        last.record(torch_stream)
        torch.cuda.synchronize()
        return first.elapsed_time(last) / count, n

    def measure(decode, case, all_ranks):
        """Times one decode object: the eager step, the step and its local part (map + local merge) replayed as CUDA
        graphs (the analogue of the reference's recorded replay program; removes the host's launch gaps). Returns
        (step ms, eager step ms, local ms, launches per step)."""
        def eager_step():
            return decode.record_step(stream, case["d_q"], case["d_pool"], case["d_table"], case["d_out"], 0)

        def eager_local():
            return decode.record_local(stream, case["d_q"], case["d_pool"], case["d_table"], 0)

        for _ in range(min(max(int(args.ramp_ms), 1), 400)):  # a count: every rank runs the same number of collectives
            eager_step()
        torch.cuda.synchronize()
        eager_ms, launches = timed(eager_step, steps, all_ranks)
        if args.no_graph:
            local_ms, _ = timed(eager_local, steps, all_ranks)
            return eager_ms, eager_ms, local_ms, launches // steps
        from khalamari_b200.device import Stream as KhStream
        side = torch.cuda.Stream()
        side_stream = KhStream(device, side.cuda_stream)

        def captured(record):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                for _ in range(3):
                    record(side_stream)
                side.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    record(side_stream)
            torch.cuda.synchronize()
            return graph

        step_graph = captured(lambda s: decode.record_step(s, case["d_q"], case["d_pool"], case["d_table"],
                                                           case["d_out"], 0))
        local_graph = captured(lambda s: decode.record_local(s, case["d_q"], case["d_pool"], case["d_table"], 0))
        step_ms, _ = timed(lambda: step_graph.replay(), steps, all_ranks)
        local_ms, _ = timed(lambda: local_graph.replay(), steps, all_ranks)
        return step_ms, eager_ms, local_ms, launches // steps

    begin, end = split_kv.split_context(context, world, PAGE)[rank]
    local_len = end - begin
    # every rank draws the SAME Q row (seed without the rank) and its own K/V pages
    case, attention, decode = build(local_len, spec["seed"] + 1000 * rank, world)
    # (a seed of its own: the page pool of rank 0 starts from spec["seed"], and a Q row equal to a cached K row
    # would make the softmax one-hot)
    q_shared = torch.randn(hq * d, generator=torch.Generator(device="cuda").manual_seed(spec["seed"] + 424243),
                           device="cuda", dtype=torch.float32).to(torch.bfloat16)
    case["q"].copy_(q_shared)
    step_ms, eager_ms, local_ms, launches = measure(decode, case, True)
    device.check(stream)
    stats = torch.tensor([step_ms, local_ms, eager_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    step_ms, local_ms, eager_ms = stats.tolist()
    # The same step with the exchange as ONE kernel over NVLink peer memory (local merge, rows stored into every
    # rank's inbox, flags, bounded wait, final merge) instead of local merge + NCCL all-gather + merge.
    nccl = {"ms_per_step": round(step_ms, 5), "eager_ms_per_step": round(eager_ms, 5), "gpu_launches_per_step": launches}
    peer = None
    if world > 1 and not args.no_peer_exchange:
        out_nccl = case["out"].clone()
        exchange = split_kv.PeerExchange(device, rank, world, hq, d)
        exchange.connect()
        decode_peer = split_kv.SplitKvDecode(device, attention, world, peer_exchange=exchange)
        decode_peer.prepare(0, local_len, partition)
        peer_ms, peer_eager_ms, _, peer_launches = measure(decode_peer, case, True)
        device.check(stream)
        peer_stats = torch.tensor([peer_ms, peer_eager_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(peer_stats, op=dist.ReduceOp.MAX)
        peer_ms, peer_eager_ms = peer_stats.tolist()
        peer = {"ms_per_step": round(peer_ms, 5), "eager_ms_per_step": round(peer_eager_ms, 5),
                "gpu_launches_per_step": peer_launches,
                "max_abs_difference_from_the_nccl_form": float((case["out"].float() - out_nccl.float()).abs().max().item())}
        step_ms, eager_ms, launches = peer_ms, peer_eager_ms, peer_launches
        dist.barrier()
        del decode_peer
        exchange.close()

    # ---- parity: every rank restates its own slice on the CPU as one partial (m, l, o) per head, rank 0 merges the
    # partials with the reducer's formula and compares the GPU result
    parity = None
    if check_parity:
        import oracle
        from concurrent.futures import ThreadPoolExecutor
        q = case["q"].float().cpu().numpy().reshape(hq, d)
        partials = None
        if local_len > 0:
            pool = case["pool"].view(torch.uint8).cpu().numpy()
            layout_o = oracle.PageTableLayout(1, 1, case["num_blocks"], 1)
            k_u8, v_u8 = oracle.gather_paged(pool, case["table"].reshape(-1), layout_o, 0, 0, PAGE, hkv, d, 2, local_len)
            k = oracle.bf16_bits_to_f32(k_u8.view(np.uint16)).reshape(local_len, hkv, d)
            v = oracle.bf16_bits_to_f32(v_u8.view(np.uint16)).reshape(local_len, hkv, d)
            with ThreadPoolExecutor(min(hq, host_threads())) as workers:
                partials = list(workers.map(
                    lambda h: oracle.partial_row(q[h], k, v, 0, local_len, hkv, d, h // (hq // hkv), scale), range(hq)))
        gathered = [partials]
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, partials)
        if rank == 0:
            expected = np.zeros((hq, d), np.float32)
            for h in range(hq):
                rows = [g[h] for g in gathered if g is not None]
                expected[h] = oracle.merge_partials([r[1] for r in rows], [r[2] for r in rows],
                                                    np.stack([r[0] for r in rows]))[0]
            actual = case["out"].float().cpu().numpy().reshape(hq, d)
            err = np.abs(actual - expected)
            ok = (err <= 2e-3) | (err <= 1e-2 * np.abs(expected))
            parity = {"max_abs": float(err.max()), "rows_checked": hq, "pass": bool(ok.all()),
                      "rule": "per element |a-b| <= 2e-3 or |a-b| <= 1e-2*|b|; oracle partial per rank over its own "
                              "pages, merged with the reducer's formula"}

    # ---- the same sequence on one GPU (rank 0 only), for the efficiency
    single_ms = step_ms
    if world > 1:
        del case, attention, decode
        torch.cuda.empty_cache()
        if rank == 0:
            case1, attention1, decode1 = build(context, spec["seed"], 1)
            single_ms = measure(decode1, case1, False)[0]
            del case1, attention1, decode1
            torch.cuda.empty_cache()
        dist.barrier()
    if rank != 0:
        return None
    total_bytes = context * 2 * hkv * d * 2
    return {"context_tokens": context, "tokens_per_gpu": local_len, "ms_per_step": round(step_ms, 5),
            "form": "eager launches" if args.no_graph else "replayed CUDA graph", "eager_ms_per_step": round(eager_ms, 5),
            "exchange": "none (one GPU)" if world == 1 else
            ("one kernel over NVLink peer memory" if peer is not None else "NCCL all-gather between two merge kernels"),
            "with_nccl_all_gather": nccl, "with_peer_memory_kernel": peer,
            "local_kernel_ms": round(local_ms, 5), "exchange_ms": round(step_ms - local_ms, 5),
            "kv_gbs_total": round(total_bytes / (step_ms * 1e-3) / 1e9, 1),
            "kv_gbs_per_gpu_local": round(local_len * 2 * hkv * d * 2 / (local_ms * 1e-3) / 1e9, 1),
            "one_gpu_ms_per_step": round(single_ms, 5),
            "efficiency_vs_one_gpu": round(single_ms / (world * step_ms), 4), "gpu_launches_per_step": launches,
            "parity": parity}


def run_split_sequence(args):
    """Workload c4 alone: the JSON line of one context length (``--context``, default 1,048,576 tokens)."""
    import torch
    import torch.distributed as dist

    from khalamari_b200 import split_kv
    from khalamari_b200.device import Device, Stream

    rank, world, local = init_ranks(torch)
    spec = dict(WORKLOADS["c4"])
    context = args.context or spec["contexts"][0]
    device = Device(local)
    torch_stream = torch.cuda.current_stream()
    stream = Stream(device, torch_stream.cuda_stream)
    props = torch.cuda.get_device_properties(local)
    sampler = ClockSampler(str(getattr(props, "uuid", "")) or None, local)
    sampler.__enter__()
    t0 = time.perf_counter()
    m = measure_split_sequence(args, torch, context, rank, world, local, device, stream, torch_stream, args.steps,
                               args.partition if args.partition > 0 else None, not args.no_parity)
    t1 = time.perf_counter()
    sampler.__exit__(None, None, None)
    if rank != 0:
        return None
    peak, peak_kind = load_peaks()
    record_bytes = split_kv.record_floats(spec["hq"], spec["d"]) * 4
    return {
        "metric": "GQA decode KV-read GB/s", "value": m["kv_gbs_total"], "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": 3, "ms_per_step": m["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": spec["label"], "context_tokens": context, "tokens_per_gpu": m["tokens_per_gpu"],
                   "l2": "inputs (KV pages read per step) larger than L2; no flush"
                   if m["tokens_per_gpu"] * 2048 > 126e6 else "per-GPU KV pages fit L2: not an HBM measurement",
                   "parallelism": f"split-KV over {world} GPUs, all-gather of {record_bytes} B per rank"},
        "tokens_per_s": round(1.0 / (m["ms_per_step"] * 1e-3), 1), "hbm_frac": round(m["kv_gbs_total"] / world / peak, 4),
        "roofline": {"bound": "hbm", "achieved": m["kv_gbs_per_gpu_local"], "peak": peak, "unit": "GB/s",
                     "frac": round(m["kv_gbs_per_gpu_local"] / peak, 4), "traffic": None, "peak_source": f"of {peak_kind}",
                     "kernel": "sdpa_map_kernel + local merge (slowest rank)", "kernel_ms": m["local_kernel_ms"]},
        "split_kv": [m], "gpu_launches": m["gpu_launches_per_step"] * args.steps,
        "clocks": sampler.summary(t0, t1), "parity": m["parity"],
    }


def cpu_inputs(spec, contexts, sample_requests, seed):
    rng = np.random.default_rng(seed)
    import oracle
    rounder = oracle.round_bf16 if spec["dtype"] == "bf16" else oracle.round_f16
    hq, hkv, d, q_len = spec["hq"], spec["hkv"], spec["d"], spec["q_len"]
    ctxs = contexts[:sample_requests]
    ks = [rounder(rng.standard_normal((c, hkv, d), dtype=np.float32))[1] for c in ctxs]
    vs = [rounder(rng.standard_normal((c, hkv, d), dtype=np.float32))[1] for c in ctxs]
    q = rounder(rng.standard_normal((len(ctxs) * q_len, hq, d), dtype=np.float32))[1]
    cu = [i * q_len for i in range(len(ctxs) + 1)]
    ti = [c - q_len for c in ctxs]
    return cu, ti, q, ks, vs


def host_threads():
    """Cores this process may run on. Launchers such as torchrun export OMP_NUM_THREADS=1, which is a default for
    their workers and not a limit of the machine, so the OpenMP default is not used."""
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def cpu_pass(spec, inputs, threads):
    import oracle
    cu, ti, q, ks, vs = inputs
    scale = spec.get("scale") or 1.0 / float(np.sqrt(spec["d"]))
    t0 = time.perf_counter()
    oracle.projected_gqa(cu, ti, q, ks, vs, spec["d"], spec["hq"], spec["hkv"], scale, threads)
    return time.perf_counter() - t0


def bounded_sample(spec, contexts, threads, passes):
    """How many of the batch's requests one CPU pass takes so that `passes` passes stay near two minutes: the whole
    batch when that fits (about 1.1 GFLOP/s per thread for the scalar restatement), else a prefix, halved until
    it does."""
    sample = len(contexts)
    rate = 1.1e9 * threads
    while sample > 1 and attention_flops(spec, contexts[:sample]) / rate * passes > 120.0:
        sample //= 2
    return sample


def cpu_baseline(spec, contexts, sample_requests):
    """The CPU restatement of the reference's GQA SDPA (oracle/, kind "port") on the host cores, contiguous
    per-request K/V as the reference's CPU path takes them, one pass over a bounded sample."""
    threads = host_threads()
    sample_requests = min(sample_requests, bounded_sample(spec, contexts, threads, 6))
    inputs = cpu_inputs(spec, contexts, sample_requests, spec["seed"])
    seconds = cpu_pass(spec, inputs, threads)
    sample_bytes = sum(contexts[:sample_requests]) * 2 * spec["hkv"] * spec["d"] * 2
    return {"value": round(sample_bytes / seconds / 1e9, 4), "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"first {sample_requests} of {len(contexts)} requests, one pass, {seconds:.2f} s",
            "tokens_per_s": round(sample_requests * spec["q_len"] / seconds, 2)}


def run_reference(args):
    """The reference arm: the reference's own CPU implementation of the path. The reference is Rust and
    cannot be built in this image, so this times its C restatement (oracle/) on all host threads: the whole batch
    of the workload per step when `steps + warmup` passes fit about two minutes, else a prefix of it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    spec = dict(WORKLOADS[args.workload])
    contexts = contexts_for(spec, 0, int(os.environ.get("WORLD_SIZE", "1")))
    threads = host_threads()
    warmup = max(args.warmup, 0)
    sample = bounded_sample(spec, contexts, threads, args.steps + warmup)
    inputs = cpu_inputs(spec, contexts, sample, spec["seed"])
    for _ in range(warmup):
        cpu_pass(spec, inputs, threads)
    times = [cpu_pass(spec, inputs, threads) for _ in range(args.steps)]
    seconds = float(np.mean(times))
    sample_bytes = sum(contexts[:sample]) * 2 * spec["hkv"] * spec["d"] * 2
    value = round(sample_bytes / seconds / 1e9, 4)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    described = (f"all {sample} requests of the batch per step" if sample == len(contexts)
                 else f"first {sample} of {len(contexts)} requests per step")
    return {
        "impl": "reference", "metric": "GQA decode KV-read GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": round(seconds * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(spec, contexts, world),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{described}, {args.steps} steps"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "tokens_per_s": round(sample * spec["q_len"] / seconds, 2),
    }


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-parity", action="store_true", help="skip the oracle check of the bench's own output")
    parser.add_argument("--no-graph", action="store_true",
                        help="one long sequence: time eager launches only, not the step replayed as a CUDA graph")
    parser.add_argument("--no-peer-exchange", action="store_true",
                        help="one long sequence: exchange through NCCL only, not through the peer-memory kernel")
    parser.add_argument("--no-split-kv", action="store_true",
                        help="default workload: skip the one-long-sequence measurements that follow the headline")
    parser.add_argument("--batch", type=int, default=0, help="override the workload's batch (profiling captures)")
    parser.add_argument("--pool-pages", type=int, default=0, help="override the page pool size (profiling captures)")
    parser.add_argument("--partition", type=int, default=-1, help="override the split-KV partition (0: selector)")
    parser.add_argument("--ramp-ms", type=float, default=500.0,
                        help="untimed load before the timed steps so that clocks settle (0 for profiler runs)")
    parser.add_argument("--fused", action="store_true",
                        help="map and reduce in one launch (last-arriver merge) instead of the reference's two")
    parser.add_argument("--uniform-context", type=int, default=0, help="give every request this context length")
    parser.add_argument("--q-len", type=int, default=0,
                        help="new tokens per request (workload c3: 2 or 4 verify tokens; default: the workload's)")
    parser.add_argument("--kv-dtype", default="io", choices=["io", "fp8"],
                        help="element type of the K/V pages: the Q/output type (default) or FP8 E4M3FN")
    parser.add_argument("--context", type=int, default=0, help="workload c4: tokens of the one sequence")
    parser.add_argument("--chunk", type=int, default=0, help="workload c5: tokens per prefill chunk (default 2048)")
    args = parser.parse_args()
    if args.impl == "reference":
        result = run_reference(args)
    elif args.workload == "c4":
        result = run_split_sequence(args)
        finish_ranks()
    elif args.workload == "c5":
        result = run_mixed(args)
        finish_ranks()
    else:
        import torch
        result, ctx = run_ours(args)
        if args.workload == "c2" and not args.no_split_kv and args.kv_dtype == "io" and not args.batch:
            # after the headline: one long sequence split over the same ranks, at the three stated context lengths
            rank, world, local = init_ranks(torch)
            torch.cuda.empty_cache()
            split = [measure_split_sequence(args, torch, context, rank, world, local, ctx["device"], ctx["stream"],
                                            ctx["torch_stream"], args.steps, None, not args.no_parity)
                     for context in SPLIT_CONTEXTS]
            if result is not None:
                result["split_kv"] = split
        finish_ranks()
    if result is not None:
        print(json.dumps(result), flush=True)


def finish_ranks():
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
