"""Benchmark of the greedy byte-level BPE path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One rank per GPU (torchrun for N > 1).  A step is one pass of the hot path over the rank's
batch of synthetic text.  Rank 0 prints ONE JSON line:

  value          whole-job input MB/s with the text already resident in HBM (device-resident call)
  e2e            the same metric through the host-buffer entry point: pinned host text -> H2D ->
                 kernels -> D2H ids + offsets, every step; e2e.copy_ceiling is a copy-only run of
                 the same bytes, slice size and stream layout without any kernel
  roofline       merge kernel: algorithmic bytes / CUDA-event time / measured HBM copy bandwidth
  cpu_baseline   the reference's CPU greedy tokenizer on a bounded sample, on this host's cores
                 (all threads, one thread, and the reference's other rule, each labelled)
  parity_check   every rank compares a seeded sample of its own shard with the CPU checker after
                 the timed regions; the line carries the AND over ranks
  latency        (N = 1) config 3: one 512-byte string per call, p50 / p99
  configs        (N = 1) short runs of configs 1, 3 (batched), 4 and 5, each with its own check
  cfg5_partition config 5 as one batch: log-normal texts, byte-range partition over the N GPUs,
                 offsets stitched on the host, per-GPU time and imbalance

Workloads (synthetic text from gputok_b200.TextGen; the reference's WikiText-103 is not available
offline):
  cfg2  256 MiB per GPU, seed 1, 4096-byte chunks   (default; the configuration the metric is quoted on)
  cfg1  1 MiB, seed 0, 1024-byte chunks
  cfg4  64 MiB, seed 3, 32 KiB chunks, multi-byte UTF-8 words and repeated-byte runs
  cfg5  512 MiB per GPU of the 4 GiB seed-4 text, log-normal text lengths (64 B..64 KiB)
  cfg3  10 000 strings of 512 B (seed 2); as a batch here, one call each in `latency`

`--impl reference` times the reference's own CPU implementation (its host functions compiled in
place into oracle/_ref, else the C restatement in oracle/) on a bounded sample of the same
workload with all host threads, and prints the same JSON shape with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "gpu-tokenizer_b200")
MERGES = os.path.join(ROOT, "tests", "golden", "gpt2_merges.txt")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

BLOCK = 65536  # generator block size

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per input byte of one k_merge_opt launch: 201.1 MB
# measured by ncu for a launch over 128 MiB of config-2 text.  Traffic grows in proportion to the tile count,
# so a launch over n bytes moves this x n.
MERGE_OPT_DRAM_BYTES_PER_INPUT_BYTE = 201.1e6 / (128 << 20)

WORKLOADS = {
    #        seed  bytes per GPU   chunk   mix  lognormal
    "cfg1": (0, 1 << 20, 1024, 0, False),
    "cfg2": (1, 256 << 20, 4096, 0, False),
    "cfg3": (2, 10000 * 512, 2048, 0, False),
    "cfg4": (3, 64 << 20, 32768, 1, False),
    "cfg5": (4, 512 << 20, 65536, 1, True),
}
SLICE_BYTES = 24 << 20  # slice size of the library's host path (the copy-only leg mirrors it)


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows: list[list[str]] = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_workload(name: str, rank: int, world: int, scale_bytes: int | None):
    """Returns (bytes uint8[n], text_offsets int64[T+1], chunk_bytes, description)."""
    from gputok_b200 import TextGen

    seed, n_bytes, chunk, mix, lognormal = WORKLOADS[name]
    if scale_bytes:
        n_bytes = scale_bytes
    n_blocks = (n_bytes + BLOCK - 1) // BLOCK
    n_bytes = n_blocks * BLOCK
    gen = TextGen(seed)
    data = gen.blocks(n_blocks, BLOCK, first_block=rank * n_blocks, mix=mix)  # weak scaling: own block range
    if name == "cfg3":
        off = np.arange(0, n_bytes + 1, 512, dtype=np.int64)
    elif lognormal:
        off = TextGen.lognormal_offsets(seed * 1000 + rank, n_bytes)
    else:
        off = np.array([0, n_bytes], dtype=np.int64)
    desc = {"workload": name, "seed": seed, "bytes_per_gpu": int(n_bytes), "chunk_bytes": chunk,
            "texts_per_gpu": int(len(off) - 1), "mix": "stress" if mix else "plain",
            "l2": "input larger than L2 (126 MB)" if n_bytes > (126 << 20) else "input smaller than L2"}
    return data, off, chunk, desc


def chunk_offsets(text_off: np.ndarray, chunk: int) -> np.ndarray:
    out = [0]
    for s, e in zip(text_off[:-1].tolist(), text_off[1:].tolist()):
        out.extend(range(s + chunk, e, chunk))
        if e > s:
            out.append(e)
    return np.array(out, dtype=np.int64)


def sample_chunks(data: np.ndarray, text_off: np.ndarray, chunk: int, budget_cpu_s: float, seed: int,
                  max_chunks: int | None = None):
    """A seeded sample of whole chunks, sized for about budget_cpu_s core-seconds of the literal
    O(n^2) greedy loop (cost model: 55 ms per 4 KiB chunk per core, quadratic in chunk length)."""
    coff = chunk_offsets(text_off, chunk) if len(text_off) < 200000 else text_off
    lens = np.diff(coff)
    cost = 0.055 * (lens / 4096.0) ** 2
    order = np.random.default_rng(seed).permutation(len(lens))
    take, acc = [], 0.0
    for c in order:
        if acc + cost[c] > budget_cpu_s and take:
            break
        take.append(int(c))
        acc += float(cost[c])
        if max_chunks and len(take) >= max_chunks:
            break
        if len(take) >= max(1, len(lens) // 100) and acc > budget_cpu_s / 3:
            break
    take = np.sort(np.array(take))
    pieces = [data[coff[c]:coff[c + 1]] for c in take]
    blob = np.concatenate(pieces) if pieces else np.zeros(0, np.uint8)
    off = np.concatenate([[0], np.cumsum([len(p) for p in pieces])]).astype(np.int64)
    return blob, off, take


def cpu_reference_runner():
    """The reference's CPU greedy tokenizer: its own host functions where oracle/_ref was built,
    else the C restatement."""
    from oracle.loader import Oracle, RefGreedy

    if RefGreedy.available():
        return RefGreedy(MERGES), "reference"
    return Oracle(MERGES), "port"


def time_cpu_baseline(data, text_off, chunk, seed, budget_cpu_s=24.0):
    """The three CPU legs on one seeded sample of the workload: the reference's greedy function on all host
    threads (the headline baseline), the same on one thread (a sub-sample), and the rule the reference's
    tokenize_batch_cpu really runs (bpe_merge_cpu: local minimum, at most 50 passes), labelled as such."""
    from oracle.loader import MODE_GREEDY, MODE_LOCALMIN

    runner, kind = cpu_reference_runner()
    blob, off, take = sample_chunks(data, text_off, chunk, budget_cpu_s, seed)
    cores = os.cpu_count() or 1
    t0 = time.perf_counter()
    ids, _ = runner.encode_chunks(blob, off, mode=MODE_GREEDY, threads=cores)
    dt = time.perf_counter() - t0
    # one thread: as many sampled chunks as about 3 s of the literal loop allow
    n1 = 1
    lens = np.diff(off)
    acc = 0.0
    for k, ln in enumerate(lens.tolist()):
        acc += 0.055 * (ln / 4096.0) ** 2
        n1 = k + 1
        if acc > 3.0:
            break
    t0 = time.perf_counter()
    runner.encode_chunks(blob[:off[n1]], off[:n1 + 1], mode=MODE_GREEDY, threads=1)
    dt1 = time.perf_counter() - t0
    t0 = time.perf_counter()
    runner.encode_chunks(blob, off, mode=MODE_LOCALMIN, max_iters=50, threads=cores)
    dtl = time.perf_counter() - t0
    return {"value": len(blob) / dt / 1e6, "unit": "MB/s", "cores": cores, "kind": kind,
            "sample": f"{len(take)} seeded chunks ({len(blob)} bytes) of the workload, literal Algorithm 1 "
                      f"(bpe_merge_cpu_greedy), one chunk per task on {cores} threads, {dt:.2f} s",
            "tokens_per_s": len(ids) / dt,
            "one_thread": {"value": int(off[n1]) / dt1 / 1e6, "unit": "MB/s", "cores": 1,
                           "sample": f"first {n1} of the sampled chunks ({int(off[n1])} bytes), {dt1:.2f} s"},
            "localmin_cap50": {"value": len(blob) / dtl / 1e6, "unit": "MB/s", "cores": cores,
                               "rule": "bpe_merge_cpu (local minimum, at most 50 passes): what the reference's "
                                       "tokenize_batch_cpu runs; NOT the greedy rule and not the parity target",
                               "sample": f"the same {len(take)} chunks, {dtl:.2f} s"}}, (blob, off, ids)


def run_reference_arm(args, rank: int, world: int):
    """--impl reference: the reference's CPU path on a bounded sample of the same workload; rank 0 only."""
    if rank != 0:
        return
    from oracle.loader import MODE_GREEDY

    data, text_off, chunk, desc = make_workload(args.workload, 0, 1, args.bytes)
    runner, kind = cpu_reference_runner()
    blob, off, take = sample_chunks(data, text_off, chunk, args.ref_budget_s, WORKLOADS[args.workload][0])
    cores = os.cpu_count() or 1
    for _ in range(args.warmup):
        runner.encode_chunks(blob[:off[min(4, len(off) - 1)]], off[:min(5, len(off))], mode=MODE_GREEDY, threads=cores)
    t0 = time.perf_counter()
    n_ids = 0
    for _ in range(args.steps):
        ids, _ = runner.encode_chunks(blob, off, mode=MODE_GREEDY, threads=cores)
        n_ids += len(ids)
    dt = time.perf_counter() - t0
    mbs = len(blob) * args.steps / dt / 1e6
    sample = (f"{len(take)} seeded chunks ({len(blob)} bytes) of the workload per step, literal Algorithm 1 "
              f"(bpe_merge_cpu_greedy), one chunk per task on {cores} threads")
    line = {"impl": "reference", "metric": "input_MB_per_s", "value": mbs, "unit": "MB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16",
            "data": "synthetic",
            "config": dict(desc, mode=args.mode, parallelism=f"byte-range shards x{world}, no collectives"),
            "tokens_per_s": n_ids / dt,
            "cpu_baseline": {"value": mbs, "unit": "MB/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": mbs, "unit": "MB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# pieces of the GPU arm
# ---------------------------------------------------------------------------------------------

class Harness:
    """torch plumbing of one rank: device, stream, barrier and scalar reductions."""

    def __init__(self, local_rank: int, world: int):
        import torch
        import torch.distributed as dist

        self.torch, self.dist, self.world = torch, dist, world
        torch.cuda.set_device(local_rank)
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        # a stream of our own (non-zero handle): the library runs its kernels on it, so the CUDA events
        # recorded on it bracket exactly those kernels
        self.stream = torch.cuda.Stream()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def _reduce(self, x: float, op) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=op)
        return float(t.item())

    def allmax(self, x):
        return self._reduce(x, self.dist.ReduceOp.MAX)

    def allmin(self, x):
        return self._reduce(x, self.dist.ReduceOp.MIN)

    def allsum(self, x):
        return self._reduce(x, self.dist.ReduceOp.SUM)

    def gather(self, x: float) -> list[float]:
        if self.world == 1:
            return [x]
        mine = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        every = [self.torch.zeros_like(mine) for _ in range(self.world)]
        self.dist.all_gather(every, mine)
        return [float(t.item()) for t in every]


def device_resident_run(hx: Harness, tok, data, text_off, chunk, mode, steps, warmup, per_stage=True):
    """Text in HBM before the timed region; K steps bracketed by barriers, CUDA events on the launching stream.
    per_stage: the library records events between its stages too (the merge kernel's own time, for the roofline);
    without it only the pipeline as a whole is timed, which is the library's default."""
    torch = hx.torch
    tok.set_stage_timing(per_stage)
    n_bytes, n_texts = len(data), len(text_off) - 1
    with torch.cuda.stream(hx.stream):
        d_bytes = torch.from_numpy(data).cuda()
        d_toff = torch.from_numpy(text_off).cuda()
        cap = n_bytes  # worst case one id per byte
        d_ids = torch.empty(cap, dtype=torch.int32, device="cuda")
        chunk_cap = n_bytes // chunk + n_texts + 2
        d_coff = torch.empty(chunk_cap, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()

    def step():
        return tok.encode_device(d_bytes.data_ptr(), n_bytes, d_toff.data_ptr(), n_texts, d_ids.data_ptr(), cap,
                                 d_coff.data_ptr(), chunk_cap, mode=mode)

    for _ in range(warmup):
        n_ids, n_chunks, _ = step()
    merge_ms, stage_acc, launches = [], np.zeros(5), 0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    hx.barrier()
    t0 = time.perf_counter()
    ev0.record(hx.stream)
    for _ in range(steps):
        n_ids, n_chunks, _ = step()
        st = tok.stage_ms()
        merge_ms.append(st["merge"])
        stage_acc += [st["chunker"], st["merge"], st["scan"], st["pack"], st["pipeline"]]
        launches += st["kernel_launches"]
    ev1.record(hx.stream)
    hx.barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    dev_ms = ev0.elapsed_time(ev1)  # CUDA events on the stream the kernels run on
    tok.set_stage_timing(False)
    with torch.cuda.stream(hx.stream):
        coff = d_coff[:n_chunks + 1].cpu().numpy()
    return {"ms_per_step": dev_ms / steps, "wall_ms_per_step": wall_ms / steps, "n_ids": int(n_ids),
            "n_chunks": int(n_chunks), "merge_ms": float(np.mean(merge_ms)),
            "stage_ms": {k: float(v / steps) for k, v in zip(("chunker", "merge", "scan", "pack", "pipeline"), stage_acc)},
            "launches": int(launches), "coff": coff}


def e2e_run(hx: Harness, tok, pin, text_off, mode, steps):
    """Pinned host text in, ids + offsets back on the host, every step (wall clock around the calls)."""
    tok.encode(pin.array, text_off, mode=mode, copy=False)
    hx.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        ids_h, toff_h, coff_h, _ = tok.encode(pin.array, text_off, mode=mode, copy=False)
        _ = int(ids_h[-1]) + int(coff_h[-1])  # touch the result on the host
    hx.torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / steps
    h2d = len(pin.array) + 8 * len(text_off)
    d2h = 4 * len(ids_h) + 8 * len(coff_h) + 8 * len(toff_h) + 32
    return ms, int(h2d), int(d2h), len(ids_h)


def copy_ceiling_run(hx: Harness, n_bytes: int, n_ids: int, steps: int):
    """Copy-only stand-in for the host path: the same bytes up (text, 24 MiB slices) and down (int32 ids of
    each slice) on two copy streams with the same slice-to-slice dependencies, and no kernel at all.  What
    this takes is what the host link allows for the call's transfers."""
    torch = hx.torch
    ns = max(1, (n_bytes + SLICE_BYTES - 1) // SLICE_BYTES)
    h_in = torch.empty(n_bytes, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(n_ids, dtype=torch.int32).pin_memory()
    d_in = torch.empty(n_bytes, dtype=torch.uint8, device="cuda")
    d_out = torch.empty(n_ids, dtype=torch.int32, device="cuda")
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ib = [min(n_bytes, i * SLICE_BYTES) for i in range(ns + 1)]
    ob = [n_ids * i // ns for i in range(ns + 1)]

    def one():
        for i in range(ns):
            with torch.cuda.stream(s_in):
                d_in[ib[i]:ib[i + 1]].copy_(h_in[ib[i]:ib[i + 1]], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_in)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev)  # the ids of a slice exist only after its text has arrived
                h_out[ob[i]:ob[i + 1]].copy_(d_out[ob[i]:ob[i + 1]], non_blocking=True)
        s_in.synchronize()
        s_out.synchronize()

    one()
    hx.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    ms = (time.perf_counter() - t0) * 1e3 / steps
    del h_in, h_out, d_in, d_out
    return ms


def parity_on_sample(tok, data, text_off, chunk, mode, seed, budget_cpu_s, threads, max_chunks=None):
    """GPU ids of a seeded sample of the workload's chunks against the literal CPU rule.  Runs after the
    timed regions; the checker never runs inside one."""
    from oracle.loader import MODE_GREEDY

    runner, _ = cpu_reference_runner()
    blob, boff, take = sample_chunks(data, text_off, chunk, budget_cpu_s, seed, max_chunks)
    want, woff = runner.encode_chunks(blob, boff, mode=MODE_GREEDY, threads=threads)
    got, _, goff, _ = tok.encode(blob, boff, mode=mode)
    return bool(np.array_equal(got, want) and np.array_equal(goff, woff)), int(len(take))


def latency_run(hx: Harness, merges, calls: int):
    """Config 3: one 512-byte string per call, batch size 1, host bytes in and ids on the host out."""
    import ctypes

    import gputok_b200
    from gputok_b200.capi import PinnedArray
    from oracle.loader import MODE_GREEDY

    seed, n_bytes, chunk, mix, _ = WORKLOADS["cfg3"]
    calls = min(calls, n_bytes // 512)
    data = gputok_b200.TextGen(seed).text(calls * 512)
    pin = PinnedArray(len(data))
    pin.array[:] = data
    tok = gputok_b200.Tokenizer(merges, chunk_tokens=chunk, device=hx.torch.cuda.current_device())
    lat, kern, raw, got = [], [], [], []
    one = np.array([0, 512], dtype=np.int64)
    ms = ctypes.c_float()
    for i in range(calls):
        s = pin.array[i * 512:(i + 1) * 512]
        t1 = time.perf_counter()
        ids, _, _, k_ms = tok.encode(s, None, copy=True)                 # the Python call a user makes
        lat.append((time.perf_counter() - t1) * 1e6)
        kern.append(k_ms * 1e3)
        got.append(ids)
        t1 = time.perf_counter()                                          # the C ABI call alone
        tok._lib.gtk_encode(tok._h, 0, s.ctypes.data, one.ctypes.data, 1, ctypes.byref(ms))
        raw.append((time.perf_counter() - t1) * 1e6)
    runner, _ = cpu_reference_runner()
    off = np.arange(0, calls * 512 + 1, 512, dtype=np.int64)
    want, woff = runner.encode_chunks(data, off, mode=MODE_GREEDY, threads=os.cpu_count() or 1)
    ok = all(np.array_equal(g, want[woff[i]:woff[i + 1]]) for i, g in enumerate(got))
    skip = min(10, calls // 2)
    lat, kern, raw = np.array(lat[skip:]), np.array(kern[skip:]), np.array(raw[skip:])
    return {"p50_us": float(np.percentile(lat, 50)), "p99_us": float(np.percentile(lat, 99)),
            "c_abi_p50_us": float(np.percentile(raw, 50)), "c_abi_p99_us": float(np.percentile(raw, 99)),
            "kernel_p50_us": float(np.percentile(kern, 50)), "calls": int(len(lat)), "bytes_per_call": 512,
            "parity_check": bool(ok), "strings_checked": int(calls),
            "note": "host bytes in, ids on the host out, batch size 1; p50/p99 through Python ctypes, "
                    "c_abi = gtk_encode alone, kernel = the kernel's own globaltimer span"}


def sub_config_run(hx: Harness, name: str, merges, steps: int):
    """A short run of another config on this GPU: device-resident and end-to-end rates and its own check."""
    import gputok_b200
    from gputok_b200.capi import PinnedArray

    data, text_off, chunk, desc = make_workload(name, 0, 1, None)
    tok = gputok_b200.Tokenizer(merges, chunk_tokens=chunk, device=hx.torch.cuda.current_device())
    tok.set_stream(hx.stream.cuda_stream)
    # timed as a caller gets it (the pipeline as a whole); the stage breakdown comes from a second, shorter pass
    dev = device_resident_run(hx, tok, data, text_off, chunk, gputok_b200.GTK_MODE_OPT, steps, 3, per_stage=False)
    dev["stage_ms"] = device_resident_run(hx, tok, data, text_off, chunk, gputok_b200.GTK_MODE_OPT, 3, 1)["stage_ms"]
    pin = PinnedArray(len(data))
    pin.array[:] = data
    e2e_ms, h2d, d2h, _ = e2e_run(hx, tok, pin, text_off, gputok_b200.GTK_MODE_OPT, max(2, steps))
    seed = WORKLOADS[name][0]
    # the literal rule is quadratic in the chunk length: a 32 KiB chunk of config 4 costs one core 3.5 s
    threads = os.cpu_count() or 1
    ok, n = parity_on_sample(tok, data, text_off, chunk, gputok_b200.GTK_MODE_OPT, seed,
                             4.0 * threads if chunk > 8192 else 8.0, threads)
    n_bytes = len(data)
    out = dict(desc, value=n_bytes / (dev["ms_per_step"] * 1e-3) / 1e6, unit="MB/s", ms_per_step=dev["ms_per_step"],
               tokens_per_s=dev["n_ids"] / (dev["ms_per_step"] * 1e-3), tokens_per_byte=dev["n_ids"] / n_bytes,
               chunks=dev["n_chunks"], stage_ms=dev["stage_ms"],
               e2e={"value": n_bytes / (e2e_ms * 1e-3) / 1e6, "unit": "MB/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
               parity_check=ok, chunks_checked=n)
    pin.free()
    return out


def partition_run(hx: Harness, rank: int, world: int, merges, total_bytes: int, steps: int):
    """Config 5 as written: ONE batch of log-normal texts, cut into `world` contiguous byte ranges balanced by
    bytes; every GPU tokenises its range on its own (no collective on the data path), the per-range offsets
    are stitched on the host.  The ranks exchange scalars and, after the timed region, their offset arrays."""
    import gputok_b200
    from gputok_b200 import TextGen, partition_by_bytes, stitch_offsets

    torch, dist = hx.torch, hx.dist
    seed, _, chunk, mix, _ = WORKLOADS["cfg5"]
    off_all = TextGen.lognormal_offsets(seed * 1000, total_bytes)   # the same on every rank
    total_bytes = int(off_all[-1])
    bounds = partition_by_bytes(off_all, world)
    t_lo, t_hi = int(bounds[rank]), int(bounds[rank + 1])
    b_lo, b_hi = int(off_all[t_lo]), int(off_all[t_hi])
    first_block = b_lo // BLOCK
    n_blocks = (b_hi + BLOCK - 1) // BLOCK - first_block
    blocks = TextGen(seed).blocks(max(n_blocks, 1), BLOCK, first_block=first_block, mix=mix)
    data = np.ascontiguousarray(blocks[b_lo - first_block * BLOCK: b_hi - first_block * BLOCK])
    text_off = (off_all[t_lo:t_hi + 1] - b_lo).astype(np.int64)
    tok = gputok_b200.Tokenizer(merges, chunk_tokens=chunk, device=torch.cuda.current_device())
    tok.set_stream(hx.stream.cuda_stream)
    dev = device_resident_run(hx, tok, data, text_off, chunk, gputok_b200.GTK_MODE_OPT, steps, 3)
    my_ms = dev["ms_per_step"]
    per_gpu_ms = hx.gather(my_ms)
    per_gpu_bytes = hx.gather(float(len(data)))
    per_gpu_ids = [int(x) for x in hx.gather(float(dev["n_ids"]))]
    per_gpu_chunks = [int(x) for x in hx.gather(float(dev["n_chunks"]))]
    step_ms = max(per_gpu_ms)
    # parity of this rank's range on a seeded sample (each text is one chunk here)
    ok, n_checked = parity_on_sample(tok, data, text_off, chunk, gputok_b200.GTK_MODE_OPT, seed + rank,
                                     6.0 if world == 1 else 2.0, max(1, (os.cpu_count() or 1) // world))
    all_ok = hx.allmin(1.0 if ok else 0.0) > 0.5
    # host-side stitch: local offsets (each range starts at 0) + ids of the ranges before it
    t0 = time.perf_counter()
    if world > 1:
        longest = max(per_gpu_chunks) + 1
        mine = torch.zeros(longest, dtype=torch.int64, device="cuda")
        mine[:len(dev["coff"])] = torch.from_numpy(dev["coff"]).cuda()
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        parts = [t[:per_gpu_chunks[r] + 1].cpu().numpy() for r, t in enumerate(every)]
    else:
        parts = [dev["coff"]]
    stitched_ok = None
    stitch_ms = None
    if rank == 0:
        stitched = stitch_offsets(parts)
        stitch_ms = (time.perf_counter() - t0) * 1e3
        bases = np.concatenate([[0], np.cumsum(per_gpu_ids)])
        cuts = np.concatenate([[0], np.cumsum(per_gpu_chunks)])
        stitched_ok = bool(len(stitched) == len(off_all) and stitched[-1] == bases[-1]
                           and np.array_equal(stitched[cuts], bases) and np.all(np.diff(stitched) > 0)
                           and sum(per_gpu_chunks) == len(off_all) - 1)
    mean_ms = sum(per_gpu_ms) / len(per_gpu_ms)
    return {"workload": "cfg5 as one batch", "seed": seed, "total_bytes": total_bytes, "texts": int(len(off_all) - 1),
            "chunk_bytes": chunk, "lognormal": "median 2048, sigma 1.0, clipped to 64..65536",
            "partition": "contiguous runs of whole texts, balanced by bytes (partition_by_bytes)",
            "value": total_bytes / (step_ms * 1e-3) / 1e6, "unit": "MB/s",
            "tokens_per_s": sum(per_gpu_ids) / (step_ms * 1e-3), "ms_per_step": step_ms, "steps": steps,
            "per_gpu_ms": per_gpu_ms, "per_gpu_bytes": [int(b) for b in per_gpu_bytes], "per_gpu_ids": per_gpu_ids,
            "imbalance": max(per_gpu_ms) / mean_ms, "byte_imbalance": max(per_gpu_bytes) / (sum(per_gpu_bytes) / world),
            "stitched_ok": stitched_ok, "stitch_ms": stitch_ms, "parity_check": bool(all_ok),
            "chunks_checked_per_gpu": n_checked}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--bytes", type=int, default=0, help="override bytes per GPU (rounded up to 64 KiB)")
    ap.add_argument("--mode", default="opt", choices=["opt", "base"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip latency, the other configs and the partition run")
    ap.add_argument("--ref-budget-s", type=float, default=24.0, help="core-seconds of CPU work per reference step")
    ap.add_argument("--latency-calls", type=int, default=2000)
    ap.add_argument("--partition-bytes", type=int, default=4 << 30, help="size of the one batch of cfg5_partition")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch

    import gputok_b200
    from gputok_b200.capi import PinnedArray

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the tokenizer has no CPU fallback")
    if not os.path.exists(gputok_b200.library_path()):
        raise SystemExit("CUDA library not built: run `python __graft_entry__.py` first")
    hx = Harness(local_rank, world)

    data, text_off, chunk, desc = make_workload(args.workload, rank, world, args.bytes)
    n_bytes, n_texts = len(data), len(text_off) - 1
    mode = gputok_b200.GTK_MODE_OPT if args.mode == "opt" else gputok_b200.GTK_MODE_BASE
    tok = gputok_b200.Tokenizer(MERGES, chunk_tokens=chunk, device=local_rank)
    tok.set_stream(hx.stream.cuda_stream)

    sampler = ClockSampler(local_rank) if rank == 0 else None  # samples through warm-up and both timed regions
    # ---- device-resident arm ----
    dev = device_resident_run(hx, tok, data, text_off, chunk, mode, args.steps, args.warmup)
    n_ids, n_chunks = dev["n_ids"], dev["n_chunks"]
    per_gpu_ms = hx.gather(dev["ms_per_step"])
    step_ms = max(per_gpu_ms)                                   # the job is as slow as its slowest rank
    imbalance = step_ms / (sum(per_gpu_ms) / len(per_gpu_ms))   # identical work per rank here: ~1.0
    total_bytes = hx.allsum(float(n_bytes))
    total_ids = hx.allsum(float(n_ids))
    value = total_bytes / (step_ms * 1e-3) / 1e6

    # ---- end-to-end arm: pinned host text in, ids + offsets back on the host, every step ----
    pin = PinnedArray(n_bytes)
    pin.array[:] = data
    e2e_ms, h2d, d2h, n_ids_h = e2e_run(hx, tok, pin, text_off, mode, args.steps)
    e2e_ms = hx.allmax(e2e_ms)
    e2e_value = total_bytes / (e2e_ms * 1e-3) / 1e6
    clocks = sampler.stop() if sampler else None
    # ---- the same transfers without any kernel: what the host link allows at this N ----
    ceil_ms = hx.allmax(copy_ceiling_run(hx, n_bytes, n_ids_h, max(3, min(args.steps, 10))))
    copy_ceiling = total_bytes / (ceil_ms * 1e-3) / 1e6

    # ---- parity of the timed path: every rank checks a seeded sample of its own shard against the literal
    #      CPU rule; at N = 1 the CPU baseline's own sample doubles as the check ----
    check, checked = None, 0
    cpu_base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_base, (blob, boff, ref_ids) = time_cpu_baseline(data, text_off, chunk, WORKLOADS[args.workload][0])
        if not args.no_check:
            g_ids, _, g_coff, _ = tok.encode(blob, boff, mode=mode)
            check, checked = bool(np.array_equal(g_ids, ref_ids)), len(boff) - 1
    elif not args.no_check:
        ok, checked = parity_on_sample(tok, data, text_off, chunk, mode, WORKLOADS[args.workload][0] + 17 * rank,
                                       4.0 if world > 1 else 12.0, max(1, (os.cpu_count() or 1) // world))
        check = hx.allmin(1.0 if ok else 0.0) > 0.5

    # ---- N = 1 extras: latency mode and the other configs ----
    latency, configs, partition = None, None, None
    extras = not args.no_extras and args.workload == "cfg2" and not args.bytes and args.mode == "opt"
    del dev["coff"]
    pin.free()
    if world == 1 and args.workload == "cfg3" and not extras and args.latency_calls > 0:
        latency = latency_run(hx, MERGES, args.latency_calls)
    if extras and world == 1:
        latency = latency_run(hx, MERGES, args.latency_calls) if args.latency_calls > 0 else None
        configs = {}
        for name, k in (("cfg1", 10), ("cfg3", 10), ("cfg4", 5), ("cfg5", 3)):
            configs[name] = sub_config_run(hx, name, MERGES, k)
    if extras:
        partition = partition_run(hx, rank, world, MERGES, args.partition_bytes, 3)

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        tau = n_ids / n_bytes
        mean_chunk = n_bytes / max(n_chunks, 1)
        algo_bytes_per_byte = 1.0 + 4.0 * tau + 8.0 / mean_chunk + (8.0 / mean_chunk if n_texts > 1 else 0.0)
        kernel_bytes_per_byte = 1.0 + 2.0 * tau  # what the merge kernel itself moves: text in, 16-bit tokens out
        avg_merge_ms = dev["merge_ms"]
        achieved = algo_bytes_per_byte * n_bytes / (avg_merge_ms * 1e-3) / 1e9
        pipeline_gbs = algo_bytes_per_byte * n_bytes / (dev["ms_per_step"] * 1e-3) / 1e9
        kernel_gbs = kernel_bytes_per_byte * n_bytes / (avg_merge_ms * 1e-3) / 1e9
        line = {
            "metric": "input_MB_per_s", "value": value, "unit": "MB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u16", "data": "synthetic",
            "config": dict(desc, mode=args.mode, parallelism=f"byte-range shards x{world}, no collectives"),
            "tokens_per_s": total_ids / (step_ms * 1e-3), "tokens_per_byte": tau, "chunks_per_gpu": int(n_chunks),
            "wall_ms_per_step": dev["wall_ms_per_step"], "per_gpu_ms": per_gpu_ms, "imbalance": imbalance,
            "stage_ms": dev["stage_ms"],
            "e2e": {"value": e2e_value, "unit": "MB/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_ms, "steps": args.steps,
                    "copy_ceiling": copy_ceiling, "copy_ceiling_ms": ceil_ms, "frac_of_copy_ceiling": e2e_value / copy_ceiling,
                    "copy_ceiling_note": "the call's transfers alone (text up in 24 MiB slices, int32 ids down per "
                                         "slice, two copy streams, no kernels), all ranks at once"},
            "gpu_launches": dev["launches"],
            "roofline": {"bound": "hbm", "kernel": "k_merge_" + args.mode, "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak,
                         "traffic": (MERGE_OPT_DRAM_BYTES_PER_INPUT_BYTE * n_bytes
                                     if args.mode == "opt" and args.workload == "cfg2" else None),
                         "traffic_note": "a constant: ncu dram__bytes_read.sum + dram__bytes_write.sum of one k_merge_opt "
                                         "launch over 128 MiB of this text (201.1 MB), scaled by input bytes",
                         "peak_source": peak_kind,
                         "algorithmic_bytes_per_input_byte": algo_bytes_per_byte,
                         "frac_note": "frac = whole-path algorithmic bytes (text + int32 ids + offsets) over the merge "
                                      "kernel's time; frac_pipeline = the same bytes over ms_per_step (all kernels); "
                                      "frac_kernel_bytes = the bytes the merge kernel itself moves (1 + 2 tau) over its time",
                         "frac_pipeline": pipeline_gbs / peak, "achieved_pipeline": pipeline_gbs,
                         "kernel_bytes_per_input_byte": kernel_bytes_per_byte,
                         "frac_kernel_bytes": kernel_gbs / peak, "achieved_kernel_bytes": kernel_gbs,
                         "kernel_ms": avg_merge_ms, "input_GB_per_s_kernel": n_bytes / (avg_merge_ms * 1e-3) / 1e9},
            "cpu_baseline": cpu_base, "parity_check": check, "parity_chunks_checked_per_gpu": int(checked),
            "clocks": clocks,
        }
        if latency:
            line["latency"] = latency
        if configs:
            line["configs"] = configs
        if partition:
            line["cfg5_partition"] = partition
        print(json.dumps(line), flush=True)
    if world > 1:
        hx.dist.barrier()
        hx.dist.destroy_process_group()


if __name__ == "__main__":
    main()
