"""Benchmark of the greedy byte-level BPE path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One rank per GPU (torchrun for N > 1).  A step is one pass of the hot path over the rank's
batch of synthetic text.  Rank 0 prints ONE JSON line:

  value          whole-job input MB/s with the text already resident in HBM (device-resident call)
  e2e            the same metric through the host-buffer entry point: pinned host text -> H2D ->
                 kernels -> D2H ids + offsets, every step
  roofline       merge kernel: algorithmic bytes / CUDA-event time / measured HBM copy bandwidth
  cpu_baseline   the reference's CPU greedy tokenizer on a bounded sample, on this host's cores

Workloads (synthetic text from gputok_b200.TextGen; the reference's WikiText-103 is not available
offline):
  cfg2  256 MiB per GPU, seed 1, 4096-byte chunks   (default; the configuration the metric is quoted on)
  cfg1  1 MiB, seed 0, 1024-byte chunks
  cfg4  64 MiB, seed 3, 32 KiB chunks, multi-byte UTF-8 words and repeated-byte runs
  cfg5  512 MiB per GPU of the 4 GiB seed-4 text, log-normal text lengths (64 B..64 KiB)
  cfg3  latency: 10 000 strings of 512 B (seed 2), one call each; reports p50/p99 in the same line

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

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per input byte of one k_merge_opt launch, from the
# ncu capture summarised in profiles/k_merge_opt_cfg2_128MiB.md (202.3 MB for 128 MiB of config-2 text);
# traffic grows in proportion to the tile count, so a launch over n bytes moves this x n.
MERGE_OPT_DRAM_BYTES_PER_INPUT_BYTE = 202.3e6 / (128 << 20)

WORKLOADS = {
    #        seed  bytes per GPU   chunk   mix  lognormal
    "cfg1": (0, 1 << 20, 1024, 0, False),
    "cfg2": (1, 256 << 20, 4096, 0, False),
    "cfg3": (2, 10000 * 512, 2048, 0, False),
    "cfg4": (3, 64 << 20, 32768, 1, False),
    "cfg5": (4, 512 << 20, 65536, 1, True),
}


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


def sample_chunks(data: np.ndarray, text_off: np.ndarray, chunk: int, budget_cpu_s: float, seed: int):
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
    from oracle.loader import MODE_GREEDY

    runner, kind = cpu_reference_runner()
    blob, off, take = sample_chunks(data, text_off, chunk, budget_cpu_s, seed)
    cores = os.cpu_count() or 1
    t0 = time.perf_counter()
    ids, _ = runner.encode_chunks(blob, off, mode=MODE_GREEDY, threads=cores)
    dt = time.perf_counter() - t0
    return {"value": len(blob) / dt / 1e6, "unit": "MB/s", "cores": cores, "kind": kind,
            "sample": f"{len(take)} seeded chunks ({len(blob)} bytes) of the workload, literal Algorithm 1, "
                      f"one chunk per task on {cores} threads, {dt:.2f} s",
            "tokens_per_s": len(ids) / dt}, (blob, off, ids)


def run_reference_arm(args, rank: int, world: int):
    """--impl reference: the reference's CPU path on a bounded sample; rank 0 only."""
    if rank != 0:
        return
    from oracle.loader import MODE_GREEDY

    data, text_off, chunk, desc = make_workload(args.workload, 0, 1, min(args.bytes or (64 << 20), 64 << 20))
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
    sample = (f"{len(take)} seeded chunks ({len(blob)} bytes) per step, literal Algorithm 1 "
              f"(bpe_merge_cpu_greedy), one chunk per task on {cores} threads")
    line = {"impl": "reference", "metric": "input_MB_per_s", "value": mbs, "unit": "MB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u16",
            "data": "synthetic", "config": desc, "tokens_per_s": n_ids / dt,
            "cpu_baseline": {"value": mbs, "unit": "MB/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": mbs, "unit": "MB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


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
    ap.add_argument("--ref-budget-s", type=float, default=24.0, help="core-seconds of CPU work per reference step")
    ap.add_argument("--latency-calls", type=int, default=2000)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    import gputok_b200
    from gputok_b200.capi import PinnedArray

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the tokenizer has no CPU fallback")
    if not os.path.exists(gputok_b200.library_path()):
        raise SystemExit("CUDA library not built: run `python __graft_entry__.py` first")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def allmax(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def allsum(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    data, text_off, chunk, desc = make_workload(args.workload, rank, world, args.bytes)
    n_bytes, n_texts = len(data), len(text_off) - 1
    mode = gputok_b200.GTK_MODE_OPT if args.mode == "opt" else gputok_b200.GTK_MODE_BASE
    tok = gputok_b200.Tokenizer(MERGES, chunk_tokens=chunk, device=local_rank)
    stream = torch.cuda.current_stream()
    tok.set_stream(stream.cuda_stream)

    # ---- device-resident arm: text in HBM before the timed region ----
    d_bytes = torch.from_numpy(data).cuda()
    d_toff = torch.from_numpy(text_off).cuda()
    cap = n_bytes  # worst case one id per byte
    d_ids = torch.empty(cap, dtype=torch.int32, device="cuda")
    chunk_cap = n_bytes // chunk + n_texts + 2
    d_coff = torch.empty(chunk_cap, dtype=torch.int64, device="cuda")

    def step_device():
        return tok.encode_device(d_bytes.data_ptr(), n_bytes, d_toff.data_ptr(), n_texts, d_ids.data_ptr(), cap,
                                 d_coff.data_ptr(), chunk_cap, mode=mode)

    sampler = ClockSampler(local_rank) if rank == 0 else None  # samples through warm-up and both timed regions
    for _ in range(args.warmup):
        n_ids, n_chunks, _ = step_device()
    merge_ms, stage_acc, launches = [], np.zeros(5), 0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.perf_counter()
    ev0.record(stream)
    for _ in range(args.steps):
        n_ids, n_chunks, _ = step_device()
        st = tok.stage_ms()
        merge_ms.append(st["merge"])
        stage_acc += [st["chunker"], st["merge"], st["scan"], st["pack"], st["pipeline"]]
        launches += st["kernel_launches"]
    ev1.record(stream)
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    dev_ms = ev0.elapsed_time(ev1)  # CUDA events on the stream the kernels run on
    step_ms = allmax(dev_ms / args.steps)
    # per-GPU load imbalance: max / mean of the ranks' own step times (1.0 = perfectly balanced)
    if world > 1:
        mine = torch.tensor([dev_ms / args.steps], dtype=torch.float64, device="cuda")
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        per_gpu_ms = [float(t.item()) for t in every]
    else:
        per_gpu_ms = [dev_ms / args.steps]
    imbalance = max(per_gpu_ms) / (sum(per_gpu_ms) / len(per_gpu_ms))
    total_bytes = allsum(float(n_bytes))
    total_ids = allsum(float(n_ids))
    value = total_bytes / (step_ms * 1e-3) / 1e6

    # ---- end-to-end arm: pinned host text in, ids + offsets back on the host, every step ----
    pin = PinnedArray(n_bytes)
    pin.array[:] = data
    e2e_steps = max(2, min(args.steps, 5))
    tok.encode(pin.array, text_off, mode=mode, copy=False)
    barrier()
    t0 = time.perf_counter()
    ev0.record(stream)
    for _ in range(e2e_steps):
        ids_h, toff_h, coff_h, _ = tok.encode(pin.array, text_off, mode=mode, copy=False)
        _ = int(ids_h[-1]) + int(coff_h[-1])  # touch the result on the host
    ev1.record(stream)
    barrier()
    e2e_ms = allmax(max(ev0.elapsed_time(ev1), 0.0) / e2e_steps)
    e2e_wall_ms = allmax((time.perf_counter() - t0) * 1e3 / e2e_steps)
    e2e_value = total_bytes / (e2e_wall_ms * 1e-3) / 1e6
    clocks = sampler.stop() if sampler else None
    h2d = n_bytes + 8 * (n_texts + 1)
    d2h = 4 * len(ids_h) + 8 * len(coff_h) + 8 * len(toff_h) + 32

    # ---- CPU baseline on rank 0 at N=1; its ids double as the parity check of the timed GPU path
    #      (the checker runs only here, never inside a timed region) ----
    check = None
    cpu_base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_base, (blob, boff, ref_ids) = time_cpu_baseline(data, text_off, chunk, WORKLOADS[args.workload][0])
        if not args.no_check:  # the GPU result on exactly the sampled chunks equals the literal rule
            g_ids, _, g_coff, _ = tok.encode(blob, boff, mode=mode)
            check = bool(np.array_equal(g_ids, ref_ids))

    # ---- latency mode (cfg3 only): one call per string, host in / host out ----
    latency = None
    if args.workload == "cfg3" and rank == 0:
        import ctypes
        lat, kern, raw = [], [], []
        one = np.array([0, 512], dtype=np.int64)
        ms = ctypes.c_float()
        for i in range(min(args.latency_calls, n_texts)):
            s = pin.array[text_off[i]:text_off[i + 1]]
            t1 = time.perf_counter()
            _, _, _, k_ms = tok.encode(s, None, mode=mode, copy=False)   # the Python call a user makes
            lat.append((time.perf_counter() - t1) * 1e6)
            kern.append(k_ms * 1e3)
            t1 = time.perf_counter()                                      # the C ABI call alone
            tok._lib.gtk_encode(tok._h, int(mode), s.ctypes.data, one.ctypes.data, 1, ctypes.byref(ms))
            raw.append((time.perf_counter() - t1) * 1e6)
        lat, kern, raw = np.array(lat[10:]), np.array(kern[10:]), np.array(raw[10:])
        latency = {"p50_us": float(np.percentile(lat, 50)), "p99_us": float(np.percentile(lat, 99)),
                   "c_abi_p50_us": float(np.percentile(raw, 50)), "c_abi_p99_us": float(np.percentile(raw, 99)),
                   "kernel_p50_us": float(np.percentile(kern, 50)),
                   "calls": int(len(lat)), "bytes_per_call": 512,
                   "note": "host bytes in, ids on the host out; p50/p99 through Python ctypes, c_abi = gtk_encode alone"}

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        tau = n_ids / n_bytes
        mean_chunk = n_bytes / max(n_chunks, 1)
        algo_bytes_per_byte = 1.0 + 4.0 * tau + 8.0 / mean_chunk + (8.0 / mean_chunk if n_texts > 1 else 0.0)
        avg_merge_ms = float(np.mean(merge_ms))
        achieved = algo_bytes_per_byte * n_bytes / (avg_merge_ms * 1e-3) / 1e9
        line = {
            "metric": "input_MB_per_s", "value": value, "unit": "MB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u16", "data": "synthetic",
            "config": dict(desc, mode=args.mode, parallelism=f"byte-range shards x{world}, no collectives"),
            "tokens_per_s": total_ids / (step_ms * 1e-3), "tokens_per_byte": tau, "chunks_per_gpu": int(n_chunks),
            "wall_ms_per_step": wall_ms / args.steps, "per_gpu_ms": per_gpu_ms, "imbalance": imbalance,
            "stage_ms": {k: float(v / args.steps) for k, v in zip(("chunker", "merge", "scan", "pack", "pipeline"),
                                                               stage_acc)},
            "e2e": {"value": e2e_value, "unit": "MB/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_wall_ms, "steps": e2e_steps},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "k_merge_" + args.mode, "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak,
                         "traffic": (MERGE_OPT_DRAM_BYTES_PER_INPUT_BYTE * n_bytes
                                     if args.mode == "opt" and args.workload == "cfg2" else None),
                         "traffic_note": "ncu DRAM bytes of a 128 MiB launch scaled by input bytes",
                         "peak_source": peak_kind,
                         "algorithmic_bytes_per_input_byte": algo_bytes_per_byte,
                         "kernel_ms": avg_merge_ms, "input_GB_per_s_kernel": n_bytes / (avg_merge_ms * 1e-3) / 1e9},
            "cpu_baseline": cpu_base, "parity_check": check, "clocks": clocks,
        }
        if latency:
            line["latency"] = latency
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
