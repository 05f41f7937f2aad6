"""Benchmark of the batched search path: QPS at recall@10 >= 0.99, k = 10, 10 000-query batches.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One process per GPU (torchrun for N > 1).  A step is one search of ONE 10 000-query batch of the
workload "descriptor-1m" (1 000 000 x 128 descriptor-like rows).  With one GPU the whole index is on
it.  With N > 1 the index is placed with `placement = shard`: the copies and the rows of the
neighbor table are split over the GPUs, every GPU runs the first round of all queries over its
copies, the kept lists are exchanged over NCCL, every GPU runs the waves of its slice of the batch
and the results are gathered — the same batch answered by all GPUs together, so the work per step
is fixed as N grows ("scaling": "strong").  The same run also reports, as secondary fields, the
throughput of N independent whole-index replicas each answering its own batches (`replicas_qps`,
no collective) and how the sharded answer compares with one GPU's and with the CPU checker's.
Data are seeded synthetic stand-ins for the public sets the reference is quoted on.

Rank 0 prints one JSON line.  `value` is measured with the queries already on the GPU (the
reference's --resident protocol, cpp/bench/octex_bench.cu:223-253 of hpdic/octex); `e2e` goes
through the host-buffer call with both copies inside the timed region.
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

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "QPS at recall@10 >= 0.99, k=10, 10k-query batch"
K = 10

# build parameters per workload (the builder's choice; the reference's paper settings for the
# matching public set are in bench/paper_build.sh:33-55) and the search-parameter ladder tried
# from cheap to expensive until recall@10 >= 0.99 (the tuning recipe of docs/guide.md:235-251)
WORKLOADS = {
    "descriptor-1m": dict(
        gen="descriptor_like", n=1_000_000, dim=128, nq=10_000,
        build=dict(copies=64, blocks=4, pca_dims=64, list_len=32, min_cell=16, log_buckets=20,
                   sketch_width=64, table_len=64)),
    # the generator of the 10M / 1B embedding configurations at a size one GPU builds in seconds
    "embedding-1m": dict(
        gen="embedding_like", n=1_000_000, dim=96, nq=10_000,
        build=dict(copies=64, blocks=4, pca_dims=64, list_len=32, min_cell=16, log_buckets=20,
                   sketch_width=64, table_len=64,  # the reference's rule gives 96: same recall, 30 % slower
                   exact_table_max=0)),  # the table by the index's own search: better recall here than the exact one
    # BASELINE.json config 1: the index at the reference's defaults
    # (cpp/include/cuvs/neighbors/octex.hpp:32-92: 200 copies, lists of 64, 2^20 buckets, table of 64,
    # sketch width chosen from the dimension) and its stated search parameters, not retuned
    "plumbing-100k": dict(
        gen="plumbing", n=100_000, dim=128, nq=1_000,
        build=dict(copies=200, blocks=4, pca_dims=64, list_len=64, min_cell=1, log_buckets=20,
                   sketch_width=0, table_len=64),
        search=dict(read=8, starts=32, waves=1, rerank=128, wave_rerank=128)),
    # BASELINE.json config 3: 960-dimensional global-descriptor-like rows, 1 000 queries
    "global-1m": dict(
        gen="global_descriptor_like", n=1_000_000, dim=960, nq=1_000,
        build=dict(copies=96, blocks=4, pca_dims=64, list_len=64, min_cell=16, log_buckets=20,
                   sketch_width=128, table_len=64)),
    # BASELINE.json config 4: 10 M embedding-like rows (shard placement with --gpus 2/4/8)
    "embedding-10m": dict(
        gen="embedding_like", n=10_000_000, dim=96, nq=10_000,
        build=dict(copies=64, blocks=4, pca_dims=64, list_len=32, min_cell=16, log_buckets=20,
                   sketch_width=64, table_len=64, exact_table_max=0)),
}
LADDER = [
    dict(read=16, starts=32, waves=1, rerank=128, wave_rerank=384),
    dict(read=8, starts=24, waves=2, rerank=128, wave_rerank=256),
    dict(read=8, starts=32, waves=2, rerank=256, wave_rerank=256),
    dict(read=32, starts=32, waves=2, rerank=256, wave_rerank=256),
    dict(read=32, starts=32, waves=3, rerank=256, wave_rerank=256),
    dict(read=32, starts=128, waves=3, rerank=256, wave_rerank=256),
    dict(read=32, starts=128, waves=2, rerank=512, wave_rerank=512),
    dict(read=32, starts=192, waves=3, rerank=384, wave_rerank=384),
    dict(read=32, starts=256, waves=3, rerank=512, wave_rerank=512),
    dict(read=32, starts=256, waves=4, rerank=512, wave_rerank=512),
    dict(read=32, starts=384, waves=4, rerank=512, wave_rerank=512),
    dict(read=64, starts=512, waves=4, rerank=512, wave_rerank=512),
]


# DRAM bytes (read + write) of one launch, from the ncu capture of this bench at its default workload
# and the first rung of LADDER (profiles/round_kernel_descriptor-1m.md). Reported as
# roofline.traffic only when the run uses exactly that workload and those parameters.
NCU_TRAFFIC = {"round_rows": 1.156e9, "round_lists": 0.651e9}


def torch_build(w):
    """Build parameters the torch restatement of the builder knows (it always makes an exact table)."""
    return {k_: v for k_, v in w["build"].items() if k_ not in ("exact_table_max", "table_passes")}


def given_search(args):
    """--search JSON over the defaults of search_params (cpp/include/cuvs/neighbors/octex.hpp:101-135)."""
    sp = dict(read=32, starts=128, waves=2, rerank=128, wave_rerank=128)
    sp.update(json.loads(args.search))
    return sp


def log(*a):
    print(*a, file=sys.stderr, flush=True)


class ClockSampler:
    """SM clock and throttle reasons of one GPU, sampled every few milliseconds from before the
    warm-up until after the timed region (read-only NVML queries; `nvidia-smi` in a loop where the
    NVML binding is missing); `summary` reports the samples that fall inside the timed region."""
    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu, uuid=None, period_s=0.002):
        self.gpu, self.uuid, self.period = gpu, uuid, period_s
        self.rows, self.proc, self.thread = [], None, None
        self.t0 = self.t1 = None
        self.stop = threading.Event()
        self.max_mhz = None
        self.how = None

    def _nvml_loop(self, nv, handle):
        while not self.stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(handle)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.rows.append((time.perf_counter(), float(mhz), int(mask)))
            except Exception:
                pass
            time.sleep(self.period)

    def _smi_loop(self):
        for line in self.proc.stdout:
            c = [x.strip() for x in line.split(",")]
            if len(c) >= 6 and c[0].replace(".", "").isdigit():
                mask = sum(bit for (_, bit), v in zip(self.REASONS, c[2:6]) if v.lower().startswith("active"))
                self.max_mhz = float(c[1]) if c[1].replace(".", "").isdigit() else self.max_mhz
                self.rows.append((time.perf_counter(), float(c[0]), mask))

    def __enter__(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            handle = None
            if self.uuid:
                for cand in (self.uuid, "GPU-" + self.uuid):
                    try:
                        handle = nv.nvmlDeviceGetHandleByUUID(cand.encode() if isinstance(cand, str) else cand)
                        break
                    except Exception:
                        handle = None
            if handle is None:
                handle = nv.nvmlDeviceGetHandleByIndex(self.gpu)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.how = "nvml"
        except Exception:
            try:
                self.proc = subprocess.Popen(
                    ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}",
                     "--format=csv,noheader,nounits", "-lms", "5"],
                    stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
                self.thread = threading.Thread(target=self._smi_loop, daemon=True)
                self.how = "nvidia-smi"
            except OSError:
                self.thread = None
        if self.thread is not None:
            self.thread.start()
        return self

    def begin(self):
        self.t0 = time.perf_counter()

    def end(self):
        self.t1 = time.perf_counter()

    def __exit__(self, *exc):
        time.sleep(0.02)
        self.stop.set()
        if self.proc is not None:
            self.proc.terminate()
            self.proc.wait(timeout=5)
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        inside = [r for r in self.rows if self.t0 is not None and self.t0 <= r[0] <= (self.t1 or r[0])]
        near = False
        if not inside and self.rows and self.t0 is not None:
            # no sample fell inside: the ones nearest to the region on either side
            mid = 0.5 * (self.t0 + (self.t1 or self.t0))
            inside = sorted(self.rows, key=lambda r: abs(r[0] - mid))[:4]
            near = True
        sm = [r[1] for r in inside]
        mask = 0
        for r in inside:
            mask |= r[2]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": [n for n, bit in self.REASONS if mask & bit],
                "samples": len(sm), "samples_total": len(self.rows), "source": self.how,
                "nearest_to_region": near}


def make_data(w, rank_seed):
    from octex_b200 import synth
    gen = getattr(synth, w["gen"])
    base = gen(w["n"], w["dim"], seed=0)
    queries = gen(w["nq"], w["dim"], seed=1 + rank_seed)
    return base, queries


def ground_truth(vectors16, queries_t, k, rows_at_once=1 << 19):
    """Exact k nearest stored rows of every query (fp32 arithmetic on the GPU, in blocks of rows)."""
    import torch
    out = []
    for q0 in range(0, queries_t.shape[0], 2048):
        q = queries_t[q0:q0 + 2048]
        best_d = best_i = None
        for r0 in range(0, vectors16.shape[0], rows_at_once):
            v = vectors16[r0:r0 + rows_at_once].float()
            d, i = ((v * v).sum(1)[None, :] - 2.0 * (q @ v.T)).topk(min(k, v.shape[0]), dim=1, largest=False)
            i = i + r0
            if best_d is not None:
                d, i = torch.cat([best_d, d], 1), torch.cat([best_i, i], 1)
                d, at = d.topk(k, dim=1, largest=False)
                i = i.gather(1, at)
            best_d, best_i = d, i
        out.append(best_i)
    return torch.cat(out).cpu().numpy()


def recall_of(ids, truth):
    hits = (ids[:, :, None] == truth[:, None, :]).any(-1).sum()
    return float(hits) / truth.size


def algorithmic_bytes(stats, sp, meta, k):
    """Bytes each kernel has to move for the batch, from the kernels' own per-query counters
    (levels tried, keys scanned, list entries, distinct ids, table rows, reranked rows)."""
    D, S, L2 = meta["dim"], meta["sketch_width"], meta.get("table_len", 0)
    KO = max(sp["starts"], k)
    n1 = stats[:, 3]
    r1 = np.minimum(n1, sp["rerank"])  # the first round starts from an empty kept list
    waves = sp["waves"]
    S4 = S + 4  # a sketch row of the first round: its codes and its fp32 constant
    lists = (4 * stats[:, 2] + n1 * S4 + r1 * 2 * D + 4 * D + 4 * S + KO * 12).sum()
    pairs = len(stats) * meta["copies"]
    # the cell lookup happens inside the projection kernel: 16-byte table slots examined and the
    # segment written per (query, copy), next to the fp16 queries read
    out = {"project": int((stats[:, 1] * 16).sum() + pairs * 8 + len(stats) * 2 * D),
           "round_lists": int(lists)}
    if waves:
        rerank_w = stats[:, 7] - r1  # rows the waves read (ids already kept are not read again)
        rows = (stats[:, 4] * 4 * L2 + stats[:, 5] * S + rerank_w * 2 * D).sum() \
            + waves * len(stats) * (4 * D + 4 * S + 2 * KO * 12)
        out["round_rows"] = int(rows / waves)  # per launch
    return out


def workload_config(args, w, sp, world):
    """The part of `config` that names the workload; both arms print the same."""
    return {"workload": args.workload, "n": w["n"], "dim": w["dim"], "queries_per_step": w["nq"],
            "k": K, "placement": "shard" if world > 1 else "one GPU", "build": w["build"], "search": sp}


def run_reference(args, rank, world):
    """The reference has no CPU search; its CPU arm is the CPU restatement of the path (oracle/),
    timed on all host threads on a bounded sample of the same workload."""
    if rank != 0:
        return
    from octex_b200 import build_index
    from oracle import oracle_py
    import torch
    w = WORKLOADS[args.workload]
    base, queries = make_data(w, 0)
    if torch.cuda.is_available() and args.builder == "native":
        # the same directory the other arm searches: the library's builder with the same seed
        import shutil
        import octex_b200
        from octex_b200 import index_dir
        path = os.path.join(args.index_dir, args.workload + "-reference-arm")
        shutil.rmtree(path, ignore_errors=True)
        octex_b200.build_native(base, path, **w["build"])
        arrays, meta = index_dir.read_index(path)
    else:
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        arrays, meta = build_index.build_arrays(base, build_index.IndexParams(**torch_build(w)), device=dev)
    ox = oracle_py.Index(arrays, meta)
    sp = given_search(args) if args.search else dict(w.get("search", LADDER[args.ladder_start]))
    sample = queries[:args.cpu_sample]
    cores = os.cpu_count() or 1
    for _ in range(max(args.warmup, 1)):
        ox.search(sample[:64], K, **sp)
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        ox.search(sample, K, **sp)
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    qps = len(sample) / t
    config = workload_config(args, w, sp, world)
    config["note"] = ("CPU restatement of the search path (the reference has no CPU search), all copies "
                      "in this process's memory")
    line = {"impl": "reference", "metric": METRIC, "value": qps, "unit": "queries/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16/f32/i8",
            "data": "synthetic", "config": config,
            "cpu_baseline": {"value": qps, "unit": "queries/s", "cores": cores, "kind": "port",
                             "sample": f"{len(sample)} of {w['nq']} queries per step, same index"},
            "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


# stdout carries exactly one line, the JSON: libraries that log there (NCCL prints its version banner
# on stdout whatever its log file is) are sent to stderr by pointing descriptor 1 at descriptor 2
# for the run, and the line is written to the saved descriptor
_STDOUT_FD = None


def claim_stdout():
    global _STDOUT_FD
    if _STDOUT_FD is None:
        sys.stdout.flush()
        _STDOUT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _STDOUT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_STDOUT_FD, data)


def timed_resident(idx, nq, sp, steps, warmup, flush, barrier, clocks=None):
    """`steps` graph replays of the batch already on the GPU, L2 flushed before each; CUDA events on
    torch's current stream (the library orders its own stream after it and signals back to it).
    Returns the milliseconds of every step and the wall time of the region."""
    import torch
    stream = torch.cuda.current_stream()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for _ in range(warmup):
        flush.fill_(1)
        idx.search_resident(nq, K, stream=stream.cuda_stream, **sp)
    barrier()
    if clocks is not None:
        clocks.begin()
    wall0 = time.perf_counter()
    for a, b in ev:
        flush.fill_(1)  # evict the index from L2 between timed steps
        a.record(stream)
        idx.search_resident(nq, K, stream=stream.cuda_stream, **sp)
        b.record(stream)
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall0
    if clocks is not None:
        clocks.end()
    return [a.elapsed_time(b) for a, b in ev], wall


def parity_against_checker(idx, arrays_host, meta, queries, ids_run, dist_run, truth, sp, n_sample, parts=1):
    """The north star's own criteria on a sample of the bench batch: the GPU's answer for the
    timed path (`ids_run`, `dist_run`: nothing kept for inspection) against the CPU checker started
    from the GPU's own projected coordinates (the inspected run gives them)."""
    from oracle import oracle_py
    sample = queries[:n_sample]
    idx.set_debug(taps=True)
    _, ids_tap = idx.search(sample, K, **sp)
    y = idx.fetch("y", np.uint16, (len(sample), -1))
    idx.set_debug(taps=False)
    ox = oracle_py.Index(arrays_host, meta)
    want_i, want_d, _ = ox.search(sample, K, y_in=y, parts=parts, **sp)
    got_i, got_d = ids_run[:len(sample)], dist_run[:len(sample)]
    same = got_i == want_i
    rel = np.abs(got_d[same] - want_d[same]) / np.maximum(np.abs(want_d[same]), 1e-30)
    return {"sample_queries": int(len(sample)),
            "ids_match_frac": float(same.mean()),
            "ids_match_frac_inspected_run": float((ids_tap == want_i).mean()),
            "dist_max_rel": float(rel.max()) if rel.size else 0.0,
            "recall_gpu": recall_of(got_i, truth[:len(sample)]),
            "recall_oracle": recall_of(want_i, truth[:len(sample)]),
            "criteria": "ids >= 0.999 of slots, distances within 1e-3 relative, |recall difference| <= 0.002"}


def reference_kernels(arrays, meta, idx, queries, ids_run, sp, kernel_ms, steps):
    """The reference's own search kernels (oracle/_ref/libref_search.so: its search_kernels.cuh
    compiled unmodified for this GPU) on the same index, batch and parameters, from the GPU's
    projected coordinates; L2 flushed before each timed stage as for the kernels of this library.
    Outside the timed region; a report beside the number, like the CPU baseline."""
    from oracle import oracle_py
    if oracle_py.ref_search() is None:
        return {"unavailable": "oracle/_ref/libref_search.so is not built (reference sources not at hand)"}
    nq = len(queries)
    idx.set_debug(taps=True)
    idx.search(queries, K, **sp)
    y = idx.fetch("y", np.uint16, (nq, -1))
    qs = idx.fetch("qs", np.float32, (nq, -1))
    idx.set_debug(taps=False)
    ref = oracle_py.ref_search_pipeline(arrays, meta, y, qs, queries, K, reps=max(3, min(steps, 10)),
                                        flush_mb=256, **sp)
    ours_first = sum(kernel_ms.get(k_, 0.0) for k_ in ("project", "cell_codes", "probe", "round_lists"))
    ours_waves = kernel_ms.get("round_rows", 0.0) * sp["waves"]
    ref_first, ref_waves = float(ref["kernel_ms"][0]), float(ref["kernel_ms"][1])
    return {"first_round_ms": ref_first, "waves_ms": ref_waves,
            "stages": "cell lookup + gather + rerank-keep | waves x (pick starts + gather + rerank-keep); "
                      "its projection GEMM (cuBLASLt) is not included",
            "this_library_first_round_ms": ours_first, "this_library_waves_ms": ours_waves,
            "this_library_stages": "projection + decode + lookup + first round | waves",
            "ratio": (ref_first + ref_waves) / max(ours_first + ours_waves, 1e-9),
            "ids_match_frac": float((ref["best_ids"] == ids_run).mean()),
            "l2": "256 MB written before each timed stage, median of the repetitions"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="octex_b200")
    ap.add_argument("--workload", default="descriptor-1m", choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-sample", type=int, default=2000)
    ap.add_argument("--ladder-start", type=int, default=0)
    ap.add_argument("--e2e-batch", type=int, default=0,
                    help="queries per captured batch of the host-buffer call (search_params.batch); 0: half the call")
    ap.add_argument("--builder", default="native", choices=["native", "torch"],
                    help="native: the library's own GPU builder writes the index directory (to "
                         "--index-dir) and the index is loaded from it; torch: the package's torch "
                         "restatement of the builder makes the arrays in GPU memory")
    ap.add_argument("--index-dir", default="/dev/shm/octex_b200_bench",
                    help="where the native builder puts the index directory of the run")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref-kernels", action="store_true")
    ap.add_argument("--copies", type=int, default=0, help="override the copies of the build")
    ap.add_argument("--table", default="", choices=["", "exact", "searched"],
                    help="override how the build makes the neighbor table (index_params.exact_table_max)")
    ap.add_argument("--search", default="", help="JSON search parameters (skips the ladder)")
    ap.add_argument("--queries", type=int, default=0,
                    help="queries per batch instead of the workload's (small profiler captures)")
    ap.add_argument("--placement", default="shard", choices=["shard", "shard-rows"],
                    help="with several GPUs: shard = copies and the neighbor table split over the GPUs, "
                         "kept lists exchanged over NCCL; shard-rows = the sketch and the fp16 vectors "
                         "dealt by rows too")
    args = ap.parse_args()
    claim_stdout()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.copies:
        WORKLOADS[args.workload]["build"]["copies"] = args.copies
    if args.table:
        WORKLOADS[args.workload]["build"]["exact_table_max"] = 0 if args.table == "searched" else 1 << 40
    if args.queries:
        WORKLOADS[args.workload]["nq"] = args.queries
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    import octex_b200
    from octex_b200 import build_index

    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    w = WORKLOADS[args.workload]
    sharded = world > 1  # one batch answered by all GPUs together
    t0 = time.time()
    base, queries = make_data(w, 0)  # every rank draws the same data: one index, one batch
    log(f"[rank {rank}] data {time.time() - t0:.1f}s")
    t0 = time.time()
    build_seconds = None
    if args.builder == "native":
        # one process builds the directory, every process loads from it
        from octex_b200 import index_dir
        import shutil
        path = os.path.join(args.index_dir, args.workload)
        if local == 0:
            shutil.rmtree(path, ignore_errors=True)
            octex_b200.build_native(base, path, verbose=(rank == 0), **w["build"])
        if world > 1:
            dist.barrier()
        host_arrays, meta = index_dir.read_index(path)
        build_seconds = meta.get("build_seconds")
        log(f"[rank {rank}] index directory ready in {time.time() - t0:.1f}s ({build_seconds})")
        whole = octex_b200.load(path, devices=[local], placement="replicate")  # the whole index on this GPU
        if sharded:
            from octex_b200 import dist as odist
            rows = args.placement == "shard-rows"
            idx = octex_b200.load(path, devices=[local], placement="shard", rank=rank, world=world,
                                  shard_vectors=rows, sketch="shard" if rows else "replicate")
            odist.connect(idx)
        else:
            idx = whole
        arrays = {"vectors": torch.as_tensor(np.asarray(host_arrays["vectors"]), device="cuda")}
        index_bytes = sum(int(v.nbytes) for v in host_arrays.values())
    else:
        arrays, meta = build_index.build_arrays(base, build_index.IndexParams(**torch_build(w)),
                                                device=f"cuda:{local}", keep_on_device=True,
                                                verbose=(rank == 0))
        torch.cuda.synchronize()
        log(f"[rank {rank}] index built in {time.time() - t0:.1f}s")
        whole = octex_b200.attach(arrays, meta, borrow=True)  # the whole index on this GPU
        if sharded:
            from octex_b200 import dist as odist
            rows = args.placement == "shard-rows"
            idx = octex_b200.attach(arrays, meta, borrow=False, rank=rank, world=world, placement="shard",
                                    shard_vectors=rows, sketch="shard" if rows else "replicate")
            odist.connect(idx)
        else:
            idx = whole
        host_arrays = None
        index_bytes = sum(v.numel() * v.element_size() for v in arrays.values())
    nq = len(queries)
    q_dev = torch.as_tensor(queries, device="cuda")
    truth = ground_truth(arrays["vectors"], q_dev, K)

    # search parameters: the cheapest rung of the ladder that reaches recall@10 >= 0.99
    chosen, rec = None, 0.0
    ids_run = dist_run = None
    fixed = [given_search(args)] if args.search else ([dict(w["search"])] if "search" in w else None)
    for sp in (fixed or LADDER[args.ladder_start:]):
        try:
            d_, i_ = idx.search(q_dev, K, **sp)
        except ValueError as e:  # a rung beyond the limits of this index (starts x table_len)
            if fixed:
                raise
            log(f"[rank {rank}] {sp} skipped: {e}")
            continue
        r = recall_of(i_.cpu().numpy(), truth)
        log(f"[rank {rank}] {sp} recall@10 {r:.4f}")
        if r > rec:
            chosen, rec = sp, r
            ids_run, dist_run = i_.cpu().numpy(), d_.cpu().numpy()
        if r >= 0.99:
            break
    sp = chosen

    # per-query counters of what the kernels read, for the algorithmic bytes
    idx.set_debug(stats=True)
    idx.search(q_dev, K, **sp)
    stats = idx.fetch("stats", np.int64, (-1, 8))
    idx.set_debug(stats=False)
    local_meta = dict(meta, copies=meta["copies"] // world if sharded else meta["copies"])
    alg = algorithmic_bytes(stats, sp, local_meta, K)

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # > L2 (126 MB)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- value: queries resident on the GPU, one graph replay per step ----
    idx.search(q_dev, K, **sp)  # leaves the batch on the GPU
    uuid = str(getattr(torch.cuda.get_device_properties(local), "uuid", "") or "")
    with ClockSampler(local, uuid) as clocks:
        step_ms, wall = timed_resident(idx, nq, sp, args.steps, args.warmup, flush, barrier, clocks)
    total_ms = sum(step_ms)
    barrier()

    # ---- per-kernel milliseconds, same batch, launched kernel by kernel ----
    prof = {}
    for _ in range(args.steps):
        flush.fill_(1)
        torch.cuda.synchronize()  # the fill runs on torch's stream, the batch on the library's
        for name, ms in idx.profile_batch(nq, K, **sp):
            key = name.split("[")[0]
            prof.setdefault(key, []).append(ms)
    kernel_ms = {k_: statistics.mean(v) for k_, v in prof.items()}
    launches_per_step = {k_: len(v) // args.steps for k_, v in prof.items()}

    # ---- e2e: host buffers, copies inside the timed region ----
    q_pin = torch.as_tensor(queries).pin_memory()
    out_i = torch.empty((nq, K), dtype=torch.int64).pin_memory()
    out_d = torch.empty((nq, K), dtype=torch.float32).pin_memory()
    qn, on, od = q_pin.numpy(), out_i.numpy(), out_d.numpy()
    def host_call_seconds(batch):
        kw = dict(sp, batch=batch) if batch else sp
        for _ in range(args.warmup):
            idx.search(qn, K, neighbors=on, distances=od, **kw)
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            idx.search(qn, K, neighbors=on, distances=od, **kw)
        torch.cuda.synchronize()
        return time.perf_counter() - t0

    # One process: the call's queries go through in captured batches of --e2e-batch on two streams
    # (search_params.batch), so the copies of one batch run under the kernels of the other; the
    # figure with the whole call as one captured batch is kept beside it. Several processes
    # exchange inside a batch and take the call as one.
    e2e_one_s = host_call_seconds(0)
    ids_one_batch = on.copy()
    e2e_s, e2e_batch, e2e_split_s = e2e_one_s, 0, None
    first = args.e2e_batch or nq // 2
    if not sharded and 1 <= first < nq:
        # half and a quarter of the call (or --e2e-batch and half of it): the slower the bus of the
        # host, the finer the batches that pay
        for b in (first, max(first // 2, 1)):
            t = host_call_seconds(b)
            if e2e_split_s is None or t < e2e_split_s[0]:
                e2e_split_s = (t, b)
        if e2e_split_s[0] < e2e_s:  # else a fast bus leaves nothing to hide: the call as one batch
            e2e_s, e2e_batch = e2e_split_s
        idx.search(qn, K, neighbors=on, distances=od, **(dict(sp, batch=e2e_batch) if e2e_batch else sp))
    rec_e2e = recall_of(on, truth)
    e2e_same = bool(np.array_equal(on, ids_run)) and bool(np.array_equal(ids_one_batch, ids_run))

    # ---- several GPUs: what the sharded answer is worth, and the replica figure beside it ----
    multi = {}
    if sharded:
        # (a) the same batch answered by this GPU alone from the whole index
        _, i_one = whole.search(q_dev, K, **sp)
        i_one = i_one.cpu().numpy()
        multi["ids_match_one_gpu"] = float((i_one == ids_run).mean())
        multi["recall_one_gpu"] = recall_of(i_one, truth)
        # (b) N independent replicas, every GPU its own batches, no collective (secondary figure)
        whole.search(q_dev, K, **sp)
        rep_ms, _ = timed_resident(whole, nq, sp, args.steps, args.warmup, flush, barrier)
        t = torch.tensor([sum(rep_ms)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        multi["replicas_qps"] = world * nq * args.steps / (float(t[0]) * 1e-3)
        multi["replicas_note"] = ("every GPU holds the whole index and answers its own batches: weak "
                                  "scaling, no data-path collective; not the headline value")
        # (c) the sharded search against the CPU checker in its sharded mode (first round per part,
        # merge of the parts' kept lists), bit for bit: the dimension-ordered projection gives
        # coordinates the checker reproduces itself
        ns = min(500, nq)
        idx.set_projection(ordered=True)
        d_s, i_s = idx.search(queries[:ns], K, **sp)
        idx.set_projection(ordered=False)
        if rank == 0:
            from oracle import oracle_py
            host = host_arrays if host_arrays is not None else {k_: v.cpu().numpy() for k_, v in arrays.items()}
            want_i, want_d, _ = oracle_py.Index(host, meta).search(queries[:ns], K, parts=world, **sp)
            multi["ids_match_checker_parts"] = float((want_i == i_s).mean())
            multi["dist_equal_checker_parts"] = bool(np.array_equal(want_d.view(np.uint32), d_s.view(np.uint32)))
            multi["checker_sample_queries"] = ns
            del host

    if world > 1:
        t = torch.tensor([total_ms, e2e_s * 1e3], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms = float(t[0]), float(t[1])
        r = torch.tensor([rec, rec_e2e], device="cuda", dtype=torch.float64)
        dist.all_reduce(r, op=dist.ReduceOp.MIN)
        rec, rec_e2e = float(r[0]), float(r[1])
        # per-kernel milliseconds of every rank (the slowest rank sets the pace of a stage)
        names = sorted(kernel_ms)
        km = torch.tensor([kernel_ms[n_] for n_ in names], device="cuda", dtype=torch.float64)
        dist.all_reduce(km, op=dist.ReduceOp.MAX)
        kernel_ms_max = {n_: float(v) for n_, v in zip(names, km)}
    else:
        e2e_ms = e2e_s * 1e3
        kernel_ms_max = kernel_ms
    if rank != 0:
        if sharded:
            idx.close()
        if world > 1:
            dist.destroy_process_group()
        return

    qps = nq * args.steps / (total_ms * 1e-3)
    e2e_qps = nq * args.steps / (e2e_ms * 1e-3)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    # sharded: the counters of this GPU's waves cover its slice of the batch only and the wave's time
    # includes the exchange, so the roofline is taken over the first-round kernels
    timed = {k_: v for k_, v in kernel_ms.items()
             if k_ in alg and not (sharded and k_ == "round_rows")}
    top = max(timed, key=lambda k_: timed[k_] * launches_per_step.get(k_, 1))
    achieved = alg[top] / (kernel_ms[top] * 1e-3) / 1e9
    captured = (args.workload == "descriptor-1m" and not args.copies and sp == LADDER[0]
                and not sharded and not args.queries)
    roofline = {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": NCU_TRAFFIC.get(top) if captured else None,
                "peak_source": "MEASURED_PEAKS.json" if peaks else "fallback 6650 GB/s",
                "algorithmic_bytes_per_launch": alg[top], "ms_per_launch": kernel_ms[top],
                "kernel_ms": kernel_ms,
                "kernels": {k_: {"GB/s": alg[k_] / (kernel_ms[k_] * 1e-3) / 1e9,
                                 "frac": alg[k_] / (kernel_ms[k_] * 1e-3) / 1e9 / peak} for k_ in timed}}
    if sharded:
        roofline["kernel_ms_slowest_rank"] = kernel_ms_max
        roofline["note"] = ("exchange = the kept lists of the first round to the GPUs that own the queries "
                            "(NCCL send / receive), merge = their merge; round_rows = the wave of this "
                            "GPU's slice of the batch; gather_results = all-gather of the results")
    config = workload_config(args, w, sp, world)
    config.update({"builder": args.builder, "build_seconds": build_seconds, "recall_at_10": rec, "recall_at_10_e2e": rec_e2e, "e2e_ids_equal_resident": e2e_same,
                   "index_bytes": index_bytes, "l2": "flushed between timed steps (256 MB fill)",
                   "memory_report": idx.memory_report(),
                   "mean_per_query": {"levels_tried": float(stats[:, 0].mean()),
                                      "list_entries": float(stats[:, 2].mean()),
                                      "distinct_first_round": float(stats[:, 3].mean()),
                                      "table_rows": float(stats[:, 4].mean()),
                                      "distinct_waves": float(stats[:, 5].mean()),
                                      "rows_reranked": float(stats[:, 6].mean())}})
    if sharded and args.placement != "shard":
        config["placement"] = args.placement
    line = {
        "metric": METRIC, "value": qps, "unit": "queries/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16/f32/i8",
        "data": "synthetic", "config": config,
        "clocks": clocks.summary(),
        "e2e": {"value": e2e_qps, "unit": "queries/s",
                "h2d_bytes_per_step": int(queries.nbytes),
                "d2h_bytes_per_step": int(on.nbytes + od.nbytes),
                "captured_batch": int(e2e_batch or nq),
                "value_one_captured_batch": (nq * args.steps / e2e_one_s) if world == 1 else None,
                "value_two_streams": (nq * args.steps / e2e_split_s[0]) if e2e_split_s else None,
                "two_streams_batch": e2e_split_s[1] if e2e_split_s else None},
        "gpu_launches": int(sum(launches_per_step.values()) * args.steps),
        "wall_s_timed_region": wall,
        "roofline": roofline,
    }
    if multi:
        line["multi_gpu"] = multi
    if world == 1:  # the comparison legs run once, beside the one-GPU number
        host = None
        if not args.no_cpu_baseline:
            try:
                host = host_arrays if host_arrays is not None else {k_: v.cpu().numpy() for k_, v in arrays.items()}
                line["cpu_baseline"] = cpu_baseline(host, meta, queries, sp, args)
                line["parity"] = parity_against_checker(idx, host, meta, queries, ids_run, dist_run, truth,
                                                        sp, args.cpu_sample)
            except Exception as e:  # a report, never a reason to lose the GPU numbers
                line.setdefault("cpu_baseline", {"value": None, "error": str(e)})
                line.setdefault("parity", {"error": str(e)})
        if not args.no_ref_kernels:
            try:
                line["ref_kernels"] = reference_kernels(host_arrays if host_arrays is not None else arrays, meta,
                                                        idx, queries, ids_run, sp, kernel_ms, args.steps)
            except Exception as e:
                line["ref_kernels"] = {"error": str(e)}
    emit(line)
    if sharded:
        idx.close()
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(host, meta, queries, sp, args):
    """The CPU restatement of the path timed on this box's host cores on a bounded sample."""
    from oracle import oracle_py
    ox = oracle_py.Index(host, meta)
    sample = queries[:args.cpu_sample]
    ox.search(sample[:64], K, **sp)
    t0 = time.perf_counter()
    ox.search(sample, K, **sp)
    t = time.perf_counter() - t0
    return {"value": len(sample) / t, "unit": "queries/s", "cores": os.cpu_count() or 1,
            "kind": "port", "sample": f"{len(sample)} of {len(queries)} queries, same index and parameters"}


if __name__ == "__main__":
    main()
