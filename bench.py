#!/usr/bin/env python
"""Benchmark of the csg reorder path (and the SpMM it feeds) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one csg reorder of the workload matrix: chunk-local transpose, sketch +
top-k, greedy.  The workload is the power-law matrix the headline target is quoted
on: R-MAT scale 22, edge factor 16, (a,b,c,d) = (.57,.19,.19,.05), duplicates
removed, seed 3 (seeded synthetic data standing in for the reference's SuiteSparse
sets), csg with the reference's default parameters (k = nnz/n clamped to [16,256],
oversampling 4, chunk 1024).

Prints ONE JSON line.  `value` is Mnnz/s with the matrix resident in HBM, timed with
CUDA events on the launching stream; `e2e` is the same metric through the host-buffer
entry point of the C ABI (pinned host CSR in, permutation out, copies inside the timed
region).  With N > 1 (launched under torchrun) the rows are cut into N chunk-aligned
shards, one per GPU, and the permutation shards are all-gathered with NCCL; the total
work is fixed, so scaling is "strong".

With N > 1 the post-reorder SpMM is row-partitioned as well (nonzero-balanced row ranges, the
dense operand replicated on every GPU, each GPU owning its rows of the result) and timed as the
maximum over ranks.  Every line carries `parity`: the permutation the timed calls produced,
compared with the CPU restatement (on a sample of whole chunks at every N, on the whole matrix
where the CPU leg runs it) and with the reference's own CUDA library, plus its SHA-256 so that
the lines of different N can be compared.

`--impl reference` times the CPU restatement of the reference's algorithm (the
reference has no CPU implementation of csg; its own code is CUDA) on the host cores,
each step on a bounded sample of whole chunks of the same matrix.
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
sys.path.insert(0, ROOT)

WORKLOAD = "rmat22"
CSG_KW = dict(k=0, oversampling=0.0, chunk_size=0)  # configs/paper.yaml:6 -> all "auto"
CHUNK = 1024


# ---------------------------------------------------------------------------------
T_START = time.time()


def log(*a):
    print("[bench %7.1fs]" % (time.time() - T_START), *a, file=sys.stderr, flush=True)


def load_workload(scale, name="rmat22"):
    """The workload matrix (host numpy int32 CSR), cached in /tmp between runs.  `rmat22`
    with another --scale is the same R-MAT recipe at that scale; the other names are the
    remaining benchmark configurations at full size."""
    from chunkedgreedy_b200 import synth
    if name != "rmat22":
        cache = "/tmp/chunkedgreedy_b200_%s.npz" % name
        if os.path.exists(cache):
            try:
                z = np.load(cache)
                return z["ptr"], z["ind"], z["val"]
            except Exception:
                pass
        w = synth.make_workload(name)
        try:
            tmp = cache + ".%d.tmp.npz" % os.getpid()
            np.savez(tmp, ptr=w["ptr"], ind=w["ind"], val=w["val"])
            os.replace(tmp, cache)
        except Exception:
            pass
        return w["ptr"], w["ind"], w["val"]
    cache = "/tmp/chunkedgreedy_b200_rmat%d_seed3.npz" % scale
    if os.path.exists(cache):
        try:
            z = np.load(cache)
            return z["ptr"], z["ind"], z["val"]
        except Exception:
            pass
    ptr, ind, val = synth.rmat(scale=scale, edge_factor=16, seed=3)
    try:
        tmp = cache + ".%d.tmp.npz" % os.getpid()
        np.savez(tmp, ptr=ptr, ind=ind, val=val)
        os.replace(tmp, cache)
    except Exception:
        pass
    return ptr, ind, val


def chunk_sample(ptr, ind, fraction, chunk=CHUNK):
    """A bounded sample of the workload made of whole chunks: chunks are sorted by their
    nonzero count and every (1/fraction)-th is taken, so light and heavy chunks appear in
    proportion.  Returns a CSR block (rows renumbered, columns kept) and the chunks taken."""
    n = ptr.size - 1
    nch = (n + chunk - 1) // chunk
    if fraction >= 1.0:
        return ptr, ind, np.arange(nch)
    edges = np.minimum(np.arange(nch + 1, dtype=np.int64) * chunk, n)
    cnt = np.diff(ptr[edges].astype(np.int64))
    order = np.argsort(-cnt, kind="stable")
    stride = max(1, int(round(1.0 / fraction)))
    take = np.sort(order[stride // 2::stride])
    take = take[take != nch - 1] if (n % chunk) else take  # keep full-size chunks only
    pieces_ptr, pieces_ind, base = [np.zeros(1, dtype=np.int64)], [], 0
    for q in take:
        r0, r1 = int(edges[q]), int(edges[q + 1])
        b, e = int(ptr[r0]), int(ptr[r1])
        pieces_ptr.append(ptr[r0 + 1:r1 + 1].astype(np.int64) - b + base)
        pieces_ind.append(ind[b:e])
        base += e - b
    return (np.concatenate(pieces_ptr).astype(np.int32),
            np.concatenate(pieces_ind) if pieces_ind else np.zeros(0, np.int32), take)


def sample_matches(order_full, sample_order, take, n, chunk=CHUNK):
    """True when the permutation of the whole matrix, restricted to the sampled chunks, is
    the permutation computed for the sample (chunks are independent problems: chunk j of the
    sample is chunk take[j] of the matrix with its rows renumbered)."""
    for j, q in enumerate(take):
        r0, r1 = int(q) * chunk, min((int(q) + 1) * chunk, n)
        if not np.array_equal(order_full[r0:r1] - r0, sample_order[j * chunk:j * chunk + (r1 - r0)] - j * chunk):
            return False
    return True


def cpu_reference_rate(ptr, ind, k, budget_s, steps_total, threads=None):
    """Times the CPU restatement (oracle/) on a sample sized so that `steps_total` steps
    fit in about `budget_s` seconds.  Returns (callable running one step -> seconds,
    sample nnz, description, chunks of the sample, holder of the last step's permutation)."""
    import oracle
    if threads:
        oracle.set_num_threads(threads)
    n = ptr.size - 1
    # probe on 1/64 of the chunks to size the real sample
    pp, pi, pc = chunk_sample(ptr, ind, 1.0 / 64)
    t0 = time.perf_counter()
    oracle.csg(pp, pi, False, k=k, ncols=n)
    probe = time.perf_counter() - t0
    rate = max(pi.size, 1) / max(probe, 1e-6)  # nnz / s
    want = rate * budget_s / max(steps_total, 1)
    fraction = min(1.0, max(1.0 / 64, want / max(ind.size, 1)))
    sp_, si_, take = chunk_sample(ptr, ind, fraction)
    last = {}

    def step():
        t = time.perf_counter()
        last["order"] = oracle.csg(sp_, si_, False, k=k, ncols=n)
        return time.perf_counter() - t

    nch = (n + CHUNK - 1) // CHUNK
    desc = "%d of %d chunks (every %d-th by nonzero count), %d nnz, full csg per step" % (
        len(take), nch, max(1, int(round(1.0 / fraction))), si_.size)
    return step, int(si_.size), desc, take, last


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)),
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------
def run_reference(args, rank, world):
    """CPU arm: rank 0 alone works; the other ranks exit 0."""
    if rank != 0:
        return
    import oracle
    # every core this process may run on: torchrun sets OMP_NUM_THREADS=1 for its ranks,
    # which would time one thread of the CPU arm at N > 1
    try:
        oracle.set_num_threads(len(os.sched_getaffinity(0)))
    except AttributeError:
        oracle.set_num_threads(os.cpu_count() or 1)
    ptr, ind, _ = load_workload(args.scale, args.workload)
    n, nnz = ptr.size - 1, ind.size
    k = min(256, max(16, nnz // n))
    step, sample_nnz, desc, _, _ = cpu_reference_rate(ptr, ind, k, args.cpu_budget,
                                                      args.steps + args.warmup)
    for _ in range(args.warmup):
        step()
    total = sum(step() for _ in range(args.steps))
    value = sample_nnz * args.steps / total / 1e6
    cores = oracle.num_threads()
    line = {
        "impl": "reference", "metric": "csg reorder throughput", "value": value, "unit": "Mnnz/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int32 indices, f32 weights", "data": "synthetic",
        "config": workload_config(n, nnz, k, args),
        "cpu_baseline": {"value": value, "unit": "Mnnz/s", "cores": cores, "kind": "port",
                         "sample": desc},
        "e2e": {"value": value, "unit": "Mnnz/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "note": "the reference implements csg only in CUDA; this arm is the OpenMP restatement "
                "of its arithmetic (oracle/csg_oracle.c) on the host cores",
    }
    emit(line)


def workload_config(n, nnz, k, args):
    names = {"rmat22": "rmat scale %d ef16 a.57 b.19 c.19 d.05 dedup seed3" % args.scale,
             "zipf65k": "zipf-banded 65536 rows seed0", "stencil1024": "9-point stencil 1024^2 relabelled seed1",
             "stencil1024nat": "9-point stencil 1024^2 natural order seed1",
             "road2m": "road lattice 2M vertices relabelled seed2",
             "rmat20gcn": "rmat scale 20 symmetrised + self loops, normalised, seed4"}
    return {"workload": "%s; csg k=%d M=%d chunk=%d"
                        % (names[args.workload], k, ((4 * k + 31) // 32) * 32, CHUNK),
            "n": int(n), "nnz": int(nnz), "parallelism": "row shards x%d" % args.gpus,
            "l2": "inputs and scratch (>1 GB) exceed L2; no explicit flush"}


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import chunkedgreedy_b200 as sp
    from chunkedgreedy_b200 import dist as csgdist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    ptr, ind, val = load_workload(args.scale, args.workload)
    n, nnz = ptr.size - 1, ind.size
    k = csgdist.resolve_k(n, nnz, 0)
    bounds = csgdist.shard_bounds(ptr, CHUNK, world)
    r0, r1 = bounds[rank]
    pl, il = csgdist.extract_shard(ptr, ind, r0, r1)
    h_ptr = torch.from_numpy(np.ascontiguousarray(pl)).pin_memory()
    h_ind = torch.from_numpy(np.ascontiguousarray(il)).pin_memory()
    d_ptr, d_ind = h_ptr.to(dev), h_ind.to(dev)
    ctx = sp.Context()
    log("rank", rank, "rows", r0, r1, "nnz", il.size, "k", k)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # a workload with a symmetric pattern is reordered with the reference's is_symmetric
    # promise when one GPU holds the whole matrix (row shards cannot use it)
    from chunkedgreedy_b200 import synth
    sym = bool(synth.WORKLOADS[args.workload][2]) and world == 1 and not args.no_symmetric_promise

    def csg_local(dp, di, **kw):
        if sym:
            return sp.chunk_similarity_greedy(dp, di, is_symmetric=True, k=k, chunk_size=CHUNK, ctx=ctx, **kw)
        return csgdist.csg_shard(dp, di, n, r0, k=k, chunk_size=CHUNK, ctx=ctx, **kw)

    def step_device():
        local = csg_local(d_ptr, d_ind)
        return csgdist.gather_shards(local, bounds) if world > 1 else local

    h_out = torch.empty(n, dtype=torch.int32).pin_memory()

    def step_e2e():
        if world == 1:  # the C ABI's host-buffer entry point: copies in, reorder, copy out
            sp.chunk_similarity_greedy_host(h_ptr, h_ind, is_symmetric=sym, k=k, chunk_size=CHUNK, out=h_out,
                                            ctx=ctx)
            return
        dp = h_ptr.to(dev, non_blocking=True)
        di = h_ind.to(dev, non_blocking=True)
        local = csg_local(dp, di)
        full = csgdist.gather_shards(local, bounds) if world > 1 else local
        h_out.copy_(full, non_blocking=True)
        torch.cuda.synchronize()

    # ---- device-resident timing --------------------------------------------------
    for _ in range(args.warmup):
        order = step_device()
        log("warm-up step done")
    barrier()
    launches0 = sp.kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        e0.record()
        for _ in range(args.steps):
            order = step_device()
        e1.record()
        barrier()
    launches = sp.kernel_launches() - launches0
    t_ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    t_ms = float(t_ms.item())
    value = nnz * args.steps / (t_ms * 1e-3) / 1e6

    log("timed: %.2f ms/step" % (t_ms / args.steps))
    # ---- stage times (CUDA events recorded by the library on the same stream) ------
    stage = {"transpose_ms": 0.0, "sketch_ms": 0.0, "greedy_ms": 0.0}
    reps = max(1, min(args.steps, 5))
    for _ in range(reps):
        _, tm = csg_local(d_ptr, d_ind, with_timing=True)
        stage["transpose_ms"] += tm["csr2csc_ms"] / reps
        stage["sketch_ms"] += tm["similarity_ms"] / reps
        stage["greedy_ms"] += tm["chunk_greedy_ms"] / reps
    n_loc, nnz_loc = r1 - r0, il.size

    log("stages", stage)
    # ---- end to end through the host-buffer path -------------------------------------
    for _ in range(min(args.warmup, 2)):
        step_e2e()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_e2e()
    barrier()
    e2e_s = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_value = nnz * args.steps / float(e2e_s.item()) / 1e6

    log("e2e done")
    # ---- post-reorder SpMM (every rank takes part: row-partitioned at N > 1) ----------
    spmm = None
    if not args.no_spmm:
        spmm = spmm_section(sp, ctx, ptr, ind, val, order, n, nnz, dev, world, rank,
                            t_ms / args.steps, with_reference=(world == 1 and not args.no_ref_cuda))
    if rank != 0:
        return
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"
    # Algorithmic bytes of the sketch/top-k stage of THIS rank's shard: the pattern read once
    # row-wise and once in transposed view, the table written once.  Two counts: with k
    # entries for every row, and with the entries of the rows that have a candidate only
    # (rows without one are known from the transpose and never touched; one untimed call
    # with statistics counts them).  The fraction uses the narrower, lower count.
    _, st_loc = csg_local(d_ptr, d_ind, with_stats=True)
    rows_written = n_loc - int(st_loc["zero_degree_rows"])
    b_sketch = 2 * (4 * (n_loc + 1) + 4 * nnz_loc) + 8 * rows_written * k
    b_sketch_all_rows = 2 * (4 * (n_loc + 1) + 4 * nnz_loc) + 8 * n_loc * k
    ach = b_sketch / (stage["sketch_ms"] * 1e-3) / 1e9 if stage["sketch_ms"] > 0 else 0.0
    order_np = order.cpu().numpy()
    line = {
        "metric": "csg reorder throughput", "value": value, "unit": "Mnnz/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int32 indices, f32 weights", "data": "synthetic",
        "config": workload_config(n, nnz, k, args), "is_symmetric_promised": sym,
        "e2e": {"value": e2e_value, "unit": "Mnnz/s",
                "h2d_bytes_per_step": int(4 * (n_loc + 1) + 4 * nnz_loc),
                "d2h_bytes_per_step": int(4 * n)},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "stages_ms": stage,
        "roofline": {"bound": "hbm",
                     "kernel": "sketch + top-k stage (heavy_expand, heavy_rounds, sketch_kernel)",
                     "achieved": ach,
                     "peak": hbm, "unit": "GB/s", "frac": ach / hbm, "peak_source": peak_src,
                     "algorithmic_bytes": int(b_sketch), "table_rows_written": int(rows_written),
                     "algorithmic_bytes_all_rows": int(b_sketch_all_rows),
                     "frac_all_rows": (b_sketch_all_rows / (stage["sketch_ms"] * 1e-3) / 1e9 / hbm
                                       if stage["sketch_ms"] > 0 else 0.0),
                     "traffic": None, "traffic_note": TRAFFIC_NOTE},
        "parity": parity_section(order_np, ptr, ind, k, n),
    }
    if world == 1 and args.workload == "rmat22" and args.scale == 22:
        line["roofline"]["traffic"] = TRAFFIC_RMAT22
    if world == 1 and not args.no_cpu_baseline:
        import oracle
        try:
            oracle.set_num_threads(len(os.sched_getaffinity(0)))
        except AttributeError:
            oracle.set_num_threads(os.cpu_count() or 1)
        step, sample_nnz, desc, take, last = cpu_reference_rate(ptr, ind, k, args.cpu_budget, 1)
        secs = step()
        line["cpu_baseline"] = {"value": sample_nnz / secs / 1e6, "unit": "Mnnz/s",
                                "cores": oracle.num_threads(), "kind": "port", "sample": desc}
        line["parity"]["vs_oracle"] = bool(sample_matches(order_np, last["order"], take, n))
        line["parity"]["vs_oracle_scope"] = desc
        log("cpu baseline done")
    if world == 1 and not args.no_ref_cuda:
        from chunkedgreedy_b200 import synth
        sym = synth.WORKLOADS[args.workload][2]
        line["reference_cuda"], ref_order = reference_cuda(d_ptr, d_ind, nnz, sym)
        if ref_order is not None:
            line["parity"]["vs_reference_cuda"] = bool(np.array_equal(ref_order.cpu().numpy(), order_np))
        # the same protocol for this library: one untimed call, a flushed L2, then the
        # library's own wall_ms and stage times (reorder_bench/methods/sporder_csg.py:41-57)
        line["same_protocol"] = same_protocol_pair(sp, ctx, d_ptr, d_ind, sym, line["reference_cuda"])
        log("reference cuda done", line["reference_cuda"])
    if spmm is not None:
        line["pillars_h16"] = spmm.pop("pillars_h16", None)
        line["apply"] = spmm.pop("apply", None)
        line["spmm"] = spmm
    if world == 1 and args.gcn:
        line["gcn"] = gcn_section(d_ptr, d_ind, torch.from_numpy(val).to(dev), n, ctx,
                                  args.gcn_epochs)
    if world == 1 and not args.no_configs and args.workload == "rmat22":
        line["configs"] = other_configs(sp, ctx, dev, args.configs_budget)
    emit(line)


# DRAM bytes (read + write) of the sketch stage's kernels per csg call at full size, from an
# ncu capture of `bench.py --steps 1 --warmup 1 --no-ref-cuda --no-cpu-baseline --no-spmm`;
# a number of the build it was captured on, not of this run
TRAFFIC_RMAT22 = 4454053376
TRAFFIC_NOTE = ("dram__bytes_read+write of heavy_expand + heavy_rounds + sketch_kernel + heavy_topk, "
                "one ncu capture at N=1 on the scale-22 matrix; null for other sizes and N")


def order_digest(order_np):
    import hashlib
    return hashlib.sha256(np.ascontiguousarray(order_np, dtype=np.int32).tobytes()).hexdigest()


def parity_section(order_np, ptr, ind, k, n):
    """What every line can say about the permutation the timed calls produced: its digest
    (equal across N when the row shards reproduce the single-GPU answer), the structural
    invariants of a csg order (a permutation; every chunk a permutation of its own rows that
    starts at the chunk's first row, sporder/src/csg/chunk_similarity_greedy.cu:31), and a
    comparison with the CPU restatement on 1/64 of the chunks."""
    import oracle
    out = {"order_sha256": order_digest(order_np)}
    full = (n // CHUNK) * CHUNK
    blocks = order_np[:full].reshape(-1, CHUNK).astype(np.int64)
    ok = bool(np.array_equal(blocks[:, 0], np.arange(0, full, CHUNK)))
    ok = ok and bool(np.array_equal(np.sort(blocks, axis=1), np.arange(full).reshape(-1, CHUNK)))
    if n > full:
        ok = ok and bool(np.array_equal(np.sort(order_np[full:]), np.arange(full, n)))
    out["structure_ok"] = ok
    try:
        oracle.set_num_threads(len(os.sched_getaffinity(0)))
    except AttributeError:
        pass
    sp_, si_, take = chunk_sample(ptr, ind, 1.0 / 64)
    want = oracle.csg(sp_, si_, False, k=k, ncols=n)
    out["vs_oracle_sample"] = bool(sample_matches(order_np, want, take, n))
    out["vs_oracle_sample_scope"] = "%d chunks (every 64-th by nonzero count)" % len(take)
    return out


def reference_cuda(d_ptr, d_ind, nnz, is_symmetric=False):
    """The reference's own CUDA library, built unchanged for sm_100a (oracle/_ref), on the
    same matrix with its benchmark protocol (one warm-up call, then the library's wall_ms;
    bench/reorder/reorder_bench/methods/sporder_csg.py:41-57).  Returns (record, order)."""
    try:
        from oracle import ref
        if not ref.available():
            return {"unavailable": "oracle/_ref/libsporder_ref.so not present"}, None
        import torch
        ref.csg(d_ptr, d_ind, is_symmetric)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=d_ptr.device)
        flush.zero_()
        order, tm = ref.csg(d_ptr, d_ind, is_symmetric, with_timing=True)
        torch.cuda.synchronize()
        return {"value": nnz / (tm["wall_ms"] * 1e-3) / 1e6, "unit": "Mnnz/s", "timing_ms": tm,
                "stage_sum_ms": tm["csr2csc_ms"] + tm["similarity_ms"] + tm["chunk_greedy_ms"],
                "kind": "reference CUDA sources compiled for sm_100a, 1 GPU"}, order
    except Exception as e:  # never let the comparison leg break the bench line
        return {"unavailable": repr(e)[:200]}, None


def same_protocol_pair(sp, ctx, d_ptr, d_ind, is_symmetric, ref_record):
    """This library under the reference harness's protocol, beside the reference's numbers
    taken the same way: wall_ms of the second call after an L2 flush, and the stage sums."""
    import torch
    try:
        sp.chunk_similarity_greedy(d_ptr, d_ind, is_symmetric=is_symmetric, ctx=ctx)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=d_ptr.device)
        flush.zero_()
        torch.cuda.synchronize()
        _, tm = sp.chunk_similarity_greedy(d_ptr, d_ind, is_symmetric=is_symmetric, with_timing=True,
                                           ctx=ctx)
        ours_sum = tm["csr2csc_ms"] + tm["similarity_ms"] + tm["chunk_greedy_ms"]
        out = {"ours_wall_ms": tm["wall_ms"], "ours_stage_sum_ms": ours_sum}
        if "timing_ms" in ref_record:
            out["reference_wall_ms"] = ref_record["timing_ms"]["wall_ms"]
            out["reference_stage_sum_ms"] = ref_record["stage_sum_ms"]
            out["wall_ratio"] = out["reference_wall_ms"] / tm["wall_ms"]
            out["stage_sum_ratio"] = out["reference_stage_sum_ms"] / ours_sum if ours_sum > 0 else None
        return out
    except Exception as e:
        return {"unavailable": repr(e)[:200]}


def _time_launches(fn, warm=3, reps=10):
    import torch
    for _ in range(warm):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def spmm_section(sp, ctx, ptr, ind, val, order, n, nnz, dev, world, rank, reorder_ms,
                 with_reference=False, widths=(32, 128, 256)):
    """Post-reorder SpMM: GFLOP/s = 2*nnz*w / t (spmatkit/spmatkit.py:2150-2155) on
    A' = P A P^T and on A with the library's fp32 kernel; at N > 1 row-partitioned
    (nonzero-balanced row ranges, dense operand replicated, results left sharded) and timed
    as the maximum over ranks.  Also: the symmetric permutation apply itself, the reference's
    quality metric before and after, cuSPARSE CSR_ALG1 on the same patterns through the
    reference's own timer (sporder/src/bench_cusparse_spmm.cu:64-90), and the number of
    launches that amortise the reorder (bench/spmm/scripts/compute_amortization.py:63-66)."""
    import torch
    import torch.distributed as dist
    from chunkedgreedy_b200 import dist as csgdist
    from chunkedgreedy_b200 import harness
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    out = {}
    d_ptr = torch.from_numpy(ptr).to(dev)
    d_ind = torch.from_numpy(ind).to(dev)
    d_val = torch.from_numpy(val).to(dev)
    p2, i2, v2 = sp.reorder(d_ptr, d_ind, order, val=d_val, symmetric=True, ctx=ctx)
    if rank == 0:
        # the permutation apply: B_apply = 2*4(n+1) + 2*4n + 2*8*nnz (read and write ptr, the
        # permutation and its inverse, indices and values once each)
        ms = _time_launches(lambda: sp.reorder(d_ptr, d_ind, order, val=d_val, symmetric=True, ctx=ctx),
                            warm=1, reps=3)
        b_apply = 2 * 4 * (n + 1) + 2 * 4 * n + 2 * 8 * nnz
        out["apply"] = {"ours_ms": ms, "algorithmic_bytes": int(b_apply),
                        "roofline_frac": b_apply / (ms * 1e-3) / 1e9 / hbm, "mode": "symmetric, with values"}
        if with_reference:
            try:
                from oracle import ref
                if ref.available():
                    rp, ri, rv = ref.reorder(d_ptr, d_ind, order, val=d_val, symmetric=True)
                    torch.cuda.synchronize()
                    out["apply"]["matches_reference"] = bool(
                        torch.equal(rp, p2) and torch.equal(ri, i2) and torch.equal(rv, v2))
                    t0 = time.perf_counter()
                    for _ in range(3):
                        ref.reorder(d_ptr, d_ind, order, val=d_val, symmetric=True)
                    torch.cuda.synchronize()
                    out["apply"]["reference_ms"] = (time.perf_counter() - t0) * 1e3 / 3
                    del rp, ri, rv
            except Exception as e:
                out["apply"]["reference_unavailable"] = repr(e)[:200]
        # the reference's quality metric (configs/paper.yaml:30-32: distinct columns per
        # window of 16 rows, fewer is better) before and after the reorder
        t0 = time.perf_counter()
        before = sp.count_pillars(d_ptr, d_ind, 16, ctx=ctx)
        ms = (time.perf_counter() - t0) * 1e3
        out["pillars_h16"] = {"original": before, "reordered": sp.count_pillars(p2, i2, 16, ctx=ctx),
                              "count_ms": ms}
    mats = (("original", (d_ptr, d_ind, d_val)), ("reordered", (p2, i2, v2)))
    bounds = {tag: csgdist.spmm_row_bounds(m[0], world) for tag, m in mats}
    for w in widths:
        B = torch.randn((n, w), device=dev, dtype=torch.float32)
        res = {}
        for tag, (pp, ii, vv) in mats:
            r0, r1 = bounds[tag][rank]
            pl, il, vl = csgdist.spmm_shard(pp, ii, vv, r0, r1) if world > 1 else (pp, ii, vv)
            C = torch.empty((max(r1 - r0, 1), w), device=dev, dtype=torch.float32)
            if r1 > r0:
                ms = _time_launches(lambda: sp.spmm(pl, il, vl, B, out=C[: r1 - r0], n_cols=n, ctx=ctx,
                                                    sync=False))
            else:
                ms = 0.0
            t = torch.tensor([ms], device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            algo = 4 * (n + 1) + 8 * nnz + 8 * n * w  # pattern + values once, B and C once
            res[tag] = {"ms": ms, "gflops": 2.0 * nnz * w / (ms * 1e6),
                        "roofline_frac": algo / (ms * 1e-3) / 1e9 / hbm,
                        "gather_bytes_frac": (4.0 * nnz * w + 8 * nnz + 4 * n * w) / (ms * 1e-3) / 1e9 / hbm}
            if with_reference and rank == 0:
                try:
                    from oracle import ref
                    if ref.available():
                        res[tag]["cusparse_ms"] = ref.cusparse_spmm(pp, ii, w, warmup=3, repeat=10)
                except Exception as e:
                    res[tag]["cusparse_unavailable"] = repr(e)[:200]
            del C
        res["speedup"] = res["original"]["ms"] / res["reordered"]["ms"]
        res["amortization_runs"] = harness.format_amortization(
            harness.amortization_runs(reorder_ms, res["original"]["ms"], res["reordered"]["ms"]))
        out["w%d" % w] = res
        del B
    out["partition"] = ("one GPU" if world == 1 else
                        "rows cut into %d nonzero-balanced ranges, dense operand replicated, "
                        "result left sharded; ms = max over ranks" % world)
    return out


def other_configs(sp, ctx, dev, budget_s):
    """The remaining benchmark configurations at full size, within a time budget: csg
    throughput, stage times and the digest of the permutation for each."""
    import torch
    from chunkedgreedy_b200 import synth
    out, t_begin = {}, time.time()
    for name in ("zipf65k", "stencil1024", "road2m", "rmat20gcn"):
        if time.time() - t_begin > budget_s:
            out[name] = {"skipped": "time budget of %.0f s used up" % budget_s}
            continue
        try:
            ptr, ind, _ = load_workload(0, name)
            sym = synth.WORKLOADS[name][2]
            d_ptr, d_ind = torch.from_numpy(ptr).to(dev), torch.from_numpy(ind).to(dev)
            n, nnz = ptr.size - 1, ind.size
            ms = _time_launches(lambda: sp.chunk_similarity_greedy(d_ptr, d_ind, is_symmetric=sym, ctx=ctx),
                                warm=2, reps=5)
            order, tm = sp.chunk_similarity_greedy(d_ptr, d_ind, is_symmetric=sym, with_timing=True, ctx=ctx)
            out[name] = {"n": int(n), "nnz": int(nnz), "ms": ms, "Mnnz_per_s": nnz / (ms * 1e-3) / 1e6,
                         "stages_ms": {"transpose_ms": tm["csr2csc_ms"], "sketch_ms": tm["similarity_ms"],
                                       "greedy_ms": tm["chunk_greedy_ms"]},
                         "order_sha256": order_digest(order.cpu().numpy())}
            del d_ptr, d_ind
        except Exception as e:
            out[name] = {"failed": repr(e)[:200]}
    return out


def gcn_section(d_ptr, d_ind, d_val, n, ctx, epochs):
    """2-layer GCN (128 -> 128 -> 16, ReLU, full-batch SGD), features N(0,1), uniform labels,
    seed 4: training on the matrix as given against reorder once + train on P A P^T."""
    import torch
    from chunkedgreedy_b200 import gcn
    g = torch.Generator(device=d_ptr.device).manual_seed(4)
    x = torch.randn((n, 128), device=d_ptr.device, generator=g)
    y = torch.randint(0, 16, (n,), device=d_ptr.device, generator=g)
    r = gcn.reorder_and_train(d_ptr, d_ind, d_val, x, y, hidden=128, classes=16, epochs=epochs,
                              optimizer="sgd", ctx=ctx)
    r.pop("order")
    for key, v in list(r.items()):  # JSON has no infinity: the harness's text form instead
        if isinstance(v, float) and (v == float("inf") or v != v):
            r[key] = "inf" if v == float("inf") else "nan"
    return r


_JSON_OUT = None


def emit(line):
    """The one JSON line, on the process's original stdout."""
    out = _JSON_OUT if _JSON_OUT is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    # Libraries write to stdout too (NCCL prints its version there at any NCCL_DEBUG level
    # the launcher may have set).  Stdout has to carry the JSON line and nothing else, so
    # file descriptor 1 is pointed at stderr for the whole run and the line goes to a
    # duplicate of the original descriptor.
    global _JSON_OUT
    sys.stdout.flush()
    _JSON_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scale", type=int, default=22, help="R-MAT scale (22 = the named workload)")
    ap.add_argument("--workload", default="rmat22",
                    choices=["rmat22", "zipf65k", "stencil1024", "stencil1024nat", "road2m", "rmat20gcn"],
                    help="rmat22 is the bench workload; the others are the remaining configurations")
    ap.add_argument("--gcn", action="store_true",
                    help="also run the reorder-then-train GCN experiment (use with --workload rmat20gcn)")
    ap.add_argument("--gcn-epochs", type=int, default=200)
    ap.add_argument("--cpu-budget", type=float, default=20.0,
                    help="seconds of CPU work the baseline sample is sized for")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref-cuda", action="store_true")
    ap.add_argument("--no-spmm", action="store_true")
    ap.add_argument("--no-symmetric-promise", action="store_true",
                    help="reorder symmetric workloads without is_symmetric (the chunk-local sort runs)")
    ap.add_argument("--no-configs", action="store_true",
                    help="skip the short runs of the other benchmark configurations")
    ap.add_argument("--configs-budget", type=float, default=90.0,
                    help="seconds the runs of the other configurations may take (generation included)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        args.cpu_budget = max(args.cpu_budget, 60.0)
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
