"""Shard a list of independent shapes over the GPUs of one box.

The reference runs every sweep serially on GPU 0 (it never calls cudaSetDevice; e.g.
scripts/Ampere_FP16/benchmark_Ampere_FP16_gemm.py:9-17).  Shapes are independent work units, so
the sweep shards with no collective: units are dealt to one worker process per GPU by
longest-processing-time-first on the cost model's prediction, every worker appends one JSON
line per finished unit to a journal (so a killed sweep resumes), and the units of a worker that
died are run by the survivors.  Workers are plain callables, which lets the scheduling logic be
tested on CPU with a fake device.
"""
import json
import multiprocessing as mp
import os
import time

from .workloads import lpt_partition


def _worker_main(rank, device, fn, units, indices, journal, queue, fn_args):
    try:
        done = 0
        for i in indices:
            t0 = time.perf_counter()
            row = fn(device, units[i], *fn_args)
            row = dict(row)
            row.update({"index": i, "device": device, "wall_s": time.perf_counter() - t0})
            if journal:
                with open(journal, "a") as f:
                    f.write(json.dumps(row) + "\n")
            queue.put(("row", rank, row))
            done += 1
        queue.put(("done", rank, done))
    except BaseException as exc:  # the parent re-queues whatever this worker did not finish
        queue.put(("fail", rank, repr(exc)))
        raise


def read_journal(path):
    """Rows of an earlier, possibly interrupted run, keyed by unit index."""
    rows = {}
    if path and os.path.exists(path):
        with open(path) as f:
            for line in f:
                try:
                    r = json.loads(line)
                    rows[int(r["index"])] = r
                except (ValueError, KeyError):
                    continue       # a torn last line of a killed run
    return rows


def run_sharded(units, fn, devices, costs=None, journal=None, fn_args=(), timeout_s=3600.0, start_method="spawn"):
    """Run fn(device, unit, *fn_args) -> dict for every unit, sharded over `devices`.

    Returns (rows_by_index, stats).  Units already present in `journal` are not re-run.
    """
    units = list(units)
    costs = list(costs) if costs is not None else [1.0] * len(units)
    rows = read_journal(journal)
    pending = [i for i in range(len(units)) if i not in rows]
    stats = {"rounds": 0, "failed_workers": [], "resumed": len(rows), "per_device_s": {}}
    alive = list(devices)
    ctx = mp.get_context(start_method)
    while pending and alive:
        stats["rounds"] += 1
        parts = lpt_partition([costs[i] for i in pending], len(alive))
        queue = ctx.Queue()
        procs = []
        t_start = time.perf_counter()
        for rank, dev in enumerate(alive):
            idx = [pending[j] for j in parts[rank]]
            p = ctx.Process(target=_worker_main, args=(rank, dev, fn, units, idx, journal, queue, tuple(fn_args)))
            p.start()
            procs.append((p, dev, idx))
        finished = set()
        failed = set()
        deadline = time.perf_counter() + timeout_s
        while len(finished) + len(failed) < len(procs):
            try:
                kind, rank, payload = queue.get(timeout=0.25)
            except Exception:
                for rank, (p, dev, idx) in enumerate(procs):
                    if rank not in finished and rank not in failed and not p.is_alive():
                        failed.add(rank)     # died without a message (killed)
                if time.perf_counter() > deadline:
                    for rank, (p, dev, idx) in enumerate(procs):
                        if rank not in finished and rank not in failed:
                            p.terminate()
                            failed.add(rank)
                continue
            if kind == "row":
                rows[payload["index"]] = payload
            elif kind == "done":
                finished.add(rank)
                stats["per_device_s"][procs[rank][1]] = (stats["per_device_s"].get(procs[rank][1], 0.0)
                                                          + time.perf_counter() - t_start)
            elif kind == "fail":
                failed.add(rank)
        for p, _, _ in procs:
            p.join(timeout=5)
        # drain rows that raced with the end-of-worker message
        while True:
            try:
                kind, rank, payload = queue.get_nowait()
            except Exception:
                break
            if kind == "row":
                rows[payload["index"]] = payload
        for rank in sorted(failed):
            stats["failed_workers"].append(procs[rank][1])
        alive = [dev for rank, (p, dev, idx) in enumerate(procs) if rank not in failed]
        pending = [i for i in pending if i not in rows]
    stats["unfinished"] = len(pending)
    return rows, stats
