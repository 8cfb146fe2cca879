"""Spawning of rank processes for the multi-process tests, with a guaranteed clean-up.

`run_ranks(target, world, args)` starts `world` children running `target(rank, world, *args, q)`;
each child reports exactly one `(rank, status, info)` tuple through `q` (use `report_and_exit`
in the child).  Whatever happens in the parent (a rank that failed while its partner sits in a
collective, a timeout, an assertion), no child survives the call: live children are terminated,
joined, and killed if they still do not leave.  A child that failed leaves with os._exit
right after reporting, so that it never blocks in destroy_process_group while its partner is
stuck in a collective it will never join.
"""
import os
import queue as _queue
import time
import traceback

import torch.multiprocessing as mp


def report_and_exit(q, rank, fn):
    """Runs fn() in a rank process, reports ("ok", result) or ("fail", traceback) and, on failure,
    leaves the process at once without touching the process group."""
    try:
        res = fn()
    except BaseException:  # noqa: BLE001
        q.put((rank, "fail", traceback.format_exc()))
        q.close()
        q.join_thread()
        os._exit(1)
    q.put((rank, "ok", res))


def run_ranks(target, world, args=(), timeout=300):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=target, args=(r, world) + tuple(args) + (q,)) for r in range(world)]
    res = []
    try:
        for p in procs:
            p.start()
        deadline = time.time() + timeout
        while len(res) < world:
            try:
                item = q.get(timeout=1.0)
            except _queue.Empty:
                if time.time() > deadline:
                    raise AssertionError(f"ranks did not report within {timeout} s; got {res}") from None
                # a child that died without reporting will never do so
                dead = [i for i, p in enumerate(procs)
                        if not p.is_alive() and p.exitcode not in (0, None) and all(r[0] != i for r in res)]
                if dead and q.empty():
                    raise AssertionError(f"ranks {dead} died without a report; got {res}") from None
                continue
            res.append(item)
            if item[1] != "ok":     # its partners may wait for it for ever: stop here
                break
        for p in procs:
            p.join(timeout=30 if all(r[1] == "ok" for r in res) else 0.1)
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
    for rank, status, info in res:
        assert status == "ok", f"rank {rank}:\n{info}"
    assert len(res) == world
    return [info for _, _, info in sorted(res, key=lambda r: r[0])]
