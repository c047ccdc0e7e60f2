"""Launches N ranks as child processes on localhost and collects their results.

A worker is a module-level function ``fn(rank, nranks, uid_bytes, *args)`` in
``tests/_workers.py`` (spawned children import it by name).  A worker that raises
reports the traceback; a worker that dies or hangs is reported as such -- the
failure-detection tests rely on that.
"""
import multiprocessing as mp
import os
import traceback


def _entry(fn_name, rank, nranks, uid_bytes, args, env, q):
    try:
        for k, v in (env or {}).items():
            os.environ[k] = str(v)
        import tests._workers as W
        res = getattr(W, fn_name)(rank, nranks, uid_bytes, *args)
        q.put((rank, "ok", res))
    except BaseException as e:  # noqa: BLE001 - report everything to the parent
        q.put((rank, "error", f"{e!r}\n{traceback.format_exc()}"))


def run_ranks(nranks, fn_name, *args, env=None, per_rank_env=None, timeout=120, expect_dead=()):
    """Returns {rank: result}.  Raises AssertionError when a rank failed (unless its
    rank is listed in expect_dead, in which case it may exit without reporting)."""
    from flagcx_b200 import capi
    ctx = mp.get_context("spawn")
    uid = capi.unique_id_bytes(capi.get_unique_id())
    q = ctx.Queue()
    procs = []
    for r in range(nranks):
        e = dict(env or {})
        if per_rank_env:
            e.update(per_rank_env.get(r, {}))
        p = ctx.Process(target=_entry, args=(fn_name, r, nranks, uid, args, e, q))
        p.start()
        procs.append(p)
    results, errors = {}, {}
    want = nranks - len(expect_dead)
    try:
        while len(results) + len(errors) < want:
            rank, status, payload = q.get(timeout=timeout)
            (results if status == "ok" else errors)[rank] = payload
    except Exception:  # queue.Empty: somebody hangs
        errors[-1] = f"timed out after {timeout}s; got {sorted(results)} ok, {sorted(errors)} failed"
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join()
    if errors:
        raise AssertionError("\n".join(f"rank {r}: {m}" for r, m in errors.items()))
    return results
