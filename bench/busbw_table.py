"""Turns the JSON-lines files that bench/busbw.py writes (--out) into markdown tables.

    python bench/busbw_table.py sweep_a.jsonl [sweep_b.jsonl ...] [--dtype bf16] [--min-bytes 1K]

One table per file: a row per message size, and per operation the time of this
library, the comparator's time, both bus bandwidths and the ratio (comparator time /
our time; above 1 means this library is faster).  Latency-mode files (--mode latency)
print microseconds per call only.  Files written with --impl reference / nccl / ours_pg
have one implementation per file; give two of them with --join to put them side by side:

    python bench/busbw_table.py --join ours_pg.jsonl reference.jsonl
"""
from __future__ import annotations

import argparse
import json
from collections import OrderedDict


def human(n: int) -> str:
    for unit, shift in (("GiB", 30), ("MiB", 20), ("KiB", 10)):
        if n >= 1 << shift:
            v = n / (1 << shift)
            return f"{v:.0f} {unit}" if v == int(v) else f"{v:.1f} {unit}"
    return f"{n} B"


def parse_size(s: str) -> int:
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    return int(float(s[:-1]) * mult[s[-1].upper()]) if s[-1].upper() in mult else int(s)


def load(path: str):
    rows = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line.startswith("{"):
                r = json.loads(line)
                # single-implementation files (--impl reference / nccl / ours_pg) name their columns "us" / "busbw"
                r.setdefault("ours_us", r.get("us"))
                r.setdefault("ours_busbw", r.get("busbw"))
                rows.append(r)
    return rows


ALGO = {-1: "auto", 0: "one-shot", 1: "two-shot", 2: "nvls-1", 3: "nvls-2", 4: "push", 5: "pull", 6: "nvls", 7: "ll", 8: "ring", 9: "copy-engine"}


def table(rows, dtype: str, min_bytes: int, show_algo: bool) -> str:
    rows = [r for r in rows if r.get("dtype", dtype) == dtype and r["bytes"] >= min_bytes]
    if not rows:
        return "(no rows)\n"
    ops = list(OrderedDict.fromkeys(r["op"] for r in rows))
    sizes = sorted({r["bytes"] for r in rows})
    by = {(r["op"], r["bytes"]): r for r in rows}
    latency = rows[0].get("mode") == "latency"
    has_cmp = any(r.get("nccl_us") for r in rows)
    out = []
    if latency:
        head = ["bytes"] + [f"{op} us" + (" (NCCL us)" if has_cmp else "") for op in ops]
    else:
        head = ["bytes"]
        for op in ops:
            head += [f"{op} GB/s"] + ([f"NCCL GB/s", "ratio"] if has_cmp else []) + (["algo/CTAs"] if show_algo else [])
    out.append("| " + " | ".join(head) + " |")
    out.append("|" + "---|" * len(head))
    for b in sizes:
        cells = [human(b)]
        for op in ops:
            r = by.get((op, b))
            if r is None:
                cells += [""] * (1 if latency else (1 + (2 if has_cmp else 0) + (1 if show_algo else 0)))
                continue
            ok = "" if r.get("correct", True) else " (WRONG)"
            if latency:
                cells.append(f"{r['ours_us']:.1f}" + (f" ({r['nccl_us']:.1f})" if r.get("nccl_us") else "") + ok)
            else:
                cells.append(f"{r['ours_busbw']:.1f}{ok}")
                if has_cmp:
                    if r.get("nccl_us"):
                        cells += [f"{r['nccl_busbw']:.1f}", f"{r['nccl_us'] / r['ours_us']:.2f}"]
                    else:
                        cells += ["", ""]
                if show_algo:
                    cells.append(f"{ALGO.get(r.get('algo', -1), r.get('algo'))}/{r.get('nctas', 0)}")
        out.append("| " + " | ".join(cells) + " |")
    return "\n".join(out) + "\n"


def joined(a_rows, b_rows, dtype: str, min_bytes: int) -> str:
    name_a = a_rows[0].get("impl", "a") if a_rows else "a"
    name_b = b_rows[0].get("impl", "b") if b_rows else "b"
    a = {(r["op"], r["bytes"]): r for r in a_rows if r.get("dtype", dtype) == dtype and r["bytes"] >= min_bytes}
    b = {(r["op"], r["bytes"]): r for r in b_rows if r.get("dtype", dtype) == dtype and r["bytes"] >= min_bytes}
    ops = list(OrderedDict.fromkeys(k[0] for k in a))
    sizes = sorted({k[1] for k in a if k in b})
    head = ["bytes"]
    for op in ops:
        head += [f"{op}: {name_a} us", f"{name_b} us", "ratio"]
    out = ["| " + " | ".join(head) + " |", "|" + "---|" * len(head)]
    for s in sizes:
        cells = [human(s)]
        for op in ops:
            ra, rb = a.get((op, s)), b.get((op, s))
            if ra and rb:
                cells += [f"{ra['ours_us']:.1f}", f"{rb['ours_us']:.1f}", f"{rb['ours_us'] / ra['ours_us']:.2f}"]
            else:
                cells += ["", "", ""]
        out.append("| " + " | ".join(cells) + " |")
    return "\n".join(out) + "\n"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("files", nargs="+")
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--min-bytes", default="1")
    ap.add_argument("--algo", action="store_true", help="add the algorithm and CTA count chosen for every row")
    ap.add_argument("--join", action="store_true", help="two files, one implementation each: side by side")
    args = ap.parse_args()
    mb = parse_size(args.min_bytes)
    if args.join:
        assert len(args.files) == 2, "--join takes exactly two files"
        print(joined(load(args.files[0]), load(args.files[1]), args.dtype, mb))
        return
    for path in args.files:
        rows = load(path)
        n = rows[0].get("n_gpus", "?") if rows else "?"
        print(f"### {path} ({n} GPUs, {args.dtype})\n")
        print(table(rows, args.dtype, mb, args.algo))


if __name__ == "__main__":
    main()
