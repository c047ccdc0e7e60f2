"""Aggregates a launch list into time shares per kernel.

The launch list is what Nsight Compute writes with

    ncu --metrics gpu__time_duration.sum --clock-control none --csv --log-file launches.csv <program>

(one row per kernel launch, one pass, cold caches, launches serialised: compare SHARES,
not absolute times).  Usage:

    python bench/launch_shares.py launches.csv [--last-step adamwFlat] [--top 25]

--last-step NAME keeps only the launches after the second-to-last burst of kernel NAME
(for a training program whose step ends with the optimizer kernel: the last whole step).
"""
from __future__ import annotations

import argparse
import csv
import io
import re
from collections import defaultdict


def read_rows(path: str):
    text = open(path, errors="replace").read()
    start = text.find('"ID"')
    if start < 0:
        raise SystemExit("no CSV header found (was the program run under ncu --csv?)")
    rows = []
    for r in csv.DictReader(io.StringIO(text[start:])):
        if r.get("Metric Name") != "gpu__time_duration.sum":
            continue
        val = float(r["Metric Value"].replace(",", ""))
        unit = r.get("Metric Unit", "ns")
        us = val / 1e3 if unit in ("ns", "nsecond") else val if unit in ("us", "usecond") else val * 1e3 if unit in ("ms", "msecond") else val * 1e6
        rows.append((int(r["ID"]), r["Kernel Name"], us))
    rows.sort()
    return rows


def short(name: str) -> str:
    name = name.replace("(anonymous namespace)::", "").replace("<unnamed>::", "")
    name = re.sub(r"\(.*", "", name)            # argument list
    name = re.sub(r"<.*", "", name)             # template arguments
    name = re.sub(r"^void\s+", "", name)
    return name.split("::")[-1][:60]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("csv")
    ap.add_argument("--last-step", default="")
    ap.add_argument("--top", type=int, default=25)
    args = ap.parse_args()
    rows = read_rows(args.csv)
    if args.last_step:
        hits = [i for i, (_, n, _) in enumerate(rows) if args.last_step in n]
        # bursts of the marker kernel: consecutive hits with no more than a few other launches between
        bursts, prev = [], None
        for i in hits:
            if prev is None or i - prev > 8:
                bursts.append([i, i])
            else:
                bursts[-1][1] = i
            prev = i
        if len(bursts) >= 2:
            rows = rows[bursts[-2][1] + 1: bursts[-1][1] + 1]
    total = sum(us for _, _, us in rows)
    agg = defaultdict(lambda: [0, 0.0])
    for _, n, us in rows:
        a = agg[short(n)]
        a[0] += 1
        a[1] += us
    print(f"{len(rows)} launches, {total / 1e3:.2f} ms of kernel time\n")
    print("| kernel | launches | total us | share | mean us |")
    print("|---|---|---|---|---|")
    for name, (cnt, us) in sorted(agg.items(), key=lambda kv: -kv[1][1])[: args.top]:
        print(f"| `{name}` | {cnt} | {us:.0f} | {100 * us / total:.1f} % | {us / cnt:.1f} |")


if __name__ == "__main__":
    main()
