"""Per-collective table from a communicator trace (flagcxCommTraceDump, `bench.py --trace-comm`).

    python bench/trace_summary.py trace.json --steps 10 [--step-ms 200.5]

Groups the records by (operation, bytes, algorithm, CTAs) and prints calls, device time
per call (CUDA events on the stream the collective ran on), and the total per training
step; with --step-ms also the share of a step that the communication stream is busy.
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict

ALGO = {-1: "-", 0: "oneshot", 1: "twoshot", 2: "nvls1", 3: "nvls2", 4: "push", 5: "pull", 6: "nvls", 7: "ll", 8: "ring", 9: "ce"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("trace")
    ap.add_argument("--steps", type=int, default=1, help="training steps the trace covers")
    ap.add_argument("--step-ms", type=float, default=0.0)
    args = ap.parse_args()
    doc = json.load(open(args.trace))
    groups = defaultdict(list)
    for r in doc["records"]:
        groups[(r["op"], r["bytes"], r["algo"], r["ctas"])].append(r["device_ms"])
    total = 0.0
    print(f"# rank {doc['rank']} of {doc['nranks']}, {len(doc['records'])} records over {args.steps} step(s)")
    print(f"{'op':>14} {'bytes':>12} {'algo':>8} {'ctas':>4} {'calls/step':>10} {'us/call':>9} {'min':>8} {'max':>8} {'ms/step':>8} {'GB/s':>7}")
    for (op, nbytes, algo, ctas), ms in sorted(groups.items(), key=lambda kv: -sum(kv[1])):
        per_step = sum(ms) / args.steps
        total += per_step
        mean = sum(ms) / len(ms) * 1e3
        n = doc["nranks"]
        moved = nbytes * (n - 1) / n  # bytes this rank receives (all-gather) or fetches (reduce-scatter)
        print(f"{op:>14} {nbytes:>12} {ALGO.get(algo, str(algo)):>8} {ctas:>4} {len(ms) / args.steps:>10.1f} {mean:>9.1f} "
              f"{min(ms) * 1e3:>8.1f} {max(ms) * 1e3:>8.1f} {per_step:>8.2f} {moved / mean / 1e3 if mean else 0:>7.0f}")
    line = f"communication stream busy: {total:.2f} ms per step"
    if args.step_ms:
        line += f" = {100 * total / args.step_ms:.1f} % of the {args.step_ms:.1f} ms step"
    print(line)


if __name__ == "__main__":
    main()
