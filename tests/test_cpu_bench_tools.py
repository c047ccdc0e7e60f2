"""The small report tools under bench/ on synthetic input (no GPU): the table maker for sweep
files, the per-collective summary of a communicator trace, the time shares of a launch list."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    res = subprocess.run([sys.executable, *args], capture_output=True, text=True, cwd=ROOT, timeout=60)
    assert res.returncode == 0, res.stdout + res.stderr
    return res.stdout


def test_busbw_table_single_and_joined(tmp_path):
    a, b = tmp_path / "a.jsonl", tmp_path / "b.jsonl"
    with open(a, "w") as f:
        for size in (1024, 1 << 20):
            f.write(json.dumps({"impl": "ours", "op": "allreduce", "dtype": "bf16", "bytes": size, "n_gpus": 8, "mode": "bandwidth",
                                "ours_us": 10.0, "nccl_us": 20.0, "ours_busbw": 1.5, "nccl_busbw": 0.75, "algo": 7, "nctas": 0,
                                "correct": True}) + "\n")
    with open(b, "w") as f:
        for size in (1024, 1 << 20):
            f.write(json.dumps({"impl": "reference", "op": "allreduce", "dtype": "bf16", "bytes": size, "n_gpus": 8,
                                "mode": "bandwidth", "us": 30.0, "busbw": 0.5}) + "\n")
    out = run("bench/busbw_table.py", str(a), "--algo")
    assert "| 1 KiB | 1.5 | 0.8 | 2.00 | ll/0 |" in out and "1 MiB" in out
    out = run("bench/busbw_table.py", "--join", str(a), str(b))
    assert "| 1 KiB | 10.0 | 30.0 | 3.00 |" in out


def test_trace_summary(tmp_path):
    p = tmp_path / "trace.json"
    recs = [{"op": "AllGather", "bytes": 1 << 20, "algo": 9, "ctas": 1, "device_ms": 0.5} for _ in range(4)]
    recs += [{"op": "ReduceScatter", "bytes": 1 << 20, "algo": 5, "ctas": 16, "device_ms": 1.0} for _ in range(2)]
    json.dump({"rank": 0, "nranks": 2, "records": recs}, open(p, "w"))
    out = run("bench/trace_summary.py", str(p), "--steps", "2", "--step-ms", "100")
    assert "AllGather" in out and "ReduceScatter" in out and "communication stream busy: 2.00 ms per step" in out


def test_launch_shares(tmp_path):
    p = tmp_path / "launches.csv"
    head = '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"\n'
    rows = []
    names = ["void <unnamed>::rmsnormFwdWarp<16>(const __nv_bfloat16 *)", "nvjet_tst_256x256", "<unnamed>::adamwFlat(__nv_bfloat16 *)"]
    i = 0
    for step in range(3):
        for name, ns in [(names[0], 1000)] * 2 + [(names[1], 900)] * 10 + [(names[2], 5000), (names[2], 6000)]:
            rows.append(f'"{i}","1","python","h","{name}","1","7","(256, 1, 1)","(8, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","ns","{ns}"')
            i += 1
    open(p, "w").write("==PROF== Connected\n" + head + "\n".join(rows) + "\n")
    out = run("bench/launch_shares.py", str(p), "--last-step", "adamwFlat")
    # the last whole step: 2 + 10 + 2 launches, 2 + 9 + 11 = 22 us
    assert "14 launches" in out and "| `adamwFlat` | 2 | 11 | 50.0 % | 5.5 |" in out and "`rmsnormFwdWarp`" in out
