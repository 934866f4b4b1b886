"""Host-side checks of bench.py that need no GPU: the workload description per world size and the reference arm's line
on a tiny stand-in configuration."""
import json
import subprocess
import sys
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_workload_config_names_the_sharding():
    sys.path.insert(0, ROOT)
    import bench
    one = bench.workload_config(1)
    assert one["parallelism"] == "single" and one["sharding"] == "single GPU" and "workload" in one
    for n in (2, 4, 8):
        c = bench.workload_config(n)
        assert c["parallelism"] == f"tp{n}" and "KV heads H/N per GPU" in c["sharding"]
        assert bench.workload_config(n, "replicas")["parallelism"] == f"dp{n}"
    # no model keys in the config: the contract wants the workload named, nothing else
    assert "model" not in one and one["context"] == 131072 and one["topk"] == 2048


def test_bench_help_lists_every_mode():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--help"], capture_output=True, text=True,
                         timeout=120)
    assert out.returncode == 0
    for word in ("--gpus", "--steps", "--warmup", "--impl", "seqshard", "varlen", "replicas", "--pdl", "--gemv"):
        assert word in out.stdout
