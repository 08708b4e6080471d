"""The exact parallel form of a sequential f32 sum of non-negative terms (RMSNorm squares, softmax
weights): its host-compilable core, built with g++ and compared with the one-accumulator loop."""
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent


def test_exact_sum_equals_sequential_sum_on_the_host(tmp_path):
    exe = tmp_path / "exact_sum_host_check"
    subprocess.run(["g++", "-O2", "-ffp-contract=off", "-o", str(exe), str(HERE / "exact_sum_host_check.cpp")], check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    print(res.stdout)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.startswith("0/6000 mismatches")
