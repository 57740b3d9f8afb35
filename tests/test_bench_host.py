"""The host-side parts of bench.py that need no GPU: the clock sampler (against a fake
nvidia-smi), the workload description that both arms print, and the promise that the
reference arm imports nothing of this repository."""
import importlib.util
import json
import os
import stat
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


FAKE_SMI = """#!/bin/sh
# prints what `nvidia-smi --query-gpu=... --format=csv,noheader,nounits -lms 25` prints, until killed
i=0
while [ $i -lt 400 ]; do
  if [ $i -lt 3 ]; then echo "0, 1200, 1965, 180.5, 0x0, Not Active, Not Active, Not Active, Not Active"
  else echo "0, 1905, 1965, 950.0, 0x4, Not Active, Not Active, Not Active, Active"; fi
  i=$((i+1)); sleep 0.02
done
"""


def test_clock_sampler_reads_median_clock_and_reasons(tmp_path, monkeypatch):
    fake = tmp_path / "nvidia-smi"
    fake.write_text(FAKE_SMI)
    fake.chmod(fake.stat().st_mode | stat.S_IXUSR)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    bench = _bench()
    s = bench.SmiSampler(0)
    s.start()
    time.sleep(0.4)
    t0 = time.time()
    time.sleep(0.5)
    t1 = time.time()
    out = s.stop(window=(t0, t1))
    assert out["sm_mhz"] == 1905.0 and out["sm_max_mhz"] == 1965.0   # the idle samples before the window do not count
    assert out["reasons"] == ["sw_power_cap"] and out["power_w_max"] == 950.0 and out["samples"] >= 3


def test_clock_sampler_without_nvidia_smi(tmp_path, monkeypatch):
    monkeypatch.setenv("PATH", str(tmp_path))
    out_of_path = _bench().SmiSampler(0)
    out_of_path.start()
    assert out_of_path.stop()["reasons"] == ["nvidia-smi unavailable"]


def test_both_arms_describe_the_same_workload():
    bench = _bench()
    a = bench.workload_config(1 << 28, 4, "float32", 8)
    assert a["placement"] == "in place, ordinary device tensor" and a["parallelism"] == "dp8" and a["op"] == "SUM"
    assert a["tensor_bytes"] == 1 << 30 and a["single_gpu_note"] is None
    assert "changes nothing" in bench.workload_config(1 << 28, 4, "float32", 1)["single_gpu_note"]
    # both arms call the one function: no second description anywhere in the file
    src = open(os.path.join(ROOT, "bench.py")).read()
    assert src.count("workload_config(") == 3   # the definition, this library's arm, the reference arm


def test_reference_arm_imports_nothing_of_this_repository():
    """Without a GPU the reference arm prints its one `unavailable` line; neither then nor while
    it gets there may it load this repository's package or library."""
    code = ("import sys, runpy; sys.argv = ['bench.py', '--impl', 'reference']; "
            "runpy.run_path(%r, run_name='__main__'); "
            "print('LOADED', sorted(m for m in sys.modules if 'switchml' in m))" % os.path.join(ROOT, "bench.py"))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    record = json.loads(lines[0])
    assert record["impl"] == "reference" and "unavailable" in record
    assert lines[-1] == "LOADED []"


def test_sweep_table_compares_each_element_type_with_its_own_nccl_column():
    spec = importlib.util.spec_from_file_location(
        "sweep_under_test", os.path.join(ROOT, "p4app-switchML_b200", "benchmarks", "allreduce_sweep.py"))
    sweep = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sweep)

    def rec(impl, numel, us, dtype="float32"):
        return {"impl": impl, "numel": numel, "us": us, "dtype": dtype, "ate_per_s": numel / us * 1e6, "bus_gbs": 1.0}
    table = sweep.markdown_table([rec("nccl", 1024, 20.0), rec("nccl-int32", 1024, 10.0, "int32"),
                                  rec("sml-float", 1024, 10.0), rec("sml-int32", 1024, 20.0, "int32"),
                                  rec("nccl", 4096, 30.0), rec("sml-float", 4096, 60.0)], 4, 100, 10)
    lines = table.splitlines()
    assert lines[2] == "| elements | nccl | nccl-int32 | sml-float | sml-int32 |"
    assert lines[4] == "| 2^10 | 20.0 | 10.0 | 10.0 (2.00x) | 20.0 (0.50x) |"   # float against nccl, int32 against nccl-int32
    assert lines[5] == "| 2^12 | 30.0 |  | 60.0 (0.50x) |  |"
