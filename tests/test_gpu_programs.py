"""The C++ programs with backend = cuda: device buffers go straight into Context::AllReduceAsync
(the reference's benchmarks can only allocate GPU buffers; none of its backends accepts them)."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "p4app-switchML_b200")
BIN = os.path.join(PKG, "bin")


@pytest.fixture
def cuda_cfg(tmp_path):
    text = open(os.path.join(PKG, "configs", "switchml-cuda.cfg")).read()
    (tmp_path / "switchml.cfg").write_text(text)
    return tmp_path


def _run(cmd, cwd, env=None):
    r = subprocess.run(cmd, cwd=cwd, capture_output=True, text=True, timeout=180, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


def test_hello_world_on_gpu(cuda_cfg):
    if not os.path.exists(os.path.join(BIN, "hello_world")):
        pytest.skip("programs not built")
    assert "Data verified successfully" in _run([os.path.join(BIN, "hello_world")], cuda_cfg)


def test_allreduce_benchmark_on_gpu(cuda_cfg):
    if not os.path.exists(os.path.join(BIN, "allreduce_benchmark")):
        pytest.skip("programs not built")
    out = _run([os.path.join(BIN, "allreduce_benchmark"), "--device", "gpu", "--tensor-type", "float",
                "--tensor-numel", "4000001", "--num-jobs", "5", "--num-warmup-jobs", "2", "--verify", "true",
                "--inplace", "false", "--random", "true", "--seed", "3"], cuda_cfg)
    assert "Results verified successfully." in out and "Aggregated tensor elements per second" in out
    out = _run([os.path.join(BIN, "allreduce_benchmark"), "--device", "gpu", "--tensor-type", "int32",
                "--tensor-numel", "1000000", "--num-jobs", "3", "--num-warmup-jobs", "1", "--verify", "true"], cuda_cfg)
    assert "Results verified successfully." in out


def test_dnn_benchmark_on_gpu(cuda_cfg):
    if not os.path.exists(os.path.join(BIN, "dnn_benchmark")):
        pytest.skip("programs not built")
    out = _run([os.path.join(BIN, "dnn_benchmark"), "--device", "gpu", "--model",
                os.path.join(PKG, "benchmarks", "models", "example.csv"), "--num-iters", "5",
                "--num-warmup-iters", "2", "--verify", "true"], cuda_cfg)
    assert "Results verified successfully." in out and "Iterations/s" in out


def test_nccl_collnet_plugin_on_gpu(cuda_cfg):
    """The collective-network plugin with device pointers (NCCL_PTR_CUDA), driven by its harness."""
    exe, plugin = os.path.join(BIN, "collnet_harness"), os.path.join(PKG, "lib", "libnccl-net-switchml.so")
    if not (os.path.exists(exe) and os.path.exists(plugin)):
        pytest.skip("plugin not built")
    out = _run([exe, "--plugin", plugin, "--device", "gpu", "--numel", "300000", "--rounds", "2"], cuda_cfg)
    assert "ptrSupport 0x3" in out and "collnet harness ok" in out and "on the gpu" in out
    out = _run([exe, "--plugin", plugin, "--device", "pinned", "--numel", "5000", "--rounds", "1"], cuda_cfg)
    assert "collnet harness ok" in out and "pinned host memory" in out
