"""The C++ programs on the dummy backend (hello_world, allreduce_benchmark, dnn_benchmark;
reference examples/hello_world, benchmarks/allreduce_benchmark, benchmarks/dnn_benchmark),
the shipped configuration templates, and workers using a stand-alone switchml_switchd."""
import glob
import multiprocessing as mp
import os
import signal
import subprocess
import time

import numpy as np
import pytest

from conftest import free_port
from switchml_b200.utils.config import check_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "p4app-switchML_b200")
BIN = os.path.join(PKG, "bin")


@pytest.fixture(scope="module")
def built():
    import importlib.util
    spec = importlib.util.spec_from_file_location("_switchml_build", os.path.join(PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()


@pytest.fixture
def cfg_dir(tmp_path):
    text = open(os.path.join(PKG, "configs", "switchml-dummy.cfg")).read()
    text = text.replace("num_workers = 1", "num_workers = 3").replace("bandwidth = 100000.0", "bandwidth = 0")
    (tmp_path / "switchml.cfg").write_text(text)
    return tmp_path


def test_shipped_templates_validate():
    files = sorted(glob.glob(os.path.join(PKG, "configs", "switchml-*.cfg")))
    assert len(files) == 3
    for f in files:
        dump = check_config(open(f).read())
        assert "backend = " + os.path.basename(f)[len("switchml-"):-len(".cfg")] in dump


def test_hello_world(built, cfg_dir):
    r = subprocess.run([os.path.join(BIN, "hello_world")], cwd=cfg_dir, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Data verified successfully" in r.stdout


@pytest.mark.parametrize("extra", [["--tensor-type", "float", "--inplace", "false"], ["--tensor-type", "int32"],
                                   ["--tensor-type", "float", "--random", "true", "--seed", "5", "--sync-every", "0"]])
def test_allreduce_benchmark_verifies(built, cfg_dir, extra):
    cmd = [os.path.join(BIN, "allreduce_benchmark"), "--tensor-numel", "200001", "--num-jobs", "4",
           "--num-warmup-jobs", "2", "--verify", "true", "--dump-stats", "true"] + extra
    r = subprocess.run(cmd, cwd=cfg_dir, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Results verified successfully." in r.stdout
    assert "Goodput min: #" in r.stdout and "Aggregated tensor elements per second: #" in r.stdout
    assert "Submitted jobs: #" in r.stdout


def test_dnn_benchmark(built, cfg_dir):
    cmd = [os.path.join(BIN, "dnn_benchmark"), "--model", os.path.join(PKG, "benchmarks", "models", "example.csv"),
           "--num-iters", "3", "--num-warmup-iters", "1", "--verify", "true"]
    r = subprocess.run(cmd, cwd=cfg_dir, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Results verified successfully." in r.stdout and "Iterations/s min: #" in r.stdout


def test_benchmark_stops_on_sigint(built, cfg_dir):
    text = (cfg_dir / "switchml.cfg").read_text().replace("bandwidth = 0", "bandwidth = 50.0")
    (cfg_dir / "switchml.cfg").write_text(text)
    p = subprocess.Popen([os.path.join(BIN, "allreduce_benchmark"), "--tensor-numel", "4000000", "--num-jobs", "50"],
                         cwd=cfg_dir, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    # Interrupt once jobs are in flight (the first lines of output say so), not after a guess
    # of how long start-up takes.
    head = ""
    while "Submitting" not in head:
        line = p.stdout.readline()
        assert line, "the benchmark ended early:\n" + head
        head += line
    time.sleep(0.5)
    p.send_signal(signal.SIGINT)
    out, _ = p.communicate(timeout=30)
    assert p.returncode == 0 and "stopping the context" in head + out


def _switchd_worker(rank, n, ctl_port, udp_port, q):
    try:
        import switchml_b200 as sml
        ctx = sml.Context.get_instance()
        assert ctx.start(sml.make_config("udp", rank=rank, num_workers=n, packet_numel=64, num_worker_threads=2,
                                         max_outstanding_packets=64, controller_port=ctl_port, switch_port=udp_port,
                                         worker_port=0, spawn_switch=False))
        x = np.full(5000, rank + 1.0, dtype=np.float32)
        ctx.all_reduce(x)
        ctx.stop()
        q.put((rank, float(x[0]), float(x[-1])))
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e), None))


def test_workers_with_standalone_switchd(built, tmp_path):
    ctl, udp = free_port(), free_port()
    log = tmp_path / "switchd.log"
    d = subprocess.Popen([os.path.join(BIN, "switchml_switchd"), "--ip", "127.0.0.1", "--port", str(ctl),
                          "--udp-port", str(udp), "--log-level", "0", "--log-file", str(log)],
                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    try:
        time.sleep(0.5)
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        procs = [ctx.Process(target=_switchd_worker, args=(r, 2, ctl, udp, q)) for r in range(2)]
        for p in procs:
            p.start()
        got = [q.get(timeout=120) for _ in range(2)]
        for p in procs:
            p.join(timeout=30)
        for rank, first, last in got:
            assert first == 3.0 and last == 3.0, (rank, first, last)
    finally:
        d.send_signal(signal.SIGTERM)
        out, _ = d.communicate(timeout=10)
    assert "broadcast" in out
    text = log.read_text()
    assert "data on UDP %d" % udp in text and "switchml_switchd stopped" in text


def test_switchd_console_on_standard_input(built, tmp_path):
    """The daemon's own shell (the reference controller runs its CLI in-process)."""
    ctl, udp = free_port(), free_port()
    cmds = "ping\nshow_switch_address\nset_drop_probabilities 0.25 0.5 7\nshow_drop_probabilities\n" \
           "show_ports\nbogus\nhelp\nexit\n"
    r = subprocess.run([os.path.join(BIN, "switchml_switchd"), "--ip", "127.0.0.1", "--port", str(ctl),
                        "--udp-port", str(udp), "--log-level", "0", "--log-file", "", "--console", "true"],
                       input=cmds, capture_output=True, text=True, timeout=60, cwd=tmp_path)
    assert r.returncode == 0, r.stdout + r.stderr
    out = r.stdout
    assert "udp_port %d" % udp in out and "ingress 0.25" in out and "egress 0.5" in out
    assert "127.0.0.1:%d/udp  up" % udp in out
    assert "unknown command: bogus" in out and "show_queue_pairs_counters" in out
    assert out.count("(switchml) ") >= 8


def test_python_hello_world_example(tmp_path):
    import sys
    script = os.path.join(PKG, "examples", "python", "hello_world.py")
    r = subprocess.run([sys.executable, script, "--num-tensors", "3", "--numel", "5000"], capture_output=True,
                       text=True, timeout=120, cwd=tmp_path)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Data verified successfully: 3 tensors of 5000 elements, 2 workers, backend dummy" in r.stdout
    assert "Finished jobs: #3#" in r.stdout


def test_dnn_model_generator_matches_parameter_counts(tmp_path):
    """benchmarks/make_dnn_model_csv.py: one line per parameter-owning module, the numel column
    adds up to the model's parameter count, and dnn_benchmark accepts the file."""
    import sys
    script = os.path.join(PKG, "benchmarks", "make_dnn_model_csv.py")
    r = subprocess.run([sys.executable, script, "--model", "resnet50", "--batch", "8"], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    rows = [l.split(",") for l in r.stdout.strip().splitlines()[1:]]
    assert sum(int(x[1]) for x in rows) == 25557032          # ResNet-50
    assert all(int(x[2]) >= 2000 and int(x[3]) >= int(x[2]) for x in rows)
    shipped = open(os.path.join(PKG, "benchmarks", "models", "bert_large.csv")).read().strip().splitlines()[1:]
    assert sum(int(l.split(",")[1]) for l in shipped) == 335174458   # BERT-large with the MLM head


def test_static_archive_links_with_plain_gcc(built, cfg_dir):
    """lib/libswitchml_b200.a (the reference ships its client library as a static archive):
    a user program links against it with g++ and the static CUDA runtime, no nvcc needed."""
    import shutil
    cuda_lib = "/usr/local/cuda/lib64"
    archive = os.path.join(PKG, "lib", "libswitchml_b200.a")
    if not (os.path.exists(archive) and os.path.exists(os.path.join(cuda_lib, "libcudart_static.a")) and shutil.which("g++")):
        pytest.skip("no static archive or no static CUDA runtime")
    src = cfg_dir / "user.cc"
    src.write_text('''
        #include <cstdio>
        #include <vector>
        #include "switchml/context.h"
        int main() {
          switchml::Context& c = switchml::Context::GetInstance();
          if (!c.Start()) return 1;
          std::vector<float> x(1000, 1.5f);
          auto job = c.AllReduce(x.data(), x.data(), x.size(), switchml::FLOAT32, switchml::SUM);
          c.Stop();
          printf("sum %g status %d\\\\n", x[0], static_cast<int>(job->GetJobStatus()));
          return 0;
        }''')
    exe = cfg_dir / "user"
    r = subprocess.run(["g++", "-std=c++17", "-I" + os.path.join(PKG, "include"), str(src), archive, "-L" + cuda_lib,
                        "-lcudart_static", "-ldl", "-lrt", "-lpthread", "-o", str(exe)], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([str(exe)], cwd=cfg_dir, capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "sum 4.5 status 3" in r.stdout, r.stdout + r.stderr   # 3 dummy workers, FINISHED
