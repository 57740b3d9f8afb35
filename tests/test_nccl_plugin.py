"""libnccl-net-switchml.so, the NCCL collective-network plugin (reference
frameworks_integration/nccl_plugin/switchml_plugin.cc), driven through its exported
`ncclCollNetPlugin_v8` table by bin/collnet_harness in the order NCCL's proxy uses:
init, devices, getProperties, reduceSupport, listen, connect, regMr, iallreduce, test,
iflush, deregMr, closeColl, closeListen. One worker on the dummy backend; two workers as
two processes on the UDP backend with the software switch."""
import ctypes
import os
import subprocess

import pytest

from conftest import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "p4app-switchML_b200")
EXE = os.path.join(PKG, "bin", "collnet_harness")
PLUGIN = os.path.join(PKG, "lib", "libnccl-net-switchml.so")


@pytest.fixture(scope="module")
def built():
    import importlib.util
    spec = importlib.util.spec_from_file_location("_switchml_build", os.path.join(PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()


def test_plugin_exports_the_v8_symbol(built):
    lib = ctypes.CDLL(PLUGIN)
    table = ctypes.c_void_p.in_dll(lib, "ncclCollNetPlugin_v8")
    name = ctypes.cast(ctypes.addressof(table), ctypes.POINTER(ctypes.c_char_p))[0]
    assert name == b"SWITCHMLv8"


def test_one_worker_on_the_dummy_backend(built, tmp_path):
    text = open(os.path.join(PKG, "configs", "switchml-dummy.cfg")).read().replace("bandwidth = 100000.0", "bandwidth = 0")
    (tmp_path / "switchml.cfg").write_text(text)
    r = subprocess.run([EXE, "--plugin", PLUGIN, "--numel", "7001"], cwd=tmp_path, capture_output=True, text=True,
                       timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "collnet harness ok: rank 0 of 1" in r.stdout
    # the refusals the harness provokes are reported through NCCL's logger
    assert "does not come from a worker of this session" in r.stderr
    assert "outside their registered regions" in r.stderr


def test_two_workers_on_the_udp_backend(built, tmp_path):
    text = open(os.path.join(PKG, "configs", "switchml-udp.cfg")).read()
    text = text.replace("num_workers = 1", "num_workers = 2").replace("controller_port = 50099",
                                                                      "controller_port = %d" % free_port())
    text = text.replace("switch_port = 48864", "switch_port = %d" % free_port()).replace("worker_port = 4000",
                                                                                         "worker_port = 0")
    text = text.replace("num_worker_threads = 4", "num_worker_threads = 2")
    (tmp_path / "switchml.cfg").write_text(text)
    xdir = tmp_path / "handles"
    xdir.mkdir()
    procs = []
    for rank in range(2):
        env = dict(os.environ, SWITCHML_RANK=str(rank))
        procs.append(subprocess.Popen([EXE, "--plugin", PLUGIN, "--exchange-dir", str(xdir), "--numel", "3000",
                                       "--rounds", "2"], cwd=tmp_path, env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=120) for p in procs]
    for rank, (p, (out, err)) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, out + err
        assert "collnet harness ok: rank %d of 2" % rank in out
