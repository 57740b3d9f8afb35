"""Runs the native unit tests (csrc/tests/core_tests.cc): static slicing, barrier, job
state machine, timeout queue, software switch pipeline, quantisation arithmetic, control
plane collectives, context lifecycle on the dummy backend."""
import importlib.util
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "p4app-switchML_b200")


def _build():
    spec = importlib.util.spec_from_file_location("_switchml_build", os.path.join(PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()


def test_core_tests_binary():
    _build()
    r = subprocess.run([os.path.join(PKG, "bin", "core_tests")], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    for name in ("logging", "numa_helpers", "simd_matches_scalar", "static_slice", "barrier", "job_fsm",
                 "timeout_queue", "soft_switch", "soft_switch_concurrent_pipes", "quant_math", "flag_protocol_model",
                 "control_plane", "context_dummy"):
        assert "ok   " + name in r.stdout
