"""Host code under ThreadSanitizer, AddressSanitizer and UndefinedBehaviorSanitizer: the native unit tests (threads of
the dummy backend, scheduler barrier, control-plane collectives, software switch) must run
clean. The reference has no sanitizer configuration; this is the race detector of the
host side."""
import importlib.util
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "p4app-switchML_b200")


def _build_module():
    spec = importlib.util.spec_from_file_location("_switchml_build", os.path.join(PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("kind", ["thread", "address", "undefined"])
def test_native_tests_under_sanitizer(kind):
    exe = _build_module().build_sanitized(kind)
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0", ASAN_OPTIONS="detect_leaks=0")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    assert "ThreadSanitizer" not in out and "AddressSanitizer" not in out and "runtime error" not in out, out[-3000:]
    assert out.count("ok  ") == 13


def test_checked_build_loads_and_exports_the_whole_c_interface():
    """build-checked/ is built from the same sources with -DSWITCHML_CHECKED; the Python
    binding must be able to load it in place of lib/ (every declared function present)."""
    import sys
    lib = _build_module().build_checked()
    code = ("import sys; sys.path.insert(0, %r); import switchml_b200; from switchml_b200._native import lib; "
            "assert lib().sml_checked_build() == 1; print('checked library ok')" % ROOT)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300,
                       env=dict(os.environ, SWITCHML_B200_LIBRARY=lib))
    assert r.returncode == 0 and "checked library ok" in r.stdout, r.stdout + r.stderr
