"""The checked build of the library (``build.py --checked``, -DSWITCHML_CHECKED): the
aggregation kernels verify the geometry of every tile before touching it and report
STATUS_BOUNDS instead of dereferencing anything out of range. Stands in for a memory
checker on machines where none may be run. Runs in child processes because the library
to load is chosen by an environment variable before the package is imported."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKED = os.path.join(ROOT, "p4app-switchML_b200", "build-checked", "libswitchml_b200.so")

BODY = """
import sys
sys.path.insert(0, %r)
import numpy as np, torch
from switchml_b200._native import lib, NativeError
from switchml_b200.ops.emulation import emulated_allreduce
from switchml_b200.ops.oracle import quant_allreduce_oracle, int_allreduce_oracle
assert lib().sml_checked_build() == 1, "not the checked build"
""" % ROOT


def _child(code, **env):
    e = dict(os.environ, SWITCHML_B200_LIBRARY=CHECKED, **env)
    r = subprocess.run([sys.executable, "-c", BODY + textwrap.dedent(code)], capture_output=True, text=True,
                       timeout=300, env=e)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    return r.stdout


@pytest.fixture(scope="module", autouse=True)
def built():
    if not os.path.exists(CHECKED):
        pytest.skip("build-checked/ is not there (python build.py --checked)")


def test_results_are_unchanged_and_no_check_fires():
    out = _child("""
        for n, numel, algo in ((2, 65, "staged"), (4, 40000, "staged"), (8, (1 << 20) + 1, "staged"),
                               (4, 4096, "oneshot"), (8, 255, "oneshot")):
            g = torch.Generator().manual_seed(numel)
            xs = [(torch.rand(numel, generator=g) * 2 - 1) * 10.0 ** (r % 3) for r in range(n)]
            outs = emulated_allreduce([x.cuda() for x in xs], mode="quant", algo=algo, block_numel=64,
                                      slot_bytes=32768)
            want = quant_allreduce_oracle([x.numpy() for x in xs], 64)
            assert all(np.array_equal(o.cpu().numpy(), want) for o in outs), (n, numel, algo)
            xi = [torch.randint(-2 ** 30, 2 ** 30, (numel,), generator=g, dtype=torch.int32) for r in range(n)]
            outs = emulated_allreduce([x.cuda() for x in xi], mode="sum", algo=algo)
            want = int_allreduce_oracle([x.numpy() for x in xi])
            assert all(np.array_equal(o.cpu().numpy(), want) for o in outs), (n, numel, algo)
        print("checked build ok")
    """)
    assert "checked build ok" in out


@pytest.mark.parametrize("algo", ["staged", "oneshot"])
def test_a_region_that_is_too_small_is_reported_not_touched(algo):
    """The kernels are told that the staging region is 4 KiB (the memory itself is as large
    as ever): every tile fails its check, the outputs stay as they were, status 3."""
    out = _child("""
        xs = [torch.ones(5000, device="cuda") * (r + 1) for r in range(4)]
        outs = [torch.full((5000,), -7.0, device="cuda") for _ in range(4)]
        try:
            emulated_allreduce(xs, mode="quant", algo=%r, block_numel=64, slot_bytes=32768, outputs=outs)
            raise SystemExit("the geometry check did not fire")
        except NativeError as e:
            msg = str(e)
        torch.cuda.synchronize()
        assert all(bool((o == -7.0).all()) for o in outs), "a refused tile was written"
        assert all(float(x[0]) == r + 1 for r, x in enumerate(xs))
        print("refused:", msg)
        # the device is fine afterwards
        y = torch.arange(10, device="cuda").sum().item()
        assert y == 45
    """ % algo, SWITCHML_CHECKED_PRETEND_STAGE_BYTES="4096")
    assert "refused:" in out and "kernel status" in out
    status = int(out.split("kernel status")[1].split()[0])
    assert status & 0xf == 3
