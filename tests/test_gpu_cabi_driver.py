"""The C ABI called from compiled C++ with nothing in between (tests/cabi_driver.cc): benchmark config 1, one tensor-core
mat_mul, one argmax and one error path, each checked against the CPU oracle inside the driver.  This is the nearest
compilable stand-in for the Rust `impl Operator` shim (no Rust toolchain in this environment)."""
import os
import subprocess

import pytest

import __graft_entry__ as graft

pytestmark = pytest.mark.gpu


def test_cpp_driver_runs_config1_through_the_c_abi(pkg, orc, dev):
    exe = graft.build_cabi_driver()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    print(r.stdout)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all checks passed" in r.stdout
    assert not os.environ.get("LD_PRELOAD")  # the driver found both libraries through its own run path
