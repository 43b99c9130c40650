"""The C++ backend plugged into the reference's own operator layer.

`wechat-tfcc_b200/plugin/_build/tfcc_b200_dropin_test` is built by `__graft_entry__.build()`
where the reference tree is available: the reference's `tfcc_core` sources compiled as they
lie, plus `plugin/tfcc_b200.cpp`, linked against `libtfcc_b200.so`.  It calls
`tfcc::blas::matmul`, `tfcc::data::set/get` and `tfcc::b200::quantization::*` on a B200 device
and checks them against host loops.  On a machine where the executable was never built the
test is skipped.
"""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
EXE = Path(__file__).resolve().parent.parent / "wechat-tfcc_b200" / "plugin" / "_build" / "tfcc_b200_dropin_test"


def test_reference_operator_layer_runs_on_the_b200_backend(pkg):
    if not EXE.exists():
        pytest.skip("drop-in executable not built (needs the reference tree at build time)")
    r = subprocess.run([str(EXE)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "DROPIN OK" in r.stdout
