"""Host-side exhaustive check behind a claim in the quantisation kernels: the row scale amax / 127 is computed
without the division routine (``scale_of_amax`` in ``pytorch_b200/csrc/dynamic_quant.cu``) and must equal the IEEE
quotient for every float the fast path accepts."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def test_amax_over_127_by_refinement_equals_the_ieee_quotient(tmp_path):
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    exe = str(tmp_path / "div127_check")
    build = subprocess.run([gcc, "-O2", "-mfma", "-ffp-contract=off", os.path.join(HERE, "div127_check.c"), "-o", exe, "-lm"],
                           capture_output=True, text=True)
    if build.returncode != 0:
        pytest.skip("this host's compiler cannot emit fused multiply-adds: " + build.stderr[-200:])
    out = subprocess.run([exe], capture_output=True, text=True, timeout=600).stdout.split()
    assert out[0] == "3c010204"                       # RN(1/127), the constant the kernel uses
    assert int(out[1]) == 0, f"{out[1]} of {out[2]} inputs differ"
    assert int(out[2]) > 1_900_000_000
