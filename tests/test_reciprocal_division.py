"""The division-free quotient of the pixel_norm / l2_normalize tile kernels (vrb_pixel_norm.cu: q = x r, e = x - d q, q + e r with r = RN(1 / d))
is the correctly rounded quotient: all 2^30 (bf16 significand, F32 significand) pairs, enumerated on the host with
IEEE single-precision arithmetic (no contraction), plus the negative control without the correction step."""
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def proof(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("proof") / "reciprocal_division_proof")
    base = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", os.path.join(HERE, "reciprocal_division_proof.c"), "-o", exe, "-lm"]
    if subprocess.run(base[:4] + ["-march=native"] + base[4:], capture_output=True).returncode != 0:
        subprocess.run(base, check=True, capture_output=True)      # without hardware FMA: slower, same answer
    return exe


def test_corrected_reciprocal_product_is_the_rounded_quotient(proof):
    run = subprocess.run([proof], capture_output=True, text=True, timeout=1500)
    assert run.returncode == 0, run.stdout
    assert run.stdout.split() == ["pairs", str(128 << 23), "mismatches", "0"]


def test_the_check_can_fail(proof):
    run = subprocess.run([proof, "uncorrected"], capture_output=True, text=True, timeout=1500)
    assert run.returncode == 1
    assert int(run.stdout.split()[3]) > (128 << 23) // 8
