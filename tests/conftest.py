"""Shared fixtures.  Tests marked ``gpu`` need a B200 and call the CUDA library through its C
ABI; everything else runs on CPU (oracle pins, host logic, ABI/symbol checks, gloo ranks)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


# ---- parity record ---------------------------------------------------------------------------
# Every tolerance comparison records what it saw: the largest bf16-ulp distance (or the largest
# relative F32 error), how many elements exceeded the tight bound, and how many of those were
# admitted by a stated exception clause.  With VRB_PARITY_REPORT=<path> the records are written
# there as JSON lines at the end of the session, so "<= 2 ulp" is a measured statement.
PARITY_RECORDS = []


def record_parity(what, dtype, count, worst, over, admitted, clause=""):
    PARITY_RECORDS.append({"case": what, "dtype": dtype, "elements": int(count), "worst": float(worst),
                           "over_tight_bound": int(over), "admitted_by_clause": int(admitted), "clause": clause})


def pytest_sessionfinish(session, exitstatus):
    path = os.environ.get("VRB_PARITY_REPORT")
    if path and PARITY_RECORDS:
        import json
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "a") as fh:
            for r in PARITY_RECORDS:
                fh.write(json.dumps(r) + "\n")


@pytest.fixture(scope="session")
def orc():
    from oracle import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def cuda_lib():
    """Build (if stale) and load libvrb.so; building needs nvcc only, not a GPU."""
    from vrhino_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def gpu():
    """(backend, ops module) on cuda:0.  Fails -- never skips -- when the extension is absent."""
    import torch
    assert torch.cuda.is_available(), "gpu-marked test collected without a CUDA device"
    from vrhino_b200 import ops
    return ops.B200Backend(), ops


# ---- helpers shared by the parity tests -----------------------------------------------------
def to_torch(t, device="cuda"):
    """Oracle tensor -> torch tensor with the same bits."""
    import torch
    if t.dtype == "bf16":
        return torch.from_numpy(t.data.view(np.int16).copy()).view(torch.bfloat16).to(device)
    if t.dtype == "u8":
        return torch.from_numpy(t.data.copy()).to(device)
    return torch.from_numpy(t.data.copy()).to(device)


def from_torch(x):
    """torch tensor -> (numpy payload, dtype tag): bf16 as uint16 bits."""
    import torch
    x = x.detach().cpu().contiguous()
    if x.dtype == torch.bfloat16:
        return x.view(torch.int16).numpy().view(np.uint16), "bf16"
    return x.numpy(), "f32"


def assert_close(orc, got, want, max_ulp=2, rel=1e-5, atol=0.0, flip_atol=0.0, flip_frac=0.0, what=""):
    """bf16 outputs: <= max_ulp on the bf16 grid (or within atol when stated).
    f32 outputs: |d| <= atol + max(rel*|ref|, 1e-8).

    flip_atol / flip_frac: an F32 output computed FROM a value the reference rounds to bf16
    mid-chain (the normalised value of rms_norm, the LayerNorm output under a bf16 hidden
    state) jumps by one bf16 ulp of that intermediate whenever rsqrtf (CUDA) and 1/sqrtf (C)
    differ in their last bit and the intermediate sits on a rounding boundary.  At most
    flip_frac of the elements may miss the tight tolerance, and those must stay within
    flip_atol (one bf16 ulp of the largest intermediate)."""
    data, tag = from_torch(got)
    assert tag == want.dtype, f"{what}: dtype {tag} != {want.dtype}"
    assert tuple(data.shape) == tuple(want.shape), f"{what}: shape {data.shape} != {want.shape}"
    if tag == "bf16":
        d = orc.bf16_ulp_distance(data, want.data)
        bad = d > max_ulp
        over = int(bad.sum())
        if atol > 0 and bad.any():
            diff = np.abs(orc.bf16_bits_to_f32(data) - want.f32())
            bad &= ~(diff <= atol)
        record_parity(what, "bf16", d.size, d.max() if d.size else 0, over, over - int(bad.sum()),
                      f"|d| <= {atol:g} absolute" if atol > 0 else "")
        if bad.any():
            i = np.unravel_index(np.argmax(np.where(bad, d, 0)), d.shape)
            raise AssertionError(f"{what}: {int(bad.sum())} of {d.size} elements differ by more than {max_ulp} bf16 ulp; "
                                 f"worst at {i}: got {orc.bf16_bits_to_f32(data)[i]!r} want {want.f32()[i]!r}")
        return float((d > 0).mean())
    ref = want.data.astype(np.float64)
    diff = np.abs(data.astype(np.float64) - ref)
    nan_mismatch = np.isnan(data) != np.isnan(want.data)
    tol = atol + np.maximum(rel * np.abs(ref), 1e-8)   # relative, with an absolute floor of 1e-8
    both_nan = np.isnan(data) & np.isnan(want.data)
    same_inf = np.isinf(data) & (data == want.data)
    bad = ~(diff <= tol) & ~both_nan & ~same_inf
    bad |= nan_mismatch
    over = int(bad.sum())
    with np.errstate(invalid="ignore", divide="ignore"):
        finite = np.isfinite(ref) & np.isfinite(data)
        worst_rel = float(np.max(np.where(finite, diff / np.maximum(np.abs(ref), 1e-3), 0.0))) if diff.size else 0.0
    if bad.any() and flip_frac > 0:
        within_flip = bad & (diff <= flip_atol) & ~nan_mismatch
        if bad.mean() <= flip_frac and within_flip.sum() == bad.sum():
            bad[:] = False
    record_parity(what, "f32 (worst = relative error, floor 1e-3)", diff.size, worst_rel, over, over - int(bad.sum()),
                  f"<= {flip_frac:g} of the elements within {flip_atol:g} (one bf16 ulp of a mid-chain value)" if flip_frac > 0 else "")
    if bad.any():
        i = np.unravel_index(np.argmax(np.where(bad, diff, 0)), diff.shape)
        raise AssertionError(f"{what}: {int(bad.sum())} of {diff.size} f32 elements out of tolerance; "
                             f"worst at {i}: got {data[i]!r} want {want.data[i]!r}")
    return float((data != want.data).mean())


def assert_bits_equal(got, want, what=""):
    data, tag = from_torch(got)
    assert tag == want.dtype and tuple(data.shape) == tuple(want.shape), what
    a = data.view(np.uint16 if tag == "bf16" else np.uint32).copy()
    b = want.data.view(np.uint16 if tag == "bf16" else np.uint32).copy()
    if tag == "f32":
        # an F32 NaN produced by arithmetic carries a platform-chosen sign / payload
        # (x86 gives 0xffc00000, the GPU 0x7fffffff); a NaN must match a NaN, bits aside
        a[np.isnan(data)] = 0x7FC00000
        b[np.isnan(want.data)] = 0x7FC00000
    if not np.array_equal(a, b):
        n = int((a != b).sum())
        raise AssertionError(f"{what}: {n} of {a.size} elements are not bit-identical")
