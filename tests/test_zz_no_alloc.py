"""GroupNorm through the entry point that carries its own scratch.

Who needs it: a caller that cannot give the library a device workspace -- every byte of its
device budget belongs to a planner-owned pool that must not grow while a step runs, or it sits on
a thread that may not enter cudaMalloc (the call synchronises the device).  The entry point
promises to allocate nothing and to behave exactly like vrb_group_norm, within a fixed limit on
batch x groups.

Checked here, through the C ABI only: the output equals the workspace-taking entry point's output
(same kernels, so bit for bit; the tolerance the other GroupNorm tests use is asserted too), on
two calls in a row with different shapes so that whatever the first call left in the shared
scratch is seen to be harmless; the limit is enforced with a clear error; and nothing is
allocated -- neither by the library's own count of its cudaMalloc calls nor by the device's free
memory, read around a call that is the FIRST use of the library in a fresh process and takes the
path a VAE decoder takes (bf16, SiLU fused, more than 4 Mi elements: the function-table kernel).
The file name sorts last on purpose: if it fails under `-x`, every other test has already run.
It does not depend on them: it also passes in a fresh process.
"""
import ctypes
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

P = ctypes.c_void_p
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _fixed(lib, x, weight, bias, out, groups, eps, silu):
    import torch
    batch, channels = x.shape[0], x.shape[1]
    spatial = x.numel() // (batch * channels)
    code = 2 if x.dtype == torch.bfloat16 else 0
    return lib.vrb_group_norm_fixed_scratch(P(x.data_ptr()), code, P(weight.data_ptr()), 0, P(bias.data_ptr()), 0,
                                            P(out.data_ptr()), batch, channels, spatial, groups, ctypes.c_float(eps), silu, None)


def _workspace(lib, x, weight, bias, out, groups, eps, silu, ws):
    import torch
    batch, channels = x.shape[0], x.shape[1]
    spatial = x.numel() // (batch * channels)
    code = 2 if x.dtype == torch.bfloat16 else 0
    return lib.vrb_group_norm(P(x.data_ptr()), code, P(weight.data_ptr()), 0, P(bias.data_ptr()), 0, P(out.data_ptr()),
                              batch, channels, spatial, groups, ctypes.c_float(eps), silu, P(ws.data_ptr()), ws.numel(), None)


def _inputs(cases, seed=11):
    import torch
    gen = torch.Generator(device="cuda").manual_seed(seed)
    made = []
    for shape, groups, dtype, silu in cases:
        x = (torch.randn(shape, device="cuda", generator=gen) * 2 + 0.3).to(dtype)
        w = torch.randn(shape[1], device="cuda", generator=gen) * 0.1 + 1
        b = torch.randn(shape[1], device="cuda", generator=gen) * 0.1
        made.append((x, w, b, groups, silu))
    return made


def test_fixed_scratch_group_norm_matches_workspace_group_norm(orc):
    import torch
    from conftest import from_torch
    from vrhino_b200 import _lib
    assert torch.cuda.is_available()
    lib = _lib.load()
    # first call: large units (multi-slice statistics); second: many small units, other dtype;
    # third: bf16 + SiLU above the size from which the normalise pass reads SiLU from the function table
    cases = [((1, 32, 3, 120, 128), 4, torch.bfloat16, 1), ((3, 64, 24, 40), 32, torch.float32, 0),
             ((1, 128, 4, 96, 96), 32, torch.bfloat16, 1)]
    made = _inputs(cases)
    buffers = []
    for x, w, b, groups, silu in made:   # every torch buffer exists before the counted window
        need = lib.vrb_group_norm_workspace_bytes(x.shape[0], groups)
        buffers.append((torch.empty_like(x), torch.full_like(x, float("nan")), torch.empty(need, dtype=torch.uint8, device="cuda")))
    torch.cuda.synchronize()
    allocations = lib.vrb_device_allocation_count()
    for (x, w, b, groups, silu), (want, got, ws) in zip(made, buffers):
        assert _workspace(lib, x, w, b, want, groups, 1e-6, silu, ws) == 0, lib.vrb_last_error()
        assert _fixed(lib, x, w, b, got, groups, 1e-6, silu) == 0, lib.vrb_last_error()
    torch.cuda.synchronize()
    assert lib.vrb_device_allocation_count() == allocations, "an operator entry point allocated device memory"
    for want, got, _ in buffers:
        view = torch.int16 if got.dtype == torch.bfloat16 else torch.int32
        assert torch.equal(got.view(view), want.view(view)), "built-in scratch and workspace entry points disagree"
        if got.dtype == torch.bfloat16:   # the tolerance of tests/test_gpu_groupnorm.py, stated explicitly
            d = orc.bf16_ulp_distance(from_torch(got)[0], from_torch(want)[0])
            assert d.max() <= 2
        else:
            assert torch.allclose(got, want, rtol=1e-5, atol=2e-6)


def _first_call_probe():
    """Body of the fresh-process check (run as `python tests/test_zz_no_alloc.py`): the very first
    call into the library is vrb_group_norm_fixed_scratch on a bf16 + SiLU tensor of 4.7 Mi
    elements.  Prints the device's free bytes before and after and the library's allocation count."""
    import torch
    sys.path.insert(0, ROOT)
    from vrhino_b200 import _lib
    lib = _lib.load()
    (x, w, b, groups, silu), = _inputs([((1, 128, 4, 96, 96), 32, torch.bfloat16, 1)])
    got, want = torch.full_like(x, float("nan")), torch.empty_like(x)
    ws = torch.empty(lib.vrb_group_norm_workspace_bytes(1, groups), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    rc = _fixed(lib, x, w, b, got, groups, 1e-6, silu)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    again = _fixed(lib, x, w, b, got, groups, 1e-6, silu)       # second call: table already resident
    torch.cuda.synchronize()
    free_again, _ = torch.cuda.mem_get_info()
    count = lib.vrb_device_allocation_count()
    rc2 = _workspace(lib, x, w, b, want, groups, 1e-6, silu, ws)
    torch.cuda.synchronize()
    print(json.dumps({"rc": [rc, again, rc2], "error": lib.vrb_last_error().decode(), "free_before": free_before,
                      "free_after": free_after, "free_again": free_again, "allocations": count,
                      "equal": bool(torch.equal(got.view(torch.int16), want.view(torch.int16)))}))


def test_first_call_in_a_fresh_process_allocates_nothing():
    # CUDA loads a kernel's code on its first launch unless told to load everything up front; with
    # eager loading the only thing left that could move the free-memory reading is an allocation.
    env = dict(os.environ, CUDA_MODULE_LOADING="EAGER")
    proc = subprocess.run([sys.executable, os.path.abspath(__file__)], capture_output=True, text=True, env=env, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    seen = json.loads(proc.stdout.strip().splitlines()[-1])
    assert seen["rc"] == [0, 0, 0], seen["error"]
    assert seen["equal"], "first call (table not yet resident) and the workspace entry point disagree"
    assert seen["allocations"] == 0, "the library called cudaMalloc"
    assert seen["free_after"] == seen["free_before"], f"device free memory moved by {seen['free_before'] - seen['free_after']} bytes"
    assert seen["free_again"] == seen["free_before"]


def test_fixed_scratch_limit_is_enforced():
    import torch
    from vrhino_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(2048, 2, 8, device="cuda")     # 2048 * 1 = 2048 units > 1024
    out = torch.empty_like(x)
    rc = lib.vrb_group_norm_fixed_scratch(P(x.data_ptr()), 0, None, 0, None, 0, P(out.data_ptr()), 2048, 2, 8, 1,
                                          ctypes.c_float(1e-5), 0, None)
    assert rc == -4
    text = lib.vrb_last_error().decode()
    assert "2048" in text and "1024" in text and "vrb_group_norm" in text
    ok = lib.vrb_group_norm_fixed_scratch(P(x.data_ptr()), 0, None, 0, None, 0, P(out.data_ptr()), 1024, 4, 8, 1,
                                          ctypes.c_float(1e-5), 0, None)   # exactly at the limit
    assert ok == 0, lib.vrb_last_error()
    torch.cuda.synchronize()


if __name__ == "__main__":
    _first_call_probe()
