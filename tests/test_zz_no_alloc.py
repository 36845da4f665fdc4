"""GroupNorm through the entry point that carries its own scratch.

Who needs it: a caller that cannot give the library a device workspace -- every byte of its
device budget belongs to a planner-owned pool that must not grow while a step runs, or it sits on
a thread that may not enter cudaMalloc (the call synchronises the device).  The entry point
promises to allocate nothing and to behave exactly like vrb_group_norm, within a fixed limit on
batch x groups.

Checked here, through the C ABI only: the output equals the workspace-taking entry point's output
(same kernels, so bit for bit; the tolerance the other GroupNorm tests use is asserted too), on
two calls in a row with different shapes so that whatever the first call left in the shared
scratch is seen to be harmless; the limit is enforced with a clear error; device memory in use does
not change across the calls.  The file name sorts last on purpose: if it fails under `-x`, every
other test has already run.  It does not depend on them: it also passes in a fresh process.
"""
import ctypes

import pytest

pytestmark = pytest.mark.gpu

P = ctypes.c_void_p


def _run_both(lib, x, weight, bias, groups, eps, silu):
    import torch
    batch, channels = x.shape[0], x.shape[1]
    spatial = x.numel() // (batch * channels)
    code = 2 if x.dtype == torch.bfloat16 else 0
    want, got = torch.empty_like(x), torch.full_like(x, float("nan"))
    need = lib.vrb_group_norm_workspace_bytes(batch, groups)
    ws = torch.empty(need, dtype=torch.uint8, device=x.device)
    rc = lib.vrb_group_norm(P(x.data_ptr()), code, P(weight.data_ptr()), 0, P(bias.data_ptr()), 0, P(want.data_ptr()),
                            batch, channels, spatial, groups, ctypes.c_float(eps), silu, P(ws.data_ptr()), need, None)
    assert rc == 0, lib.vrb_last_error()
    rc = lib.vrb_group_norm_fixed_scratch(P(x.data_ptr()), code, P(weight.data_ptr()), 0, P(bias.data_ptr()), 0,
                                          P(got.data_ptr()), batch, channels, spatial, groups, ctypes.c_float(eps), silu, None)
    assert rc == 0, lib.vrb_last_error()
    torch.cuda.synchronize()
    return got, want


def test_fixed_scratch_group_norm_matches_workspace_group_norm(orc):
    import torch
    from conftest import from_torch
    from vrhino_b200 import _lib
    assert torch.cuda.is_available()
    lib = _lib.load()
    gen = torch.Generator(device="cuda").manual_seed(11)
    # first call: large units (multi-slice statistics); second: many small units, other dtype
    cases = [((1, 32, 3, 120, 128), 4, torch.bfloat16, 1), ((3, 64, 24, 40), 32, torch.float32, 0)]
    inputs = []
    for shape, groups, dtype, silu in cases:
        x = (torch.randn(shape, device="cuda", generator=gen) * 2 + 0.3).to(dtype)
        w = torch.randn(shape[1], device="cuda", generator=gen) * 0.1 + 1
        b = torch.randn(shape[1], device="cuda", generator=gen) * 0.1
        inputs.append((x, w, b, groups, silu))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    results = [_run_both(lib, x, w, b, groups, 1e-6, silu) for x, w, b, groups, silu in inputs]
    free_after, _ = torch.cuda.mem_get_info()
    for got, want in results:
        view = torch.int16 if got.dtype == torch.bfloat16 else torch.int32
        assert torch.equal(got.view(view), want.view(view)), "built-in scratch and workspace entry points disagree"
        if got.dtype == torch.bfloat16:   # the tolerance of tests/test_gpu_groupnorm.py, stated explicitly
            d = orc.bf16_ulp_distance(from_torch(got)[0], from_torch(want)[0])
            assert d.max() <= 2
        else:
            assert torch.allclose(got, want, rtol=1e-5, atol=2e-6)
    # the per-call workspaces of _run_both were torch's; the entry point itself took nothing
    assert free_before - free_after <= 64 << 20, "device memory shrank by more than torch's own test buffers"


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
