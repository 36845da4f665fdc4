"""The host-buffer entry points give bit-identical results to the device entry points (they run
the same kernels on row blocks), for pinned and for pageable host memory."""
import ctypes

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("pinned,batch", [(True, 1), (False, 1), (True, 2)])
def test_host_chain_matches_device_chain(gpu, pinned, batch):
    import torch
    be, ops = gpu
    from vrhino_b200 import _lib, workloads
    # 3000 rows x 1536 bf16 = 9 MB per tensor: two row blocks, the second one partial; batch 2 = both
    # CFG branches with their own modulation vectors, run branch by branch on the host side
    blk = workloads.WanBlock(be, tokens=3000, grid=(1, 30, 100), ffn=1024, text_tokens=40, seed=3, batch=batch)
    for l in blk.launches():
        l.fn()
    torch.cuda.synchronize()
    host = workloads.WanBlockHost(blk)
    if not pinned:
        for name in ("x", "q", "k", "proj", "cross_q", "cross_k", "cross", "ffn_out", "ffn_hidden", "cos", "sin"):
            setattr(host, name, getattr(host, name).clone())       # pageable copies
        host.out = {k: torch.empty_like(v) for k, v in host.out.items()}
    host.step()
    host.step()   # second call reuses the staging buffers
    for key, want in blk.out.items():
        got = host.out[key]
        assert got.dtype == want.dtype and got.shape == want.shape, key
        view = torch.int16 if want.dtype == torch.bfloat16 else torch.int32
        assert torch.equal(got.view(view), want.cpu().view(view)), f"{key}: host pipeline != device launch"
    _lib.load().vrb_host_release()
    host.step()   # works again after release
    assert torch.equal(host.out["A"].view(torch.int16), blk.out["A"].cpu().view(torch.int16))
    _lib.load().vrb_host_release()


def test_host_entry_rejects_bad_arguments(gpu):
    from vrhino_b200 import _lib
    lib = _lib.load()
    assert lib.vrb_host_activation(2, None, None, 2, 4, 8) == -1
    assert b"null tensor" in lib.vrb_last_error()
    buf = (ctypes.c_uint16 * 64)()
    assert lib.vrb_host_activation(2, buf, buf, 2, 0, 8) == -1
    assert lib.vrb_host_activation(2, buf, buf, 5, 8, 8) == -2
