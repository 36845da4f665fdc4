"""Parity at the FULL sizes of the headline configurations, where the CPU oracle cannot evaluate
the whole tensor in seconds.  Two kinds of checks:

* sampled units against the oracle: token rows of the DiT chains and (batch, group) units of
  GroupNorm are independent of one another, so the oracle evaluates a few dozen sampled rows /
  two sampled groups of the very tensors the kernels processed;
* size-independent properties over EVERY element: a table-driven unary result must equal the
  65536-entry function table gathered at the input's bit pattern (the table itself is checked
  exhaustively elsewhere); SwiGLU must equal one bf16 multiply of the value half with the table
  value of the gate half; dequantisation must equal one F32 multiply of the decoded code with its
  row scale (numpy); the fused CFG+Euler update must equal the unfused oracle chain; repeated
  launches must be bit-identical.
"""
import numpy as np
import pytest

from conftest import assert_close, from_torch, to_torch

pytestmark = pytest.mark.gpu


def _bits(t):
    import torch
    return t.contiguous().view(torch.int16)


def _orc_rows(orc, t, rows):
    """Oracle tensor holding the sampled rows of a [1, S, D] torch tensor."""
    import torch
    sub = t[0, rows].contiguous().cpu()
    if sub.dtype == torch.bfloat16:
        return orc.T(sub.view(torch.int16).numpy().view(np.uint16).reshape(1, len(rows), -1), "bf16")
    return orc.T(sub.numpy().reshape(1, len(rows), -1), "f32")


def _cmp_rope(orc, got, want, what):
    """bf16 RoPE outputs: <= 2 ulp, except where the two products of the rotation cancel -- there the
    result inherits one bf16 ulp of the (much larger) rounded normalised operands; such elements
    must be rare (<= 0.2 %) and within 8 * 2^-8 absolutely (the bound test_golden.py uses)."""
    from conftest import record_parity
    data, tag = from_torch(got)
    assert tag == "bf16" and tuple(data.shape) == tuple(want.shape), what
    d = orc.bf16_ulp_distance(data, want.data)
    bad = d > 2
    record_parity(what, "bf16", d.size, d.max(), int(bad.sum()), int(bad.sum()),
                  "<= 0.2 % of the elements within 8 * 2^-8 absolute (RoPE cancellation after the bf16-rounded norm)" if bad.any() else "")
    if bad.any():
        diff = np.abs(orc.bf16_bits_to_f32(data).astype(np.float64) - want.f32().astype(np.float64))
        assert bad.mean() <= 2e-3 and (diff[bad] <= 2.0 ** -8 * 8.0).all(), (what, int(bad.sum()), int(d.max()))


def _cmp_rows(orc, got, rows, want, what, **kw):
    sub = got[0, rows].contiguous().reshape(want.shape)
    assert_close(orc, sub, want, what=what, **kw)


def _check_wan_chain(orc, gpu, blk, tag):
    """Runs the eleven launches of a Wan block and compares 48 sampled token rows per launch with the
    oracle's unfused chain (the reference's operator sequence)."""
    import torch
    be, ops = gpu
    S = blk.x.shape[1]
    for l in blk.launches():
        l.fn()
    torch.cuda.synchronize()
    rng = np.random.default_rng(0)
    rows = np.sort(np.concatenate([[0, 1, S - 1], rng.choice(S, 45, replace=False)]))
    rows_t = torch.from_numpy(rows).cuda()
    obe, pol = orc.OracleBackend(), orc.Policy.unqualified_default("bf16")
    f32 = lambda t: orc.T(t.detach().cpu().float().numpy(), "f32")
    x = _orc_rows(orc, blk.x, rows_t)
    mod = [f32(r) for r in blk.rows]
    eps = blk.eps

    def chain_ln_mod(shift, scale):
        return obe.cast(orc.modulate(obe, pol, obe.layer_norm(x, None, None, eps), shift, scale), "bf16")

    _cmp_rows(orc, blk.out["A"], rows_t, chain_ln_mod(mod[0], mod[1]), f"{tag} A ln_modulate")
    _cmp_rows(orc, blk.out["G"], rows_t, chain_ln_mod(mod[3], mod[4]), f"{tag} G ln_modulate")
    d = blk.cos.shape[-1]
    cos = orc.T(blk.cos.reshape(-1, d)[rows_t].cpu().numpy().reshape(1, len(rows), 1, d), "f32")
    sin = orc.T(blk.sin.reshape(-1, d)[rows_t].cpu().numpy().reshape(1, len(rows), 1, d), "f32")
    for name, src, w in (("Bq", blk.q, blk.wq), ("Bk", blk.k, blk.wk)):
        n = orc.attention_norm(obe, pol, _orc_rows(orc, src, rows_t), f32(w), eps, rows_for_schedule=S)
        r = orc.operation_rope(obe, pol, obe.reshape(n, (1, len(rows), blk.heads, d)), cos, sin)
        want = obe.cast(r, "bf16")
        got = blk.out[name][0, rows_t].reshape(1, len(rows), blk.heads, d)
        _cmp_rope(orc, got, want, f"{tag} {name} rms_rope")
    n = orc.attention_norm(obe, pol, _orc_rows(orc, blk.cross_q, rows_t), f32(blk.wcq), eps, rows_for_schedule=S)
    _cmp_rows(orc, blk.out["Eq"], rows_t, obe.cast(n, "bf16"), f"{tag} E rms cross q")
    want = obe.layer_norm(x, f32(blk.gamma3), f32(blk.beta3), eps)
    _cmp_rows(orc, blk.out["D"], rows_t, want, f"{tag} D ln_affine")
    for name, branch, gate in (("C", blk.proj, mod[2]), ("I", blk.ffn_out, mod[5])):
        want = orc.gated_residual(obe, pol, x, _orc_rows(orc, branch, rows_t), gate)
        got = blk.out[name][0, rows_t]
        assert torch.equal(_bits(got).cpu(), torch.from_numpy(want.data.view(np.int16).reshape(got.shape))), name
    want = orc.residual_add(obe, pol, x, _orc_rows(orc, blk.cross, rows_t))
    got = blk.out["F"][0, rows_t]
    assert torch.equal(_bits(got).cpu(), torch.from_numpy(want.data.view(np.int16).reshape(got.shape))), "F"
    # size-independent: a second pass over the whole tensors is bit-identical (no order-dependent sums)
    first = {k: v.clone() for k, v in blk.out.items() if k in ("A", "Bq", "D")}
    for l in blk.launches():
        if l.name.split()[0] in ("A", "B", "D"):
            l.fn()
    torch.cuda.synchronize()
    for k, v in first.items():
        assert torch.equal(_bits(v), _bits(blk.out[k])), f"{tag} {k}: repeated launch differs"


def test_wan21_chain_full_size_sampled_rows(orc, gpu):
    """Config 2: the eleven launches on 32760 tokens x 1536."""
    from vrhino_b200 import workloads
    _check_wan_chain(orc, gpu, workloads.WanBlock(gpu[0], tokens=32760, seed=11), "wan2.1")


def test_wan22_chain_full_size_sampled_rows(orc, gpu):
    """Config 3: the same chain at D = 5120 (40 heads x 128), FFN 13824, 32760 tokens on the real
    21 x 30 x 52 RoPE grid.  A 5120-wide row spans several warps, so this is the full-size exercise of
    the cross-warp reduction of the row kernels (layer_norm_parallel_kernel, native/src/backend/cuda/
    cuda_backend.cu:910-943, and rms_norm_contiguous_f32_kernel, :853-907, are what it replaces)."""
    import torch
    from vrhino_b200 import workloads
    blk = workloads.WanBlock(gpu[0], tokens=32760, dim=5120, heads=40, ffn=13824, seed=13)
    _check_wan_chain(orc, gpu, blk, "wan2.2")
    # GELU-tanh [32760, 13824]: every element equals the function table at the input's bit pattern
    be = gpu[0]
    codes = torch.arange(65536, dtype=torch.int32, device="cuda").to(torch.int16).view(torch.bfloat16)
    table = be.activation(codes, 2).view(torch.int16)
    x, out = blk.ffn_hidden[0], blk.out["H"][0]
    bad = 0
    for r0 in range(0, x.shape[0], 2048):
        sl = slice(r0, min(r0 + 2048, x.shape[0]))
        index = (x[sl].contiguous().view(torch.int16).to(torch.int32) & 0xFFFF).long()
        bad += int((table[index.reshape(-1)].reshape(index.shape) != out[sl].view(torch.int16)).sum())
    assert bad == 0


def test_wan21_merged_residual_norm_full_size(orc, gpu):
    """Config 2 with both CFG branches batched and each residual update merged into the LayerNorm that
    follows it (9 launches): over EVERY element the updated streams equal the separate residual
    kernels' and the normalised tensors equal the norm kernels run on those streams; 48 sampled rows
    of the merged launches against the oracle's unfused chain."""
    import torch
    from vrhino_b200 import workloads
    be, ops = gpu
    blk = workloads.WanBlock(be, tokens=32760, seed=12, batch=2)
    for l in blk.launches(fuse_residual_norm=True):
        l.fn()
    torch.cuda.synchronize()
    o, r, e = blk.out, blk.rows, blk.eps
    pol = blk.policy
    c = ops.fused_gated_residual(be, pol, blk.x, blk.proj, r[2])
    assert torch.equal(_bits(o["C"]), _bits(c)), "C stream"
    assert torch.equal(_bits(o["D"]), _bits(be.layer_norm(c, blk.gamma3, blk.beta3, e))), "D on the updated stream"
    f = ops.fused_gated_residual(be, pol, blk.x, blk.cross, None)
    assert torch.equal(_bits(o["F"]), _bits(f)), "F stream"
    assert torch.equal(_bits(o["G"]), _bits(ops.fused_layer_norm_modulate(be, f, None, None, e, r[3], r[4]))), "G on the updated stream"
    del c, f
    rng = np.random.default_rng(1)
    rows = np.sort(np.concatenate([[0, 32759], rng.choice(32760, 22, replace=False)]))
    rows_t = torch.from_numpy(rows).cuda()
    obe, opol = orc.OracleBackend(), orc.Policy.unqualified_default("bf16")
    f32 = lambda t: orc.T(t.detach().cpu().float().numpy(), "f32")
    for b in range(2):
        x = _orc_rows(orc, blk.x[b:b + 1], rows_t)
        state = orc.gated_residual(obe, opol, x, _orc_rows(orc, blk.proj[b:b + 1], rows_t), f32(r[2][b:b + 1]))
        got = o["C"][b, rows_t]
        assert torch.equal(_bits(got).cpu(), torch.from_numpy(state.data.view(np.int16).reshape(got.shape))), "C"
        _cmp_rows(orc, o["D"][b:b + 1], rows_t, obe.layer_norm(state, f32(blk.gamma3), f32(blk.beta3), e), "C+D normalised")
        state = orc.residual_add(obe, opol, x, _orc_rows(orc, blk.cross[b:b + 1], rows_t))
        got = o["F"][b, rows_t]
        assert torch.equal(_bits(got).cpu(), torch.from_numpy(state.data.view(np.int16).reshape(got.shape))), "F"
        want = obe.cast(orc.modulate(obe, opol, obe.layer_norm(state, None, None, e), f32(r[3][b:b + 1]), f32(r[4][b:b + 1])), "bf16")
        _cmp_rows(orc, o["G"][b:b + 1], rows_t, want, "F+G normalised")


@pytest.mark.parametrize("kind", [2, 0])
def test_table_unary_full_size_every_element(gpu, kind):
    """[32760, 8960] bf16 (GELU-tanh of config 2; SiLU for the VAE): out == table[in] everywhere,
    the table being the direct kernel's result on all 65536 codes; and a second launch is
    bit-identical."""
    import torch
    be, ops = gpu
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((32760, 8960), device="cuda", generator=g).to(torch.bfloat16)
    codes = torch.arange(65536, dtype=torch.int32, device="cuda").to(torch.int16).view(torch.bfloat16)
    table = be.activation(codes, kind).view(torch.int16)          # 65536 elements: direct kernel
    out = be.activation(x, kind)
    index = x.view(torch.int16).to(torch.int32) & 0xFFFF
    bad = 0
    for r0 in range(0, 32760, 4096):                              # gather in slabs to bound scratch memory
        sl = slice(r0, min(r0 + 4096, 32760))
        bad += int((table[index[sl].reshape(-1).long()].reshape(index[sl].shape) != out[sl].view(torch.int16)).sum())
    assert bad == 0
    again = be.activation(x, kind)
    assert torch.equal(out.view(torch.int16), again.view(torch.int16))


def test_swiglu_full_size_every_element(gpu):
    """Config 4: proj [1, 44520, 16384] -> [1, 44520, 8192]; value half times SiLU table of the gate
    half, one bf16 multiply (= the reference's F32 multiply followed by the bf16 store)."""
    import torch
    be, ops = gpu
    g = torch.Generator(device="cuda").manual_seed(4)
    proj = torch.randn((1, 44520, 16384), device="cuda", generator=g).to(torch.bfloat16)
    codes = torch.arange(65536, dtype=torch.int32, device="cuda").to(torch.int16).view(torch.bfloat16)
    silu = be.activation(codes, 0)
    out = ops.fused_swiglu(be, proj)
    bad = 0
    for r0 in range(0, 44520, 4096):
        sl = slice(r0, min(r0 + 4096, 44520))
        a, gate = proj[0, sl, :8192], proj[0, sl, 8192:]
        s = silu[(gate.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF).long()]
        want = (a.float() * s.float()).to(torch.bfloat16)
        bad += int((want.view(torch.int16) != out[0, sl].view(torch.int16)).sum())
    assert bad == 0


def test_mochi_rows_full_size_sampled(orc, gpu):
    """Config 4 row launches on 44520 tokens x 3072: sampled rows against the oracle."""
    import torch
    from vrhino_b200 import workloads
    be, ops = gpu
    blk = workloads.MochiBlock(be, tokens=44520, hidden=64, seed=5)      # SwiGLU is covered above
    launches = {l.name: l for l in blk.launches()}
    for name in ("rms_scale", "head rms_rope q", "rms_gated_residual"):
        launches[name].fn()
    torch.cuda.synchronize()
    rng = np.random.default_rng(1)
    rows = np.sort(np.concatenate([[0, 44519], rng.choice(44520, 30, replace=False)]))
    rows_t = torch.from_numpy(rows).cuda()
    obe, pol = orc.OracleBackend(), orc.Policy.unqualified_default("bf16")
    f32 = lambda t: orc.T(t.detach().cpu().float().numpy(), "f32")
    want = orc.mochi_norm_scale(obe, _orc_rows(orc, blk.h, rows_t), f32(blk.scale.reshape(1, -1)))
    _cmp_rows(orc, blk.out["pre"], rows_t, want, "rms_scale")
    H, d = blk.heads, blk.cos.shape[-1]
    q = obe.reshape(_orc_rows(orc, blk.q, rows_t), (1, len(rows), H, d))
    n = orc.attention_norm(obe, pol, q, f32(blk.wq), 1e-5, rows_for_schedule=44520 * H)
    cos = orc.T(blk.cos[0, rows_t].cpu().numpy().reshape(1, len(rows), H, d), "f32")
    sin = orc.T(blk.sin[0, rows_t].cpu().numpy().reshape(1, len(rows), H, d), "f32")
    want = obe.cast(orc.operation_rope(obe, pol, n, cos, sin), "bf16")
    got = blk.out["q"][0, rows_t].reshape(1, len(rows), H, d)
    _cmp_rope(orc, got, want, "head rms_rope q")
    want = orc.gated_residual(obe, pol, _orc_rows(orc, blk.x, rows_t),
                              obe.rms_norm(_orc_rows(orc, blk.branch, rows_t), None, 1e-6), f32(blk.gate))
    _cmp_rows(orc, blk.out["res"], rows_t, want, "rms_gated_residual")


def test_fp8_dequant_full_size_every_element(orc, gpu):
    """Config 3: 5120 x 13824 codes, per-channel scales: every output equals bf16(decode(code) * scale)."""
    import torch
    be, ops = gpu
    g = torch.Generator(device="cuda").manual_seed(6)
    codes = torch.randint(0, 256, (5120, 13824), device="cuda", dtype=torch.int16, generator=g).to(torch.uint8)
    scales = (torch.rand((5120, 1), device="cuda", generator=g) * 9e-3 + 1e-3).float()
    decoded = torch.tensor([orc.lib().orc_decode_fp8(int(c)) for c in range(256)], dtype=torch.float32, device="cuda")
    for dtype in (torch.bfloat16, torch.float32):
        out = be.dequantize(codes, scales, 13824, dtype=dtype)
        want = (decoded[codes.long()] * scales).to(dtype)         # one F32 multiply, one rounding
        view = torch.int16 if dtype == torch.bfloat16 else torch.int32
        assert torch.equal(out.view(view), want.view(view)), dtype


def test_cfg_euler_full_size(orc, gpu):
    """Config 3: F32 latent [1,16,21,60,104], guidance 5.0, dt -0.02: fused kernel == the oracle's
    unfused cfg_combine + euler_update chain, bit for bit."""
    import torch
    from vrhino_b200 import synth
    be, ops = gpu
    shape = (1, 16, 21, 60, 104)
    x, u, c = (orc.tensor(synth.normal(shape, seed=s)) for s in (1, 2, 3))
    obe = orc.OracleBackend(execution_dtype="f32")
    pol = orc.Policy.fp32()
    guided = orc.cfg_combine(obe, pol, u, c, 5.0)
    want = orc.euler_update(obe, pol, x, guided, orc.scalar_f32(0.02), True)
    be32 = ops.B200Backend(execution_dtype=torch.float32)
    got = ops.fused_cfg_euler(be32, ops.Policy.fp32(), to_torch(x), to_torch(u), to_torch(c), 5.0, 0.02, True)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.data.view(np.uint32))


def test_group_norm_full_size_two_groups_against_oracle(orc, gpu):
    """Config 5: [1, 256, 28, 240, 424] bf16, 32 groups.  Units are independent, so the oracle
    evaluates groups 0 and 31 (2 x 22.8 M elements) of the tensor the kernel normalised.

    The 2-ulp bound is checked where it is meaningful, on the GroupNorm output y: SiLU at very
    negative y behaves like y * exp(y), so ONE bf16 ulp of y (which any two correct
    implementations of the statistics may differ by) moves silu(y) by many ulps.  The fused
    operator is therefore checked as: y within 2 ulp of the oracle, and fused output ==
    silu_table[y] for EVERY element (y = this library's unfused GroupNorm output), plus a
    bit-identical repeat of the whole 1.46 GB operator."""
    import torch
    be, ops = gpu
    g = torch.Generator(device="cuda").manual_seed(7)
    shape = (1, 256, 28, 240, 424)
    x = (torch.randn(shape, device="cuda", generator=g) * 2.0).to(torch.bfloat16)
    gamma = (torch.randn(256, device="cuda", generator=g) * 0.1 + 1.0).float()
    beta = (torch.randn(256, device="cuda", generator=g) * 0.1).float()
    out = ops.fused_group_norm_silu(be, x, 32, gamma, beta, 1e-6)
    again = ops.fused_group_norm_silu(be, x, 32, gamma, beta, 1e-6)
    assert torch.equal(out.view(torch.int16), again.view(torch.int16))
    del again
    y = be.group_norm(x, 32, gamma, beta, 1e-6)
    codes = torch.arange(65536, dtype=torch.int32, device="cuda").to(torch.int16).view(torch.bfloat16)
    silu = be.activation(codes, 0).view(torch.int16)
    yv, ov = y.view(torch.int16).reshape(256, -1), out.view(torch.int16).reshape(256, -1)
    bad = 0
    for c in range(0, 256, 8):
        index = (yv[c:c + 8].to(torch.int32) & 0xFFFF).long()
        bad += int((silu[index] != ov[c:c + 8]).sum())
    assert bad == 0
    obe = orc.OracleBackend()
    for group in (0, 31):
        ch = slice(group * 8, group * 8 + 8)
        xs = x[:, ch].contiguous().cpu()
        xo = orc.T(xs.view(torch.int16).numpy().view(np.uint16), "bf16")
        w = orc.T(gamma[ch].cpu().numpy(), "f32")
        b = orc.T(beta[ch].cpu().numpy(), "f32")
        want = obe.group_norm(xo, 1, w, b, 1e-6)
        got, _ = from_torch(y[:, ch])
        d = orc.bf16_ulp_distance(got.reshape(-1), want.data.reshape(-1))
        # outputs next to zero come from (x - mean) * inv * gamma cancelling against beta: absolute 2e-6
        # there (the bound the small GroupNorm tests use), 2 bf16 ulp everywhere else
        diff = np.abs(orc.bf16_bits_to_f32(got.reshape(-1)).astype(np.float64) - want.f32().reshape(-1).astype(np.float64))
        bad = (d > 2) & (diff > 2e-6)
        assert not bad.any(), (group, int(bad.sum()), int(d[bad].max()))
        assert (d == 0).mean() > 0.99
