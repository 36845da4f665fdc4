"""The benchmark workloads: the non-GEMM operator chains of one DiT block / sampler step / VAE
norm at the sizes the headline configurations name, expressed as lists of fused launches with
their algorithmic HBM bytes.

Algorithmic bytes of one launch = every distinct input tensor read once + every output
written once, at storage dtype; broadcast vectors counted once.  GroupNorm, whose reduction
unit is far larger than on-chip memory, counts its input twice (statistics pass + apply pass).

Inputs are synthetic: activations ~N(0,1) (seeded on the device), modulation vectors
~N(0,0.1), norm weights ~N(1,0.1); the "GEMM outputs" the chain consumes are synthesised too,
since GEMMs and attention are not part of this path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List

import torch

from . import ops, synth

BF16, F32 = torch.bfloat16, torch.float32


@dataclass
class Launch:
    name: str
    fn: Callable[[], object]
    bytes: int
    kernels: int = 1


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


def _randn(shape, dtype, gen, mean=0.0, std=1.0):
    return (torch.randn(shape, device="cuda", dtype=torch.float32, generator=gen) * std + mean).to(dtype)


class WanBlock:
    """Wan2.1-1.3B style DiT block, one CFG branch: B=1, S tokens, D = heads*head_dim, FFN F.

    Chain (native/src/architectures/wan_self_attention_graph.h:46-70 and wan.cpp:68-119 of the
    reference): A LN->modulate->bf16; B rms(q),rms(k)->RoPE->bf16; C x + proj*gate;
    D LN(gamma,beta); E rms(cross q), rms(cross k on the text rows); F x + cross;
    G LN->modulate->bf16 (rows 3,4); H GELU-tanh on [S,F]; I x + ffn*gate.
    """

    def __init__(self, be, tokens=32760, dim=1536, heads=12, ffn=8960, grid=(21, 30, 52), text_tokens=512,
                 hidden_dtype=BF16, seed=0, batch=1):
        """batch > 1: the CFG branches as one batched tensor [batch, S, D] with one modulation
        vector set per batch entry (the RoPE tables are shared by the batch)."""
        assert grid[0] * grid[1] * grid[2] == tokens
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.be, S, D, B = be, tokens, dim, batch
        self.policy = ops.Policy(BF16, hidden_dtype)
        hd = hidden_dtype
        self.x = _randn((B, S, D), hd, g)
        self.mod = _randn((B, 6, D), F32, g, std=0.1)                 # combined modulation rows
        self.rows = [self.mod[:, i:i + 1, :].contiguous() for i in range(6)]
        self.q, self.k, self.proj, self.cross_q, self.cross, self.ffn_out = (_randn((B, S, D), BF16, g) for _ in range(6))
        self.cross_k = _randn((B, text_tokens, D), BF16, g)
        self.ffn_hidden = _randn((B, S, ffn), BF16, g)
        self.wq, self.wk, self.wcq, self.wck, self.gamma3 = (_randn((D,), F32, g, 1.0, 0.1) for _ in range(5))
        self.beta3 = _randn((D,), F32, g, 0.0, 0.1)
        cos, sin = synth.wan_rope_tables(*grid, head_dim=dim // heads)
        self.cos, self.sin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
        self.heads, self.eps = heads, 1e-6
        self.out = {}

    # DRAM bytes (read + write) per element the table-driven GELU-tanh kernel moves, from an ncu
    # capture of one [32760, 8960] bf16 launch (1 124.7 MB for 293.5 M elements: the 4 algorithmic
    # bytes minus the part of the output still dirty in L2 when the kernel ends); the kernel streams,
    # so its traffic grows in proportion to the element count.
    GELU_DRAM_BYTES_PER_ELEMENT = 1_124_700_000 / (32760 * 8960)

    def token_shard(self, rank: int, world: int) -> "WanBlock":
        """The same block restricted to rank `rank`'s contiguous token rows [r*S/world, (r+1)*S/world)
        of every per-token tensor (and its rows of the RoPE tables and of the text tokens); vectors
        shared by all rows are shared with the parent.  The operators are row-independent, so the
        shard's outputs are the parent's outputs on those rows, bit for bit."""
        S, T = self.x.shape[1], self.cross_k.shape[1]
        r0, r1 = rank * S // world, (rank + 1) * S // world
        t0, t1 = rank * T // world, (rank + 1) * T // world
        blk = object.__new__(WanBlock)
        blk.__dict__.update(self.__dict__)
        for name in ("x", "q", "k", "proj", "cross_q", "cross", "ffn_out", "ffn_hidden"):
            setattr(blk, name, getattr(self, name)[:, r0:r1].contiguous())
        blk.cross_k = self.cross_k[:, t0:t1].contiguous()
        d = self.cos.shape[-1]
        blk.cos = self.cos.reshape(S, d)[r0:r1].reshape(1, r1 - r0, 1, d).contiguous()
        blk.sin = self.sin.reshape(S, d)[r0:r1].reshape(1, r1 - r0, 1, d).contiguous()
        blk.out = {}
        blk.token_rows, blk.text_rows = (r0, r1), (t0, t1)
        return blk

    def launches(self, fuse_residual_norm: bool = False, pair_qk: bool = False) -> List[Launch]:
        """pair_qk: the q and k projections normalised and rotated by ONE launch (they are independent
        and share the RoPE tables, which then cross HBM once), likewise the cross-attention q and k: two
        launches fewer, bit-identical outputs.
        fuse_residual_norm: C+D and F+G each as ONE launch (residual update + the LayerNorm that
        reads the updated stream, wan.cpp:95-107 of the reference) -- 9 launches instead of 11.  Such a
        launch reads residual and branch and writes stream and normalised output: 4 passes where
        the two launches it replaces make 5."""
        be, p, r, e, o = self.be, self.policy, self.rows, self.eps, self.out
        B, S, D = self.x.shape
        act = B * S * D
        hb = self.x.element_size()
        vec = B * D * 4

        def A(): o["A"] = ops.fused_layer_norm_modulate(be, self.x, None, None, e, r[0], r[1], out=o.get("A"))
        def Bq(): o["Bq"] = ops.fused_rms_norm_rope(be, self.q, self.wq, e, self.cos, self.sin, heads=self.heads, out=o.get("Bq"))
        def Bk(): o["Bk"] = ops.fused_rms_norm_rope(be, self.k, self.wk, e, self.cos, self.sin, heads=self.heads, out=o.get("Bk"))
        def C(): o["C"] = ops.fused_gated_residual(be, p, self.x, self.proj, r[2], out=o.get("C"))
        def Dn(): o["D"] = be.layer_norm(self.x, self.gamma3, self.beta3, e, out=o.get("D")) if self.x.dtype == BF16 else \
            ops.fused_layer_norm_cast(be, self.x, self.gamma3, self.beta3, e, out=o.get("D"))
        def Eq(): o["Eq"] = ops.fused_rms_norm_rope(be, self.cross_q, self.wcq, e, None, None, heads=self.heads, out=o.get("Eq"))
        def Ek(): o["Ek"] = ops.fused_rms_norm_rope(be, self.cross_k, self.wck, e, None, None, heads=self.heads, out=o.get("Ek"))
        def Fr(): o["F"] = ops.fused_gated_residual(be, p, self.x, self.cross, None, out=o.get("F"))
        def G(): o["G"] = ops.fused_layer_norm_modulate(be, self.x, None, None, e, r[3], r[4], out=o.get("G"))
        def H(): o["H"] = be.activation(self.ffn_hidden, ops.GELU_TANH, out=o.get("H"))
        def I(): o["I"] = ops.fused_gated_residual(be, p, self.x, self.ffn_out, r[5], out=o.get("I"))

        def Bqk(): o["Bq"], o["Bk"] = ops.fused_rms_norm_rope_pair(be, self.q, self.wq, self.k, self.wk, e, self.cos, self.sin,
                                                                   heads=self.heads, out=(o.get("Bq"), o.get("Bk")))
        def Eqk(): o["Eq"], o["Ek"] = ops.fused_rms_norm_rope_pair(be, self.cross_q, self.wcq, self.cross_k, self.wck, e, None, None,
                                                                   heads=self.heads, out=(o.get("Eq"), o.get("Ek")))

        def CD(): o["C"], o["D"] = ops.fused_gated_residual_layer_norm(be, p, self.x, self.proj, r[2], self.gamma3, self.beta3, e,
                                                                       state_out=o.get("C"), out=o.get("D"))
        def FG(): o["F"], o["G"] = ops.fused_gated_residual_layer_norm(be, p, self.x, self.cross, None, None, None, e, r[3], r[4],
                                                                       state_out=o.get("F"), out=o.get("G"))

        table = self.cos.numel() * 4 * 2
        # q / k norm + RoPE and the cross-attention norms: two launches each, or one pair launch that reads
        # the RoPE tables once
        if pair_qk:
            b_launches = [Launch("B rms_rope q+k", Bqk, 2 * (act * 4 + vec) + table // 2)]
            e_launches = [Launch("E rms cross q+k", Eqk, act * 4 + self.cross_k.numel() * 4 + 2 * vec)]
        else:
            b_launches = [Launch("B rms_rope q", Bq, act * 4 + vec + table // 2), Launch("B rms_rope k", Bk, act * 4 + vec + table // 2)]
            e_launches = [Launch("E rms cross q", Eq, act * 4 + vec), Launch("E rms cross k", Ek, self.cross_k.numel() * 4 + vec)]
        if fuse_residual_norm:
            return [Launch("A ln_modulate", A, act * (hb + 2) + 2 * vec)] + b_launches + [
                Launch("C+D gated_residual ln_affine", CD, act * (hb + 2 + hb + 2) + 3 * vec)] + e_launches + [
                Launch("F+G residual_add ln_modulate", FG, act * (hb + 2 + hb + 2) + 2 * vec),
                Launch("H gelu_tanh", H, self.ffn_hidden.numel() * 4),
                Launch("I gated_residual", I, act * (hb + 2 + hb) + vec),
            ]
        return [Launch("A ln_modulate", A, act * (hb + 2) + 2 * vec)] + b_launches + [
            Launch("C gated_residual", C, act * (hb + 2 + hb) + vec),
            Launch("D ln_affine", Dn, act * (hb + 2) + 2 * vec)] + e_launches + [
            Launch("F residual_add", Fr, act * (hb + 2 + hb)),
            Launch("G ln_modulate", G, act * (hb + 2) + 2 * vec),
            Launch("H gelu_tanh", H, self.ffn_hidden.numel() * 4),
            Launch("I gated_residual", I, act * (hb + 2 + hb) + vec),
        ]


def compile_launches(launches: List[Launch]) -> List[Launch]:
    """The same launches with the Python above the C ABI taken out of the loop: every launch is run
    once while the C-ABI calls it makes are recorded (entry point + argument objects, the current
    stream included), and the returned launches replay exactly those calls.  Outputs must already
    exist (run every launch once before), so that the recorded pointers stay valid; the tensors are
    kept alive by the original launches' closures.  Replay on the stream that was current here."""
    from . import _lib
    lib = _lib.load()
    compiled = []
    for l in launches:
        calls = []
        original = ops.call

        def recording(name, *args, _calls=calls):
            _calls.append((getattr(lib, name), args, name))
            original(name, *args)

        ops.call = recording
        try:
            l.fn()
        finally:
            ops.call = original

        def replay(_calls=calls, _keep=l.fn):
            for fn, args, name in _calls:
                if fn(*args) != 0:
                    _lib.check(-1)

        compiled.append(Launch(l.name, replay, l.bytes, l.kernels))
    return compiled


def time_launches(launches: List[Launch], steps: int, warmup: int):
    """Device times with CUDA events on the current stream, the C-ABI calls recorded once and replayed
    so that no Python sits between two launches: the whole list back to back (`steps` repetitions,
    one event pair), and every launch on its own, `steps` repetitions back to back -- a launch of a few
    microseconds bracketed by its own event pair through the Python layer would mostly measure the
    host.  Returns (list_ms_per_step, {name: ms_per_launch})."""
    for l in launches:
        l.fn()
    torch.cuda.synchronize()
    compiled = compile_launches(launches)

    def timed(fns, reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            for fn in fns:
                fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    every = [l.fn for l in compiled]
    for _ in range(max(warmup, 1)):
        for fn in every:
            fn()
    torch.cuda.synchronize()
    total = timed(every, steps)
    per = {}
    for l in compiled:
        l.fn()
        per[l.name] = timed([l.fn], steps)
    return total, per


class Wan22Step:
    """Wan2.2-A14B step pieces: the D=5120 / FFN=13824 block chain, the FP8-e4m3 weight dequant
    [5120, 13824] with per-output-channel F32 scales (copy_to_device's quantised branch,
    native/src/backend/cuda/cuda_backend.cu:3214-3296), and cfg_combine + euler_update on the
    F32 latent [1,16,21,60,104] (native/src/sampling.cpp:181-193)."""

    def __init__(self, be, tokens=32760, seed=0, with_block=True):
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.be = be
        self.block = WanBlock(be, tokens=tokens, dim=5120, heads=40, ffn=13824, grid=(1, 1, tokens), seed=seed) if with_block else None
        rows, cols = 5120, 13824
        codes = torch.randint(0, 254, (rows, cols), device="cuda", dtype=torch.int16, generator=g)
        self.packed = (codes + (codes >= 127).to(torch.int16)).to(torch.uint8)   # the 254 finite codes: no 0x7f, 0xff
        self.scales = (torch.rand((rows, 1), device="cuda", generator=g) * 9e-3 + 1e-3).float()
        self.latent, self.uncond, self.cond = (_randn((1, 16, 21, 60, 104), F32, g) for _ in range(3))
        self.policy = ops.Policy.fp32()
        self.out = {}

    def launches(self, pair_qk: bool = False) -> List[Launch]:
        """pair_qk: as in WanBlock.launches (q and k, and the cross-attention q and text k, as one launch each)."""
        be, o = self.be, self.out
        n = self.latent.numel()

        def dq(): o["dequant"] = be.dequantize(self.packed, self.scales, self.packed.shape[1], out=o.get("dequant"))
        def cfg(): o["cfg"] = ops.fused_cfg_combine(be, self.policy, self.uncond, self.cond, 5.0, out=o.get("cfg"))
        def euler(): o["euler"] = ops.fused_euler_update(be, self.policy, self.latent, self.uncond, 0.02, True, out=o.get("euler"))
        def both(): o["cfg_euler"] = ops.fused_cfg_euler(be, self.policy, self.latent, self.uncond, self.cond, 5.0, 0.02, True, out=o.get("cfg_euler"))

        extra = [
            Launch("fp8 dequant", dq, self.packed.numel() * 3 + self.scales.numel() * 4),
            Launch("cfg_combine", cfg, n * 12),
            Launch("euler_update", euler, n * 12),
            Launch("cfg+euler fused", both, n * 16),
        ]
        return (self.block.launches(pair_qk=pair_qk) if self.block is not None else []) + extra


class MochiBlock:
    """Mochi-style visual stream, per rank: S tokens of dim 3072, 24 heads x 128, SwiGLU hidden
    8192 (native/src/architectures/mochi.cpp:182-231): RMS(no weight) -> *(1+scale) -> bf16;
    per-head RMS(w, 1e-5) -> RoPE with per-head tables -> bf16 for q and k; SwiGLU;
    residual + RMS(branch) * tanh-bounded gate."""

    def __init__(self, be, tokens=44520, dim=3072, heads=24, hidden=8192, seed=0, hidden_dtype=BF16):
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.be, S, D = be, tokens, dim
        self.heads = heads
        self.policy = ops.Policy(BF16, hidden_dtype)
        self.x = _randn((1, S, D), hidden_dtype, g)
        self.h, self.q, self.k, self.branch = (_randn((1, S, D), BF16, g) for _ in range(4))
        self.scale = _randn((1, 1, D), F32, g, std=0.1)
        self.raw_gate = _randn((1, 1, D), F32, g, std=0.1)
        self.gate = torch.tanh(self.raw_gate)
        self.wq, self.wk = (_randn((D // heads,), F32, g, 1.0, 0.1) for _ in range(2))
        phase = torch.rand((1, S, heads, D // heads), device="cuda", generator=g) * 6.2831853
        self.cos, self.sin = torch.cos(phase), torch.sin(phase)
        del phase
        self.proj = _randn((1, S, 2 * hidden), BF16, g)
        self.out = {}

    def launches(self, merge_tail: bool = False) -> List[Launch]:
        """merge_tail: the residual update and the pre-norm of the layer that follows it (mochi.cpp:204-211,
        :228-231) as ONE launch with the tanh of the gate folded in, q and k as one pair launch."""
        be, p, o = self.be, self.policy, self.out
        act = self.h.numel()
        hb = self.x.element_size()
        vec = self.scale.numel() * 4
        table = self.cos.numel() * 4 * 2
        if merge_tail:
            def qk(): o["q"], o["k"] = ops.fused_rms_norm_rope_pair(be, self.q, self.wq, self.k, self.wk, 1e-5, self.cos, self.sin,
                                                                    heads=self.heads, per_head_norm=True, out=(o.get("q"), o.get("k")))
            def sw2(): o["swiglu"] = ops.fused_swiglu(be, self.proj, out=o.get("swiglu"))
            def tail(): o["res"], o["pre_next"] = ops.fused_rms_norm_gated_residual_norm_scale(
                be, p, self.x, self.branch, self.raw_gate, self.scale, state_out=o.get("res"), out=o.get("pre_next"))
            return [
                Launch("head rms_rope q+k", qk, 2 * (act * 4 + 512) + table),
                Launch("swiglu", sw2, self.proj.numel() * 2 + self.proj.numel()),
                Launch("rms_gated_residual + next rms_scale", tail, act * (2 + 3 * hb) + 2 * vec),
            ]

        def pre(): o["pre"] = ops.fused_rms_norm_scale(be, self.h, self.scale, 1e-6, out=o.get("pre"))
        def q(): o["q"] = ops.fused_rms_norm_rope(be, self.q, self.wq, 1e-5, self.cos, self.sin, heads=self.heads, per_head_norm=True, out=o.get("q"))
        def k(): o["k"] = ops.fused_rms_norm_rope(be, self.k, self.wk, 1e-5, self.cos, self.sin, heads=self.heads, per_head_norm=True, out=o.get("k"))
        def sw(): o["swiglu"] = ops.fused_swiglu(be, self.proj, out=o.get("swiglu"))
        def res(): o["res"] = ops.fused_rms_norm_gated_residual(be, p, self.x, self.branch, self.gate, 1e-6, out=o.get("res"))

        return [
            Launch("rms_scale", pre, act * 4 + vec),
            Launch("head rms_rope q", q, act * 4 + table + 512),
            Launch("head rms_rope k", k, act * 4 + table + 512),
            Launch("swiglu", sw, self.proj.numel() * 2 + self.proj.numel()),
            Launch("rms_gated_residual", res, act * (2 + 2 * hb) + vec),
        ]


class LtxBlock:
    """LTX-Video transformer block, both CFG branches as the batch the reference evaluates them in
    (native/src/architectures/ltx.cpp:100-151, ltx_self_attention_graph.cpp:30-44): B=2, S tokens of
    dim 2048, 32 heads x 64, FFN 8192, 128 text tokens.  A rms_norm(no weight, 1e-6) -> modulate -> bf16;
    B q, k: rms_norm(w, 1e-5) over 2048 -> RoPE with per-batch tables [B, S, 2048] (the fractional
    positions make them as large as q in F32) -> bf16; C x + proj * gate; E rms_norm(w) of the
    cross-attention q and of the text k; F x + cross; G rms_norm -> modulate; H GELU-tanh on [B, S, 8192];
    I x + ffn * gate.  per_token: modulation vectors [B, S, 2048] (one set per token) instead of [B, 1, 2048]."""

    def __init__(self, be, tokens=6144, dim=2048, heads=32, ffn=8192, text_tokens=128, batch=2, hidden_dtype=BF16,
                 per_token=False, seed=0):
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.be, S, D, B = be, tokens, dim, batch
        self.policy = ops.Policy(BF16, hidden_dtype)
        self.x = _randn((B, S, D), hidden_dtype, g)
        m = S if per_token else 1
        self.rows = [_randn((B, m, D), F32, g, std=0.1) for _ in range(6)]
        self.q, self.k, self.proj, self.cross_q, self.cross, self.ffn_out = (_randn((B, S, D), BF16, g) for _ in range(6))
        self.cross_k = _randn((B, text_tokens, D), BF16, g)
        self.ffn_hidden = _randn((B, S, ffn), BF16, g)
        self.wq, self.wk, self.wcq, self.wck = (_randn((D,), F32, g, 1.0, 0.1) for _ in range(4))
        phase = torch.rand((B, S, heads, D // heads), device="cuda", generator=g) * 6.2831853
        self.cos, self.sin = torch.cos(phase), torch.sin(phase)
        del phase
        self.heads = heads
        self.out = {}

    def launches(self) -> List[Launch]:
        be, p, r, o = self.be, self.policy, self.rows, self.out
        act = self.x.numel()
        hb = self.x.element_size()
        vec = r[0].numel() * 4
        table = self.cos.numel() * 4 * 2

        def A(): o["A"] = ops.fused_rms_norm_modulate(be, self.x, 1e-6, r[0], r[1], out=o.get("A"))
        def Bqk(): o["Bq"], o["Bk"] = ops.fused_rms_norm_rope_pair(be, self.q, self.wq, self.k, self.wk, 1e-5, self.cos, self.sin,
                                                                   heads=self.heads, out=(o.get("Bq"), o.get("Bk")))
        def C(): o["C"] = ops.fused_gated_residual(be, p, self.x, self.proj, r[2], out=o.get("C"))
        def Eqk(): o["Eq"], o["Ek"] = ops.fused_rms_norm_rope_pair(be, self.cross_q, self.wcq, self.cross_k, self.wck, 1e-5, None, None,
                                                                   heads=self.heads, out=(o.get("Eq"), o.get("Ek")))
        def Fr(): o["F"] = ops.fused_gated_residual(be, p, self.x, self.cross, None, out=o.get("F"))
        def G(): o["G"] = ops.fused_rms_norm_modulate(be, self.x, 1e-6, r[3], r[4], out=o.get("G"))
        def H(): o["H"] = be.activation(self.ffn_hidden, ops.GELU_TANH, out=o.get("H"))
        def I(): o["I"] = ops.fused_gated_residual(be, p, self.x, self.ffn_out, r[5], out=o.get("I"))

        return [
            Launch("A rms_modulate", A, act * (hb + 2) + 2 * vec),
            Launch("B rms_rope q+k (tables as large as q)", Bqk, 2 * act * 4 + table),
            Launch("C gated_residual", C, act * (hb + 2 + hb) + vec),
            Launch("E rms cross q+k", Eqk, act * 4 + self.cross_k.numel() * 4),
            Launch("F residual_add", Fr, act * (hb + 2 + hb)),
            Launch("G rms_modulate", G, act * (hb + 2) + 2 * vec),
            Launch("H gelu_tanh", H, self.ffn_hidden.numel() * 4),
            Launch("I gated_residual", I, act * (hb + 2 + hb) + vec),
        ]


class VaeGroupNorm:
    """VAE decoder GroupNorm(32 groups, eps 1e-6) + SiLU on [N, 256, T, H, W] bf16 ~N(0, 2)
    (native/src/components/autoencoder_kl.cpp:31-41).  Statistics pass + apply pass: the input
    counts twice in the algorithmic bytes, the output once."""

    def __init__(self, be, shape=(1, 256, 28, 240, 424), groups=32, seed=0, per_frame=False):
        """per_frame: statistics per (batch entry, frame, group) on the [N, C, T, H, W] tensor as it
        lies (frame_group_norm, native/src/architectures/mochi.cpp:365-371, minus its permutes)."""
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.be, self.groups, self.per_frame = be, groups, per_frame
        self.x = _randn(shape, BF16, g, 0.0, 2.0)
        self.gamma = _randn((shape[1],), F32, g, 1.0, 0.1)
        self.beta = _randn((shape[1],), F32, g, 0.0, 0.1)
        self.out = {}

    def launches(self) -> List[Launch]:
        def gn(): self.out["gn"] = ops.fused_group_norm_silu(self.be, self.x, self.groups, self.gamma, self.beta, 1e-6, out=self.out.get("gn"))
        def gf(): self.out["gn"] = self.be.group_norm_frames(self.x, self.groups, self.gamma, self.beta, 1e-5, fuse_silu=True,
                                                             out=self.out.get("gn"))
        if self.per_frame:
            return [Launch("group_norm_frames_silu", gf, self.x.numel() * 6, kernels=4)]
        return [Launch("group_norm_silu", gn, self.x.numel() * 6, kernels=4)]


class LinearEpilogues:
    """The bf16 linear's epilogue merged with the operator that reads its result, at the sizes of the
    DiT blocks: FFN up-projection -> GELU-tanh [B*S, 8960] (wan.cpp:109-112), FFN down-projection ->
    gated residual [B, S, 1536] (wan.cpp:113-116), Mochi FFN -> SwiGLU [S, 2*8192] (mochi.cpp:197-200).
    Inputs are F32 "GEMM accumulators" ~N(0,1); algorithmic bytes = accumulation + bias (+ residual)
    read once, result written once.  merged=False runs epilogue and consumer as two launches."""

    def __init__(self, be, tokens=32760, batch=2, dim=1536, ffn=8960, swiglu_hidden=8192, seed=0, merged=True):
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.be, self.merged = be, merged
        self.policy = ops.Policy(BF16, BF16)
        self.acc_up = _randn((batch, tokens, ffn), F32, g)
        self.bias_up = _randn((ffn,), BF16, g, 0.0, 0.5)
        self.acc_down = _randn((batch, tokens, dim), F32, g)
        self.bias_down = _randn((dim,), BF16, g, 0.0, 0.5)
        self.res = _randn((batch, tokens, dim), BF16, g)
        self.gate = _randn((batch, 1, dim), F32, g, std=0.3)
        self.acc_glu = _randn((1, tokens, 2 * swiglu_hidden), F32, g)
        self.out = {}

    def launches(self) -> List[Launch]:
        be, p, o = self.be, self.policy, self.out
        up, down, glu = self.acc_up.numel(), self.acc_down.numel(), self.acc_glu.numel()

        def gelu(): o["gelu"] = ops.linear_output_activation(be, self.acc_up, self.bias_up, ops.GELU_TANH, out=o.get("gelu"))
        def gated(): o["gated"] = ops.linear_output_gated_residual(be, p, self.res, self.acc_down, self.bias_down, self.gate, out=o.get("gated"))
        def swiglu(): o["swiglu"] = ops.linear_output_swiglu(be, self.acc_glu, None, out=o.get("swiglu"))
        def lin_up(): o["lin_up"] = ops.linear_output(be, self.acc_up, self.bias_up, out=o.get("lin_up"))
        def lin_down(): o["lin_down"] = ops.linear_output(be, self.acc_down, self.bias_down, out=o.get("lin_down"))
        def lin_glu(): o["lin_glu"] = ops.linear_output(be, self.acc_glu, None, out=o.get("lin_glu"))
        def gelu2(): o["gelu"] = be.activation(o["lin_up"], ops.GELU_TANH, out=o.get("gelu"))
        def gated2(): o["gated"] = ops.fused_gated_residual(be, p, self.res, o["lin_down"], self.gate, out=o.get("gated"))
        def swiglu2(): o["swiglu"] = ops.fused_swiglu(be, o["lin_glu"], out=o.get("swiglu"))

        if self.merged:
            return [Launch("linear_output gelu_tanh", gelu, up * 6), Launch("linear_output gated_residual", gated, down * 8),
                    Launch("linear_output swiglu", swiglu, glu * 4 + glu)]
        return [Launch("epilogue up", lin_up, up * 6), Launch("gelu_tanh", gelu2, up * 4),
                Launch("epilogue down", lin_down, down * 6), Launch("gated_residual", gated2, down * 6),
                Launch("epilogue glu", lin_glu, glu * 6), Launch("swiglu", swiglu2, glu * 3)]


class LtxVaeNorm:
    """The head of LTX's decoder_residual (native/src/architectures/ltx.cpp:221-227) on a VAE decoder
    feature map [1, C, T, H, W] bf16 ~N(0.2, 1.5): pixel_norm over the channels, then modulate with
    per-channel (shift, scale) ~N(0, 0.2) and SiLU.  Algorithmic bytes: input read once, result
    written once (F32 as modulate's contract gives it, or bf16 with the consumer's operand cast)."""

    def __init__(self, be, shape=(1, 128, 16, 256, 384), dtype=BF16, seed=0):
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.be = be
        self.x = _randn(shape, dtype, g, 0.2, 1.5)
        vec = (shape[0], shape[1], 1, 1, 1)
        self.shift, self.scale = _randn(vec, F32, g, 0.0, 0.2), _randn(vec, F32, g, 0.0, 0.2)
        self.out = {}

    def launches(self) -> List[Launch]:
        be, o, x = self.be, self.out, self.x
        n, eb = x.numel(), x.element_size()

        def norm(): o["norm"] = be.pixel_norm(x, 1, 1e-8, out=o.get("norm"))
        def f32(): o["f32"] = ops.fused_pixel_norm_modulate(be, x, self.shift, self.scale, 1e-8, out=o.get("f32"))
        def bf16(): o["bf16"] = ops.fused_pixel_norm_modulate(be, x, self.shift, self.scale, 1e-8, out_dtype=BF16, out=o.get("bf16"))

        return [Launch("pixel_norm", norm, n * 2 * eb), Launch("pixel_norm modulate silu f32", f32, n * (eb + 4)),
                Launch("pixel_norm modulate silu bf16", bf16, n * (eb + 2))]


class LtxDepthToSpace:
    """LTX decoder up-block tail (native/src/architectures/ltx.cpp:250-259) on a feature map [1, C, T, H, W]
    bf16: the convolution output [1, 4C, T, H, W] and the block input, shuffled, repeated, sliced and
    added in one pass; plus pixel_shuffle_nd alone.  Algorithmic bytes: inputs once + result once."""

    def __init__(self, be, shape=(1, 256, 16, 128, 192), dtype=BF16, seed=0):
        g = torch.Generator(device="cuda").manual_seed(seed)
        b, c, t, h, w = shape
        self.be = be
        self.x = _randn(shape, dtype, g)
        self.y = _randn((b, 4 * c, t, h, w), dtype, g)
        self.out = {}

    def launches(self) -> List[Launch]:
        be, o = self.be, self.out
        eb = self.x.element_size()
        b, c, t, h, w = self.x.shape
        out_elems = b * (c // 2) * (2 * t - 1) * 4 * h * w

        def d2s(): o["d2s"] = ops.fused_depth_to_space_residual(be, self.y, self.x, out=o.get("d2s"))
        def shuffle(): o["shuffle"] = be.pixel_shuffle_nd(self.y, (2, 2, 2), out=o.get("shuffle"))

        return [Launch("depth_to_space residual", d2s, (self.y.numel() + self.x.numel() + out_elems) * eb),
                Launch("pixel_shuffle 2x2x2", shuffle, self.y.numel() * 2 * eb)]


class WanVaeRmsChannel:
    """Wan VAE rms_channel (+ SiLU) (native/src/components/executor.cpp:90-93 as used by wan.cpp:225-297):
    RMSNorm over the channel axis of [1, C, T, H, W] bf16 ~N(0,1) with gamma [C] ~N(1,0.1), eps 1e-12.
    Algorithmic bytes: input once + result once."""

    def __init__(self, be, shape=(1, 192, 4, 240, 416), dtype=BF16, seed=0):
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.be = be
        self.x = _randn(shape, dtype, g)
        self.gamma = _randn((shape[1],), F32, g, 1.0, 0.1)
        self.out = {}

    def launches(self) -> List[Launch]:
        be, x = self.be, self.x
        n = x.numel() * x.element_size() * 2

        def plain(): self.out["plain"] = be.rms_norm(x, self.gamma, 1e-12, 1)
        def silu(): self.out["silu"] = ops.fused_rms_channel_silu(be, x, self.gamma, 1e-12)

        return [Launch("rms_channel", plain, n), Launch("rms_channel silu", silu, n)]


class LayoutOps:
    """The layout operators at the sizes the video paths call them with: the Wan patch embedding's transposition
    [1, 1536, 32760] -> [1, 32760, 1536] (native/src/architectures/wan.cpp:159), Mochi's frames-first permute of a VAE
    feature map and its channels-last permute (mochi.cpp:368, :384), LTX's causal replicate padding of the time axis and
    its spatial zero padding (ltx.cpp:210-214), SwiGLU's two halves as slices (mochi.cpp:197-198) and a concat along the
    channel axis.  Algorithmic bytes: what is read + what is written."""

    def __init__(self, be, frames=8, dtype=BF16, seed=0):
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.be = be
        self.patches = _randn((1, 1536, 32760), dtype, g)
        self.feature = _randn((1, 128, frames, 256, 384), dtype, g)
        self.proj = _randn((1, 8192, 16384), dtype, g)
        self.out = {}

    def launches(self) -> List[Launch]:
        be, o = self.be, self.out
        size = lambda t: t.numel() * t.element_size()
        f = self.feature
        b, c, t, h, w = f.shape
        padded_t = size(f) * (t + 4) // t
        padded_hw = size(f) * ((h + 2) * (w + 2)) // (h * w)

        def transpose(): o["tokens"] = be.permute(self.patches, (0, 2, 1), out=o.get("tokens"))
        def frames_first(): o["frames"] = be.permute(f, (0, 2, 1, 3, 4), out=o.get("frames"))
        def channels_last(): o["last"] = be.permute(f, (0, 2, 3, 4, 1), out=o.get("last"))
        def causal(): o["causal"] = be.pad(f, [0, 0, 0, 0, 2, 2], 0.0, True, out=o.get("causal"))
        def spatial(): o["spatial"] = be.pad(f, [1, 1, 1, 1], 0.0, False, out=o.get("spatial"))
        def edge(): o["edge"] = ops.fused_edge_time_pad(be, f, 1, 1, 1, out=o.get("edge"))
        def nearest(): o["nearest"] = be.interpolate_nearest(f.view(c * t // 8, 8, h, w), [2.0, 2.0], out=o.get("nearest"))
        def half(): o["half"] = be.slice(self.proj, 2, 8192, 16384, out=o.get("half"))
        def joined(): o["joined"] = be.concat([f, f], 1, out=o.get("joined"))

        return [
            Launch("permute tokens<->channels", transpose, 2 * size(self.patches)),
            Launch("permute frames first", frames_first, 2 * size(f)),
            Launch("permute channels last", channels_last, 2 * size(f)),
            Launch("pad time replicate", causal, size(f) + padded_t),
            Launch("pad H, W zero", spatial, size(f) + padded_hw),
            Launch("pad T replicate + H, W zero, one pass", edge, size(f) + size(f) * ((t + 2) * (h + 2) * (w + 2)) // (t * h * w)),
            Launch("nearest 2x in H and W (Wan VAE upsample)", nearest, 5 * size(f)),
            Launch("slice second half", half, size(self.proj)),
            Launch("concat channels (2 launches)", joined, 4 * size(f)),
        ]


def build_config(be, config: int, tokens=None, hidden_dtype=BF16, frames=None, batch=1):
    """The launch list of headline configuration 2..5 (optionally at a reduced token / frame count),
    or of the additional measurement configurations 6..13."""
    if config == 2:
        t = tokens or 32760
        return WanBlock(be, tokens=t, grid=(21, 30, 52) if t == 32760 else (1, 1, t), hidden_dtype=hidden_dtype, batch=batch)
    if config == 3:
        return Wan22Step(be, tokens=tokens or 32760)
    if config == 4:
        return MochiBlock(be, tokens=tokens or 44520, hidden_dtype=hidden_dtype)
    if config == 5:
        return VaeGroupNorm(be, shape=(1, 256, frames or 28, 240, 424))
    if config == 6:
        return VaeGroupNorm(be, shape=(frames or 28, 256, 1, 240, 424))
    if config == 7:
        return VaeGroupNorm(be, shape=(1, 256, frames or 28, 240, 424), per_frame=True)
    if config in (8, 9):
        return LinearEpilogues(be, tokens=tokens or 32760, batch=batch, merged=config == 8)
    if config == 10:
        return LtxVaeNorm(be, shape=(1, 128, frames or 16, 256, 384), dtype=hidden_dtype)
    if config == 11:
        return LtxDepthToSpace(be, shape=(1, 256, frames or 16, 128, 192), dtype=hidden_dtype)
    if config == 12:
        return WanVaeRmsChannel(be, shape=(1, 192, frames or 4, 240, 416), dtype=hidden_dtype)
    if config == 13:
        return LayoutOps(be, frames=frames or 8, dtype=hidden_dtype)
    if config in (14, 15):
        return LtxBlock(be, tokens=tokens or 6144, batch=batch if batch > 1 else 2, hidden_dtype=hidden_dtype, per_token=config == 15)
    raise ValueError("config must be 2..15 (6 = config 5 as a pre-permuted per-frame tensor, 7 = per-frame statistics "
                     "on the unpermuted [N,C,T,H,W] tensor, 8 = linear epilogues merged with their consumers, "
                     "9 = the same as separate launches, 10 = LTX VAE pixel_norm -> modulate -> SiLU, "
                     "11 = LTX VAE depth_to_space, 12 = Wan VAE rms_channel + SiLU, 13 = layout operators, "
                     "14 = LTX block chain, 15 = the same with per-token modulation)")


def _main():
    """python -m vrhino_b200.workloads [--config C] [--tokens N] [--frames T] [--only PREFIX]
    [--repeat R] [--hidden bf16|f32] [--batch B] [--fuse-residual-norm] [--pair-qk] [--merge-tail]

    Runs (selected) launches of one configuration a few times and prints their device times; a
    small, self-contained command for profilers."""
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, default=2)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--frames", type=int, default=None)
    ap.add_argument("--only", default="")
    ap.add_argument("--repeat", type=int, default=3)
    ap.add_argument("--hidden", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--batch", type=int, default=1, help="config 2: CFG branches batched into one tensor")
    ap.add_argument("--fuse-residual-norm", action="store_true",
                    help="config 2: residual update + following LayerNorm as one launch (9 launches per block)")
    ap.add_argument("--pair-qk", action="store_true", help="config 2: q and k RMSNorm+RoPE as one launch")
    ap.add_argument("--merge-tail", action="store_true", help="Mochi: residual update + next pre-norm as one launch")
    a = ap.parse_args()
    be = ops.B200Backend()
    work = build_config(be, a.config, tokens=a.tokens, hidden_dtype=BF16 if a.hidden == "bf16" else F32, frames=a.frames,
                        batch=a.batch)
    chosen = {k: True for k, on in (("fuse_residual_norm", a.fuse_residual_norm), ("pair_qk", a.pair_qk),
                                          ("merge_tail", a.merge_tail)) if on}
    listed = work.launches(**chosen)
    launches = [l for l in listed if l.name.startswith(a.only)]
    total, per = time_launches(launches, steps=a.repeat, warmup=1)
    for l in launches:
        print(f"{l.name:32s} {per[l.name] * 1e3:9.1f} us {l.bytes / per[l.name] / 1e6:9.1f} GB/s {l.bytes / 1e6:9.1f} MB")
    print(f"{'total':32s} {total * 1e3:9.1f} us {sum(l.bytes for l in launches) / total / 1e6:9.1f} GB/s")


class WanBlockHost:
    """The same chain with every operand in page-locked HOST memory, run through the host-buffer
    entry points of the C ABI (upload, kernel, download pipelined inside each call).  A batched block
    (both CFG branches) is run branch by branch: each branch has its own modulation vectors, and the
    host entry points take one vector set per call."""

    def __init__(self, blk: WanBlock):
        import ctypes
        from . import _lib
        self._c, self._lib = ctypes, _lib
        self.blk = blk

        def pin(t):
            return t.detach().cpu().contiguous().pin_memory()

        self.x, self.q, self.k, self.proj = pin(blk.x), pin(blk.q), pin(blk.k), pin(blk.proj)
        self.cross_q, self.cross_k, self.cross, self.ffn_out = pin(blk.cross_q), pin(blk.cross_k), pin(blk.cross), pin(blk.ffn_out)
        self.ffn_hidden = pin(blk.ffn_hidden)
        self.rows = [pin(r) for r in blk.rows]
        self.wq, self.wk, self.wcq, self.wck = pin(blk.wq), pin(blk.wk), pin(blk.wcq), pin(blk.wck)
        self.gamma3, self.beta3 = pin(blk.gamma3), pin(blk.beta3)
        B, S = blk.x.shape[0], blk.x.shape[1]
        self.cos, self.sin = pin(blk.cos.reshape(S, -1)), pin(blk.sin.reshape(S, -1))
        hd = blk.x.dtype

        def out_like(t, dtype=BF16):
            return torch.empty(t.shape, dtype=dtype).pin_memory()

        self.out = {k: out_like(self.x) for k in ("A", "Bq", "Bk", "D", "Eq", "G")}
        self.out.update({k: out_like(self.x, hd) for k in ("C", "F", "I")})
        self.out["Ek"] = out_like(self.cross_k)
        self.out["H"] = out_like(self.ffn_hidden)
        ins = [self.x] * 6 + [self.q, self.k, self.proj, self.cross_q, self.cross_k, self.cross, self.ffn_out, self.ffn_hidden] + \
              [self.cos, self.sin, self.cos, self.sin] * B
        self.h2d_bytes = _nbytes(*ins) + B * (6 * self.rows[0][0].numel() * 4 + 6 * self.wq.numel() * 4)
        self.d2h_bytes = _nbytes(*self.out.values())
        self.bytes_per_step = sum(l.bytes for l in blk.launches())

    def step(self):
        P = lambda t: None if t is None else self._c.c_void_p(t.data_ptr())
        code = lambda t: 0 if t is None else (2 if t.dtype == BF16 else 0)
        call, o, r = self._lib.call, self.out, self.rows
        B, S, D = self.x.shape
        eps = self._c.c_float(1e-6)
        F = self.ffn_hidden.shape[-1]
        T = self.cross_k.shape[1]
        d = self.cos.shape[-1]
        for b in range(B):
            x = self.x[b]

            def ln_mod(out, shift, scale, w=None, bias=None):
                call("vrb_host_layer_norm_modulate", P(x), code(x), P(w), code(w), P(bias), code(bias),
                     None if scale is None else P(scale[b]), None if shift is None else P(shift[b]), 0,
                     P(out[b]), code(out), S, D, eps)

            def rms_rope(src, w, out, rows, rope=True):
                call("vrb_host_rms_norm_rope", P(src[b]), code(src), P(w), 0, P(self.cos) if rope else None, P(self.sin) if rope else None,
                     d, P(out[b]), code(out), rows, D, D, eps)

            def gated(branch, gate, out):
                call("vrb_host_gated_residual", P(x), code(x), P(branch[b]), code(branch), None if gate is None else P(gate[b]), 0,
                     P(out[b]), code(out), S, D)

            ln_mod(o["A"], r[0], r[1])
            rms_rope(self.q, self.wq, o["Bq"], S)
            rms_rope(self.k, self.wk, o["Bk"], S)
            gated(self.proj, r[2], o["C"])
            ln_mod(o["D"], None, None, self.gamma3, self.beta3)
            rms_rope(self.cross_q, self.wcq, o["Eq"], S, rope=False)
            rms_rope(self.cross_k, self.wck, o["Ek"], T, rope=False)
            gated(self.cross, None, o["F"])
            ln_mod(o["G"], r[3], r[4])
            call("vrb_host_activation", 2, P(self.ffn_hidden[b]), P(o["H"][b]), 2, S, F)
            gated(self.ffn_out, r[5], o["I"])


if __name__ == "__main__":
    _main()
