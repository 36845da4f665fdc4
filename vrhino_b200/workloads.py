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
                 hidden_dtype=BF16, seed=0):
        assert grid[0] * grid[1] * grid[2] == tokens
        g = torch.Generator(device="cuda").manual_seed(seed)
        self.be, S, D = be, tokens, dim
        self.policy = ops.Policy(BF16, hidden_dtype)
        hd = hidden_dtype
        self.x = _randn((1, S, D), hd, g)
        self.mod = _randn((1, 6, D), F32, g, std=0.1)                 # combined modulation rows
        self.rows = [self.mod[:, i:i + 1, :].contiguous() for i in range(6)]
        self.q, self.k, self.proj, self.cross_q, self.cross, self.ffn_out = (_randn((1, S, D), BF16, g) for _ in range(6))
        self.cross_k = _randn((1, text_tokens, D), BF16, g)
        self.ffn_hidden = _randn((1, S, ffn), BF16, g)
        self.wq, self.wk, self.wcq, self.wck, self.gamma3 = (_randn((D,), F32, g, 1.0, 0.1) for _ in range(5))
        self.beta3 = _randn((D,), F32, g, 0.0, 0.1)
        cos, sin = synth.wan_rope_tables(*grid, head_dim=dim // heads)
        self.cos, self.sin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
        self.heads, self.eps = heads, 1e-6
        self.out = {}

    def launches(self) -> List[Launch]:
        be, p, r, e, o = self.be, self.policy, self.rows, self.eps, self.out
        S, D = self.x.shape[1], self.x.shape[2]
        act = S * D
        hb = self.x.element_size()
        vec = D * 4

        def A(): o["A"] = ops.fused_layer_norm_modulate(be, self.x, None, None, e, r[0], r[1])
        def Bq(): o["Bq"] = ops.fused_rms_norm_rope(be, self.q, self.wq, e, self.cos, self.sin, heads=self.heads)
        def Bk(): o["Bk"] = ops.fused_rms_norm_rope(be, self.k, self.wk, e, self.cos, self.sin, heads=self.heads)
        def C(): o["C"] = ops.fused_gated_residual(be, p, self.x, self.proj, r[2])
        def Dn(): o["D"] = be.layer_norm(self.x, self.gamma3, self.beta3, e) if self.x.dtype == BF16 else \
            ops.fused_layer_norm_cast(be, self.x, self.gamma3, self.beta3, e)
        def Eq(): o["Eq"] = ops.fused_rms_norm_rope(be, self.cross_q, self.wcq, e, None, None, heads=self.heads)
        def Ek(): o["Ek"] = ops.fused_rms_norm_rope(be, self.cross_k, self.wck, e, None, None, heads=self.heads)
        def Fr(): o["F"] = ops.fused_gated_residual(be, p, self.x, self.cross, None)
        def G(): o["G"] = ops.fused_layer_norm_modulate(be, self.x, None, None, e, r[3], r[4])
        def H(): o["H"] = be.activation(self.ffn_hidden, ops.GELU_TANH)
        def I(): o["I"] = ops.fused_gated_residual(be, p, self.x, self.ffn_out, r[5])

        table = self.cos.numel() * 4 * 2
        return [
            Launch("A ln_modulate", A, act * (hb + 2) + 2 * vec),
            Launch("B rms_rope q", Bq, act * 4 + vec + table // 2),
            Launch("B rms_rope k", Bk, act * 4 + vec + table // 2),
            Launch("C gated_residual", C, act * (hb + 2 + hb) + vec),
            Launch("D ln_affine", Dn, act * (hb + 2) + 2 * vec),
            Launch("E rms cross q", Eq, act * 4 + vec),
            Launch("E rms cross k", Ek, self.cross_k.numel() * 4 + vec),
            Launch("F residual_add", Fr, act * (hb + 2 + hb)),
            Launch("G ln_modulate", G, act * (hb + 2) + 2 * vec),
            Launch("H gelu_tanh", H, self.ffn_hidden.numel() * 4),
            Launch("I gated_residual", I, act * (hb + 2 + hb) + vec),
        ]


def time_launches(launches: List[Launch], steps: int, warmup: int):
    """Per-launch device time with CUDA events on the current stream; returns
    (total_ms_per_step, {name: mean_ms})."""
    for _ in range(warmup):
        for l in launches:
            l.fn()
    torch.cuda.synchronize()
    per = {l.name: 0.0 for l in launches}
    events = []
    for _ in range(steps):
        for l in launches:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            l.fn()
            b.record()
            events.append((l.name, a, b))
    torch.cuda.synchronize()
    for name, a, b in events:
        per[name] += a.elapsed_time(b) / steps
    return sum(per.values()), per


def _main():
    """python -m vrhino_b200.workloads [--tokens N] [--only PREFIX] [--repeat R] [--hidden bf16|f32]

    Runs (selected) launches of the Wan block chain a few times and prints their device times; a
    small, self-contained command for profilers."""
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--only", default="")
    ap.add_argument("--repeat", type=int, default=3)
    ap.add_argument("--hidden", default="bf16", choices=["bf16", "f32"])
    a = ap.parse_args()
    be = ops.B200Backend()
    blk = WanBlock(be, tokens=a.tokens, grid=(1, 1, a.tokens), hidden_dtype=BF16 if a.hidden == "bf16" else F32)
    launches = [l for l in blk.launches() if l.name.startswith(a.only)]
    total, per = time_launches(launches, steps=a.repeat, warmup=1)
    for l in launches:
        print(f"{l.name:20s} {per[l.name] * 1e3:9.1f} us {l.bytes / per[l.name] / 1e6:9.1f} GB/s {l.bytes / 1e6:9.1f} MB")


class WanBlockHost:
    """The same chain with every operand in page-locked HOST memory, run through the host-buffer
    entry points of the C ABI (upload, kernel, download pipelined inside each call)."""

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
        S = blk.x.shape[1]
        self.cos, self.sin = pin(blk.cos.reshape(S, -1)), pin(blk.sin.reshape(S, -1))
        hd = blk.x.dtype

        def out_like(t, dtype=BF16):
            return torch.empty(t.shape, dtype=dtype).pin_memory()

        self.out = {k: out_like(self.x) for k in ("A", "Bq", "Bk", "D", "Eq", "G")}
        self.out.update({k: out_like(self.x, hd) for k in ("C", "F", "I")})
        self.out["Ek"] = out_like(self.cross_k)
        self.out["H"] = out_like(self.ffn_hidden)
        ins = [self.x] * 6 + [self.q, self.k, self.proj, self.cross_q, self.cross_k, self.cross, self.ffn_out, self.ffn_hidden,
                              self.cos, self.sin, self.cos, self.sin]
        self.h2d_bytes = _nbytes(*ins) + 6 * self.rows[0].numel() * 4 + 6 * self.wq.numel() * 4
        self.d2h_bytes = _nbytes(*self.out.values())
        self.bytes_per_step = sum(l.bytes for l in blk.launches())

    def step(self):
        P = lambda t: None if t is None else self._c.c_void_p(t.data_ptr())
        code = lambda t: 0 if t is None else (2 if t.dtype == BF16 else 0)
        call, o, r = self._lib.call, self.out, self.rows
        S, D = self.x.shape[1], self.x.shape[2]
        eps = self._c.c_float(1e-6)
        F = self.ffn_hidden.shape[-1]
        T = self.cross_k.shape[1]
        d = self.cos.shape[-1]

        def ln_mod(out, shift, scale, w=None, b=None):
            call("vrb_host_layer_norm_modulate", P(self.x), code(self.x), P(w), code(w), P(b), code(b), P(scale), P(shift), 0,
                 P(out), code(out), S, D, eps)

        def rms_rope(x, w, out, rows, rope=True):
            call("vrb_host_rms_norm_rope", P(x), code(x), P(w), 0, P(self.cos) if rope else None, P(self.sin) if rope else None,
                 d, P(out), code(out), rows, D, D, eps)

        def gated(branch, gate, out):
            call("vrb_host_gated_residual", P(self.x), code(self.x), P(branch), code(branch), P(gate), 0, P(out), code(out), S, D)

        ln_mod(o["A"], r[0], r[1])
        rms_rope(self.q, self.wq, o["Bq"], S)
        rms_rope(self.k, self.wk, o["Bk"], S)
        gated(self.proj, r[2], o["C"])
        ln_mod(o["D"], None, None, self.gamma3, self.beta3)
        rms_rope(self.cross_q, self.wcq, o["Eq"], S, rope=False)
        rms_rope(self.cross_k, self.wck, o["Ek"], T, rope=False)
        gated(self.cross, None, o["F"])
        ln_mod(o["G"], r[3], r[4])
        call("vrb_host_activation", 2, P(self.ffn_hidden), P(o["H"]), 2, S, F)
        gated(self.ffn_out, r[5], o["I"])


if __name__ == "__main__":
    _main()
