"""The Wan DiT-block non-GEMM chain on the CPU oracle, timed: the benchmark's CPU baseline.

TEST / BASELINE INFRASTRUCTURE ONLY.  Runs the chain the way the reference runs it -- one
operator at a time, every intermediate materialised (modulate = cast, add, mul, add, cast;
gated_residual = casts, mul, add; ...) -- on a bounded sample of token rows, with the C
restatement's OpenMP loops spread over the host cores.  Algorithmic bytes are counted exactly as
for the GPU arm (each distinct input once + each output once), so the two GB/s figures are the
same metric.
"""
from __future__ import annotations

import os
import time

import numpy as np

from . import oracle as orc


def _normal(shape, dtype, seed, mean=0.0, std=1.0):
    rng = np.random.default_rng(seed)
    return orc.tensor((rng.standard_normal(shape, dtype=np.float32) * std + mean), dtype)


class WanBlockCpu:
    """Same tensors and chain as vrhino_b200.workloads.WanBlock, on `tokens` sampled rows."""

    def __init__(self, tokens=1024, dim=1536, heads=12, ffn=8960, text_tokens=512, hidden="bf16", seed=0):
        S, D = tokens, dim
        self.be = orc.OracleBackend(execution_dtype=orc.BF16)
        self.policy = orc.Policy(requested=orc.BF16, residual=hidden)
        self.x = _normal((1, S, D), hidden, seed)
        mod = _normal((1, 6, D), orc.F32, seed + 1, std=0.1)
        self.rows = [self.be.slice(mod, 1, i, i + 1) for i in range(6)]
        self.q, self.k, self.proj, self.cross_q, self.cross, self.ffn_out = (
            _normal((1, S, D), orc.BF16, seed + 2 + i) for i in range(6))
        self.cross_k = _normal((1, min(text_tokens, S), D), orc.BF16, seed + 9)
        self.ffn_hidden = _normal((1, S, ffn), orc.BF16, seed + 10)
        self.wq, self.wk, self.wcq, self.wck, self.gamma3 = (_normal((D,), orc.F32, seed + 11 + i, 1.0, 0.1) for i in range(5))
        self.beta3 = _normal((D,), orc.F32, seed + 16, 0.0, 0.1)
        d = D // heads
        ph = np.random.default_rng(seed + 17).uniform(-3, 3, size=(1, S, 1, d)).astype(np.float32)
        self.cos, self.sin = orc.tensor(np.cos(ph)), orc.tensor(np.sin(ph))
        self.heads = heads

    def algorithmic_bytes(self) -> int:
        S, D = self.x.shape[1], self.x.shape[2]
        act, hb, vec = S * D, (2 if self.x.dtype == orc.BF16 else 4), D * 4
        table = self.cos.numel * 4
        return (3 * (act * (hb + 2) + 2 * vec) + 2 * (act * 4 + vec + table) + 3 * (act * (2 * hb + 2)) + 2 * vec
                + (act * 4 + vec) + (self.cross_k.numel * 4 + vec) + self.ffn_hidden.numel * 4)

    def step(self):
        be, p, r = self.be, self.policy, self.rows
        H, d = self.heads, self.x.shape[2] // self.heads
        S = self.x.shape[1]
        out = {}
        out["A"] = be.cast(orc.modulate(be, p, be.layer_norm(self.x, None, None, 1e-6), r[0], r[1]), orc.BF16)
        for name, t, w in (("Bq", self.q, self.wq), ("Bk", self.k, self.wk)):
            n = orc.attention_norm(be, p, t, w, 1e-6).reshape((1, S, H, d))
            out[name] = be.cast(orc.operation_rope(be, p, n, self.cos, self.sin), orc.BF16)
        out["C"] = orc.gated_residual(be, p, self.x, self.proj, r[2])
        out["D"] = be.cast(be.layer_norm(self.x, self.gamma3, self.beta3, 1e-6), orc.BF16)
        out["Eq"] = be.cast(orc.attention_norm(be, p, self.cross_q, self.wcq, 1e-6), orc.BF16)
        out["Ek"] = be.cast(orc.attention_norm(be, p, self.cross_k, self.wck, 1e-6), orc.BF16)
        out["F"] = orc.residual_add(be, p, self.x, self.cross)
        out["G"] = be.cast(orc.modulate(be, p, be.layer_norm(self.x, None, None, 1e-6), r[3], r[4]), orc.BF16)
        out["H"] = be.activation(self.ffn_hidden, orc.GELU_TANH)
        out["I"] = orc.gated_residual(be, p, self.x, self.ffn_out, r[5])
        return out


def time_chain(tokens: int, steps: int, warmup: int, hidden: str = "bf16"):
    """Returns (seconds per step, algorithmic bytes per step, threads used)."""
    threads = int(os.environ.get("OMP_NUM_THREADS", "0")) or (os.cpu_count() or 1)
    orc.build()
    blk = WanBlockCpu(tokens=tokens, hidden=hidden)
    for _ in range(warmup):
        blk.step()
    t0 = time.perf_counter()
    for _ in range(steps):
        blk.step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return dt, blk.algorithmic_bytes(), threads
