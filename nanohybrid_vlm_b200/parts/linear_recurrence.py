"""Mixers whose memory is a matrix per head that decays per key channel: S <- diag(w) S + k v^T (``ops.decay_scan``).

``wkv``: time mixing in the manner of RWKV-6.  Parameters: ``num_heads`` (H), ``head_dim`` (d, of r, k and v alike),
``decay_rank`` (the inner size of the decay's two-step projection), ``eps`` (of the output norm).
With x' the input of the token before (zeros before a request's first token), each of r, k, v, g, w reads its own mix
x + (x' - x) * mu_s.  r, k, v = projections of their mixes [H d]; gate = silu(g(mix_g)); the decay per head and key
channel is exp(-exp(w2 tanh(w1 mix_w) + w0)).  Per head: o = (S + diag(u) k v^T)^T r with the bonus u for the current
token only, then S <- diag(decay) S + k v^T.  Each head's o is divided by its root mean square, multiplied by ``norm``
[H d] and by the gate; then the output projection.
Tensors: ``mu`` [5, width] stacked from the checkpoint's ``mu.r``, ``mu.k``, ``mu.v``, ``mu.g``, ``mu.w``; ``rkvg``
[4, H d, width] stacked from ``r``, ``k``, ``v``, ``g`` (four products with four inputs: one batched product); ``w1``
[rank, width]; ``w2`` [H d, rank]; ``w0`` [H d]; ``u`` [H, d]; ``norm`` [H d]; ``o`` [width, H d].  Per request the
mixer keeps the last input (float32) and S (float32).  The inner projection of the decay keeps its 32-bit sums; tanh,
the second product, both exponentials, the recurrence and the output norm are 32-bit.

``lightning_attention``: linear attention with one constant decay per head.  Parameters: ``num_heads`` (H),
``head_dim`` (d of q and k), ``v_head_dim`` (dv), ``decay`` (H numbers), ``eps``.
q = silu(q(x)), k = silu(k(x)) [H d], v = silu(v(x)) [H dv].  Per head S <- decay_h S + k v^T, o = S^T q (the current
token counted).  The concatenated heads are divided by the root mean square of them all together, multiplied by ``norm``
[H dv] and by sigmoid(g(x)); then the output projection.
Tensors: ``qkvg`` [2 H d + 2 H dv, width] packed from ``q``, ``k``, ``v``, ``g``; ``norm`` [H dv]; ``o`` [width, H dv].
Per request the mixer keeps S in float32.  SiLU is applied to the projections' rounded output in 32-bit as the scan
reads it; the recurrence and the output norm are 32-bit.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import MIXERS, CompositeNeed, FixedStateNeed, Mixer
from .spec import ParamDecl, Source

MIXES = ("r", "k", "v", "g", "w")


class WKV(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.H = int(spec["num_heads"])
        self.d = int(spec["head_dim"])
        self.rank = int(spec["decay_rank"])
        self.eps = float(spec["eps"])
        if min(self.H, self.d, self.rank) <= 0:
            raise ValueError("wkv: heads, head_dim and decay_rank must be positive")
        self.n = self.H * self.d

    def params(self):
        W, n = self.env.hidden_size, self.n
        return [
            ParamDecl("mu", (len(MIXES), W), init="mix_share",
                      sources=tuple(Source("mu." + s, i, 1, squeeze=True) for i, s in enumerate(MIXES))),
            ParamDecl("rkvg", (4, n, W), sources=tuple(Source(s, i, 1, squeeze=True) for i, s in enumerate("rkvg"))),
            ParamDecl("w1", (self.rank, W)),
            ParamDecl("w2", (n, self.rank), init="unit"),
            ParamDecl("w0", (n,), init="gate_bias"),
            ParamDecl("u", (self.H, self.d), init="unit"),
            ParamDecl("norm", (n,), init="norm"),
            ParamDecl("o", (W, n)),
        ]

    def cache_need(self):
        return CompositeNeed((FixedStateNeed((self.env.hidden_size,)), FixedStateNeed((self.H * self.d * self.d,))))

    def streamed_weights(self):
        return [(self.w_o, 0)]

    def forward(self, x, batch, cache):
        T, n, W = x.shape[0], self.n, self.env.hidden_size
        last_input, memory = cache.children[0].state, cache.children[1].state
        mixes = self.new(len(MIXES), T, W)              # one contiguous plane per mix
        ops.token_shift_mix(mixes, x, self.w_mu, last_input, batch)
        proj = self.new(4, T, n)                        # r, k, v, g: four products in one batched launch
        ops.linear_heads(proj.transpose(0, 1), mixes[:4].transpose(0, 1), self.w_rkvg)
        inner = self.new(T, self.rank, dtype=torch.float32)
        ops.linear_f32(inner, mixes[4], self.w_w1)
        decay = self.new(T, n, dtype=torch.float32)
        ops.decay_lowrank(decay, inner, self.w_w2, self.w_w0)
        o = self.new(T, n, dtype=torch.float32)
        ops.decay_scan(o, proj[0], proj[1], proj[2], memory, batch, self.H, self.d, self.d, decay_tokens=decay,
                       bonus=self.w_u)
        gated = self.new(T, n)
        ops.gated_rmsnorm(gated, o, proj[3], self.w_norm, self.H, self.eps, gate_first=False, gate="silu")
        out = self.new(T, W)
        ops.linear(out, gated, self.w_o)
        return out


class LightningAttention(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.H = int(spec["num_heads"])
        self.d = int(spec["head_dim"])
        self.dv = int(spec.get("v_head_dim") or self.d)
        self.eps = float(spec["eps"])
        decay = [float(v) for v in spec["decay"]]
        if min(self.H, self.d, self.dv) <= 0 or len(decay) != self.H:
            raise ValueError(f"lightning attention: positive sizes and one decay per head ({self.H}), got {len(decay)}")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=env.device)
        self.qk_size, self.v_size = self.H * self.d, self.H * self.dv

    def params(self):
        W, qk, v = self.env.hidden_size, self.qk_size, self.v_size
        return [
            ParamDecl("qkvg", (2 * qk + 2 * v, W), sources=(Source("q", 0, qk), Source("k", qk, qk), Source("v", 2 * qk, v),
                                                            Source("g", 2 * qk + v, v))),
            ParamDecl("norm", (v,), init="norm"),
            ParamDecl("o", (W, v)),
        ]

    def cache_need(self):
        return FixedStateNeed((self.H * self.d * self.dv,))

    def streamed_weights(self):
        return [(self.w_qkvg, 0), (self.w_o, 0)]

    def forward(self, x, batch, cache):
        T, qk, v = x.shape[0], self.qk_size, self.v_size
        proj = self.new(T, 2 * qk + 2 * v)
        ops.linear(proj, x, self.w_qkvg)
        o = self.new(T, v, dtype=torch.float32)
        ops.decay_scan(o, proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + v], cache.state, batch, self.H, self.d,
                       self.dv, decay_heads=self.decay, silu=True, read_after=True)
        gated = self.new(T, v)
        ops.gated_rmsnorm(gated, o, proj[:, 2 * qk + v:], self.w_norm, 1, self.eps, gate_first=False, gate="sigmoid")
        out = self.new(T, self.env.hidden_size)
        ops.linear(out, gated, self.w_o)
        return out


MIXERS.register("wkv", WKV)
MIXERS.register("lightning_attention", LightningAttention)
