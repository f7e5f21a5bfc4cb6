"""Attention whose keys and values are expanded from one latent vector per token.

Parameters: ``num_heads`` (H), ``head_dim`` (dn: the part of a query / key head that is not rotated), ``rot_dim`` (dr:
the rotated part), ``v_head_dim`` (dv), ``q_rank``, ``kv_rank``, ``scale`` (on the scores), ``position`` (a PartSpec of a
position encoding with a rotary table over at most dr elements), ``eps`` (of the two latent norms), ``sink`` (True: a
learned number per head joins the softmax denominator), ``output_gate`` (None, or "sigmoid_head": head h's output times
sigmoid(g(x))_h, one number per head).

With x the mixer's input:  c_q = rmsnorm(dq x) * dq.norm;  q = uq c_q, per head [dn | dr];  dkv x = [latent | key part]:
c = rmsnorm(latent) * dkv.norm, k_r = the key part, rotated, shared by all heads.  Head h has keys [uk_h c | k_r] and
values uv_h c; the score is q . k * scale.  Since q_h . (uk_h c) = (uk_h^T q_h) . c and sum_j p_j (uv_h c_j) =
uv_h (sum_j p_j c_j), the heads attend over the latents themselves: the cache holds one row [c | k_r] per token
(pages with one plane), the query of head h becomes [uk_h^T q_h | rotated q_r] (a product per head), the attention
kernel reads a row as key and its first kv_rank elements as value, and its output per head goes through uv_h.

Tensors: ``dq`` [q_rank, width], ``dq.norm`` [q_rank], ``uq`` [H (dn + dr), q_rank], ``dkvg`` [kv_rank + dr (+ H), width]
packed from the checkpoint's ``dkv`` and ``g``, ``dkv.norm`` [kv_rank], ``uk`` [H dn, kv_rank], ``uv`` [H dv, kv_rank],
``sink`` [H] (float32), ``o`` [width, H dv].  Norms, rotation, scores and softmax are computed in 32-bit.

Two forms of one step.  Single tokens (and float32) attend over the latents as above.  A bfloat16 step with prompt
portions expands the latents of its requests into keys [uk_h c | k_r] and values uv_h c per head, padded to a common
head size D, in temporary pages, and runs the tensor-core attention kernels over those: a query then costs
dn + dr + dv operations per key and head instead of 2 kv_rank + dr, and the expansion is one product over the
requests' tokens.  The two forms differ by rounding only (which of the factors is rounded to bfloat16 on the way).
"""
from __future__ import annotations

import torch

from ..kernels import attention_mma, ops
from .base import MIXERS, Mixer, PagedKVNeed
from .spec import ParamDecl, Source


class LatentAttention(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.H = int(spec["num_heads"])
        self.dn, self.dr, self.dv = int(spec["head_dim"]), int(spec["rot_dim"]), int(spec["v_head_dim"])
        self.q_rank, self.rank = int(spec["q_rank"]), int(spec["kv_rank"])
        self.scale = float(spec["scale"])
        self.eps = float(spec["eps"])
        self.has_sink = bool(spec.get("sink", True))
        self.gate = spec.get("output_gate")
        if self.gate not in (None, "sigmoid_head"):
            raise ValueError(f"an output gate is None or 'sigmoid_head', not {self.gate!r}")
        self.position = env.position(spec.get("position"))
        if min(self.H, self.dn + self.dr, self.dv, self.q_rank, self.rank) <= 0 or self.dn < 0 or self.dr < 0:
            raise ValueError("latent attention: sizes must be positive")
        self.row = self.rank + self.dr

    def params(self):
        W, H = self.env.hidden_size, self.H
        dkvg = [Source("dkv", 0, self.row)] + ([Source("g", self.row, H)] if self.gate else [])
        decls = [
            ParamDecl("dq", (self.q_rank, W)),
            ParamDecl("dq.norm", (self.q_rank,), init="norm"),
            ParamDecl("uq", (H * (self.dn + self.dr), self.q_rank)),
            ParamDecl("dkvg", (self.row + (H if self.gate else 0), W), sources=tuple(dkvg)),
            ParamDecl("dkv.norm", (self.rank,), init="norm"),
            ParamDecl("uk", (H * self.dn, self.rank)),
            ParamDecl("uv", (H * self.dv, self.rank)),
            ParamDecl("o", (W, H * self.dv)),
        ]
        if self.has_sink:
            decls.append(ParamDecl("sink", (H,), init="gate_bias", storage="float32"))
        return decls

    def bind(self, tensors):
        super().bind(tensors)
        # uk per head with the latent along the rows, so that uk_h^T q_h is a product of the usual form
        self.uk_t = self.w_uk.view(self.H, self.dn, self.rank).transpose(1, 2).contiguous() if self.dn else None
        self.uv_heads = self.w_uv.view(self.H, self.dv, self.rank)
        # the expanded form: both expansions as one matrix, heads padded to a size the tensor-core kernels take
        self.D = -(-max(self.dn + self.dr, self.dv) // 16) * 16
        self.ukv = None
        if self.w_uk.dtype == torch.bfloat16 and self.w_uk.is_cuda and attention_mma.supports(self.D, self.H, self.H):
            self.ukv = torch.cat([self.w_uk, self.w_uv]).contiguous()

    def cache_need(self):
        return PagedKVNeed(1, self.row, v_head_dim=self.rank, planes=1)

    def streamed_weights(self):
        return [(self.w_dq, 0), (self.w_uq, 0), (self.w_dkvg, 0), (self.w_o, 0)]

    def forward(self, x, batch, cache):
        T, H = x.shape[0], self.H
        qa = self.new(T, self.q_rank)
        ops.linear(qa, x, self.w_dq)
        cq = self.new(T, self.q_rank)
        ops.rmsnorm(cq, qa, self.w_dq_norm, self.eps)
        q = self.new(T, H * (self.dn + self.dr))
        ops.linear(q, cq, self.w_uq)
        kvg = self.new(T, self.w_dkvg.shape[0])
        ops.linear(kvg, x, self.w_dkvg)
        rot = self.position.rotary() if self.position is not None else None
        table, rotary_dim = rot if rot is not None else (None, 0)
        q_lat = self.new(T, H * self.row)
        ops.latent_rope_store(kvg[:, :self.row], q, q_lat, cache.pages if cache.writes else None,
                              cache.tables.slot_mapping, batch.positions, table, rotary_dim, H, self.dn, self.dr,
                              self.rank, self.eps, self.w_dkv_norm)
        gate = kvg[:, self.row:] if self.gate else None
        if (self.ukv is not None and EXPAND_PROMPT_PORTIONS and batch.n_prefill_tokens > 0
                and attention_mma.supports(self.D, H, H, batch.n_seqs)):
            return self._expanded(q, q_lat, gate, batch, cache)
        if self.dn:
            ops.linear_heads(q_lat.view(T, H, self.row)[:, :, :self.rank], q.view(T, H, self.dn + self.dr)[:, :, :self.dn],
                             self.uk_t)
        else:
            q_lat.view(T, H, self.row)[:, :, :self.rank].zero_()
        o_lat = self.new(T, H * self.rank)
        ops.latent_attention(o_lat, q_lat, cache.pages, cache.tables, batch, H, self.rank, self.row, self.scale,
                             self.w_sink if self.has_sink else None)
        o = self.new(T, H * self.dv)
        ops.linear_heads(o.view(T, H, self.dv), o_lat.view(T, H, self.rank), self.uv_heads)
        if self.gate:
            ops.sigmoid_mul_heads(o, o, gate, self.dv)
        y = self.new(T, self.env.hidden_size)
        ops.linear(y, o, self.w_o)
        return y

    def _expanded(self, q, q_lat, gate, batch, cache):
        """The step's attention over keys and values expanded per head (bfloat16 steps that bring prompt portions;
        their single tokens ride along)."""
        T, H, D = q.shape[0], self.H, self.D
        qp, pages, tables = ops.latent_expand(cache.pages, cache.tables, batch, q, q_lat, self.ukv, H, self.dn, self.dr,
                                              self.dv, self.rank, D)
        padded = self.new(T, H * D)
        ops.attention_tensor_core(padded, qp, pages, tables, batch.cu_q, batch.kv_len, batch.n_seqs,
                                  batch.n_prefill_tokens, batch.n_prefill_seqs, batch.n_decode_seqs, batch.max_kv_len, H, H,
                                  D, self.scale, 0, self.w_sink if self.has_sink else None)
        o = self.new(T, H * self.dv)
        if self.gate:
            ops.sigmoid_mul_heads(o, padded, gate, self.dv, x_head=D)
        else:
            o.view(T, H, self.dv).copy_(padded.view(T, H, D)[:, :, :self.dv])
        y = self.new(T, self.env.hidden_size)
        ops.linear(y, o, self.w_o)
        return y


EXPAND_PROMPT_PORTIONS = True       # tests switch it off to compare the two forms


MIXERS.register("latent_attention", LatentAttention)
