"""Grouped-query attention with options that several designs combine differently: a learned sink per head, rotation
before a weightless q/k norm, value heads whose size may differ from the key heads', values that are the keys
themselves, a window or chunks, projection biases, and a sigmoid gate on the output.

Parameters: ``num_heads``, ``num_kv_heads``, ``head_dim`` (queries and keys), ``v_head_dim`` (values; default
``head_dim``), ``scale`` (on q . k; None: head_dim ** -0.5), ``position`` (a PartSpec of a position encoding with a
rotary table, or None), ``unit_norm_eps`` (after the rotation each q and k head is divided by its root mean square
with this eps inside the root; None: no norm), ``sink`` (True: the softmax denominator of head h also holds
exp(sink_h), a learned number with no key and no value, unscaled, counted once), ``window`` (None: all keys; n: the
last n), ``chunk`` (None, or n: a query sees only the keys of its own chunk of n positions, chunks counted from
position 0 of the request), ``values`` ("projected": a projection of their own; "keys": the values are the key heads as
projected, bias included, before the rotation, and there is no value projection), ``bias`` (True: q, k and the output
projection have biases ``q.b``, ``k.b``, ``o.b``), ``output_gate`` (None, or "sigmoid": the concatenated heads are
multiplied by sigmoid(g(x)) before the output projection, g a projection of the mixer's input; "sigmoid_head": g has one
output per head and head h is multiplied by sigmoid(g(x))_h), ``qk_norm_weight`` (True: after the unit norm each
q and k head is multiplied by a learned weight [head_dim], ``q.norm`` / ``k.norm``, shared by the heads),
``distance_slope_base`` (None, or b: the score of head h at distance n behind the query loses 2^(-b (h + 1) / H) * n),
``own_kv`` (False: the layer has no key / value projections, norms or pages of its own and reads the keys and values
that another run stored, ``LayerRun.cache_from``), ``keep_window`` (how many keys the pages keep, where that is more
than this layer's own ``window`` shows: a layer whose pages another layer with a wider window reads; None: all),
``keep_first`` (n, with a window: the keys at positions below n stay visible to every later query, at their true
positions, and their pages are kept), ``sink_constant`` (a number: the denominator of every head holds exp of it, as a
learned sink would, but no tensor is read; 0.0 adds one), ``qk_norm_order`` ("after_rotation", the default, or
"before_rotation": the unit norm and its weight come before the rotation), ``rope_layout`` ("half": element i turns
with element i + dims / 2, the default; "interleaved": element 2i with element 2i + 1), ``bias`` may also be "qk":
biases on q and k only.

Tensors: ``qkv`` [(nq + nkv) d (+ nkv dv) (+ nq dv), width], rows q then k then v then g, packed from the
checkpoint's ``q``, ``k``, ``v``, ``g`` (those that exist); ``qk_bias`` [(nq + nkv) d] from ``q.b``, ``k.b``; ``sink``
[nq] (float32); ``o`` [width, nq dv]; ``o.b`` [width].  Scores, softmax, rotation, bias and norm are computed in 32-bit.
"""
from __future__ import annotations

from ..kernels import ops
from .base import MIXERS, Mixer, PagedKVNeed
from .spec import ParamDecl, Source


class SinkAttention(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.nq = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        self.dv = int(spec.get("v_head_dim") or self.d)
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads do not divide into {self.nkv} KV heads")
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else self.d ** -0.5
        eps = spec.get("unit_norm_eps")
        self.eps = None if eps is None else float(eps)
        self.has_sink = bool(spec.get("sink", True))
        self.sink_constant = spec.get("sink_constant")
        if self.sink_constant is not None:
            if spec.get("sink", False):
                raise ValueError("a sink is learned (sink=True) or a constant (sink_constant), not both")
            import torch
            self.has_sink = False
            self.fixed_sinks = torch.full((self.nq,), float(self.sink_constant), dtype=torch.float32, device=env.device)
        self.keep_first = int(spec.get("keep_first", 0) or 0)
        self.norm_order = spec.get("qk_norm_order", "after_rotation")
        self.rope_layout = spec.get("rope_layout", "half")
        if self.norm_order not in ("after_rotation", "before_rotation") or self.rope_layout not in ("half", "interleaved"):
            raise ValueError(f"unknown qk_norm_order {self.norm_order!r} or rope_layout {self.rope_layout!r}")
        self.window = spec.get("window")
        self.keep_window = spec.get("keep_window", self.window)
        if self.keep_window is not None and (self.window is None or self.keep_window < self.window):
            raise ValueError("the pages must keep at least the keys that the layer's window shows")
        self.chunk = spec.get("chunk")
        if self.keep_first and (self.window is None or self.keep_window != self.window):
            raise ValueError("kept first keys go with a window of the layer's own")
        self.values = spec.get("values", "projected")
        if self.values not in ("projected", "keys"):
            raise ValueError(f"values are 'projected' or 'keys', not {self.values!r}")
        if self.values == "keys" and self.dv != self.d:
            raise ValueError(f"values that are the keys have the keys' size {self.d}, not {self.dv}")
        self.bias = bool(spec.get("bias", False))
        self.out_bias = self.bias and spec.get("bias") != "qk"
        self.gate = spec.get("output_gate")
        if self.gate not in (None, "sigmoid", "sigmoid_head"):
            raise ValueError(f"an output gate is None, 'sigmoid' or 'sigmoid_head', not {self.gate!r}")
        self.position = env.position(spec.get("position"))
        self.own_kv = bool(spec.get("own_kv", True))
        self.norm_weight = bool(spec.get("qk_norm_weight", False))
        if self.norm_weight and self.eps is None:
            raise ValueError("a weight on the q/k norm needs the norm (unit_norm_eps)")
        base = spec.get("distance_slope_base")
        self.slopes = None
        if base is not None:
            import torch
            self.slopes = torch.tensor([2.0 ** (-float(base) * (h + 1) / self.nq) for h in range(self.nq)],
                                       dtype=torch.float32, device=env.device)
        self.q_size = self.nq * self.d
        self.k_size = self.nkv * self.d if self.own_kv else 0
        self.v_size = self.nkv * self.dv if self.values == "projected" and self.own_kv else 0
        self.g_size = (self.nq if self.gate == "sigmoid_head" else self.nq * self.dv) if self.gate else 0

    def params(self):
        H = self.env.hidden_size
        sources = [Source("q", 0, self.q_size)]
        if self.k_size:
            sources.append(Source("k", self.q_size, self.k_size))
        if self.v_size:
            sources.append(Source("v", self.q_size + self.k_size, self.v_size))
        if self.g_size:
            sources.append(Source("g", self.q_size + self.k_size + self.v_size, self.g_size))
        decls = [
            ParamDecl("qkv", (self.q_size + self.k_size + self.v_size + self.g_size, H), sources=tuple(sources)),
            ParamDecl("o", (H, self.nq * self.dv)),
        ]
        if self.has_sink:
            decls.append(ParamDecl("sink", (self.nq,), storage="float32"))
        if self.norm_weight:
            decls.append(ParamDecl("q.norm", (self.d,), init="norm"))
            if self.own_kv:
                decls.append(ParamDecl("k.norm", (self.d,), init="norm"))
        if self.bias:
            if not self.own_kv:
                raise ValueError("projection biases are not offered for a layer without keys of its own")
            decls.append(ParamDecl("qk_bias", (self.q_size + self.k_size,), init="zeros_noise",
                                   sources=(Source("q.b", 0, self.q_size), Source("k.b", self.q_size, self.k_size))))
            if self.out_bias:
                decls.append(ParamDecl("o.b", (H,), init="zeros_noise"))
        return decls

    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.keep_window, v_head_dim=self.dv, chunk=self.chunk,
                           keep_first=self.keep_first)

    def streamed_weights(self):
        return [(self.w_qkv, 0), (self.w_o, 0)]

    def forward(self, x, batch, cache):
        T = x.shape[0]
        qkv = self.new(T, self.q_size + self.k_size + self.v_size + self.g_size)
        ops.linear(qkv, x, self.w_qkv)
        rot = self.position.rotary() if self.position is not None else None
        table, rotary_dim = rot if rot is not None else (None, 0)
        q = self.new(T, self.q_size)
        if cache.writes != self.own_kv:
            raise ValueError("a layer with keys of its own writes its pages; one without reads another run's (cache_from)")
        ops.rope_norm_store(qkv, q, cache.pages if cache.writes else None, cache.tables.slot_mapping, batch.positions,
                            table, rotary_dim, self.nq, self.nkv, self.d, self.dv, self.eps,
                            bias=self.w_qk_bias if self.bias else None, values_from_keys=self.values == "keys",
                            q_weight=self.w_q_norm if self.norm_weight else None,
                            k_weight=self.w_k_norm if self.norm_weight and self.own_kv else None,
                            norm_first=self.norm_order == "before_rotation", interleaved=self.rope_layout == "interleaved")
        o = self.new(T, self.nq * self.dv)
        ops.attention_sink(o, q, cache.pages, cache.tables, batch, self.nq, self.nkv, self.d, self.dv, self.scale,
                           self.w_sink if self.has_sink else getattr(self, "fixed_sinks", None), self.window or 0,
                           self.chunk or 0, self.slopes, self.keep_first)
        if self.gate == "sigmoid_head":
            ops.sigmoid_mul_heads(o, o, qkv[:, self.q_size + self.k_size + self.v_size:], self.dv)
        elif self.gate:
            ops.sigmoid_mul(o, o, qkv[:, self.q_size + self.k_size + self.v_size:])
        y = self.new(T, self.env.hidden_size)
        ops.linear(y, o, self.w_o)
        if self.out_bias:
            ops.add_row_bias(y, self.w_o_b)
        return y


MIXERS.register("sink_attention", SinkAttention)
