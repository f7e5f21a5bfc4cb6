"""Norms: RMSNorm with the residual add fused in (nanovllm/layers/layernorm.py:5-50), and Dynamic Tanh.

Parameters: ``width``, ``eps``, ``weight_offset`` (0 for ``x * w``; 1 for the ``x * (1 + w)``
convention some models store), ``source`` (the checkpoint's name of the weight, default "weight"), ``groups`` (the
row is cut into this many equal consecutive parts and each is divided by the root mean square of its own elements;
default 1; over a float32 stream only), ``post_scale`` (the checkpoint's name of a second vector [width] that multiplies
the normed output after the weight, a scale per channel on a sub-block's contribution; only where the norm adds a
sub-block's output onto a float32 stream, ``add_normed``).

Over a residual stream kept in float32 (``forward_add`` / ``forward_add_rows`` given a :class:`Pending`) the terms
are added in 32-bit, the statistics and the product with the weight are 32-bit, and the result is rounded once.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import NORMS, Norm, Pending
from .spec import ParamDecl, Source


class RMSNorm(Norm):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.width = spec["width"]
        self.eps = float(spec["eps"])
        self.weight_offset = float(spec.get("weight_offset", 0.0))
        self.source = spec.get("source", "weight")
        self.groups = int(spec.get("groups", 1))
        if self.groups < 1 or self.width % self.groups:
            raise ValueError(f"a norm over {self.width} elements does not divide into {self.groups} parts")
        self.post_scale = spec.get("post_scale")

    def _plain_only(self):
        if self.groups != 1:
            raise TypeError("a norm in groups works over a float32 residual stream: it takes a Pending")
        if self.post_scale is not None:
            raise TypeError("a norm with a scale per channel adds a sub-block's output onto a float32 stream (add_normed)")

    def params(self):
        # the tensors carry the checkpoint's names where a scale comes with the norm, so that two such norms can share
        # a layer's prefix
        name = "weight" if self.post_scale is None else self.source
        decls = [ParamDecl(name, (self.width,), init="norm" if self.weight_offset == 0.0 else "zeros_noise",
                           sources=(Source(self.source, 0, self.width),))]
        if self.post_scale is not None:
            decls.append(ParamDecl(self.post_scale, (self.width,), init="layer_scale",
                                   sources=(Source(self.post_scale, 0, self.width),)))
        return decls

    def bind(self, tensors):
        if self.post_scale is None:
            return super().bind(tensors)
        self.w_weight, self.w_post_scale = tensors[self.source], tensors[self.post_scale]

    def add_normed(self, terms, residual, side_eps=None, want_rounded=True):
        if self.groups != 1 or self.weight_offset != 0.0:
            raise TypeError("the output norm is a plain RMS norm (one group, the weight as it is stored)")
        rounded = self.new(*residual.shape) if want_rounded else None
        ops.postnorm_stream(residual, rounded, terms, self.w_weight, getattr(self, "w_post_scale", None), self.eps, side_eps)
        return rounded

    def forward(self, x):
        self._plain_only()
        out = self.new(*x.shape)
        ops.rmsnorm(out, x, self.w_weight, self.eps, weight_offset=self.weight_offset)
        return out

    def forward_add(self, x, residual):
        if isinstance(x, Pending):
            if self.post_scale is not None:
                self._plain_only()
            x = x.settled()
            out = self.new(*residual.shape)
            ops.rmsnorm_stream(out, residual, self.w_weight, self.eps, addends=x.terms, weight_offset=self.weight_offset,
                               groups=self.groups)
            return out
        self._plain_only()
        out = self.new(*x.shape)
        ops.rmsnorm(out, x, self.w_weight, self.eps, residual=residual, weight_offset=self.weight_offset)
        return out

    def forward_add_rows(self, x, residual, rows):
        if isinstance(x, Pending):
            x = x.settled()
            out = self.new(rows.numel(), residual.shape[-1])
            ops.rmsnorm_stream(out, residual, self.w_weight, self.eps, addends=x.terms, rows=rows, write_stream=False,
                               weight_offset=self.weight_offset, groups=self.groups)
            return out
        self._plain_only()
        out = self.new(rows.numel(), x.shape[-1])
        ops.rmsnorm(out, x, self.w_weight, self.eps, residual=residual, rows=rows, write_residual=False,
                    weight_offset=self.weight_offset)
        return out


class DynamicTanh(Norm):
    """y = tanh(alpha * x) * w + b: a norm without statistics (a learned scalar ``alpha``, learned vectors ``w``, ``b``).

    Parameters: ``width``, ``source`` (the checkpoint's name of the weight; the bias is ``<source>.b`` and alpha, stored
    without a shape, ``<source>.alpha``; the part's own tensors carry the same names, so several norms can share a
    prefix).  Computed in 32-bit.  Over a float32 residual stream (``forward_add`` / ``forward_add_rows`` given a
    :class:`Pending`) the kernel also adds the sub-block output that is pending, after the Dynamic Tanh norm that this
    output still has to pass (``Pending.post``), all in 32-bit: one launch between two sub-blocks."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.width = int(spec["width"])
        self.source = spec.get("source", "weight")

    def params(self):
        s = self.source
        return [ParamDecl(s, (self.width,), init="norm", sources=(Source(s, 0, self.width),)),
                ParamDecl(s + ".b", (self.width,), init="zeros_noise", sources=(Source(s + ".b", 0, self.width),)),
                ParamDecl(s + ".alpha", (1,), init="dyntanh_alpha", sources=(Source(s + ".alpha", 0, 1, squeeze=True),))]

    def bind(self, tensors):
        s = self.source
        self.w_weight, self.w_bias, self.w_alpha = tensors[s], tensors[s + ".b"], tensors[s + ".alpha"]

    @property
    def triple(self):
        return self.w_alpha, self.w_weight, self.w_bias

    def forward(self, x):
        out = self.new(*x.shape)
        ops.dyntanh(out, x, *self.triple)
        return out

    def forward_embedding(self, table, token_ids):
        """The looked-up rows of ``table`` through this norm, as a float32 stream [T, width]."""
        out = self.new(token_ids.numel(), self.width, dtype=torch.float32)
        ops.embed_dyntanh(out, table, token_ids, *self.triple)
        return out

    def _stream(self, x, residual, rows, n_rows):
        if not isinstance(x, Pending) or residual.dtype != torch.float32:
            raise TypeError("the Dynamic Tanh norm adds into a float32 residual stream: it takes a Pending")
        if x.post is not None and not isinstance(x.post, DynamicTanh):
            x = x.settled()
        if len(x.terms) > 1 or any(c != 1.0 for _, c in x.terms):
            raise ValueError("the Dynamic Tanh norm adds at most one pending sub-block output, with factor 1")
        out = self.new(n_rows, self.width)
        addend = x.terms[0][0] if x.terms else None
        ops.dyntanh_stream(out, residual, self.triple, addend, x.post.triple if x.post is not None else None, rows=rows,
                           write_stream=rows is None)
        return out

    def forward_add(self, x, residual):
        return self._stream(x, residual, None, residual.shape[0])

    def forward_add_rows(self, x, residual, rows):
        return self._stream(x, residual, rows, rows.numel())


NORMS.register("rmsnorm", RMSNorm)
NORMS.register("dyntanh", DynamicTanh)
