"""Token embedding and output head (nanovllm/layers/embed_head.py:9-66).

The head takes only the rows whose logits are wanted and returns them in fp32.  A tied head
owns no tensor: it is given the embedding's table.

Embedding parameters: ``vocab_size``, ``scale`` (a factor on the looked-up rows, default none), ``stream`` ("model":
rows in the model's dtype; "float32": rows in 32-bit, for blocks that keep their residual stream in float32),
``source`` (the checkpoint's name of the table, default "weight"), ``norm`` (a PartSpec of a norm that the looked-up
rows pass before they become the stream, its tensors under the same prefix; the stream is then float32).  Head
parameters: ``vocab_size``, ``tied``, ``exact`` (True: the 32-bit sums of the product are the logits; False: rounded to
the model's dtype first and then widened, as the reference's head does), ``source`` (the checkpoint's name of an untied
head's table; the part's own tensor then carries that name instead of "weight"), ``scale`` (a factor on the logits),
``softcap`` (c: the scaled logits become c * tanh(logits / c); both in 32-bit, on the rows that are asked for).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import EMBEDDINGS, HEADS, NORMS, Embedding, Head
from .spec import ParamDecl, Source


class TokenEmbedding(Embedding):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec["vocab_size"])
        self.scale = spec.get("scale")
        self.stream = spec.get("stream", "model")
        self.source = spec.get("source", "weight")
        if self.stream not in ("model", "float32"):
            raise ValueError(f"an embedding's stream is 'model' or 'float32', not {self.stream!r}")
        if self.scale is not None and self.stream != "float32":
            raise ValueError("a scaled embedding writes a float32 stream")
        norm = spec.get("norm")
        self.norm = NORMS.get(norm.kind)(norm, env) if norm is not None else None
        if self.norm is not None and (self.stream != "float32" or self.scale is not None):
            raise ValueError("an embedding with a norm writes a float32 stream and has no scale")

    def params(self):
        own = [ParamDecl("weight", (self.vocab, self.env.hidden_size), sources=(Source(self.source, 0, self.vocab),))]
        return own + (self.norm.params() if self.norm is not None else [])

    def bind(self, tensors):
        self.w_weight = tensors["weight"]
        if self.norm is not None:
            self.norm.bind({name: t for name, t in tensors.items() if name != "weight"})

    def forward(self, token_ids, batch=None):
        if self.norm is not None:
            if hasattr(self.norm, "forward_embedding"):
                return self.norm.forward_embedding(self.w_weight, token_ids)
            rows = self.new(token_ids.numel(), self.env.hidden_size)
            ops.embed(rows, self.w_weight, token_ids)
            out = self.new(token_ids.numel(), self.env.hidden_size, dtype=torch.float32)
            ops.to_f32(out, self.norm.forward(rows))
            return out
        if self.stream == "float32":
            out = self.new(token_ids.numel(), self.env.hidden_size, dtype=torch.float32)
            ops.embed_scaled_f32(out, self.w_weight, token_ids, 1.0 if self.scale is None else float(self.scale))
            return out
        out = self.new(token_ids.numel(), self.env.hidden_size)
        ops.embed(out, self.w_weight, token_ids)
        return out


class LMHead(Head):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec["vocab_size"])
        self.tied = bool(spec.get("tied", False))
        self.exact = bool(spec.get("exact", False))
        self.source = spec.get("source")
        self.scale = float(spec.get("scale") or 1.0)
        self.softcap = spec.get("softcap")
        if self.softcap is not None and float(self.softcap) <= 0:
            raise ValueError("a soft cap on the logits must be positive")

    def params(self):
        if self.tied:
            return []
        if self.source is None:
            return [ParamDecl("weight", (self.vocab, self.env.hidden_size))]
        return [ParamDecl(self.source, (self.vocab, self.env.hidden_size), sources=(Source(self.source, 0, self.vocab),))]

    def bind(self, tensors):
        (self.w_weight,) = tensors.values()

    def tie(self, embedding) -> None:
        self.w_weight = embedding.w_weight

    def streamed_weights(self):
        return [] if self.exact else [(self.w_weight, 1)]

    def forward(self, rows_hidden):
        logits = self.new(rows_hidden.shape[0], self.vocab, dtype=torch.float32)
        if self.exact:
            ops.linear_f32(logits, rows_hidden, self.w_weight)
        else:
            ops.linear(logits, rows_hidden, self.w_weight)
        if self.scale != 1.0 or self.softcap is not None:
            ops.scale_softcap(logits, self.scale, self.softcap)
        return logits


EMBEDDINGS.register("token_embedding", TokenEmbedding)
HEADS.register("lm_head", LMHead)
