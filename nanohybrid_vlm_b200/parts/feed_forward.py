"""SwiGLU feed-forward (nanovllm/models/qwen3.py:91-117, nanovllm/layers/activation.py:6-11).

Parameters: ``intermediate_size``.  Tensors: ``gate_up_proj.weight`` [2 I, width], rows gate
then up, packed from gate_proj / up_proj (nanovllm/layers/linear.py:102-108);
``down_proj.weight`` [width, I].
"""
from __future__ import annotations

from ..kernels import ops
from .base import FEED_FORWARDS, FeedForward
from .spec import ParamDecl, Source


class SwiGLU(FeedForward):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.inter = int(spec["intermediate_size"])

    def params(self):
        H, I = self.env.hidden_size, self.inter
        return [
            ParamDecl("gate_up_proj.weight", (2 * I, H), sources=(
                Source("gate_proj.weight", 0, I), Source("up_proj.weight", I, I))),
            ParamDecl("down_proj.weight", (H, I)),
        ]

    def streamed_weights(self):
        return [(self.w_gate_up_proj_weight, 2), (self.w_down_proj_weight, 0)]

    def forward(self, x, batch):
        T = x.shape[0]
        act = self.new(T, self.inter)
        if not ops.swiglu_first_half(act, x, self.w_gate_up_proj_weight):
            gate_up = self.new(T, 2 * self.inter)
            ops.linear(gate_up, x, self.w_gate_up_proj_weight)
            ops.silu_mul(act, gate_up)
        y = self.new(T, self.env.hidden_size)
        ops.linear(y, act, self.w_down_proj_weight)
        return y


class GatedMLP(FeedForward):
    """down(act(gate(x)) * up(x)) with a choice of activation.  Parameters: ``intermediate_size``, ``activation``
    ("silu" or "gelu_tanh"), ``names`` (the checkpoint's names of the gate, up and down matrices; default
    ("gate", "up", "down")).  Tensors: ``gate_up`` [2 I, width], rows gate then up; ``down`` [width, I]."""
    ACTIVATIONS = {"silu": "silu_mul", "gelu_tanh": "gelu_tanh_mul"}

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.inter = int(spec["intermediate_size"])
        self.activation = spec.get("activation", "silu")
        if self.activation not in self.ACTIVATIONS:
            raise ValueError(f"unknown activation {self.activation!r}; known: {sorted(self.ACTIVATIONS)}")
        self.names = tuple(spec.get("names", ("gate", "up", "down")))

    def params(self):
        H, I = self.env.hidden_size, self.inter
        gate, up, down = self.names
        return [ParamDecl("gate_up", (2 * I, H), sources=(Source(gate, 0, I), Source(up, I, I))),
                ParamDecl("down", (H, I), sources=(Source(down, 0, H),))]

    def streamed_weights(self):
        return [(self.w_gate_up, 2 if self.activation == "silu" else 0), (self.w_down, 0)]

    def forward(self, x, batch):
        T = x.shape[0]
        act = self.new(T, self.inter)
        if self.activation != "silu" or not ops.swiglu_first_half(act, x, self.w_gate_up):
            gate_up = self.new(T, 2 * self.inter)
            ops.linear(gate_up, x, self.w_gate_up)
            getattr(ops, self.ACTIVATIONS[self.activation])(act, gate_up)
        y = self.new(T, self.env.hidden_size)
        ops.linear(y, act, self.w_down)
        return y


class DenseMLP(FeedForward):
    """down(act(up(x))): a feed-forward without a gate.  Parameters: ``intermediate_size``, ``activation`` ("relu2": the
    square of relu; "gelu_tanh": the tanh form of GELU), ``names`` (the checkpoint's names of the two matrices; default ("up", "down")).  Tensors: ``up``
    [I, width], ``down`` [width, I]."""
    ACTIVATIONS = {"relu2": "relu_squared", "gelu_tanh": "gelu_tanh"}

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.inter = int(spec["intermediate_size"])
        self.activation = spec.get("activation", "relu2")
        if self.activation not in self.ACTIVATIONS:
            raise ValueError(f"unknown activation {self.activation!r}; known: {sorted(self.ACTIVATIONS)}")
        self.names = tuple(spec.get("names", ("up", "down")))

    def params(self):
        H, I = self.env.hidden_size, self.inter
        up, down = self.names
        return [ParamDecl("up", (I, H), sources=(Source(up, 0, I),)), ParamDecl("down", (H, I), sources=(Source(down, 0, H),))]

    def streamed_weights(self):
        return [(self.w_up, 0), (self.w_down, 0)]

    def forward(self, x, batch):
        T = x.shape[0]
        act = self.new(T, self.inter)
        ops.linear(act, x, self.w_up)
        getattr(ops, self.ACTIVATIONS[self.activation])(act)
        y = self.new(T, self.env.hidden_size)
        ops.linear(y, act, self.w_down)
        return y


FEED_FORWARDS.register("dense_mlp", DenseMLP)
FEED_FORWARDS.register("swiglu", SwiGLU)
FEED_FORWARDS.register("gated_mlp", GatedMLP)
