"""A plain, slow restatement of the Ginodra design in float64 on the CPU: one function per mechanism, loops over
tokens where the design has a recurrence, no cache, no batching.  The tests compare the engine with it; it shares
nothing with the engine's code.

Notation.  x [T, W] is the residual stream of one request, h a sublayer's input.  Linear weights are [out, in] and
applied as h @ W.T.  ``cfg`` is the config.json dictionary, ``w`` maps tensor names to float64 tensors.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ---------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """x over the root of (its mean square + eps), along the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def grouped_norm(x, weight, groups, eps):
    """The row cut into ``groups`` equal consecutive parts, each brought to unit root mean square by itself; the
    whole row then times the weight."""
    T, W = x.shape
    return unit_rms(x.reshape(T, groups, W // groups), eps).reshape(T, W) * weight


def time_filter(h, taps_weight):
    """h + a causal filter over time on every channel: out_t = h_t + sum_j f[:, j] h_(t - K + 1 + j), with zeros in
    front of the sequence.  taps_weight [W, K]; its last column multiplies the current token."""
    T, W = h.shape
    K = taps_weight.shape[1]
    padded = torch.cat([torch.zeros(K - 1, W, dtype=h.dtype), h], 0)
    out = h.clone()
    for j in range(K):
        out = out + padded[j:j + T] * taps_weight[:, j]
    return out


def relu_squared_mlp(h, up, down):
    return (torch.relu(h @ up.T) ** 2) @ down.T


def rotate_half(x, positions, dims, base):
    """x [T, heads, n]: the first ``dims`` elements of each head turn by position * base^(-2i/dims), element i paired
    with element i + dims/2; the rest stay."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = positions.to(F64)[:, None] * freq[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], -1)


def softmax_rows(scores, visible, sink=None):
    """scores [T, S] for one head; ``visible`` a boolean mask; ``sink``: a number whose exponential joins the
    denominator without a key or a value.  Returns the weights [T, S]."""
    s = scores.masked_fill(~visible, -math.inf)
    top = s.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, torch.full_like(top, float(sink)))
    e = torch.exp(s - top)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink - top)
    return e / den


# ---------------------------------------------------------------- mixers
def latent_attention(h, m, w, p, eps, positions=None):
    """Attention whose queries pass a normed latent and whose keys and values are expanded from one normed latent per
    token; one rotated key part is shared by all heads; a sink per head; a sigmoid gate per head."""
    T = h.shape[0]
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T) if positions is None else positions
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_half(q[..., dn:], pos, m["rot"]["dims"], m["rot"]["base"])
    kv = h @ w[p + "dkv"].T
    c = unit_rms(kv[:, :rank], eps) * w[p + "dkv.norm"]
    k_rot = rotate_half(kv[:, None, rank:], pos, m["rot"]["dims"], m["rot"]["base"])[:, 0]
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    causal = pos[:, None] >= pos[None, :]
    gate = torch.sigmoid(h @ w[p + "g"].T)                      # [T, H]
    heads = []
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        heads.append((softmax_rows(s, causal, w[p + "sink"][a]) @ v[:, a]) * gate[:, a:a + 1])
    return torch.cat(heads, -1) @ w[p + "o"].T


def window_keys(h, m, w, p, eps):
    """The keys (normed per head) and values of a windowed attention layer, as its cache holds them."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = unit_rms((h @ w[p + "k"].T).reshape(T, G, d), eps) * w[p + "k.norm"]
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    return k, v


def window_attention(h, m, w, p, eps, kv=None):
    """Grouped-query attention inside a sliding window, no rotation: the score loses slope_head * distance; q and k
    are normed per head with a weight; a sigmoid gate per head.  ``kv``: keys and values of another layer, used in the
    place of this layer's own."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = unit_rms((h @ w[p + "q"].T).reshape(T, H, d), eps) * w[p + "q.norm"]
    k, v = kv if kv is not None else window_keys(h, m, w, p, eps)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    dist = (i - j).to(F64)
    visible = (dist >= 0) & (dist < m["mask"]["size"])
    gate = torch.sigmoid(h @ w[p + "g"].T)
    heads = []
    for a in range(H):
        slope = 2.0 ** (-8.0 * (a + 1) / H)
        s = (q[:, a] @ k[:, a // (H // G)].T) * m["scale"] - slope * dist
        heads.append((softmax_rows(s, visible) @ v[:, a // (H // G)]) * gate[:, a:a + 1])
    return torch.cat(heads, -1) @ w[p + "o"].T


def general_delta(h, m, w, p, eps):
    """The generalised delta rule: per head a matrix S [d, d] that decays per key channel, forgets along the unit key
    at a learned rate per channel, and takes in k v^T; both the decay and the forgetting read the state of the token
    before.  The read-out r^T S sees the current token's write."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = (h @ w[p + "r"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, H, d)
    v = (h @ w[p + "v"].T).reshape(T, H, d)
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]))
    decay = decay.reshape(T, H, d)
    rate = torch.sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).reshape(T, H, d)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, d, d, dtype=F64)
    out = torch.zeros(T, H, d, dtype=F64)
    for t in range(T):
        seen = torch.einsum("hk,hkv->hv", u[t], S)                         # u^T S of the old state
        S = decay[t][:, :, None] * S - (rate[t] * u[t])[:, :, None] * seen[:, None, :] \
            + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hk,hkv->hv", r[t], S)
    o = unit_rms(out, eps).reshape(T, H * d) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# ---------------------------------------------------------------- the model
def layer_states(cfg, w, tokens):
    """The residual stream after every layer, [layers, T, W]."""
    eps, groups, mult = cfg["norm"]["eps"], cfg["norm"]["groups"], cfg["residual_mult"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept = {}
    states = []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        h = grouped_norm(x, w[f"l{i}.norm1"], groups, eps)
        hm = time_filter(h, w[f"l{i}.canon1"])
        if layer["type"] == "latent_attention":
            y = latent_attention(hm, m, w, p, eps)
        elif layer["type"] == "attention":
            if m.get("kv_from") is None:
                kept[i] = window_keys(hm, m, w, p, eps)
                y = window_attention(hm, m, w, p, eps)
            else:
                y = window_attention(hm, m, w, p, eps, kv=kept[m["kv_from"]])
        elif layer["type"] == "general_delta":
            y = general_delta(hm, m, w, p, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            y = y + relu_squared_mlp(time_filter(h, w[f"l{i}.canon2"]), w[f"l{i}.mlp.up"], w[f"l{i}.mlp.down"])
        x = x + mult * y
        states.append(x)
    return torch.stack(states)


def forward(cfg, w, tokens):
    """Logits [T, vocab] of one request, every position."""
    x = layer_states(cfg, w, tokens)[-1]
    x = grouped_norm(x, w["final.norm"], cfg["norm"]["groups"], cfg["norm"]["eps"])
    z = (x @ w["embed"].T) * cfg["logit_scale"]
    cap = cfg["logit_softcap"]
    return cap * torch.tanh(z / cap)


# ---------------------------------------------------------------- random weights for the tests
def tensor_shapes(cfg):
    W = cfg["width"]
    K = cfg["canon"]["taps"]
    shapes = {"embed": (cfg["vocab"], W), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        shapes[f"l{i}.norm1"] = (W,)
        shapes[f"l{i}.canon1"] = (W, K)
        if layer["type"] == "latent_attention":
            H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            shapes.update({p + "dq": (m["q_rank"], W), p + "dq.norm": (m["q_rank"],), p + "uq": (H * (dn + dr), m["q_rank"]),
                           p + "dkv": (m["kv_rank"] + dr, W), p + "dkv.norm": (m["kv_rank"],),
                           p + "uk": (H * dn, m["kv_rank"]), p + "uv": (H * dv, m["kv_rank"]), p + "sink": (H,),
                           p + "g": (H, W), p + "o": (W, H * dv)})
        elif layer["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "q": (H * d, W), p + "q.norm": (d,), p + "g": (H, W), p + "o": (W, H * dv)})
            if m.get("kv_from") is None:
                shapes.update({p + "k": (G * d, W), p + "v": (G * dv, W), p + "k.norm": (d,)})
        else:
            n = m["heads"] * m["dim"]
            rank = m["decay_rank"]
            shapes.update({p + "r": (n, W), p + "k": (n, W), p + "v": (n, W), p + "g": (n, W), p + "a": (n, W),
                           p + "a.b": (n,), p + "w1": (rank, W), p + "w2": (n, rank), p + "w0": (n,), p + "norm": (n,),
                           p + "o": (W, n)})
        if layer.get("mlp") is not None:
            shapes.update({f"l{i}.canon2": (W, K), f"l{i}.mlp.up": (layer["mlp"]["ff"], W),
                           f"l{i}.mlp.down": (W, layer["mlp"]["ff"])})
    return shapes


def random_weights(cfg, seed):
    """bfloat16 tensors under the checkpoint's names: matrices N(0, 1/in), norms near 1, filters, biases and sinks of
    a size that shows in the logits."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("norm") or name.endswith("norm1"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
        elif "canon" in name:
            t = 0.4 * torch.randn(shape, generator=gen)
        elif name.endswith((".sink", ".a.b", ".w0")):
            t = torch.randn(shape, generator=gen)
        elif name == "embed":
            t = torch.randn(shape, generator=gen)
        elif name.endswith((".w2",)):
            t = torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out
