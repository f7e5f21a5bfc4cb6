"""A plain, slow restatement of the Beputar design in float64 on the CPU: one function per mechanism, loops over
tokens where the design has a recurrence, no cache, no batching.  The tests compare the engine with it; it shares
nothing with the engine's code.

Notation.  x [T, W] is the residual stream of one request, h a sublayer's input (the stream itself: this design norms
what a sublayer returns, not what it reads).  Linear weights are [out, in] and applied as h @ W.T.  ``cfg`` is the
config.json dictionary, ``w`` maps tensor names to float64 tensors.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ---------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """x over the root of (its mean square + eps), along the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def base_frequencies(dims, base):
    return torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)


def yarn_frequencies(dims, base, scaling):
    """The frequencies rescaled between two wavelengths, and the factor on cosines and sines."""
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    f = base_frequencies(dims, base)
    i = torch.arange(dims // 2, dtype=F64)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, dims, freq, layout, mult=1.0):
    """x [T, heads, n]: the first ``dims`` elements of each head turn by position * freq_i; "half" pairs element i
    with element i + dims/2, "interleaved" pairs 2i with 2i + 1.  ``mult`` multiplies cosines and sines."""
    ang = positions.to(F64)[:, None] * freq[None, :]
    cos, sin = (ang.cos() * mult)[:, None, :], (ang.sin() * mult)[:, None, :]
    half = dims // 2
    if layout == "half":
        a, b = x[..., :half], x[..., half:dims]
        return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], -1)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([a * cos - b * sin, b * cos + a * sin], -1).reshape(*x.shape[:-1], dims)
    return torch.cat([turned, x[..., dims:]], -1)


def visible_keys(positions, size, keep_first=0):
    """[T, T] booleans: query i sees key j if j <= i and (i - j < size or j < keep_first); size None: every earlier key."""
    i, j = positions[:, None], positions[None, :]
    seen = j <= i
    if size is not None:
        seen = seen & ((i - j < size) | (j < keep_first))
    return seen


def softmax_rows(scores, visible, extra_one=False):
    """scores [T, S] for one head.  ``extra_one``: the denominator also holds exp(0) = 1, a term without a value."""
    s = scores.masked_fill(~visible, -math.inf)
    top = s.max(-1, keepdim=True).values
    if extra_one:
        top = top.clamp(min=0.0)
    e = torch.exp(s - top)
    den = e.sum(-1, keepdim=True)
    if extra_one:
        den = den + torch.exp(-top)
    return e / den


def grouped_attention(q, k, v, scale, visible, extra_one=False):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key head h // (H / G) -> [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        p = softmax_rows((q[:, h] @ k[:, g].T) * scale, visible, extra_one)
        out[:, h] = p @ v[:, g]
    return out


# ---------------------------------------------------------------- mixers
def windowed_attention(h, m, w, p, eps, positions=None):
    """The 'attention' mixer: biased q and k, values that are the keys as projected, interleaved rotation with
    rescaled frequencies, then a weightless unit norm per head, a sliding window, ordinary softmax."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(T) if positions is None else positions
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = k
    rot = m["rot"]
    if rot.get("scaling") is not None:
        freq, mult = yarn_frequencies(rot["dims"], rot["base"], rot["scaling"])
    else:
        freq, mult = base_frequencies(rot["dims"], rot["base"]), 1.0
    q = unit_rms(rotate(q, pos, rot["dims"], freq, "interleaved", mult), eps)
    k = unit_rms(rotate(k, pos, rot["dims"], freq, "interleaved", mult), eps)
    size = m["mask"]["size"] if m.get("mask") is not None else None
    o = grouped_attention(q, k, v, m["scale"], visible_keys(pos, size))
    return o.reshape(T, H * m["vdim"]) @ w[p + "o"].T


def kept_first_attention(h, m, w, p, eps, positions=None):
    """The left side of the 'parallel' mixer: values that are the keys as projected, a weighted norm of q and k before
    a rotate-half rotation, a sliding window that also keeps the first tokens, a softmax whose denominator holds one
    more, a sigmoid gate per head."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(T) if positions is None else positions
    q = (h @ w[p + "q"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, G, d)
    v = k
    rot = m["rot"]
    freq = base_frequencies(rot["dims"], rot["base"])
    q = rotate(unit_rms(q, eps) * w[p + "q.norm"], pos, rot["dims"], freq, "half")
    k = rotate(unit_rms(k, eps) * w[p + "k.norm"], pos, rot["dims"], freq, "half")
    mask = m.get("mask")
    seen = visible_keys(pos, mask["size"] if mask else None, mask.get("keep_first", 0) if mask else 0)
    o = grouped_attention(q, k, v, m["scale"], seen, extra_one=True)
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * m["vdim"]) @ w[p + "o"].T


def lightning_attention(h, m, w, p, eps, state=None):
    """The right side: S <- decay_h S + k v^T per head, o = S^T q with the current token counted; all heads normed
    together, a sigmoid gate, the output projection."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(T, H, d)
    k = silu(h @ w[p + "k"].T).reshape(T, H, d)
    v = silu(h @ w[p + "v"].T).reshape(T, H, dv)
    S = torch.zeros(H, d, dv, dtype=F64) if state is None else state
    o = torch.zeros(T, H, dv, dtype=F64)
    decay = torch.tensor(m["decay"], dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    y = unit_rms(o.reshape(T, H * dv), eps) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def side_by_side(h, m, w, p, eps):
    """The 'parallel' mixer: half the sum of both sides, each normed over the model width first."""
    left = unit_rms(kept_first_attention(h, m["left"], w, p + "left.", eps), eps) * w[p + "left.out"]
    right = unit_rms(lightning_attention(h, m["right"], w, p + "right.", eps), eps) * w[p + "right.out"]
    return 0.5 * (left + right)


def wkv(h, m, w, p, eps):
    """Time mixing with a decay per key channel made from the input, and a bonus for the current token."""
    T, W = h.shape
    H, d = m["heads"], m["dim"]
    before = torch.cat([torch.zeros(1, W, dtype=F64), h[:-1]], 0)

    def mix(s):
        return h + (before - h) * w[p + "mu." + s]

    r = (mix("r") @ w[p + "r"].T).reshape(T, H, d)
    k = (mix("k") @ w[p + "k"].T).reshape(T, H, d)
    v = (mix("v") @ w[p + "v"].T).reshape(T, H, d)
    gate = silu(mix("g") @ w[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix("w") @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).reshape(T, H, d)
    u = w[p + "u"]
    S = torch.zeros(H, d, d, dtype=F64)
    o = torch.zeros(T, H, d, dtype=F64)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t])
        S = decay[t][:, :, None] * S + kv
    y = unit_rms(o, eps).reshape(T, H * d) * w[p + "norm"] * gate
    return y @ w[p + "o"].T


# ---------------------------------------------------------------- feed-forwards
def dense_ff(h, w, p):
    return gelu_tanh(h @ w[p + "up"].T) @ w[p + "down"].T


def gated_unit(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def mixture(h, mlp, w, p):
    """Sigmoid scores, the ``top`` largest chosen, each chosen expert fed with score * h; a shared expert for all."""
    scores = torch.sigmoid(h @ w[p + "router"].T)
    top = scores.topk(mlp["router"]["top"], dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for s, e in zip(top.values[t], top.indices[t]):
            out[t] += gated_unit((s * h[t])[None], w, f"{p}e{int(e)}.")[0]
    if mlp.get("shared") is not None:
        out = out + gated_unit(h, w, p + "shared.")
    return out


# ---------------------------------------------------------------- the model
MIXERS = {"wkv": wkv, "parallel": side_by_side,
          "attention": lambda h, m, w, p, eps: windowed_attention(h, m, w, p, eps)}


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one request given whole (and the stream after every layer, if asked)."""
    eps = cfg["norm"]["eps"]
    w = {k: v.to(F64) for k, v in w.items()}
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        a = MIXERS[layer["type"]](x, layer["mixer"], w, p + "mix.", eps)
        x = x + unit_rms(a, eps) * w[p + "norm1"] * w[p + "ls1"]
        mlp = layer.get("mlp")
        if mlp is not None:
            f = dense_ff(x, w, p + "mlp.") if mlp["kind"] == "dense" else mixture(x, mlp, w, p + "mlp.")
            x = x + unit_rms(f, eps) * w[p + "norm2"] * w[p + "ls2"]
        streams.append(x)
    logits = (unit_rms(x, eps) * w["final.norm"]) @ w["embed"].T
    return (logits, torch.stack(streams)) if return_layers else logits


def random_weights(cfg, seed=0):
    """Random tensors of the design's names and shapes (float32 values that bfloat16 holds exactly)."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    w = {}

    def mat(name, *shape, std=None):
        std = std if std is not None else 1.0 / math.sqrt(shape[-1])
        w[name] = (torch.randn(*shape, generator=g) * std).bfloat16().float()

    def vec(name, n, mean=1.0, std=0.1):
        w[name] = (mean + torch.randn(n, generator=g) * std).bfloat16().float()

    mat("embed", cfg["vocab"], W, std=0.05)
    vec("final.norm", W)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for n in ("norm1", "norm2"):
            vec(p + n, W)
        for n in ("ls1", "ls2"):
            vec(p + n, W, mean=0.6, std=0.2)
        q = p + "mix."
        if layer["type"] == "parallel":
            a, s = m["left"], m["right"]
            mat(q + "left.q", a["heads"] * a["dim"], W)
            mat(q + "left.k", a["kv_heads"] * a["dim"], W)
            vec(q + "left.q.norm", a["dim"])
            vec(q + "left.k.norm", a["dim"])
            mat(q + "left.g", a["heads"], W)
            mat(q + "left.o", W, a["heads"] * a["vdim"])
            for n, rows in (("q", s["dim"]), ("k", s["dim"]), ("v", s["vdim"]), ("g", s["vdim"])):
                mat(q + "right." + n, s["heads"] * rows, W)
            mat(q + "right.o", W, s["heads"] * s["vdim"])
            vec(q + "right.norm", s["heads"] * s["vdim"])
            vec(q + "left.out", W)
            vec(q + "right.out", W)
        elif layer["type"] == "attention":
            mat(q + "q", m["heads"] * m["dim"], W)
            mat(q + "k", m["kv_heads"] * m["dim"], W)
            vec(q + "q.b", m["heads"] * m["dim"], mean=0.0, std=0.3)
            vec(q + "k.b", m["kv_heads"] * m["dim"], mean=0.0, std=0.3)
            mat(q + "o", W, m["heads"] * m["vdim"])
        else:
            n, rank = m["heads"] * m["dim"], m.get("decay_rank", 8)
            for s in "rkvgw":
                vec(q + "mu." + s, W, mean=0.5, std=0.25)
            for s in "rkvg":
                mat(q + s, n, W)
            mat(q + "w1", rank, W)
            mat(q + "w2", n, rank, std=0.5)
            vec(q + "w0", n, mean=-1.0, std=1.0)
            # A head's first output is sign(c) v / rms(v) with c = sum_k r_k u_k k_k (the memory is still empty), so a c
            # near zero would leave the sign to rounding.  Keys that lean on the receptance's projection and a bonus
            # around one keep c away from zero; nothing else depends on it.
            w[q + "k"] = (w[q + "r"] + 0.5 * w[q + "k"]).bfloat16().float()
            w[q + "u"] = (1.0 + torch.randn(m["heads"], m["dim"], generator=g) * 0.3).bfloat16().float()
            vec(q + "norm", n)
            mat(q + "o", W, n)
        mlp = layer.get("mlp")
        if mlp is None:
            del w[p + "norm2"], w[p + "ls2"]
            continue
        f = p + "mlp."
        if mlp["kind"] == "dense":
            mat(f + "up", mlp["ff"], W)
            mat(f + "down", W, mlp["ff"])
        else:
            units = [(f"{f}e{j}.", mlp["expert"]["ff"]) for j in range(mlp["router"]["experts"])]
            if mlp.get("shared") is not None:
                units.append((f + "shared.", mlp["shared"]["ff"]))
            for pre, ff in units:
                mat(pre + "gate", ff, W)
                mat(pre + "up", ff, W)
                mat(pre + "down", W, ff)
            mat(f + "router", mlp["router"]["experts"], W, std=2.0 / math.sqrt(W))
    return w
