"""Beputar: a decoder-only model whose layers are listed one by one in config.json.

config.json: ``architecture`` "Beputar"; ``vocab``, ``width``; ``embedding.scale``; ``norm.eps``; ``layers``: a list of
{``type``, ``mixer``, ``mlp``}.  Every layer norms what a sub-block returns, not what it reads: x <- x + ls1 * norm1(mixer(x)),
then, if the layer has a feed-forward, x <- x + ls2 * norm2(mlp(x)); the stream x is float32, the norms are RMS norms with
a plain weight and ls1, ls2 are scales per channel.  Layer types:

* ``wkv`` (``mixer``: heads, dim): time mixing with mixes of each token's input and the input before it, a decay per
  key channel made from the input, and a bonus for the current token.  The inner size of its decay projection is the
  first dimension of the checkpoint's ``w1``; a configuration without a checkpoint names it as ``decay_rank``.
* ``parallel``: two mixers on the same input, each output RMS-normed over the width (``left.out``, ``right.out``), half
  their sum.  ``mixer.left`` (heads, kv_heads, dim, vdim, scale, rot {base, dims}, mask {size, keep_first}): attention
  whose values are the keys as projected, q and k normed per head with a weight before a rotate-half rotation, a window
  that also keeps the first tokens, one more in the softmax denominator, a sigmoid gate per head.  ``mixer.right``
  (heads, dim, vdim, decay [one per head]): linear attention with a constant decay per head, SiLU on q, k and v, all
  heads normed together, a sigmoid gate.
* ``attention`` (``mixer``: heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling {factor, original, fast, slow}},
  mask {size}): q and k with biases, values that are the keys as projected, rotation of neighbouring pairs with
  frequencies rescaled along a ramp, then a weightless unit norm per head, a sliding window, ordinary softmax.

``mlp`` is null, {``kind``: "dense", ``ff``}: down(gelu_tanh(up h)), or {``kind``: "moe", ``router`` {experts, top},
``expert`` {ff}, ``shared`` {ff} or null}: sigmoid scores, the ``top`` largest chosen, each chosen expert fed with score * h
(a plain gated unit with SiLU), a shared expert for every token.

The logits are the last norm (``final.norm``) times the embedding table itself, without its scale.  Tensors: ``embed``,
``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.ls1``, ``l<i>.norm2``, ``l<i>.ls2``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass

from ..config.model_config import ConfigError, ModelConfig, parse_dtype, take
from ..config.registry import register_architecture
from ..parts.spec import LayerRun, LayerSpec, ModelSpec, PartUse, part

ARCHITECTURE = "Beputar"
NO_POSITION_LIMIT = 1 << 20     # the design names no longest sequence; the engine's max_model_len is the limit in use
LAYER_TYPES = ("wkv", "parallel", "attention")
SINK_SCORE = 0.0                # the left attention's denominator holds exp(0) = 1 more: fixed by the design
YARN_MAGNITUDE_SLOPE = 0.1      # cosines and sines are multiplied by 0.1 ln(factor) + 1: fixed by the design


def _sub(raw: dict, key: str, where: str) -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: key {key!r} must be an object")
    return v


def _positive(m: dict, keys, where: str) -> list[int]:
    vals = [take(m, k, int, where=where) for k in keys]
    if min(vals) <= 0:
        raise ConfigError(f"{where}: {', '.join(keys)} must be positive")
    return vals


def _check_softmax_attention(m: dict, where: str, kept_first: bool) -> None:
    heads, kv, dim, vdim = _positive(m, ("heads", "kv_heads", "dim", "vdim"), where)
    if heads % kv:
        raise ConfigError(f"{where}: heads {heads} must be a multiple of kv_heads {kv}")
    if vdim != dim:
        raise ConfigError(f"{where}: the values are the keys, so vdim {vdim} must equal dim {dim}")
    take(m, "scale", float, where=where)
    rot = _sub(m, "rot", where)
    dims = take(rot, "dims", int, where=where + ".rot")
    if take(rot, "base", float, where=where + ".rot") <= 1.0:
        raise ConfigError(f"{where}.rot: base must be above 1")
    if dims <= 0 or dims % 2 or dims > dim:
        raise ConfigError(f"{where}.rot: dims {dims} must be even and at most dim {dim}")
    if rot.get("scaling") is not None:
        sc = _sub(rot, "scaling", where + ".rot")
        if min(take(sc, k, float, where=where + ".rot.scaling") for k in ("factor", "original", "fast", "slow")) <= 0:
            raise ConfigError(f"{where}.rot.scaling: factor, original, fast and slow must be positive")
    if m.get("mask") is not None:
        mask = _sub(m, "mask", where)
        if take(mask, "size", int, where=where + ".mask") <= 0:
            raise ConfigError(f"{where}.mask: size must be positive")
        if kept_first and take(mask, "keep_first", int, 0, where=where + ".mask") < 0:
            raise ConfigError(f"{where}.mask: keep_first must not be negative")


def _check_lightning(m: dict, where: str) -> None:
    heads, _, _ = _positive(m, ("heads", "dim", "vdim"), where)
    decay = m.get("decay")
    if not isinstance(decay, list) or len(decay) != heads or not all(isinstance(v, (int, float)) and 0 <= v <= 1 for v in decay):
        raise ConfigError(f"{where}: decay must list one number in [0, 1] per head ({heads})")


def _check_wkv(m: dict, where: str) -> None:
    _positive(m, ("heads", "dim"), where)
    if m.get("decay_rank") is not None and take(m, "decay_rank", int, where=where) <= 0:
        raise ConfigError(f"{where}: decay_rank must be positive")


def _check_mlp(mlp, where: str) -> None:
    if mlp is None:
        return
    if not isinstance(mlp, dict):
        raise ConfigError(f"{where} must be an object or null")
    kind = take(mlp, "kind", str, where=where)
    if kind == "dense":
        if take(mlp, "ff", int, where=where) <= 0:
            raise ConfigError(f"{where}: ff must be positive")
    elif kind == "moe":
        r = _sub(mlp, "router", where)
        experts, top = take(r, "experts", int, where=where + ".router"), take(r, "top", int, where=where + ".router")
        if experts <= 0 or not 0 < top <= experts:
            raise ConfigError(f"{where}.router: {experts} experts, top {top}")
        for key in ("expert",) + (("shared",) if mlp.get("shared") is not None else ()):
            if take(_sub(mlp, key, where), "ff", int, where=f"{where}.{key}") <= 0:
                raise ConfigError(f"{where}.{key}: ff must be positive")
    else:
        raise ConfigError(f"{where}: unknown kind {kind!r} (known: 'dense', 'moe', or null)")


def sizes_from_checkpoint(raw: dict, shape_of) -> dict:
    """config.json completed by the sizes that only a tensor's shape gives: a ``wkv`` mixer's ``decay_rank`` is the
    first dimension of its ``w1``.  ``shape_of(name)`` is the shape of a checkpoint tensor, or None."""
    layers = raw.get("layers")
    if not isinstance(layers, list):
        return raw
    out = []
    for i, layer in enumerate(layers):
        if (isinstance(layer, dict) and layer.get("type") == "wkv" and isinstance(layer.get("mixer"), dict)
                and layer["mixer"].get("decay_rank") is None):
            shape = shape_of(f"l{i}.mix.w1")
            if shape is not None and len(shape) == 2:
                layer = {**layer, "mixer": {**layer["mixer"], "decay_rank": int(shape[0])}}
        out.append(layer)
    return {**raw, "layers": out}


@dataclass(frozen=True)
class BeputarConfig(ModelConfig):
    layers_json: str = "[]"         # the ``layers`` list as canonical JSON (the dataclass stays hashable)
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0

    @property
    def layers(self) -> list:
        return json.loads(self.layers_json)

    @classmethod
    def from_json_dict(cls, raw: dict) -> "BeputarConfig":
        vocab, width = take(raw, "vocab", int), take(raw, "width", int)
        if vocab <= 0 or width <= 0:
            raise ConfigError("config.json: vocab and width must be positive")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, layer in enumerate(layers):
            where = f"config.json: layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"{where} must be an object")
            kind = take(layer, "type", str, where=where)
            mixer = _sub(layer, "mixer", where)
            if kind == "wkv":
                _check_wkv(mixer, where + ".mixer")
                if mixer.get("decay_rank") is None:
                    raise ConfigError(f"{where}.mixer: the decay projection's inner size is unknown: the checkpoint has "
                                      f"no tensor l{i}.mix.w1 and config.json no key 'decay_rank'")
            elif kind == "parallel":
                _check_softmax_attention(_sub(mixer, "left", where + ".mixer"), where + ".mixer.left", kept_first=True)
                _check_lightning(_sub(mixer, "right", where + ".mixer"), where + ".mixer.right")
            elif kind == "attention":
                _check_softmax_attention(mixer, where + ".mixer", kept_first=False)
            else:
                raise ConfigError(f"{where}: unknown layer type {kind!r} (known: {LAYER_TYPES})")
            _check_mlp(layer.get("mlp"), where + ".mlp")
        eos = raw.get("eos_token_id")
        return cls(
            architecture=ARCHITECTURE, model_type=take(raw, "model_type", str, "beputar"), vocab_size=vocab,
            hidden_size=width, max_position_embeddings=take(raw, "max_position_embeddings", int, NO_POSITION_LIMIT),
            dtype=parse_dtype(raw.get("dtype", raw.get("torch_dtype", "bfloat16"))),
            eos_token_id=eos if isinstance(eos, int) and not isinstance(eos, bool) else None,
            layers_json=json.dumps(layers, sort_keys=True),
            norm_eps=take(_sub(raw, "norm", "config.json"), "eps", float),
            embedding_scale=take(raw.get("embedding") or {}, "scale", float, 1.0))

    def to_json_dict(self) -> dict:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "layers": self.layers,
                "dtype": str(self.dtype).replace("torch.", ""),
                **({"eos_token_id": self.eos_token_id} if self.eos_token_id is not None else {})}


def _rotary(rot: dict):
    sc = rot.get("scaling")
    if sc is None:
        return part("rope_banded", theta=float(rot["base"]), rotary_dim=int(rot["dims"]))
    return part("rope_ramped", theta=float(rot["base"]), rotary_dim=int(rot["dims"]), factor=float(sc["factor"]),
                original=float(sc["original"]), fast=float(sc["fast"]), slow=float(sc["slow"]),
                magnitude_slope=YARN_MAGNITUDE_SLOPE)


def _kept_first_attention(a: dict, eps: float):
    mask = a.get("mask")
    return part("sink_attention", num_heads=a["heads"], num_kv_heads=a["kv_heads"], head_dim=a["dim"], v_head_dim=a["vdim"],
                scale=float(a["scale"]), position=_rotary(a["rot"]), unit_norm_eps=eps, qk_norm_weight=True,
                qk_norm_order="before_rotation", sink=False, sink_constant=SINK_SCORE, values="keys",
                window=None if mask is None else int(mask["size"]),
                keep_first=0 if mask is None else int(mask.get("keep_first", 0)), output_gate="sigmoid_head")


def _mixer(kind: str, m: dict, eps: float):
    if kind == "wkv":
        return part("wkv", num_heads=m["heads"], head_dim=m["dim"], decay_rank=m["decay_rank"], eps=eps)
    if kind == "attention":
        mask = m.get("mask")
        return part("sink_attention", num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                    v_head_dim=m["vdim"], scale=float(m["scale"]), position=_rotary(m["rot"]), rope_layout="interleaved",
                    unit_norm_eps=eps, sink=False, values="keys", bias="qk",
                    window=None if mask is None else int(mask["size"]))
    s = m["right"]
    right = part("lightning_attention", num_heads=s["heads"], head_dim=s["dim"], v_head_dim=s["vdim"],
                 decay=tuple(float(v) for v in s["decay"]), eps=eps)
    return part("parallel_mixers", left=_kept_first_attention(m["left"], eps), right=right, left_scale=0.5,
                right_scale=0.5, side_norm_eps=eps)


def _feed_forward(mlp: dict):
    if mlp["kind"] == "dense":
        return part("dense_mlp", intermediate_size=int(mlp["ff"]), activation="gelu_tanh")
    r, s = mlp["router"], mlp.get("shared")
    shared = None if s is None else part("gated_mlp", intermediate_size=int(s["ff"]), activation="silu")
    return part("routed_moe", experts=int(r["experts"]), top=int(r["top"]), correction=False, scores="sigmoid",
                renorm=False, weight_on="input", intermediate_size=int(mlp["expert"]["ff"]), limit=None, alpha=1.0,
                up_shift=0.0, shared=shared, shared_gate=False)


def build_spec(cfg: BeputarConfig) -> ModelSpec:
    """Beputar as data: per layer a block that norms and scales each sub-block's output onto a float32 stream."""
    block = part("postnorm_residual")
    layers, unused = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."

        def norm(name: str, scale: str):
            return PartUse(part("rmsnorm", width=cfg.hidden_size, eps=cfg.norm_eps, source=name, post_scale=scale), p)

        uses = dict(mixer=PartUse(_mixer(layer["type"], layer["mixer"], cfg.norm_eps), p + "mix."),
                    mixer_norm=norm("norm1", "ls1"))
        if layer.get("mlp") is not None:
            uses.update(ffn=PartUse(_feed_forward(layer["mlp"]), p + "mlp."), ffn_norm=norm("norm2", "ls2"))
        else:
            unused += [p + "norm2", p + "ls2"]      # a checkpoint may carry them for a layer that has no use for them
        layers.append(LayerSpec(block, **uses))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        embedding=PartUse(part("token_embedding", vocab_size=cfg.vocab_size, scale=cfg.embedding_scale,
                               stream="float32", source="embed"), ""),
        layers=tuple(layers), order=tuple(LayerRun(i) for i in range(len(layers))),
        final_norm=PartUse(part("rmsnorm", width=cfg.hidden_size, eps=cfg.norm_eps, source="norm"), "final."),
        head=PartUse(part("lm_head", vocab_size=cfg.vocab_size, tied=True, exact=True), "head."),
        ignored_checkpoint_tensors=tuple(unused))


register_architecture(ARCHITECTURE, model_types=("beputar",), parse_config=BeputarConfig.from_json_dict,
                      build_spec=build_spec, complete_config=sizes_from_checkpoint)
