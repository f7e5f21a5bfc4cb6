"""Ginodra: a decoder-only model whose layers are listed one by one in config.json.

config.json: ``architecture`` "Ginodra"; ``vocab``, ``width``; ``norm`` {``eps``, ``groups``}; ``residual_mult``;
``canon.taps``; ``logit_scale``, ``logit_softcap``; ``layers``: a list of {``type``, ``mixer``, ``mlp``}.  Every layer
is a parallel block: with h = norm1(x), x <- x + residual_mult * (mixer(f1(h)) + mlp(f2(h))), the stream x in float32,
the norm an RMS norm in ``norm.groups`` parts, f1 and f2 short causal filters over time added to their input
(``canon1``, ``canon2``, [width, taps]).  Layer types:

* ``latent_attention`` (``mixer``: heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot {base, dims}): queries
  through a normed latent, keys and values expanded from one normed latent per token, one rotated key part for all
  heads, a sink per head, a sigmoid gate per head;
* ``attention`` (``mixer``: heads, kv_heads, dim, vdim, scale, mask {size}, kv_from): grouped-query attention in a
  sliding window without rotation, q and k normed per head with a weight, the score less 2^(-8 (h + 1) / H) times
  the distance, a sigmoid gate per head; ``kv_from``: j makes the layer read layer j's keys and values;
* ``general_delta`` (``mixer``: heads, dim): the generalised delta rule.  The inner size of its decay projection is
  the first dimension of the checkpoint's ``w1``; a configuration without a checkpoint names it as ``decay_rank``.

``mlp`` is null or {``kind``: "dense", ``ff``}: down(relu(up h)^2).  The logits are the last norm (``final.norm``)
times the embedding table, times ``logit_scale``, then capped as cap * tanh(z / cap).  Tensors: ``embed``,
``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.canon1``, ``l<i>.canon2``, ``l<i>.mix.*``, ``l<i>.mlp.{up,down}``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass

from ..config.model_config import ConfigError, ModelConfig, parse_dtype, take
from ..config.registry import register_architecture
from ..parts.spec import LayerRun, LayerSpec, ModelSpec, PartUse, part

ARCHITECTURE = "Ginodra"
NO_POSITION_LIMIT = 1 << 20     # the design names no longest sequence; the engine's max_model_len is the limit in use
SLOPE_BASE = 8.0                # head h of H loses 2^(-SLOPE_BASE (h + 1) / H) per position of distance
LAYER_TYPES = ("latent_attention", "attention", "general_delta")


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


def _check_latent(m: dict, where: str) -> None:
    _positive(m, ("heads", "vdim", "q_rank", "kv_rank"), where)
    dim, rot_dim = take(m, "dim", int, where=where), take(m, "rot_dim", int, where=where)
    if dim < 0 or rot_dim < 0 or dim + rot_dim <= 0:
        raise ConfigError(f"{where}: dim {dim} and rot_dim {rot_dim} must not be negative, nor both zero")
    take(m, "scale", float, where=where)
    if rot_dim:
        rot = _sub(m, "rot", where)
        dims = take(rot, "dims", int, where=where + ".rot")
        take(rot, "base", float, where=where + ".rot")
        if dims <= 0 or dims % 2 or dims > rot_dim:
            raise ConfigError(f"{where}.rot: dims {dims} must be even and at most rot_dim {rot_dim}")


def _check_attention(m: dict, where: str, index: int, layers: list) -> None:
    heads, kv, dim, vdim = _positive(m, ("heads", "kv_heads", "dim", "vdim"), where)
    if heads % kv:
        raise ConfigError(f"{where}: heads {heads} must be a multiple of kv_heads {kv}")
    take(m, "scale", float, where=where)
    if m.get("mask") is not None and take(_sub(m, "mask", where), "size", int, where=where + ".mask") <= 0:
        raise ConfigError(f"{where}.mask: size must be positive")
    src = m.get("kv_from")
    if src is None:
        return
    if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < index:
        raise ConfigError(f"{where}: kv_from must name an earlier layer, got {src!r}")
    other = layers[src]
    om = other.get("mixer") if isinstance(other, dict) else None
    if other.get("type") != "attention" or not isinstance(om, dict) or om.get("kv_from") is not None:
        raise ConfigError(f"{where}: kv_from {src} must name an attention layer with keys and values of its own")
    if (om.get("kv_heads"), om.get("dim"), om.get("vdim")) != (kv, dim, vdim):
        raise ConfigError(f"{where}: layer {src}'s kv_heads, dim and vdim differ from this layer's")


def _check_delta(m: dict, where: str) -> None:
    _positive(m, ("heads", "dim"), where)
    if m.get("decay_rank") is not None and take(m, "decay_rank", int, where=where) <= 0:
        raise ConfigError(f"{where}: decay_rank must be positive")


def sizes_from_checkpoint(raw: dict, shape_of) -> dict:
    """config.json completed by the sizes that only a tensor's shape gives: a ``general_delta`` mixer's ``decay_rank``
    is the first dimension of its ``w1``.  ``shape_of(name)`` is the shape of a checkpoint tensor, or None."""
    layers = raw.get("layers")
    if not isinstance(layers, list):
        return raw
    out = []
    for i, layer in enumerate(layers):
        if (isinstance(layer, dict) and layer.get("type") == "general_delta" and isinstance(layer.get("mixer"), dict)
                and layer["mixer"].get("decay_rank") is None):
            shape = shape_of(f"l{i}.mix.w1")
            if shape is not None and len(shape) == 2:
                layer = {**layer, "mixer": {**layer["mixer"], "decay_rank": int(shape[0])}}
        out.append(layer)
    return {**raw, "layers": out}


@dataclass(frozen=True)
class GinodraConfig(ModelConfig):
    layers_json: str = "[]"         # the ``layers`` list as canonical JSON (the dataclass stays hashable)
    norm_eps: float = 1e-6
    norm_groups: int = 1
    residual_mult: float = 1.0
    filter_taps: int = 1
    logit_scale: float = 1.0
    logit_softcap: float | None = None

    @property
    def layers(self) -> list:
        return json.loads(self.layers_json)

    @classmethod
    def from_json_dict(cls, raw: dict) -> "GinodraConfig":
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
            if kind == "latent_attention":
                _check_latent(mixer, where + ".mixer")
            elif kind == "attention":
                _check_attention(mixer, where + ".mixer", i, layers)
            elif kind == "general_delta":
                _check_delta(mixer, where + ".mixer")
                if mixer.get("decay_rank") is None:
                    raise ConfigError(f"{where}.mixer: the decay projection's inner size is unknown: the checkpoint has "
                                      f"no tensor l{i}.mix.w1 and config.json no key 'decay_rank'")
            else:
                raise ConfigError(f"{where}: unknown layer type {kind!r} (known: {LAYER_TYPES})")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or take(mlp, "kind", str, where=where + ".mlp") != "dense":
                    raise ConfigError(f"{where}.mlp: only kind 'dense' (or null) is known")
                if take(mlp, "ff", int, where=where + ".mlp") <= 0:
                    raise ConfigError(f"{where}.mlp: ff must be positive")
        norm = _sub(raw, "norm", "config.json")
        groups = take(norm, "groups", int, 1, where="config.json: norm")
        if groups <= 0 or width % groups:
            raise ConfigError(f"config.json: norm.groups {groups} must divide the width {width}")
        taps = take(raw.get("canon") or {}, "taps", int, 1, where="config.json: canon")
        if not 1 <= taps <= 8:
            raise ConfigError(f"config.json: canon.taps must be 1 to 8, got {taps}")
        cap = take(raw, "logit_softcap", float, None)
        if cap is not None and cap <= 0:
            raise ConfigError("config.json: logit_softcap must be positive")
        eos = raw.get("eos_token_id")
        return cls(
            architecture=ARCHITECTURE, model_type=take(raw, "model_type", str, "ginodra"), vocab_size=vocab,
            hidden_size=width, max_position_embeddings=take(raw, "max_position_embeddings", int, NO_POSITION_LIMIT),
            dtype=parse_dtype(raw.get("dtype", raw.get("torch_dtype", "bfloat16"))),
            eos_token_id=eos if isinstance(eos, int) and not isinstance(eos, bool) else None,
            layers_json=json.dumps(layers, sort_keys=True), norm_eps=take(norm, "eps", float), norm_groups=groups,
            residual_mult=take(raw, "residual_mult", float, 1.0), filter_taps=taps,
            logit_scale=take(raw, "logit_scale", float, 1.0), logit_softcap=cap)

    def to_json_dict(self) -> dict:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "residual_mult": self.residual_mult,
                "canon": {"taps": self.filter_taps}, "logit_scale": self.logit_scale,
                "logit_softcap": self.logit_softcap, "layers": self.layers,
                "dtype": str(self.dtype).replace("torch.", ""),
                **({"eos_token_id": self.eos_token_id} if self.eos_token_id is not None else {})}


def _kept_window(layers: list, index: int):
    """How many keys the pages of attention layer ``index`` must keep: the widest window among the layer itself and the
    layers that read its keys (None: all, when one of them has no window)."""
    sizes = []
    for i, layer in enumerate(layers):
        m = layer["mixer"]
        if layer["type"] == "attention" and (i == index or m.get("kv_from") == index):
            if m.get("mask") is None:
                return None
            sizes.append(int(m["mask"]["size"]))
    return max(sizes)


def _mixer(layers: list, index: int, eps: float):
    kind, m = layers[index]["type"], layers[index]["mixer"]
    if kind == "latent_attention":
        rope = None
        if m["rot_dim"]:
            rope = part("rope_banded", theta=float(m["rot"]["base"]), rotary_dim=int(m["rot"]["dims"]))
        return part("latent_attention", num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"],
                    v_head_dim=m["vdim"], q_rank=m["q_rank"], kv_rank=m["kv_rank"], scale=float(m["scale"]),
                    position=rope, eps=eps, sink=True, output_gate="sigmoid_head")
    if kind == "attention":
        src = m.get("kv_from")
        return part("sink_attention", num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                    v_head_dim=m["vdim"], scale=float(m["scale"]), position=None, unit_norm_eps=eps, sink=False,
                    window=None if m.get("mask") is None else int(m["mask"]["size"]),
                    keep_window=_kept_window(layers, index if src is None else src), qk_norm_weight=True,
                    distance_slope_base=SLOPE_BASE, output_gate="sigmoid_head", own_kv=src is None)
    return part("general_delta_rule", num_heads=m["heads"], head_dim=m["dim"], decay_rank=m["decay_rank"], eps=eps)


def build_spec(cfg: GinodraConfig) -> ModelSpec:
    """Ginodra as data: per layer a parallel block (one grouped norm; mixer and feed-forward side by side, each behind
    its input filter; float32 stream); a layer with ``kv_from`` runs on the pages of the layer it names."""
    block = part("parallel_residual", residual_mult=cfg.residual_mult)
    layers, order = [], []
    raw_layers = cfg.layers
    for i, layer in enumerate(raw_layers):
        uses = dict(mixer=PartUse(_mixer(raw_layers, i, cfg.norm_eps), f"l{i}.mix."),
                    norm=PartUse(part("rmsnorm", width=cfg.hidden_size, eps=cfg.norm_eps, groups=cfg.norm_groups,
                                      source="norm1"), f"l{i}."))
        uses["mixer_filter"] = PartUse(part("causal_filter_add", width=cfg.hidden_size, taps=cfg.filter_taps,
                                            source="canon1"), f"l{i}.")
        if layer.get("mlp") is not None:
            uses["ffn"] = PartUse(part("dense_mlp", intermediate_size=layer["mlp"]["ff"], activation="relu2"),
                                  f"l{i}.mlp.")
            uses["ffn_filter"] = PartUse(part("causal_filter_add", width=cfg.hidden_size, taps=cfg.filter_taps,
                                              source="canon2"), f"l{i}.")
        layers.append(LayerSpec(block, **uses))
        order.append(LayerRun(i, cache_from=layer["mixer"].get("kv_from") if layer["type"] == "attention" else None))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        embedding=PartUse(part("token_embedding", vocab_size=cfg.vocab_size, stream="float32", source="embed"), ""),
        layers=tuple(layers), order=tuple(order),
        final_norm=PartUse(part("rmsnorm", width=cfg.hidden_size, eps=cfg.norm_eps, groups=cfg.norm_groups,
                                source="norm"), "final."),
        head=PartUse(part("lm_head", vocab_size=cfg.vocab_size, tied=True, exact=True, scale=cfg.logit_scale,
                          softcap=cfg.logit_softcap), "head."))


register_architecture(ARCHITECTURE, model_types=("ginodra",), parse_config=GinodraConfig.from_json_dict,
                      build_spec=build_spec, complete_config=sizes_from_checkpoint)
