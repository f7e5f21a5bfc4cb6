"""Ginodra on the CPU: its config.json keys and their checks, the tensor table against the design's tensor names, what
each layer keeps between steps (pages with one plane for the latents, a window's pages that a later layer shares,
the delta rule's state, the input filters' last tokens), and the sizes that only the checkpoint gives."""
import copy

import pytest
import torch

import plain_ginodra as pg
from nanohybrid_vlm_b200.config.model_config import ConfigError
from nanohybrid_vlm_b200.config.registry import ARCHITECTURES
from nanohybrid_vlm_b200.engine.model import CausalLM
from nanohybrid_vlm_b200.parts.base import FixedStateNeed, PagedKVNeed, SharedPagesNeed, need_leaves


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, base, scale):
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale,
                rot=dict(base=base, dims=rot_dim))


def window(heads, kv, dim, vdim, size, scale, kv_from=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, mask=dict(size=size))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


CFG = dict(architecture="Ginodra", vocab=120, width=48, norm=dict(eps=1e-5, groups=3), residual_mult=0.5,
           canon=dict(taps=4), logit_scale=1.5, logit_softcap=20.0, layers=[
    dict(type="attention", mixer=window(4, 2, 8, 12, 10, 0.3), mlp=dict(kind="dense", ff=40)),
    dict(type="latent_attention", mixer=latent(3, 12, 4, 10, 20, 28, 10000.0, 0.2), mlp=None),
    dict(type="general_delta", mixer=dict(heads=3, dim=8, decay_rank=6), mlp=dict(kind="dense", ff=56)),
    dict(type="attention", mixer=window(4, 2, 8, 12, 25, 0.2, kv_from=0), mlp=dict(kind="dense", ff=40)),
])


def build(cfg):
    import nanohybrid_vlm_b200.models  # noqa: F401
    entry = ARCHITECTURES.resolve(cfg)
    parsed = entry.parse_config(cfg)
    return parsed, entry.build_spec(parsed)


def test_tensor_table_names_and_shapes_are_the_designs():
    parsed, spec = build(CFG)
    model = CausalLM(spec, torch.bfloat16, "cpu")
    got = {}
    for bp in model.param_table():
        for src in bp.decl.sources:
            got[src.name] = tuple(src.checkpoint_shape(bp.decl.shape))
    assert got == {k: tuple(v) for k, v in pg.tensor_shapes(CFG).items()}
    assert "l3.mix.k" not in got and "l3.mix.k.norm" not in got and "l1.canon2" not in got
    assert parsed.to_json_dict()["layers"] == CFG["layers"]


def test_cache_needs_follow_the_layers():
    _, spec = build(CFG)
    needs = [need_leaves(n) for n in CausalLM(spec, torch.float32, "cpu").cache_needs()]
    kept = FixedStateNeed((3 * 48,))                    # the last taps - 1 inputs of the layer's norm, in every layer
    assert all(n[0] == kept for n in needs)
    # layer 0's pages keep the keys that layer 3's wider window still reads
    assert needs[0][1] == PagedKVNeed(2, 8, 25, v_head_dim=12)
    assert needs[1][1] == PagedKVNeed(1, 28 + 4, v_head_dim=28, planes=1)
    assert needs[2][1] == FixedStateNeed((3 * 8 * 8,)) or needs[2][1].shape == (3 * 8 * 8,)
    assert isinstance(needs[3][1], SharedPagesNeed)
    assert spec.order[3].cache_from == 0 and all(spec.order[i].cache_from is None for i in range(3))


def test_decay_rank_comes_from_the_checkpoint():
    from nanohybrid_vlm_b200.models.ginodra import sizes_from_checkpoint
    cfg = copy.deepcopy(CFG)
    del cfg["layers"][2]["mixer"]["decay_rank"]
    with pytest.raises(ConfigError, match="w1"):
        build(cfg)
    done = sizes_from_checkpoint(cfg, lambda name: (11, 48) if name == "l2.mix.w1" else None)
    assert done["layers"][2]["mixer"]["decay_rank"] == 11 and "decay_rank" not in cfg["layers"][2]["mixer"]
    build(done)


@pytest.mark.parametrize("path,value,words", [
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "mask", "size"), 0, "size"),
    (("layers", 3, "mixer", "kv_from"), 3, "earlier"),
    (("layers", 3, "mixer", "kv_from"), 1, "attention layer"),
    (("layers", 3, "mixer", "vdim"), 8, "differ"),
    (("layers", 1, "mixer", "rot", "dims"), 3, "dims"),
    (("layers", 1, "mixer", "kv_rank"), 0, "positive"),
    (("layers", 2, "mixer", "dim"), 0, "positive"),
    (("layers", 2, "mlp", "kind"), "moe", "dense"),
    (("layers", 2, "type"), "conv", "unknown layer type"),
    (("norm", "groups"), 5, "groups"),
    (("canon", "taps"), 0, "taps"),
    (("logit_softcap",), 0.0, "softcap"),
    (("width",), 0, "positive"),
])
def test_bad_values_are_refused(path, value, words):
    cfg = copy.deepcopy(CFG)
    at = cfg
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=words):
        build(cfg)


def test_optional_keys():
    cfg = copy.deepcopy(CFG)
    cfg["canon"] = dict(taps=1)                         # one tap: nothing to keep between steps
    cfg["logit_softcap"] = None
    cfg["layers"][0]["mixer"]["mask"] = None            # no window: every key is kept, also for the layer that shares
    del cfg["norm"]["groups"]
    _, spec = build(cfg)
    needs = [need_leaves(n) for n in CausalLM(spec, torch.float32, "cpu").cache_needs()]
    assert needs[0] == [PagedKVNeed(2, 8, None, v_head_dim=12)]
    assert len(needs[2]) == 1 and isinstance(needs[2][0], FixedStateNeed)
