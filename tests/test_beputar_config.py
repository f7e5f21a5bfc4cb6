"""Beputar on the CPU: its config.json keys and their checks, the tensor table against the design's tensor names, what
each layer keeps between steps (pages of a window with kept first keys, the linear attention's and the time mixing's
memories, the last input), the sizes that only the checkpoint gives, and the cache manager's handling of pages whose keys
are kept for good."""
import copy

import pytest
import torch

import plain_beputar as pb
from nanohybrid_vlm_b200.cache.manager import CacheManager, GroupSpec
from nanohybrid_vlm_b200.config.model_config import ConfigError
from nanohybrid_vlm_b200.config.registry import ARCHITECTURES
from nanohybrid_vlm_b200.engine.model import CausalLM
from nanohybrid_vlm_b200.parts.base import FixedStateNeed, PagedKVNeed, need_leaves

LEFT = dict(heads=4, kv_heads=2, dim=8, vdim=8, scale=0.3, rot=dict(base=10000.0, dims=4), mask=dict(size=12, keep_first=3))
RIGHT = dict(heads=2, dim=4, vdim=6, decay=[0.9, 0.5])
ATTN = dict(heads=4, kv_heads=2, dim=8, vdim=8, scale=0.2, mask=dict(size=25),
            rot=dict(base=1000.0, dims=8, scaling=dict(factor=4.0, original=16, fast=4.0, slow=1.0)))
MOE = dict(kind="moe", router=dict(experts=4, top=2), expert=dict(ff=12), shared=dict(ff=16))
CFG = dict(architecture="Beputar", vocab=120, width=48, embedding=dict(scale=3.0), norm=dict(eps=1e-5), layers=[
    dict(type="parallel", mixer=dict(left=LEFT, right=RIGHT), mlp=dict(kind="dense", ff=40)),
    dict(type="wkv", mixer=dict(heads=3, dim=8, decay_rank=6), mlp=MOE),
    dict(type="attention", mixer=ATTN, mlp=None),
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
    assert got == {k: tuple(v.shape) for k, v in pb.random_weights(CFG).items()}
    assert "l2.norm2" not in got and "l2.ls2" not in got and "l2.mix.o.b" not in got and "l2.mix.v" not in got
    assert set(spec.ignored_checkpoint_tensors) == {"l2.norm2", "l2.ls2"}
    assert parsed.to_json_dict()["layers"] == CFG["layers"]


def test_cache_needs_follow_the_layers():
    _, spec = build(CFG)
    needs = [need_leaves(n) for n in CausalLM(spec, torch.float32, "cpu").cache_needs()]
    assert needs[0] == [PagedKVNeed(2, 8, 12, v_head_dim=8, keep_first=3), FixedStateNeed((2 * 4 * 6,))]
    assert needs[1] == [FixedStateNeed((48,)), FixedStateNeed((3 * 8 * 8,))]
    assert needs[2] == [PagedKVNeed(2, 8, 25, v_head_dim=8)]


def test_decay_rank_comes_from_the_checkpoint():
    from nanohybrid_vlm_b200.models.beputar import sizes_from_checkpoint
    cfg = copy.deepcopy(CFG)
    del cfg["layers"][1]["mixer"]["decay_rank"]
    with pytest.raises(ConfigError, match="w1"):
        build(cfg)
    done = sizes_from_checkpoint(cfg, lambda name: (11, 48) if name == "l1.mix.w1" else None)
    assert done["layers"][1]["mixer"]["decay_rank"] == 11 and "decay_rank" not in cfg["layers"][1]["mixer"]
    build(done)


@pytest.mark.parametrize("path,value,words", [
    (("layers", 0, "mixer", "left", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "left", "vdim"), 12, "values are the keys"),
    (("layers", 0, "mixer", "left", "mask", "size"), 0, "size"),
    (("layers", 0, "mixer", "left", "mask", "keep_first"), -1, "keep_first"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 3, "dims"),
    (("layers", 0, "mixer", "right", "decay"), [0.5], "decay"),
    (("layers", 0, "mixer", "right", "dim"), 0, "positive"),
    (("layers", 1, "mixer", "dim"), 0, "positive"),
    (("layers", 1, "mlp", "router", "top"), 5, "top"),
    (("layers", 1, "mlp", "expert", "ff"), 0, "ff"),
    (("layers", 1, "mlp", "kind"), "glu", "unknown kind"),
    (("layers", 2, "mixer", "rot", "scaling", "factor"), 0.0, "positive"),
    (("layers", 2, "mixer", "rot", "base"), 1.0, "base"),
    (("layers", 2, "type"), "conv", "unknown layer type"),
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
    del cfg["layers"][0]["mixer"]["left"]["mask"]["keep_first"]     # a window without kept keys
    cfg["layers"][2]["mixer"]["mask"] = None                        # no window: every key is kept
    del cfg["layers"][2]["mixer"]["rot"]["scaling"]                 # plain frequencies
    cfg["layers"][1]["mlp"]["shared"] = None
    del cfg["embedding"]
    parsed, spec = build(cfg)
    assert parsed.embedding_scale == 1.0
    model = CausalLM(spec, torch.float32, "cpu")
    needs = [need_leaves(n) for n in model.cache_needs()]
    assert needs[0][0] == PagedKVNeed(2, 8, 12, v_head_dim=8) and needs[2] == [PagedKVNeed(2, 8, None, v_head_dim=8)]
    names = {s.name for bp in model.param_table() for s in bp.decl.sources}
    assert not any(n.startswith("l1.mlp.shared") for n in names) and "l1.mlp.e3.down" in names


def test_pages_of_kept_first_keys_are_never_given_back():
    """A window of 20 with 10 kept first keys over pages of 8: pages 0 and 1 stay for the life of the request, the pages
    between them and the window go back as the window passes, and a freed request returns all of them."""
    cm = CacheManager([GroupSpec(20, None, 10), GroupSpec(20)], 8, [12, 12])
    cm.allocate("a", 70)
    assert cm.release_behind_window("a", 70) == 4 + 6
    kept, plain = cm.block_table("a", 0), cm.block_table("a", 1)
    assert [p >= 0 for p in kept] == [True, True, False, False, False, False, True, True, True]
    assert [p >= 0 for p in plain] == [False] * 6 + [True] * 3
    cm.allocate("a", 90)
    assert cm.release_behind_window("a", 90) == 2 + 2
    assert [p >= 0 for p in cm.block_table("a", 0)][:3] == [True, True, False]
    cm.check()
    cm.free("a")
    cm.check()
    assert cm.pools[0].num_free == 12 and cm.pools[1].num_free == 12
    short = CacheManager([GroupSpec(4, None, 3)], 8, 4)     # the kept keys and the window share the first page
    short.allocate("b", 30)
    assert short.release_behind_window("b", 30) == 2 and [p >= 0 for p in short.block_table("b")] == [True, False, False, True]
