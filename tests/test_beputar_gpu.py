"""Beputar through the engine against the plain model (float64): the same requests whole, with their last tokens
decoded one by one, in portions down to two tokens, and mixed with other requests in a pool so small that pages and
state slots are used again; long decoding from a single token; greedy generation through ``LLM.generate`` and the
scheduler, and through the command line.  Small configurations that differ in every size, in the order of their layers
and in what the design leaves open: windows smaller and larger than a page, more kept first keys than the window is
wide and none at all, an attention layer without a mask, rotation of a part of a head and of all of it, rescaled
frequencies and plain ones, one to four experts chosen, a mixture without a shared expert, layers without a
feed-forward, one recurrent head and several, value heads smaller and larger than key heads in the linear attention,
a decay of exactly one, sizes that are no multiple of 8."""
import json
import os

import numpy as np
import pytest
import torch

import plain_beputar as pb
import trace_tools as tt

pytestmark = pytest.mark.gpu


def left(heads, kv, dim, rot_dims, base, size, keep_first, scale):
    mask = None if size is None else dict(size=size, keep_first=keep_first)
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=scale, rot=dict(base=base, dims=rot_dims), mask=mask)


def right(heads, dim, vdim, decay):
    return dict(heads=heads, dim=dim, vdim=vdim, decay=decay)


def attn(heads, kv, dim, rot_dims, base, size, scale, scaling=None):
    rot = dict(base=base, dims=rot_dims)
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=scale, rot=rot,
                mask=None if size is None else dict(size=size))


def wkv(heads, dim, rank):
    return dict(heads=heads, dim=dim, decay_rank=rank)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, shared):
    return dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff),
                shared=None if shared is None else dict(ff=shared))


BEP_A = dict(architecture="Beputar", vocab=300, width=96, embedding=dict(scale=4.0), norm=dict(eps=1e-5), layers=[
    dict(type="parallel", mixer=dict(left=left(4, 2, 16, 8, 10000.0, 12, 3, 0.3), right=right(2, 8, 12, [0.9, 0.5])),
         mlp=dense(80)),
    dict(type="wkv", mixer=wkv(3, 16, 8), mlp=moe(4, 2, 24, 32)),
    dict(type="attention", mixer=attn(4, 2, 16, 16, 1000.0, 25, 0.2, scaling=(4.0, 16, 4.0, 1.0)), mlp=None),
    dict(type="parallel", mixer=dict(left=left(2, 1, 32, 32, 500.0, 7, 20, 0.15), right=right(1, 16, 8, [1.0])),
         mlp=moe(3, 1, 16, None)),
])
BEP_B = dict(architecture="Beputar", vocab=211, width=64, embedding=dict(scale=1.0), norm=dict(eps=1e-6), layers=[
    dict(type="wkv", mixer=wkv(1, 40, 5), mlp=None),
    dict(type="attention", mixer=attn(6, 6, 8, 4, 1000000.0, None, 0.4), mlp=moe(6, 4, 8, 16)),
    dict(type="parallel", mixer=dict(left=left(3, 3, 16, 16, 50.0, 33, 0, 0.25), right=right(4, 8, 8, [0.3, 0.99, 0.7, 0.0])),
         mlp=None),
    dict(type="attention", mixer=attn(2, 1, 32, 8, 300.0, 9, 0.2, scaling=(8.0, 32, 8.0, 2.0)), mlp=dense(40)),
    dict(type="wkv", mixer=wkv(4, 8, 16), mlp=dense(32)),
    dict(type="parallel", mixer=dict(left=left(2, 2, 8, 2, 10.0, None, 0, 0.5), right=right(2, 24, 4, [0.8, 0.95])),
         mlp=moe(2, 2, 12, 20)),
])
# sizes that are no multiple of 8 anywhere: every product and the attention take their general paths
BEP_C = dict(architecture="Beputar", vocab=97, width=100, embedding=dict(scale=7.5), norm=dict(eps=1e-6), layers=[
    dict(type="attention", mixer=attn(3, 1, 20, 6, 20000.0, 50, 0.25, scaling=(2.0, 40, 16.0, 0.5)), mlp=moe(5, 3, 18, 14)),
    dict(type="parallel", mixer=dict(left=left(3, 1, 10, 10, 7000.0, 19, 5, 0.3), right=right(3, 6, 10, [0.5, 0.75, 0.9])),
         mlp=dense(36)),
    dict(type="wkv", mixer=wkv(2, 34, 3), mlp=moe(7, 1, 10, None)),
])
MODELS = {"A": (BEP_A, 41), "B": (BEP_B, 42), "C": (BEP_C, 43)}
LENGTHS = (70, 41, 97, 2, 33, 129, 1, 9, 55)
F32_TOL = 1e-4          # float32 sums in another order than float64
BF16_TOL = 0.05         # activations rounded to 8 bits of mantissa after every op


def write_model(folder, cfg, seed):
    from safetensors.torch import save_file
    w = pb.random_weights(cfg, seed)
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(folder, "model.safetensors"))
    on_disk = json.loads(json.dumps(cfg))
    for layer in on_disk["layers"]:                     # the decay projection's inner size is read off the checkpoint
        layer["mixer"].pop("decay_rank", None)
        for side in ("left",):                          # a mask that is absent is left out, not null
            if isinstance(layer["mixer"].get(side), dict) and layer["mixer"][side].get("mask") is None:
                layer["mixer"][side].pop("mask", None)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(on_disk, f)
    return {k: v.to(torch.float64) for k, v in w.items()}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, seed) in MODELS.items():
        d = str(tmp_path_factory.mktemp(f"beputar_{name}"))
        out[name] = (d, cfg, write_model(d, cfg, seed))
    return out


def requests_for(name):
    cfg, seed = MODELS[name]
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, cfg["vocab"], n).tolist() for i, n in enumerate(LENGTHS)}


@pytest.fixture(scope="module")
def references(models):
    return {name: {rid: pb.forward(cfg, w, t).numpy() for rid, t in requests_for(name).items()}
            for name, (_, cfg, w) in models.items()}


def check(got, ref, reqs, dtype):
    """float32: every position within the limit.  bfloat16: the rounding of a router's input can tip a choice between two
    experts whose scores are nearly equal (the scores also scale the experts' inputs, and the stream carries a few per
    cent of rounding by the later layers), which changes that token (and, less, the later ones of its request) by more
    than rounding does elsewhere; so the typical position stays within the limit and few are far over it.  What is cut
    or placed wrongly shows in float32, where nothing is left to chance."""
    for rid, toks in reqs.items():
        assert sorted(got[rid]) == list(range(len(toks))), f"{rid}: positions missing"
        g = np.stack([got[rid][p] for p in range(len(toks))])
        assert np.isfinite(g).all(), f"{rid}: position {int((~np.isfinite(g)).any(axis=1).argmax())} is not finite"
        diff = g - ref[rid]
        err = (diff - diff.mean(axis=1, keepdims=True)).std(axis=1) / ref[rid].std()
        if dtype == "float32":
            assert err.max() <= F32_TOL, f"{rid}: first bad position {int((err > F32_TOL).argmax())}, worst {err.max():.2e}"
        else:
            over = err > 2 * BF16_TOL
            middle = np.sort(err)[(len(toks) - 1) // 2]
            assert middle <= BF16_TOL and over.sum() <= max(2, len(toks) // 5), \
                f"{rid}: first bad position {int(over.argmax())}, {int(over.sum())} far over, median {middle:.2e}"


def pairs(requests, n=2):
    return tt.portions(requests, sizes=(n,))


MODES = {"whole": tt.whole, "decode_tail": tt.decode_tail, "portions": tt.portions, "pairs": pairs, "mixed": tt.mixed}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("name", list(MODELS))
def test_replay_matches_plain(name, mode, dtype, models, references, tmp_path):
    folder, cfg, _ = models[name]
    reqs = requests_for(name)
    got = tt.run_trace(folder, dtype, MODES[mode](reqs), str(tmp_path), vocab=cfg["vocab"],
                       page_size=16 if name == "A" else 5)
    check(got, references[name], reqs, dtype)


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_logits_do_not_depend_on_the_cutting(name, models, tmp_path):
    """Every kernel fixes the order of its sums per output, so in float32 a position's logits agree to the last few
    bits however its tokens were cut and batched and wherever its pages and its state slot lie."""
    folder, cfg, _ = models[name]
    reqs = requests_for(name)
    outs = []
    for i, mode in enumerate(("whole", "portions", "mixed", "pairs")):
        d = tmp_path / mode
        d.mkdir()
        outs.append(tt.run_trace(folder, "float32", MODES[mode](reqs), str(d), page_size=(8, 16, 3, 64)[i]))
    for rid, toks in reqs.items():
        a = np.stack([outs[0][rid][p] for p in range(len(toks))])
        for other in outs[1:]:
            b = np.stack([other[rid][p] for p in range(len(toks))])
            worst = np.abs(a - b).max(axis=1)
            assert worst.max() <= 2e-5 * np.abs(a).max(), f"{rid} position {int(worst.argmax())} differs between cuttings"


def test_bfloat16_with_pages_of_64_agrees_with_float32(models, tmp_path):
    """Pages of 64 keys: the shapes at which bfloat16 steps take the engine's widest kernels.  The same trace in
    float32 is the comparison."""
    folder, cfg, _ = models["A"]
    reqs = {k: v for k, v in requests_for("A").items() if len(v) > 30}
    steps = tt.mixed(reqs, live=3, first=40)
    out = {}
    for dtype in ("float32", "bfloat16"):
        d = tmp_path / dtype
        d.mkdir()
        out[dtype] = tt.run_trace(folder, dtype, steps, str(d), vocab=cfg["vocab"], page_size=64)
    ref = {rid: np.stack([out["float32"][rid][p] for p in range(len(t))]) for rid, t in reqs.items()}
    check(out["bfloat16"], ref, reqs, "bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_from_one_token(name, dtype, models, tmp_path):
    """One token of prompt, then 200 tokens one by one: states, the last input and the cache written by single-token
    steps only, with every window passing over decoded tokens and many page borders; pages behind the windows go back
    to the pool meanwhile, those of the kept first keys stay."""
    folder, cfg, w = models[name]
    toks = np.random.default_rng(3).integers(0, cfg["vocab"], 201).tolist()
    reqs = {"long": toks}
    got = tt.run_trace(folder, dtype, tt.decode_tail(reqs, tail=200), str(tmp_path), vocab=cfg["vocab"], page_size=16)
    check(got, {"long": pb.forward(cfg, w, toks).numpy()}, reqs, dtype)


def plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(pb.forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("eager", [True, False])
def test_greedy_generation_through_the_engine(eager, name, models):
    """``LLM.generate`` with more prompts than state slots and a token budget that cuts prompts into portions: the
    scheduler admits, batches, frees and reuses pages and slots; tokens equal the plain model's greedy choice, with
    and without captured decode steps."""
    from nanohybrid_vlm_b200 import LLM, SamplingParams
    folder, cfg, w = models[name]
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (23, 5, 41, 1, 12)]
    llm = LLM(folder, dtype="float32", kvcache_block_size=8, num_kvcache_blocks=40, max_num_batched_tokens=16,
              max_num_seqs=3, max_model_len=64, enforce_eager=eager)
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=7, ignore_eos=True), use_tqdm=False)
    for p, o in zip(prompts, out):
        assert o["token_ids"] == plain_greedy(cfg, w, p, 7)


def test_command_line_generates_the_plain_models_tokens(models):
    """``python -m nanohybrid_vlm_b200.cli generate`` on a Beputar folder: the registry picks the model by config.json."""
    import subprocess
    import sys
    folder, cfg, w = models["C"]
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, cfg["vocab"], n).tolist() for n in (6, 19)]
    args = [sys.executable, "-m", "nanohybrid_vlm_b200.cli", "generate", "--model", folder, "--dtype", "float32",
            "--temperature", "0", "--max-tokens", "5", "--ignore-eos", "--kvcache-block-size", "16", "--num-kvcache-blocks",
            "16", "--max-num-seqs", "2", "--max-model-len", "64", "--max-num-batched-tokens", "32", "--quiet"]
    for p in prompts:
        args += ["--prompt-ids", ",".join(map(str, p))]
    env = dict(os.environ, PYTHONPATH=tt.ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run(args, capture_output=True, text=True, env=env, cwd=tt.ROOT)
    assert r.returncode == 0, r.stderr[-3000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [l["token_ids"] for l in lines] == [plain_greedy(cfg, w, p, 5) for p in prompts]


def test_random_weights_folder_round_trip(tmp_path):
    """The random-weights mode writes a Beputar folder from its configuration that the engine loads and runs."""
    from nanohybrid_vlm_b200.weights import write_random_model
    folder = str(tmp_path / "m")
    write_random_model(folder, dict(BEP_B, dtype="bfloat16"), seed=5)
    reqs = {"a": list(range(40)), "b": [7, 3, 9]}
    out = tmp_path / "o"
    out.mkdir()
    got = tt.run_trace(folder, "bfloat16", tt.mixed(reqs, live=2, first=8), str(out), vocab=BEP_B["vocab"])
    assert all(np.isfinite(row).all() for rows in got.values() for row in rows.values())
