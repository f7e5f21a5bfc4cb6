"""The mechanisms of the Ginodra design one at a time: each part or kernel against the plain function of the same
mechanism (float64 on the CPU), in packed batches of unequal requests, in portions down to one token, with pages in a
poisoned pool that is so small that pages and state slots are used again.  Where random numbers would hide a fault (a
key just outside a window, a far key among hundreds, a sink that is left out, a filter tap that reaches before the
request's start), the weights or inputs are made so that it shows."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_ginodra as pg

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
F64 = torch.float64


@pytest.fixture(scope="module")
def ops():
    from nanohybrid_vlm_b200.kernels import ops
    return ops


def dev(t):
    return t.cuda()


def i32(x):
    return torch.tensor(x, dtype=torch.int32).cuda()


def tol(dtype, f32=2e-5, bf16=2e-2):
    return dict(rtol=f32, atol=f32) if dtype == torch.float32 else dict(rtol=bf16, atol=bf16)


def step_batch(news, starts, slots):
    cu = [0, *np.cumsum(news).tolist()]
    return SimpleNamespace(cu_q=i32(cu), q_start=i32(starts), state_slots=i32(slots), n_seqs=len(news),
                           n_tokens=int(sum(news)))


def portions_of(lengths, cuts):
    """Step i brings the i-th portion of every request that still has one: (requests, their starts, their sizes)."""
    bounds = [[0, *c, L] for L, c in zip(lengths, cuts)]
    for i in range(max(len(b) for b in bounds) - 1):
        who = [r for r, b in enumerate(bounds) if i + 1 < len(b)]
        yield who, [bounds[r][i] for r in who], [bounds[r][i + 1] - bounds[r][i] for r in who]


def make_part(registry, spec, width, dtype, seed, max_position=1024, scale=None):
    """A part with random weights; returns (part, its tensors under the checkpoint's names in float64)."""
    from nanohybrid_vlm_b200.parts import BuildEnv
    env = BuildEnv(width, dtype, "cuda", max_position)
    obj = registry.get(spec.kind)(spec, env)
    g = torch.Generator().manual_seed(seed)
    host, named = {}, {}
    for decl in obj.params():
        if decl.init == "norm":
            t = 1 + 0.3 * torch.randn(decl.shape, generator=g)
        elif len(decl.shape) == 1 or decl.init in ("gate_bias", "unit", "filter_taps"):
            t = torch.randn(decl.shape, generator=g) * (0.5 if decl.init == "filter_taps" else 1.0)
        else:
            t = torch.randn(decl.shape, generator=g) / math.sqrt(decl.shape[-1])
        if scale and decl.name in scale:
            t = t * scale[decl.name]
        t = t.to(torch.bfloat16)                        # checkpoints are bfloat16; float32 runs use the same numbers
        store = torch.float32 if getattr(decl, "storage", None) == "float32" else dtype
        host[decl.name] = t.to(store)
        for src in (decl.sources or (SimpleNamespace(name=decl.name, row=0, rows=decl.shape[0]),)):
            named[src.name] = t[src.row:src.row + src.rows].to(F64)
    obj.bind({k: v.cuda() for k, v in host.items()})
    return obj, named


class Rig:
    """Cache manager, storage and batch builder for parts tested alone: one run per need, requests by name, a pool
    filled with NaN."""

    def __init__(self, needs, cache_from=None, page_size=8, num_pages=64, slots=3, dtype=torch.float32):
        from nanohybrid_vlm_b200.cache import CacheLayout, CacheManager, CacheStorage
        from nanohybrid_vlm_b200.engine.batch import BatchBuilder
        from nanohybrid_vlm_b200.parts import LayerRun
        self.layout = CacheLayout.from_needs(needs)
        self.order = [LayerRun(i, cache_from=(cache_from or {}).get(i)) for i in range(len(needs))]
        n_groups = max(1, len(self.layout.groups))
        self.cm = CacheManager(self.layout.groups, page_size, num_pages, slots if self.layout.needs_state_slots else 0)
        self.storage = CacheStorage(self.layout, self.order, page_size, [num_pages] * n_groups,
                                    slots if self.layout.needs_state_slots else 0, dtype, "cuda", poison=True)
        self.builder = BatchBuilder(self.cm, 1000, "cuda", 4096, 8, 1024)
        self.held = {}

    def batch(self, items):
        from nanohybrid_vlm_b200.engine.batch import StepItem
        built = []
        for rid, start, n in items:
            self.cm.allocate(rid, start + n)
            self.held[rid] = start + n
            built.append(StepItem(rid, [0] * n, start, []))
        return self.builder.build(built)

    def view(self, run, batch):
        return self.storage.view(run, self.order[run].cache_from, batch)

    def after_step(self):
        for rid, n in self.held.items():
            self.cm.release_behind_window(rid, n)

    def free(self, rid):
        self.cm.free(rid)
        del self.held[rid]
        self.cm.check()


def run_in_steps(rig, lengths, cuts, step, order=None):
    """Run requests of ``lengths`` cut at ``cuts`` through ``step(batch, rows)`` (rows: per request in the batch its
    (request index, start, size)); returns per request the concatenated outputs.  A request is freed when it ends, so
    that a later one gets its pages and slot."""
    outs = [[] for _ in lengths]
    for who, starts, news in portions_of(lengths, cuts):
        b = rig.batch([(f"r{r}", s, n) for r, s, n in zip(who, starts, news)])
        y = step(b, list(zip(who, starts, news)))
        at = 0
        for r, s, n in zip(who, starts, news):
            outs[r].append(y[at:at + n].float().cpu())
            at += n
            if s + n == lengths[r]:
                rig.free(f"r{r}")
        rig.after_step()
    return [torch.cat(o) for o in outs]


# ---------------------------------------------------------------- the norm in groups, over the float32 stream
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,groups", [(96, 3), (100, 5), (1032, 1), (64, 64)])
def test_grouped_norm_over_the_stream(dtype, width, groups):
    from nanohybrid_vlm_b200.parts import NORMS, part
    from nanohybrid_vlm_b200.parts.base import Pending
    norm, w = make_part(NORMS, part("rmsnorm", width=width, eps=1e-5, groups=groups), width, dtype, seed=width)
    g = torch.Generator().manual_seed(1)
    T = 7
    stream = 3 * torch.randn(T, width, generator=g)
    stream[:, :width // groups] *= 50                    # one loud group must not quieten the others
    a, b = (torch.randn(T, width, generator=g).to(dtype) for _ in range(2))
    weight = w["weight"]
    s_dev = dev(stream.clone())
    out = norm.forward_add(Pending(), s_dev)
    torch.testing.assert_close(out.cpu().to(F64), pg.grouped_norm(stream.to(F64), weight, groups, 1e-5), **tol(dtype))
    assert torch.equal(s_dev.cpu(), stream)
    out = norm.forward_add(Pending(((dev(a), 0.5), (dev(b), -1.25))), s_dev)
    summed = stream.to(F64) + 0.5 * a.to(F64) - 1.25 * b.to(F64)
    torch.testing.assert_close(s_dev.cpu().to(F64), summed, rtol=1e-6, atol=1e-5)           # the stream stays 32-bit
    torch.testing.assert_close(out.cpu().to(F64), pg.grouped_norm(summed, weight, groups, 1e-5), **tol(dtype))
    rows = i32([5, 0])
    before = s_dev.clone()
    out = norm.forward_add_rows(Pending(((dev(a), 2.0),)), s_dev, rows)
    want = pg.grouped_norm(summed + 2.0 * a.to(F64), weight, groups, 1e-5)[[5, 0]]
    torch.testing.assert_close(out.cpu().to(F64), want, **tol(dtype))
    assert torch.equal(s_dev, before)


# ---------------------------------------------------------------- input filters over time
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,taps", [(96, 4), (100, 2), (40, 1), (264, 8)])
def test_filter_pair_in_portions_and_reused_slots(ops, dtype, width, taps):
    """Two filters over one input share the state of the last taps - 1 inputs.  Portions shorter than the filter (one and
    two tokens) make a tap reach through several earlier steps; the first tokens of a request must see zeros, not the
    request that held the slot before."""
    g = torch.Generator().manual_seed(taps)
    w1, w2 = (torch.randn(width, taps, generator=g).to(dtype) for _ in range(2))
    lengths = [23, 9, 31, 5, 12]
    cuts = [[1, 2, 4, 11], [3], [16, 17, 19, 20], [], [2, 3]]
    xs = [(torch.randn(L, width, generator=g) + 3).to(dtype) for L in lengths]      # an offset: a leaked input shows
    state = torch.full((2, max(1, (taps - 1) * width)), float("nan"), device="cuda")
    free, slot_of = [0, 1], {}
    got = [[[], []] for _ in lengths]
    waiting = list(range(len(lengths)))
    progress = {r: 0 for r in waiting}
    bounds = [[0, *c, L] for L, c in zip(lengths, cuts)]
    while waiting or slot_of:
        while waiting and free:
            slot_of[waiting.pop(0)] = free.pop(0)
        who = sorted(slot_of)
        starts = [bounds[r][progress[r]] for r in who]
        news = [bounds[r][progress[r] + 1] - s for r, s in zip(who, starts)]
        x = torch.cat([xs[r][s:s + n] for r, s, n in zip(who, starts, news)])
        o1, o2 = (torch.empty(x.shape, dtype=dtype, device="cuda") for _ in range(2))
        ops.causal_filter_add(o1, o2, dev(x), dev(w1), dev(w2), state, step_batch(news, starts, [slot_of[r] for r in who]))
        at = 0
        for r, s, n in zip(who, starts, news):
            got[r][0].append(o1[at:at + n].cpu())
            got[r][1].append(o2[at:at + n].cpu())
            at += n
            progress[r] += 1
            if s + n == lengths[r]:
                free.append(slot_of.pop(r))
    for r, x in enumerate(xs):
        for k, w in enumerate((w1, w2)):
            torch.testing.assert_close(torch.cat(got[r][k]).to(F64), pg.time_filter(x.to(F64), w.to(F64)), **tol(dtype, bf16=4e-2))
    # one filter alone writes the same numbers
    o = torch.empty(xs[0].shape, dtype=dtype, device="cuda")
    ops.causal_filter_add(o, None, dev(xs[0]), dev(w1), None, state, step_batch([lengths[0]], [0], [0]))
    torch.testing.assert_close(o.cpu(), torch.cat(got[0][0]), rtol=0, atol=0)


# ---------------------------------------------------------------- small steps
@pytest.mark.parametrize("dtype", DTYPES)
def test_head_gates_squared_relu_and_capped_logits(ops, dtype):
    g = torch.Generator().manual_seed(5)
    T, H, dv, skip = 6, 5, 12, 3
    x = torch.randn(T, H * dv, generator=g).to(dtype)
    wide = (3 * torch.randn(T, skip + H, generator=g)).to(dtype)
    out = torch.empty(T, H * dv, dtype=dtype, device="cuda")
    ops.sigmoid_mul_heads(out, dev(x), dev(wide)[:, skip:], dv)
    want = (x.to(F64).view(T, H, dv) * torch.sigmoid(wide[:, skip:].to(F64))[:, :, None]).view(T, H * dv)
    torch.testing.assert_close(out.cpu().to(F64), want, **tol(dtype))
    y = dev((2 * torch.randn(T, 70, generator=g)).to(dtype))
    ref = torch.relu(y.cpu().to(F64)) ** 2
    ops.relu_squared(y)
    torch.testing.assert_close(y.cpu().to(F64), ref, **tol(dtype))
    z = 40 * torch.randn(T, 33, generator=g)
    for cap in (15.0, None):
        zz = dev(z.clone())
        ops.scale_softcap(zz, 0.7, cap)
        want = 0.7 * z.to(F64) if cap is None else cap * torch.tanh(0.7 * z.to(F64) / cap)
        torch.testing.assert_close(zz.cpu().to(F64), want, rtol=1e-5, atol=1e-5)


# ---------------------------------------------------------------- attention kernels: window, distance bias, sink, one plane
def plain_heads(q, k, v, nq, nkv, scale, window, slopes, sinks):
    """q [L, nq, dk], k [L, nkv, dk], v [L, nkv, dv] of one request -> [L, nq * dv]."""
    L = q.shape[0]
    i, j = torch.arange(L)[:, None], torch.arange(L)[None, :]
    dist = (i - j).to(F64)
    visible = (dist >= 0) & ((dist < window) if window else torch.ones_like(dist, dtype=torch.bool))
    heads = []
    for a in range(nq):
        kh = a // (nq // nkv)
        s = (q[:, a] @ k[:, kh].T) * scale
        if slopes is not None:
            s = s - float(slopes[a]) * dist
        heads.append(pg.softmax_rows(s, visible, None if sinks is None else sinks[a].to(F64)) @ v[:, kh])
    return torch.cat(heads, -1)


def planted_qk(g, L, nq, nkv, dk, window, dtype):
    """Random queries and keys in which some queries would, but for the mask, give nearly all their weight to one key:
    the key just outside their window; the first key inside it takes a large share; without a window the key at
    position 2, hundreds of tokens back, does."""
    q, k = 0.5 * torch.randn(L, nq, dk, generator=g), 0.5 * torch.randn(L, nkv, dk, generator=g)
    if window:
        for i in range(window, L, max(3, window // 2 + 1)):
            q[i, :, dk - 1] += 4.0
            k[i - window, :, dk - 1] += 6.0             # just outside
            k[i - window + 1, :, dk - 1] += 3.0         # the first key the window keeps
    elif L > 2:
        k[2, :, dk - 1] += 5.0
        q[L - 1, :, dk - 1] += 4.0
        q[L // 2, :, dk - 1] += 4.0
    return q.to(dtype), k.to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("simt", [True, False], ids=["cuda_cores", "dispatcher"])
@pytest.mark.parametrize("nq,nkv,dk,dv,page,window,planes,sink,slope", [
    (4, 2, 16, 24, 8, 12, 2, False, True), (6, 6, 8, 8, 5, 33, 2, False, True), (3, 1, 32, 16, 16, 7, 2, False, True),
    (4, 4, 64, 64, 64, 40, 2, False, True), (8, 2, 128, 128, 64, 100, 2, True, True), (2, 2, 64, 64, 16, 1, 2, False, True),
    (3, 1, 48, 40, 8, 0, 1, True, False), (5, 1, 16, 12, 3, 0, 1, True, False), (2, 1, 80, 64, 64, 0, 1, True, False),
    (4, 1, 24, 24, 16, 9, 1, False, True), (2, 1, 320, 288, 16, 0, 1, True, False), (4, 1, 576, 512, 64, 0, 1, True, False),
    (2, 1, 1040, 1030, 8, 0, 1, False, False), (20, 1, 72, 56, 16, 0, 1, True, False), (16, 1, 32, 32, 4, 0, 1, False, False)])
def test_attention_kernels_in_portions_against_plain(ops, dtype, simt, nq, nkv, dk, dv, page, window, planes, sink, slope):
    """Portions that start and end inside windows and pages, single tokens (a decoded token whose window's edge lies
    on a page border among them), a request of two tokens and one of several hundred; pages in shuffled places of a
    pool of NaN.  One plane: a page row is the key and its leading dv elements are the value (latents)."""
    g = torch.Generator().manual_seed(nq * 10 + dk)
    w = window or 40
    lengths = [3 * w + 5, w + 1, 2, 2 * w, 300 if not window else 2 * w + 3]
    cuts = [[w - 1, w, w + 1, 2 * w - 2, 2 * w - 1, 2 * w, 3 * w + 4], [w], [1], [3, 5, max(6, w - 1), 2 * w - 1],
            [lengths[4] - 3, lengths[4] - 2, lengths[4] - 1]]
    cuts = [sorted({c for c in cs if 0 < c < L}) for cs, L in zip(cuts, lengths)]
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / nq) for h in range(nq)]) if slope else None
    sinks = 2 + torch.randn(nq, generator=g) if sink else None
    scale = 0.3
    row = max(dk, dv) if planes == 2 else dk
    n_pages = sum(-(-L // page) for L in lengths) + 3
    pages = torch.full((n_pages, planes, nkv, page, row), float("nan"), dtype=dtype, device="cuda")
    perm = torch.randperm(n_pages, generator=g).tolist()
    qs, wants, tables = [], [], []
    for L in lengths:
        q, k = planted_qk(g, L, nq, nkv, dk, window, dtype)
        v = k[..., :dv] if planes == 1 else torch.randn(L, nkv, dv, generator=g).to(dtype)
        mine = [perm.pop() for _ in range(-(-L // page))]
        for t in range(L):
            pages[mine[t // page], 0, :, t % page, :dk] = dev(k[t])
            if planes == 2:
                pages[mine[t // page], 1, :, t % page, :dv] = dev(v[t])
        qs.append(q)
        tables.append(mine)
        wants.append(plain_heads(q.to(F64), k.to(F64), v.to(F64), nq, nkv, scale, window, slopes, sinks))
    width = max(len(t) for t in tables)
    got = [torch.zeros(L, nq * dv) for L in lengths]
    for who, starts, news in portions_of(lengths, cuts):
        q = torch.cat([qs[r][s:s + n] for r, s, n in zip(who, starts, news)]).reshape(-1, nq * dk)
        bt = torch.tensor([tables[r] + [-1] * (width - len(tables[r])) for r in who], dtype=torch.int32)
        out = torch.full((q.shape[0], nq * dv), float("nan"), dtype=dtype, device="cuda")
        b = step_batch(news, starts, [-1] * len(who))
        b.kv_len = i32([s + n for s, n in zip(starts, news)])
        b.n_prefill_tokens = sum(n for n in news if n > 1)
        b.n_prefill_seqs = sum(1 for n in news if n > 1)
        b.n_decode_seqs = sum(1 for n in news if n == 1)
        b.max_kv_len = max(s + n for s, n in zip(starts, news))
        if simt:
            ops.attention_sink_simt(out, dev(q), pages, dev(bt), b.cu_q, b.kv_len, len(who), q.shape[0], nq, nkv, dk, dv,
                                    scale, None if sinks is None else dev(sinks), window, 0,
                                    None if slopes is None else dev(slopes))
        elif planes == 1 and not window and slopes is None:     # latents: the tensor-core kernel where the sizes allow it
            ops.latent_attention(out, dev(q), pages, SimpleNamespace(block_tables=dev(bt)), b, nq, dv, dk, scale,
                                 None if sinks is None else dev(sinks))
        else:       # the dispatcher: the tensor-core kernels where the shape allows them
            ops.attention_sink(out, dev(q), pages, SimpleNamespace(block_tables=dev(bt)), b, nq, nkv, dk, dv, scale,
                               None if sinks is None else dev(sinks), window, 0, None if slopes is None else dev(slopes))
        at = 0
        for r, s, n in zip(who, starts, news):
            got[r][s:s + n] = out[at:at + n].float().cpu()
            at += n
    for r in range(len(lengths)):
        # bfloat16: a planted score carries the rounding of its query and key, so a weight is off by up to a few
        # percent; a key that is wrongly seen or missed moves the outputs by whole units
        torch.testing.assert_close(got[r].to(F64), wants[r], **(tol(dtype) if dtype == torch.float32 else dict(rtol=5e-2, atol=8e-2)))


# ---------------------------------------------------------------- the mixers as parts, with the engine's cache
def latent_spec(H, dn, dr, dv, q_rank, rank, base, scale, eps, sink=True):
    from nanohybrid_vlm_b200.parts import part
    rope = part("rope_banded", theta=base, rotary_dim=dr) if dr else None
    return part("latent_attention", num_heads=H, head_dim=dn, rot_dim=dr, v_head_dim=dv, q_rank=q_rank, kv_rank=rank,
                scale=scale, position=rope, eps=eps, sink=sink, output_gate="sigmoid_head")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dn,dr,dv,q_rank,rank,width,page", [
    (3, 24, 8, 20, 48, 40, 96, 8), (5, 8, 4, 8, 16, 12, 64, 5), (2, 16, 16, 32, 24, 64, 80, 16), (3, 10, 6, 14, 18, 22, 100, 3),
    (1, 64, 32, 64, 96, 128, 128, 64), (2, 32, 32, 48, 64, 272, 128, 16), (20, 16, 8, 16, 32, 48, 64, 16)])
@pytest.mark.parametrize("form", ["expanded_prompts", "latents_tensor_cores", "latents_cuda_cores"])
def test_latent_attention_part(ops, dtype, form, H, dn, dr, dv, q_rank, rank, width, page, monkeypatch):
    """Whole against portions in unequal batches, in a pool that only holds what is live.  The sinks are large, so a
    sink that is left out, counted per key or scaled moves every output.  In bfloat16 a step with prompt portions
    expands the latents into keys and values per head for the tensor-core kernels (single tokens of the same step
    ride along), a step of single tokens attends over the latents, on the tensor cores (a token's keys cut into
    pieces that are merged) or the CUDA cores; every form is run for every step shape."""
    from nanohybrid_vlm_b200.parts import MIXERS
    from nanohybrid_vlm_b200.parts import latent_attention as la
    monkeypatch.setattr(la, "EXPAND_PROMPT_PORTIONS", form == "expanded_prompts")
    monkeypatch.setattr(ops, "LATENTS_ON_TENSOR_CORES", form != "latents_cuda_cores")
    eps, base, scale = 1e-5, 5000.0, 0.2
    mixer, w = make_part(MIXERS, latent_spec(H, dn, dr, dv, q_rank, rank, base, scale, eps), width, dtype, seed=H * 7 + dn,
                         scale={"sink": 2.0})
    m = dict(heads=H, dim=dn, rot_dim=dr, vdim=dv, kv_rank=rank, q_rank=q_rank, scale=scale, rot=dict(dims=dr, base=base))
    g = torch.Generator().manual_seed(3)
    lengths = [70, 2, 33, 130, 9]
    cuts = [[13, 15, 16, 40, 69], [1], [32], [64, 65, 127, 128, 129], []]
    xs = [torch.randn(L, width, generator=g).to(dtype) for L in lengths]
    wp = {"m." + k: v for k, v in w.items()}
    wants = [pg.latent_attention(x.to(F64), m, wp, "m.", eps) for x in xs]
    live = -(-70 // page) + 1 + -(-33 // page) + -(-130 // page) + -(-9 // page)
    rig = Rig([mixer.cache_need()], page_size=page, num_pages=live, dtype=dtype)

    def step(b, rows):
        x = torch.cat([xs[r][s:s + n] for r, s, n in rows])
        return mixer.forward(dev(x), b, rig.view(0, b))

    got = run_in_steps(rig, lengths, cuts, step)
    again = run_in_steps(rig, lengths[:3], [[], [], []], step)           # the freed pages, whole this time
    for r in range(len(lengths)):
        torch.testing.assert_close(got[r].to(F64), wants[r], **tol(dtype, f32=5e-5, bf16=4e-2))
    for r in range(3):
        torch.testing.assert_close(again[r].to(F64), wants[r], **tol(dtype, f32=5e-5, bf16=4e-2))


def window_spec(nq, nkv, d, dv, window, keep, scale, eps, own=True):
    from nanohybrid_vlm_b200.parts import part
    return part("sink_attention", num_heads=nq, num_kv_heads=nkv, head_dim=d, v_head_dim=dv, scale=scale, position=None,
                unit_norm_eps=eps, sink=False, window=window, keep_window=keep, qk_norm_weight=True,
                distance_slope_base=8.0, output_gate="sigmoid_head", own_kv=own)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,dv,w_own,w_other,width,page", [
    (4, 2, 16, 24, 12, 25, 96, 8), (6, 6, 8, 8, 33, 9, 64, 5), (3, 1, 20, 10, 50, 50, 100, 16), (4, 4, 64, 64, 40, 17, 128, 64)])
def test_window_attention_parts_share_pages(dtype, nq, nkv, d, dv, w_own, w_other, width, page):
    """A layer with keys of its own and one that reads them through another window (wider or narrower) with its own
    queries, norm weight, gate and scale.  The pages keep the wider of the two windows and go back to the pool
    behind it; the pool holds little more than that."""
    from nanohybrid_vlm_b200.parts import MIXERS
    from nanohybrid_vlm_b200.parts.base import with_shared_pages
    eps, keep = 1e-5, max(w_own, w_other)
    owner, wo = make_part(MIXERS, window_spec(nq, nkv, d, dv, w_own, keep, 0.3, eps), width, dtype, seed=nq + d)
    reader, wr = make_part(MIXERS, window_spec(nq, nkv, d, dv, w_other, keep, 0.2, eps, own=False), width, dtype, seed=nq + d + 1)
    assert set(wr) == {"q", "q.norm", "g", "o"}
    mo = dict(heads=nq, kv_heads=nkv, dim=d, vdim=dv, scale=0.3, mask=dict(size=w_own))
    mr = dict(mo, scale=0.2, mask=dict(size=w_other))
    g = torch.Generator().manual_seed(4)
    lengths = [3 * keep + 5, 2, keep + 1, 2 * keep]
    cuts = [[keep - 1, keep, keep + 1, 2 * keep, 3 * keep + 3, 3 * keep + 4], [1], [keep], [3, 5, 2 * keep - 1]]
    cuts = [sorted({c for c in cs if 0 < c < L}) for cs, L in zip(cuts, lengths)]
    xs = [(torch.randn(L, width, generator=g).to(dtype), torch.randn(L, width, generator=g).to(dtype)) for L in lengths]
    w1 = {"a." + k: v for k, v in wo.items()}
    w2 = {"b." + k: v for k, v in wr.items()}
    want1 = [pg.window_attention(x.to(F64), mo, w1, "a.", eps) for x, _ in xs]
    want2 = [pg.window_attention(y.to(F64), mr, w2, "b.", eps, kv=pg.window_keys(x.to(F64), mo, w1, "a.", eps)) for x, y in xs]
    rig = Rig([owner.cache_need(), with_shared_pages(reader.cache_need())], cache_from={1: 0}, page_size=page,
              num_pages=4 * (-(-keep // page) + 2) + 2 * (-(-keep // page)), dtype=dtype)

    def step(b, rows):
        x = torch.cat([xs[r][0][s:s + n] for r, s, n in rows])
        y = torch.cat([xs[r][1][s:s + n] for r, s, n in rows])
        return torch.cat([owner.forward(dev(x), b, rig.view(0, b)), reader.forward(dev(y), b, rig.view(1, b))], 1)

    got = run_in_steps(rig, lengths, cuts, step)
    for r in range(len(lengths)):
        torch.testing.assert_close(got[r][:, :width].to(F64), want1[r], **tol(dtype, f32=5e-5, bf16=4e-2))
        torch.testing.assert_close(got[r][:, width:].to(F64), want2[r], **tol(dtype, f32=5e-5, bf16=4e-2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d,rank,width", [(3, 16, 8, 96), (1, 40, 5, 64), (4, 8, 16, 64), (2, 34, 3, 100), (2, 64, 40, 128),
                                            (1, 130, 7, 72)])
def test_general_delta_part_over_portions_and_reused_slots(dtype, H, d, rank, width):
    """Five requests through three state slots in portions of 1, 2 and more tokens: a request that takes over a slot
    starts from zeros.  The state after many tokens depends on every earlier one, so a token that is lost, doubled or
    out of order shows at all later positions."""
    from nanohybrid_vlm_b200.parts import MIXERS, part
    eps = 1e-5
    mixer, w = make_part(MIXERS, part("general_delta_rule", num_heads=H, head_dim=d, decay_rank=rank, eps=eps), width, dtype,
                         seed=H * 100 + d)
    m = dict(heads=H, dim=d, decay_rank=rank)
    g = torch.Generator().manual_seed(6)
    lengths = [41, 19, 6, 80, 3]
    cuts = [[2, 3, 20, 37], [18], [1, 2, 3, 4, 5], [16, 17, 33, 64, 79], []]
    xs = [torch.randn(L, width, generator=g).to(dtype) for L in lengths]
    wp = {"m." + k: v for k, v in w.items()}
    wants = [pg.general_delta(x.to(F64), m, wp, "m.", eps) for x in xs]
    rig = Rig([mixer.cache_need()], slots=3, dtype=dtype)
    got = [[] for _ in lengths]
    bounds = [[0, *c, L] for L, c in zip(lengths, cuts)]
    waiting, running = list(range(len(lengths))), {}
    while waiting or running:
        while waiting and len(running) < 3:
            running[waiting.pop(0)] = 0
        rows = [(r, bounds[r][i], bounds[r][i + 1] - bounds[r][i]) for r, i in sorted(running.items())]
        b = rig.batch([(f"r{r}", s, n) for r, s, n in rows])
        y = mixer.forward(dev(torch.cat([xs[r][s:s + n] for r, s, n in rows])), b, rig.view(0, b))
        at = 0
        for r, s, n in rows:
            got[r].append(y[at:at + n].float().cpu())
            at += n
            running[r] += 1
            if s + n == lengths[r]:
                del running[r]
                rig.free(f"r{r}")
    for r in range(len(lengths)):
        torch.testing.assert_close(torch.cat(got[r]).to(F64), wants[r], **tol(dtype, f32=1e-4, bf16=5e-2))
