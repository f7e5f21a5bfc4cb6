"""The mechanisms of the Beputar design one at a time: each part or kernel against the plain function of the same
mechanism (float64 on the CPU), in packed batches of unequal requests, in portions down to one token, with pages in a
poisoned pool that is so small that pages and state slots are used again.  Where random numbers would hide a fault (a
key just outside a window, a kept first key hundreds of tokens back, the one more in the denominator, a state that
leaks from the request that held the slot before), the weights or inputs are made so that it shows."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_beputar as pb

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


def make_part(registry, spec, width, dtype, seed, max_position=1024, scale=None):
    """A part with random weights; returns (part, its tensors under the checkpoint's names in float64)."""
    from nanohybrid_vlm_b200.parts import BuildEnv
    env = BuildEnv(width, dtype, "cuda", max_position)
    obj = registry.get(spec.kind)(spec, env)
    g = torch.Generator().manual_seed(seed)
    host, named = {}, {}
    for decl in obj.params():
        if decl.init in ("norm", "layer_scale", "mix_share"):
            t = {"norm": 1.0, "layer_scale": 0.6, "mix_share": 0.5}[decl.init] + 0.3 * torch.randn(decl.shape, generator=g)
        elif len(decl.shape) == 1 or decl.init in ("gate_bias", "unit"):
            t = torch.randn(decl.shape, generator=g)
        else:
            t = torch.randn(decl.shape, generator=g) / math.sqrt(decl.shape[-1])
        for key, factor in (scale or {}).items():
            if decl.name == key:
                t = t * factor
        t = t.to(torch.bfloat16)                        # checkpoints are bfloat16; float32 runs use the same numbers
        host[decl.name] = t.to(torch.float32 if decl.storage == "float32" else dtype)
        for src in decl.resolved_sources():
            piece = t.narrow(src.dim, src.row, src.rows)
            named[src.name] = (piece.squeeze(src.dim) if src.squeeze else piece).to(F64)
    obj.bind({k: v.cuda() for k, v in host.items()})
    return obj, named


class Rig:
    """Cache manager, storage and batch builder for parts tested alone: one run per need, requests by name, a pool
    filled with NaN."""

    def __init__(self, needs, page_size=8, num_pages=64, slots=3, dtype=torch.float32):
        from nanohybrid_vlm_b200.cache import CacheLayout, CacheManager, CacheStorage
        from nanohybrid_vlm_b200.engine.batch import BatchBuilder
        from nanohybrid_vlm_b200.parts import LayerRun
        self.layout = CacheLayout.from_needs(needs)
        self.order = [LayerRun(i) for i in range(len(needs))]
        n_groups = max(1, len(self.layout.groups))
        n_slots = slots if self.layout.needs_state_slots else 0
        self.cm = CacheManager(self.layout.groups, page_size, num_pages, n_slots)
        self.storage = CacheStorage(self.layout, self.order, page_size, [num_pages] * n_groups, n_slots, dtype, "cuda",
                                    poison=True)
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
        return self.storage.view(run, None, batch)

    def after_step(self):
        for rid, n in self.held.items():
            self.cm.release_behind_window(rid, n)

    def free(self, rid):
        self.cm.free(rid)
        del self.held[rid]
        self.cm.check()


def run_through_slots(rig, lengths, cuts, step, live=3):
    """Requests of ``lengths`` cut at ``cuts``, at most ``live`` at a time (the others wait for a slot), through
    ``step(batch, rows)`` with rows = per request of the step (index, start, size); returns each request's outputs."""
    got = [[] for _ in lengths]
    bounds = [[0, *c, L] for L, c in zip(lengths, cuts)]
    waiting, running = list(range(len(lengths))), {}
    while waiting or running:
        while waiting and len(running) < live:
            running[waiting.pop(0)] = 0
        rows = [(r, bounds[r][i], bounds[r][i + 1] - bounds[r][i]) for r, i in sorted(running.items())]
        b = rig.batch([(f"r{r}", s, n) for r, s, n in rows])
        y = step(b, rows)
        at = 0
        for r, s, n in rows:
            got[r].append(y[at:at + n].float().cpu())
            at += n
            running[r] += 1
            if s + n == lengths[r]:
                del running[r]
                rig.free(f"r{r}")
        rig.after_step()
    return [torch.cat(o) for o in got]


LENGTHS = [41, 19, 6, 80, 3]
CUTS = [[2, 3, 20, 37], [18], [1, 2, 3, 4, 5], [16, 17, 33, 64, 79], []]


# ---------------------------------------------------------------- the recurrent mixers
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d,rank,width", [(3, 16, 8, 96), (1, 40, 5, 64), (4, 8, 16, 64), (2, 34, 3, 100), (2, 64, 40, 128),
                                            (1, 130, 7, 72)])
def test_wkv_part_over_portions_and_reused_slots(dtype, H, d, rank, width):
    """Five requests through three state slots in portions of 1, 2 and more tokens: a request that takes over a slot
    starts from zeros and from a zero 'token before'.  The memory after many tokens depends on every earlier one, so a
    token that is lost, doubled or out of order shows at all later positions; the inputs carry an offset, so that a last
    input leaked from another request shows in the mixes."""
    from nanohybrid_vlm_b200.parts import MIXERS, part
    eps = 1e-5
    mixer, w = make_part(MIXERS, part("wkv", num_heads=H, head_dim=d, decay_rank=rank, eps=eps), width, dtype,
                         seed=H * 100 + d, scale={"w0": 0.7, "u": 0.5})
    m = dict(heads=H, dim=d)
    g = torch.Generator().manual_seed(6)
    xs = [(torch.randn(L, width, generator=g) + 0.5).to(dtype) for L in LENGTHS]
    wp = {"m." + k: v for k, v in w.items()}
    wants = [pb.wkv(x.to(F64), m, wp, "m.", eps) for x in xs]
    rig = Rig([mixer.cache_need()], slots=3, dtype=dtype)
    got = run_through_slots(rig, LENGTHS, CUTS, lambda b, rows: mixer.forward(
        dev(torch.cat([xs[r][s:s + n] for r, s, n in rows])), b, rig.view(0, b)))
    for r in range(len(LENGTHS)):
        torch.testing.assert_close(got[r].to(F64), wants[r], **tol(dtype, f32=1e-4, bf16=6e-2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d,dv,width,decay", [(2, 24, 40, 96, [0.55, 0.98]), (1, 16, 8, 64, [1.0]), (4, 8, 24, 64, [0.3, 0.0, 0.9, 0.99]),
                                                (3, 6, 10, 100, [0.5, 0.75, 0.9]), (1, 130, 20, 72, [0.97]), (2, 64, 128, 128, [0.9, 0.95])])
def test_lightning_attention_part_over_portions_and_reused_slots(dtype, H, d, dv, width, decay):
    """The same through the linear attention with a constant decay per head (a decay of one keeps everything, one of
    zero only the current token)."""
    from nanohybrid_vlm_b200.parts import MIXERS, part
    eps = 1e-5
    mixer, w = make_part(MIXERS, part("lightning_attention", num_heads=H, head_dim=d, v_head_dim=dv, decay=tuple(decay), eps=eps),
                         width, dtype, seed=H * 10 + dv)
    m = dict(heads=H, dim=d, vdim=dv, decay=decay)
    g = torch.Generator().manual_seed(7)
    xs = [torch.randn(L, width, generator=g).to(dtype) for L in LENGTHS]
    wp = {"m." + k: v for k, v in w.items()}
    wants = [pb.lightning_attention(x.to(F64), m, wp, "m.", eps) for x in xs]
    rig = Rig([mixer.cache_need()], slots=3, dtype=dtype)
    got = run_through_slots(rig, LENGTHS, CUTS, lambda b, rows: mixer.forward(
        dev(torch.cat([xs[r][s:s + n] for r, s, n in rows])), b, rig.view(0, b)))
    for r in range(len(LENGTHS)):
        torch.testing.assert_close(got[r].to(F64), wants[r], **tol(dtype, f32=1e-4, bf16=6e-2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dk,dv", [(2, 56, 56), (3, 10, 6), (1, 200, 17)])
def test_decay_scan_kernel_both_reads(ops, dtype, H, dk, dv):
    """The recurrence alone, in both forms of its read, one token at a time against whole."""
    g = torch.Generator().manual_seed(dk)
    T = 37
    r, k, v = (torch.randn(T, n, generator=g).to(dtype) for n in (H * dk, H * dk, H * dv))
    w = torch.rand(T, H * dk, generator=g) * 0.5 + 0.5
    u = torch.randn(H * dk, generator=g).to(dtype)
    wh = torch.rand(H, generator=g)
    proj = dev(torch.cat([r, k, v], 1))
    views = (proj[:, :H * dk], proj[:, H * dk:2 * H * dk], proj[:, 2 * H * dk:])
    r64, k64, v64 = (t.to(F64).view(T, H, -1) for t in (r, k, v))
    for read_after in (False, True):
        S = torch.zeros(H, dk, dv, dtype=F64)
        want = torch.zeros(T, H, dv, dtype=F64)
        dec = wh.to(F64)[None, :, None].expand(T, H, dk) if read_after else w.to(F64).view(T, H, dk)
        for t in range(T):
            kv = k64[t][:, :, None] * v64[t][:, None, :]
            if read_after:
                S = dec[t][:, :, None] * S + kv
                want[t] = torch.einsum("hkv,hk->hv", S, r64[t])
            else:
                want[t] = torch.einsum("hkv,hk->hv", S + u.to(F64).view(H, dk, 1) * kv, r64[t])
                S = dec[t][:, :, None] * S + kv
        kw = dict(decay_heads=dev(wh), read_after=True) if read_after else dict(decay_tokens=dev(w), bonus=dev(u))
        state = torch.full((2, H * dk * dv), float("nan"), device="cuda")
        whole = torch.empty(T, H * dv, device="cuda")
        ops.decay_scan(whole, *views, state, step_batch([T], [0], [1]), H, dk, dv, **kw)
        torch.testing.assert_close(whole.cpu().to(F64), want.view(T, H * dv), **tol(dtype, f32=1e-4, bf16=1e-4))
        state2 = torch.full((2, H * dk * dv), float("nan"), device="cuda")
        single = torch.empty(T, H * dv, device="cuda")
        for t in range(T):
            kw_t = dict(kw)
            if not read_after:
                kw_t["decay_tokens"] = kw["decay_tokens"][t:t + 1]
            ops.decay_scan(single[t:t + 1], *(x[t:t + 1] for x in views), state2, step_batch([1], [t], [0]), H, dk, dv, **kw_t)
        torch.testing.assert_close(single, whole, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(state2[0], state[1], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,n_mix", [(96, 5), (100, 1), (520, 3)])
def test_token_shift_mixes_with_reused_slots(ops, dtype, width, n_mix):
    g = torch.Generator().manual_seed(width)
    mu = torch.rand(n_mix, width, generator=g).to(dtype)
    xs = [(torch.randn(L, width, generator=g) + 3).to(dtype) for L in LENGTHS]
    state = torch.full((2, width), float("nan"), device="cuda")
    got = [[] for _ in LENGTHS]
    bounds = [[0, *c, L] for L, c in zip(LENGTHS, CUTS)]
    free, slot_of, waiting, progress = [0, 1], {}, list(range(len(LENGTHS))), {r: 0 for r in range(len(LENGTHS))}
    while waiting or slot_of:
        while waiting and free:
            slot_of[waiting.pop(0)] = free.pop(0)
        who = sorted(slot_of)
        starts = [bounds[r][progress[r]] for r in who]
        news = [bounds[r][progress[r] + 1] - s for r, s in zip(who, starts)]
        x = torch.cat([xs[r][s:s + n] for r, s, n in zip(who, starts, news)])
        out = torch.empty(n_mix, x.shape[0], width, dtype=dtype, device="cuda")
        ops.token_shift_mix(out, dev(x), dev(mu), state, step_batch(news, starts, [slot_of[r] for r in who]))
        at = 0
        for r, s, n in zip(who, starts, news):
            got[r].append(out[:, at:at + n].transpose(0, 1).cpu())
            at += n
            progress[r] += 1
            if s + n == LENGTHS[r]:
                free.append(slot_of.pop(r))
    for r, x in enumerate(xs):
        x64 = x.to(F64)
        before = torch.cat([torch.zeros(1, width, dtype=F64), x64[:-1]])
        want = x64[:, None, :] + (before - x64)[:, None, :] * mu.to(F64)[None]
        torch.testing.assert_close(torch.cat(got[r]).to(F64), want, **tol(dtype, bf16=4e-2))


# ---------------------------------------------------------------- the attention mixers
def left_spec(nq, nkv, d, rot, base, size, keep_first, scale, eps):
    from nanohybrid_vlm_b200.parts import part
    return part("sink_attention", num_heads=nq, num_kv_heads=nkv, head_dim=d, v_head_dim=d, scale=scale,
                position=part("rope_banded", theta=base, rotary_dim=rot), unit_norm_eps=eps, qk_norm_weight=True,
                qk_norm_order="before_rotation", sink=False, sink_constant=0.0, values="keys", window=size,
                keep_first=keep_first, output_gate="sigmoid_head")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rot,size,keep,width,page", [
    (4, 2, 16, 8, 12, 3, 96, 8), (2, 1, 32, 32, 7, 20, 64, 8), (3, 1, 10, 10, 19, 5, 100, 5), (8, 2, 128, 32, 33, 9, 64, 16),
    (4, 4, 64, 64, 40, 1, 64, 16), (2, 2, 8, 2, 5, 0, 64, 4)])
def test_kept_first_attention_part(dtype, nq, nkv, d, rot, size, keep, width, page):
    """Attention that keeps the first keys beside its window, as a part: portions whose edges fall just before, at and
    just behind the window's width and the kept keys' count, pages that the window has passed go back to a pool that
    holds little more than the window, those of the kept keys stay.  The loud key weights make single keys matter."""
    from nanohybrid_vlm_b200.parts import MIXERS
    eps = 1e-5
    mixer, w = make_part(MIXERS, left_spec(nq, nkv, d, rot, 10000.0, size, keep, 0.5, eps), width, dtype, seed=nq + d,
                         scale={"qkv": 2.0})
    m = dict(heads=nq, kv_heads=nkv, dim=d, vdim=d, scale=0.5, rot=dict(base=10000.0, dims=rot),
             mask=dict(size=size, keep_first=keep))
    g = torch.Generator().manual_seed(4)
    lengths = [3 * size + keep + 5, 2, size + 1, 2 * size + keep]
    cuts = [[keep, keep + 1, size - 1, size, size + 1, 2 * size, 3 * size + 3, 3 * size + 4], [1], [size], [3, 5, 2 * size - 1]]
    cuts = [sorted({c for c in cs if 0 < c < L}) for cs, L in zip(cuts, lengths)]
    xs = [torch.randn(L, width, generator=g).to(dtype) for L in lengths]
    wp = {"a." + k: v for k, v in w.items()}
    wants = [pb.kept_first_attention(x.to(F64), m, wp, "a.", eps) for x in xs]
    per_request = -(-size // page) + -(-keep // page) + 3
    rig = Rig([mixer.cache_need()], page_size=page, num_pages=3 * per_request + 2 * (-(-lengths[0] // page)), dtype=dtype)
    got = run_through_slots(rig, lengths, cuts, lambda b, rows: mixer.forward(
        dev(torch.cat([xs[r][s:s + n] for r, s, n in rows])), b, rig.view(0, b)))
    for r in range(len(lengths)):
        torch.testing.assert_close(got[r].to(F64), wants[r], **tol(dtype, f32=5e-5, bf16=5e-2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rot,size,scaling,width,page", [
    (4, 2, 16, 16, 25, (4.0, 16, 4.0, 1.0), 96, 8), (6, 6, 8, 4, None, None, 64, 5), (2, 1, 32, 8, 9, (8.0, 32, 8.0, 2.0), 64, 8),
    (3, 1, 20, 6, 50, (2.0, 40, 16.0, 0.5), 100, 16), (8, 4, 64, 48, 72, (3.0, 512, 16.0, 2.0), 64, 16)])
def test_windowed_attention_part(dtype, nq, nkv, d, rot, size, scaling, width, page):
    """The attention with biases, neighbouring pairs rotated by rescaled frequencies, and a unit norm after the rotation."""
    from nanohybrid_vlm_b200.parts import MIXERS, part
    eps, base = 1e-5, 5000.0
    if scaling is None:
        rope = part("rope_banded", theta=base, rotary_dim=rot)
    else:
        rope = part("rope_ramped", theta=base, rotary_dim=rot, factor=scaling[0], original=float(scaling[1]), fast=scaling[2],
                    slow=scaling[3])
    spec = part("sink_attention", num_heads=nq, num_kv_heads=nkv, head_dim=d, v_head_dim=d, scale=0.4, position=rope,
                rope_layout="interleaved", unit_norm_eps=eps, sink=False, values="keys", bias="qk", window=size)
    mixer, w = make_part(MIXERS, spec, width, dtype, seed=nq * 7 + d)
    assert set(w) == {"q", "k", "q.b", "k.b", "o"}
    rotd = dict(base=base, dims=rot)
    if scaling is not None:
        rotd["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = dict(heads=nq, kv_heads=nkv, dim=d, vdim=d, scale=0.4, rot=rotd, mask=None if size is None else dict(size=size))
    g = torch.Generator().manual_seed(5)
    span = size or 30
    lengths = [3 * span + 5, 2, span + 1, 2 * span]
    cuts = [[span - 1, span, span + 1, 2 * span, 3 * span + 3, 3 * span + 4], [1], [span], [3, 5, 2 * span - 1]]
    cuts = [sorted({c for c in cs if 0 < c < L}) for cs, L in zip(cuts, lengths)]
    xs = [torch.randn(L, width, generator=g).to(dtype) for L in lengths]
    wp = {"a." + k: v for k, v in w.items()}
    wants = [pb.windowed_attention(x.to(F64), m, wp, "a.", eps) for x in xs]
    rig = Rig([mixer.cache_need()], page_size=page, num_pages=5 * (-(-lengths[0] // page)), dtype=dtype)
    got = run_through_slots(rig, lengths, cuts, lambda b, rows: mixer.forward(
        dev(torch.cat([xs[r][s:s + n] for r, s, n in rows])), b, rig.view(0, b)))
    for r in range(len(lengths)):
        torch.testing.assert_close(got[r].to(F64), wants[r], **tol(dtype, f32=5e-5, bf16=5e-2))


def plain_heads(q, k, v, nq, nkv, scale, window, keep_first, extra_one):
    L = q.shape[0]
    seen = pb.visible_keys(torch.arange(L), window, keep_first)
    return pb.grouped_attention(q, k, v, scale, seen, extra_one).reshape(L, -1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("simt", [True, False], ids=["cuda_cores", "dispatcher"])
@pytest.mark.parametrize("nq,nkv,d,page,window,keep", [(4, 2, 16, 8, 24, 5), (8, 2, 128, 16, 80, 7), (2, 2, 64, 16, 40, 33),
                                                       (8, 1, 64, 64, 70, 64), (3, 1, 48, 16, 10, 17), (4, 1, 128, 16, 32, 0),
                                                       (4, 2, 128, 64, 100, 9), (2, 1, 64, 128, 130, 70)])
def test_attention_kernels_keep_first_keys(ops, dtype, simt, nq, nkv, d, page, window, keep, monkeypatch):
    """The attention kernels with kept first keys, in portions and single tokens over a cache whose pages between the kept
    keys and the window are gone (NaN in the pool).  Planted: some queries would, but for the mask, give nearly all
    their weight to the first key that is not kept or to the key just outside their window; the last kept key and the
    first key of the window take a large share; with all scores low the one more in the denominator decides."""
    from nanohybrid_vlm_b200.parts.base import PagedKVNeed
    if simt:
        monkeypatch.setattr(ops, "SINK_ATTENTION_ON_TENSOR_CORES", False)
    g = torch.Generator().manual_seed(window + keep)
    L = 5 * window + keep + 3
    q, k = 0.5 * torch.randn(L, nq, d, generator=g), 0.5 * torch.randn(L, nkv, d, generator=g)
    v = torch.randn(L, nkv, d, generator=g)
    for i in range(window + keep + 1, L, max(3, window // 2 + 1)):
        q[i, :, d - 1] += 4.0
        k[i - window, :, d - 1] += 6.0                  # just outside the window
        k[i - window + 1, :, d - 1] += 3.0              # the first key the window keeps
    k[keep, :, d - 2] += 6.0                            # the first key that is not kept
    if keep:
        k[keep - 1, :, d - 2] += 3.0                    # the last kept key
    q[2 * window::7, :, d - 2] += 4.0
    q[3 * window + 1::11] *= 0.01                       # all scores near zero: the extra one is a large share
    q, k, v = (t.to(dtype) for t in (q, k, v))
    want = plain_heads(q.to(F64), k.to(F64), v.to(F64), nq, nkv, 0.4, window, keep, True)
    rig = Rig([PagedKVNeed(nkv, d, window, keep_first=keep)], page_size=page,
              num_pages=-(-window // page) + -(-keep // page) + -(-L // page) // 2 + 4, dtype=dtype)
    sinks = torch.zeros(nq, device="cuda")
    cuts = sorted({c for c in (keep, keep + 1, window, window + 1, 2 * window + 3, *range(4 * window, L)) if 0 < c < L})
    outs, at = [], 0
    for end in [*cuts, L]:
        b = rig.batch([("r", at, end - at)])
        view = rig.view(0, b)
        pages = view.pages
        slots = view.tables.slot_mapping[:end - at].long()
        pg_, off = slots // page, slots % page
        pages[pg_, 0, :, off] = dev(k[at:end]).to(dtype)
        pages[pg_, 1, :, off] = dev(v[at:end]).to(dtype)
        o = torch.empty(end - at, nq * d, dtype=dtype, device="cuda")
        ops.attention_sink(o, dev(q[at:end].reshape(end - at, nq * d)), pages, view.tables, b, nq, nkv, d, d, 0.4, sinks,
                           window, 0, None, keep)
        outs.append(o.float().cpu())
        rig.after_step()
        at = end
    torch.testing.assert_close(torch.cat(outs).to(F64), want, **tol(dtype, f32=5e-5, bf16=3e-2))


# ---------------------------------------------------------------- position tables
def test_ramped_rotary_table_against_plain():
    from nanohybrid_vlm_b200.parts import POSITIONS, BuildEnv, part
    for dims, base, sc in ((48, 30000.0, (3.0, 512, 16.0, 2.0)), (16, 1000.0, (4.0, 16, 4.0, 1.0)), (6, 20000.0, (2.0, 40, 16.0, 0.5)),
                           (8, 300.0, (8.0, 32, 8.0, 2.0))):
        spec = part("rope_ramped", theta=base, rotary_dim=dims, factor=sc[0], original=float(sc[1]), fast=sc[2], slow=sc[3])
        table, rd = POSITIONS.get("rope_ramped")(spec, BuildEnv(32, torch.float32, "cuda", 300)).rotary()
        freq, mult = pb.yarn_frequencies(dims, base, dict(zip(("factor", "original", "fast", "slow"), sc)))
        ang = torch.arange(300, dtype=F64)[:, None] * freq[None]
        want = torch.cat([ang.cos(), ang.sin()], -1) * mult
        assert rd == dims and 1.0 < mult
        torch.testing.assert_close(table.cpu().to(F64), want, rtol=0, atol=1e-6)


# ---------------------------------------------------------------- output norms onto the stream
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [96, 100, 1032, 4096])
def test_output_norm_adds_onto_the_stream(ops, dtype, width):
    g = torch.Generator().manual_seed(width)
    T, eps = 5, 1e-5
    stream = 3 * torch.randn(T, width, generator=g)
    a, b = (4 * torch.randn(T, width, generator=g)).to(dtype), (0.3 * torch.randn(T, width, generator=g)).to(dtype)
    wa, wb, w, ls = ((1 + 0.3 * torch.randn(width, generator=g)).to(dtype) for _ in range(4))
    s64, a64, b64, wa64, wb64, w64, ls64 = (t.to(F64) for t in (stream, a, b, wa, wb, w, ls))
    cases = [
        ([(a, 1.0, None)], ls, pb.unit_rms(a64, eps) * w64 * ls64),
        ([(a, 1.0, None)], None, pb.unit_rms(a64, eps) * w64),
        ([(a, 0.5, wa), (b, 0.5, wb)], ls,
         pb.unit_rms(0.5 * (pb.unit_rms(a64, eps) * wa64 + pb.unit_rms(b64, eps) * wb64), eps) * w64 * ls64),
    ]
    for terms, scale, add in cases:
        s = dev(stream.clone())
        rounded = torch.empty(T, width, dtype=dtype, device="cuda")
        ops.postnorm_stream(s, rounded, [(dev(t), c, None if x is None else dev(x)) for t, c, x in terms], dev(w),
                            None if scale is None else dev(scale), eps)
        torch.testing.assert_close(s.cpu().to(F64), s64 + add, rtol=2e-6, atol=2e-5)          # the stream stays 32-bit
        assert torch.equal(rounded, s.to(dtype))
    out = torch.empty(T, width, dtype=dtype, device="cuda")
    ops.stream_round(out, dev(stream))
    assert torch.equal(out.cpu(), stream.to(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_gelu_tanh_in_place(ops, dtype):
    g = torch.Generator().manual_seed(2)
    for n in (70, 64):
        y = (3 * torch.randn(6, n, generator=g)).to(dtype)
        z = dev(y.clone())
        ops.gelu_tanh(z)
        torch.testing.assert_close(z.cpu().to(F64), pb.gelu_tanh(y.to(F64)), **tol(dtype))


# ---------------------------------------------------------------- the mixture of experts
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tensor_cores", [True, False])
@pytest.mark.parametrize("E,top,ff,shared,width,T", [(4, 2, 24, 32, 96, 50), (10, 1, 48, 80, 256, 300), (5, 3, 18, None, 100, 33),
                                                     (6, 6, 8, 16, 64, 7), (3, 1, 16, 8, 64, 1), (4, 2, 64, 64, 128, 900)])
def test_sigmoid_router_with_weights_on_the_inputs(ops, dtype, tensor_cores, E, top, ff, shared, width, T, monkeypatch):
    """Sigmoid scores, the largest chosen, each chosen expert fed with score * x, no renormalisation.  The router's
    weights are loud and the inputs' rounding is what both sides see, so that no choice is a close call."""
    from nanohybrid_vlm_b200.parts import FEED_FORWARDS, part
    monkeypatch.setattr(ops, "MOE_ON_TENSOR_CORES", tensor_cores)
    sh = None if shared is None else part("gated_mlp", intermediate_size=shared, activation="silu")
    spec = part("routed_moe", experts=E, top=top, correction=False, scores="sigmoid", renorm=False, weight_on="input",
                intermediate_size=ff, limit=None, alpha=1.0, up_shift=0.0, shared=sh, shared_gate=False)
    ffn, w = make_part(FEED_FORWARDS, spec, width, dtype, seed=E * 10 + top, scale={"router": 3.0})
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, width, generator=g).to(dtype)
    mlp = dict(router=dict(experts=E, top=top), shared=None if shared is None else dict(ff=shared))
    wp = {"f." + k: v for k, v in w.items()}
    want = pb.mixture(x.to(F64), mlp, wp, "f.")
    z = (x.to(F64) @ wp["f.router"].T).sort(-1, descending=True).values          # the order of the logits is the scores'
    sure = (z[:, top - 1] - z[:, top]) > 0.1 if top < E else torch.ones(T, dtype=torch.bool)
    got = ffn.forward(dev(x), None).float().cpu().to(F64)
    assert sure.float().mean() > 0.5
    torch.testing.assert_close(got[sure], want[sure], **tol(dtype, f32=5e-5, bf16=6e-2))
