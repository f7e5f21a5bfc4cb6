"""Tensor-level wrappers of the CUDA entry points.

Each wrapper checks what its kernel assumes (device, dtype, contiguity, sizes) and then
launches on the current CUDA stream.  Outputs are passed in by the caller, so a step can
run from preallocated buffers.  bfloat16 matrix products go to cuBLAS through
``torch.mm`` (the reference's own projections are library calls too,
nanovllm/layers/linear.py:66); float32 products use this library's fixed-order kernel so
that the 32-bit path never sees a reduced-precision matrix mode.
"""
from __future__ import annotations

import os
import weakref

import torch

from . import attention_decode, attention_mma, attention_tcgen05, library
from .library import KernelError, call

F32, BF16 = 0, 1


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}")


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("this engine computes on the GPU only: got a CPU tensor (there is no CPU fallback)")


def _contig(name: str, t: torch.Tensor) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _ptr(t):
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def embed(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
    _need_cuda(out, table, ids)
    _contig("out", out); _contig("table", table)
    assert ids.dtype == torch.int32 and out.dtype == table.dtype and out.shape[1] == table.shape[1]
    call("nhv_embed", dtype_code(out), out.data_ptr(), table.data_ptr(), ids.data_ptr(), ids.numel(),
         table.shape[1], table.shape[0], stream_ptr())


def feed_tokens(token_ids, feed_src, chosen, vocab: int) -> None:
    """token_ids[t] = chosen[feed_src[t]] where feed_src[t] >= 0 (tokens that the step before chose, taken on the
    device); the other entries keep what the host wrote."""
    _need_cuda(token_ids, feed_src, chosen)
    assert token_ids.dtype == feed_src.dtype == chosen.dtype == torch.int32 and feed_src.numel() >= token_ids.numel()
    call("nhv_feed_tokens", token_ids.data_ptr(), feed_src.data_ptr(), chosen.data_ptr(), token_ids.numel(), chosen.numel(),
         int(vocab), stream_ptr())


def rmsnorm(out, x, weight, eps: float, residual=None, rows=None, write_residual: bool = True,
            weight_offset: float = 0.0) -> None:
    """out[r] = norm(x[src] (+ residual[src])) * (weight + weight_offset), src = rows[r] or r.
    With a residual and write_residual the rounded sum replaces residual[src]."""
    _need_cuda(out, x, weight, residual, rows)
    _contig("out", out); _contig("x", x)
    width = x.shape[-1]
    assert weight.numel() == width and weight.dtype == x.dtype and out.dtype == x.dtype
    n_rows = rows.numel() if rows is not None else x.numel() // width
    assert out.numel() == n_rows * width
    if residual is not None:
        _contig("residual", residual)
        assert residual.shape == x.shape and residual.dtype == x.dtype
    if rows is not None:
        assert rows.dtype == torch.int32
    call("nhv_rmsnorm", dtype_code(x), out.data_ptr(), x.data_ptr(), _ptr(residual), weight.data_ptr(), _ptr(rows),
         n_rows, width, float(eps), int(bool(write_residual and residual is not None and rows is None)),
         float(weight_offset), stream_ptr())


def silu_mul(out, gate_up) -> None:
    _need_cuda(out, gate_up)
    _contig("out", out); _contig("gate_up", gate_up)
    inter = gate_up.shape[-1] // 2
    assert gate_up.shape[-1] == 2 * inter and out.shape[-1] == inter and out.dtype == gate_up.dtype
    call("nhv_silu_mul", dtype_code(out), out.data_ptr(), gate_up.data_ptr(), out.numel() // inter, inter, stream_ptr())


def gelu_tanh_mul(out, gate_up) -> None:
    """out = gelu_tanh(gate) * up for gate_up [n, 2 * inter] with the gate in the first half of each row."""
    _need_cuda(out, gate_up)
    _contig("out", out); _contig("gate_up", gate_up)
    inter = gate_up.shape[-1] // 2
    assert gate_up.shape[-1] == 2 * inter and out.shape[-1] == inter and out.dtype == gate_up.dtype
    call("nhv_gelu_tanh_mul", dtype_code(out), out.data_ptr(), gate_up.data_ptr(), out.numel() // inter, inter, stream_ptr())


def embed_scaled_f32(out, table, ids, scale: float) -> None:
    """out [T, width] float32 = table[ids] * scale: the start of a residual stream kept in 32-bit."""
    _need_cuda(out, table, ids)
    _contig("out", out); _contig("table", table)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and out.shape[1] == table.shape[1]
    call("nhv_embed_scaled_f32", dtype_code(table), out.data_ptr(), table.data_ptr(), ids.data_ptr(), ids.numel(),
         table.shape[1], table.shape[0], float(scale), stream_ptr())


def rmsnorm_stream(out, stream, weight, eps: float, addends=(), rows=None, write_stream: bool = True,
                   weight_offset: float = 0.0, groups: int = 1) -> None:
    """The norm over a float32 residual stream [T, width]: s = stream[src] + sum(coef * tensor[src]) in 32-bit over up
    to three ``addends`` (tensor in the storage type, coef), written back to the stream unless ``rows`` gathers, and
    out[r] = s / rms(s) * (weight + weight_offset) rounded once to the storage type; src = rows[r] or r.  ``groups``
    > 1: the row is cut into that many equal consecutive parts, each divided by its own root mean square."""
    tensors = [t for t, _ in addends]
    _need_cuda(out, stream, weight, rows, *tensors)
    _contig("out", out); _contig("stream", stream)
    width = stream.shape[-1]
    assert stream.dtype == torch.float32 and weight.numel() == width and weight.dtype == out.dtype
    if len(addends) > 3:
        raise KernelError("the stream norm adds at most three tensors")
    for t in tensors:
        _contig("addend", t)
        assert t.shape == stream.shape and t.dtype == out.dtype
    n_rows = rows.numel() if rows is not None else stream.numel() // width
    assert out.numel() == n_rows * width and (rows is None or rows.dtype == torch.int32)
    ptrs = [t.data_ptr() for t in tensors] + [None] * (3 - len(tensors))
    coefs = [float(c) for _, c in addends] + [0.0] * (3 - len(tensors))
    call("nhv_rmsnorm_stream", dtype_code(out), out.data_ptr(), *ptrs, *coefs, stream.data_ptr(), weight.data_ptr(),
         _ptr(rows), n_rows, width, float(eps), int(bool(write_stream and tensors and rows is None)),
         float(weight_offset), int(groups), stream_ptr())


def scaled_sum(out, a, b, ca: float, cb: float) -> None:
    """out = ca * a + cb * b elementwise (sums in 32-bit)."""
    _need_cuda(out, a, b)
    _contig("out", out); _contig("a", a); _contig("b", b)
    assert out.shape == a.shape == b.shape and out.dtype == a.dtype == b.dtype
    call("nhv_scaled_sum", dtype_code(out), out.data_ptr(), a.data_ptr(), b.data_ptr(), float(ca), float(cb), out.numel(),
         stream_ptr())


def short_conv_silu(out, x, weight, bias, state, batch) -> None:
    """out [T, C] = silu(causal convolution over time of x [T, C] (a view with unit column stride) with weight [C, K]
    (+ bias)); ``state`` [slots, (K - 1) * C] float32 holds each request's last K - 1 inputs and is moved on.  ``out`` is
    of x's type, or float32 (for a recurrence that reads it next)."""
    _need_cuda(out, x, weight, bias, state)
    C, K = weight.shape
    assert x.dim() == 2 and x.shape[1] == C and x.stride(1) == 1 and out.shape == x.shape and out.stride(1) == 1
    assert x.dtype == weight.dtype and out.dtype in (x.dtype, torch.float32) and weight.is_contiguous()
    assert state.dtype == torch.float32
    assert state.dim() == 2 and state.stride(1) == 1 and (bias is None or (bias.dtype == x.dtype and bias.numel() == C))
    call("nhv_short_conv_silu", dtype_code(x), dtype_code(out), out.data_ptr(), out.stride(0), x.data_ptr(), x.stride(0), weight.data_ptr(),
         _ptr(bias), state.data_ptr(), state.stride(0), batch.cu_q.data_ptr(), batch.q_start.data_ptr(),
         batch.state_slots.data_ptr(), batch.n_seqs, x.shape[0], C, K, stream_ptr())


SCAN_COLUMNS = 0    # columns of a scan's state per lane: 0 is the kernel's choice; tests set 1, 2, 4
SCAN_GROUP4 = -1    # the delta rule's scan four tokens per round of its chain: -1 is the kernel's choice (off); tests set 1
SCAN_LANES = 0      # lanes per state column in the recurrent scans: 0 is the kernels' own choice; tests set 4, 8, 16, 32


def delta_rule(o, qkv, ba, a_log, dt_bias, state, batch, G: int, H: int, d: int, dv: int) -> None:
    """The gated delta rule over the step's tokens.  qkv [T, 2*G*d + H*dv] (q, k, v after their convolutions), ba
    [T, 2*H] float32 (inputs of beta's sigmoid, then of the decay's softplus), a_log / dt_bias [H] float32, state
    [slots, H*dv*d] float32 -> o [T, H*dv] float32 (before its norm and gate)."""
    _need_cuda(o, qkv, ba, a_log, dt_bias, state)
    T = qkv.shape[0]
    assert qkv.stride(1) == 1 and qkv.shape[1] == 2 * G * d + H * dv
    assert o.dtype == ba.dtype == a_log.dtype == dt_bias.dtype == state.dtype == torch.float32
    assert o.is_contiguous() and o.shape == (T, H * dv) and ba.is_contiguous() and ba.shape == (T, 2 * H)
    scratch = torch.empty(T * (2 * G * d + 9 * G + H * dv + 2 * H), dtype=torch.float32, device=qkv.device)
    at, ptrs = 0, []
    # qn, kn, v32, pairs (16-byte aligned for d, dv in steps of 4), then kq, beta, decay
    for n in (T * G * d, T * G * d, T * H * dv, T * G * 8, T * G, T * H, T * H):
        ptrs.append(scratch.data_ptr() + 4 * at)
        at += n
    qn, kn, v32, pairs, kq, beta, decay = ptrs
    call("nhv_delta_rule", dtype_code(qkv), o.data_ptr(), qkv.data_ptr(), qkv.stride(0), ba.data_ptr(), a_log.data_ptr(),
         dt_bias.data_ptr(), state.data_ptr(), state.stride(0), qn, kn, kq, v32, beta, decay, batch.cu_q.data_ptr(),
         batch.q_start.data_ptr(), batch.state_slots.data_ptr(), batch.n_seqs, T, G, H, d, dv, SCAN_LANES, SCAN_GROUP4, pairs,
         SCAN_COLUMNS, stream_ptr())


def ssd_scan(y, xbc, dt_raw, dt_bias, a_log, d_skip, state, batch, H: int, P: int, N: int, G: int) -> None:
    """The Mamba-2 recurrence over the step's tokens.  xbc [T, H*P + 2*G*N] (x, B, C after the convolution), dt_raw
    [T, H] float32 (before bias and softplus), state [slots, H*P*N] float32 -> y [T, H*P] float32."""
    _need_cuda(y, xbc, dt_raw, dt_bias, a_log, d_skip, state)
    T = xbc.shape[0]
    assert xbc.stride(1) == 1 and xbc.shape[1] == H * P + 2 * G * N and dt_raw.stride(1) == 1 and dt_raw.shape == (T, H)
    assert y.dtype == dt_raw.dtype == dt_bias.dtype == a_log.dtype == d_skip.dtype == state.dtype == torch.float32
    assert y.is_contiguous() and y.shape == (T, H * P)
    call("nhv_ssd_scan", dtype_code(xbc), y.data_ptr(), xbc.data_ptr(), xbc.stride(0), dt_raw.data_ptr(), dt_raw.stride(0),
         dt_bias.data_ptr(), a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(), state.stride(0), batch.cu_q.data_ptr(),
         batch.q_start.data_ptr(), batch.state_slots.data_ptr(), batch.n_seqs, T, H, P, N, G, SCAN_LANES,
         SCAN_COLUMNS, stream_ptr())


def gated_rmsnorm(out, y, z, weight, n_groups: int, eps: float, gate_first: bool, gate: str = "silu") -> None:
    """y [T, n_groups * size] float32, gate z [T, same] (a view with unit column stride), weight of any length that
    divides the row (indexed by column mod its length).  gate_first: out = unit_rms(y * silu(z)) * weight per group;
    else out = unit_rms(y) * weight * silu(z).  ``gate`` "sigmoid" puts sigmoid(z) in the place of silu(z)."""
    assert gate in ("silu", "sigmoid")
    _need_cuda(out, y, z, weight)
    T, width = y.shape
    assert y.dtype == torch.float32 and y.is_contiguous() and width % n_groups == 0
    assert z.shape == y.shape and z.stride(1) == 1 and out.shape == y.shape and out.stride(1) == 1
    assert out.dtype == z.dtype == weight.dtype and width % weight.numel() == 0
    call("nhv_gated_rmsnorm", dtype_code(out), out.data_ptr(), out.stride(0), y.data_ptr(), z.data_ptr(), z.stride(0),
         weight.data_ptr(), weight.numel(), T, n_groups, width // n_groups, float(eps), int(bool(gate_first)),
         1 if gate == "sigmoid" else 0, stream_ptr())


def dyntanh(out, x, alpha, weight, bias) -> None:
    """out = tanh(alpha * x) * weight + bias (Dynamic Tanh), elementwise over rows of ``weight.numel()`` elements, computed
    in 32-bit.  ``x`` and ``out`` are each float32 or of the parameters' type; ``alpha`` has one element."""
    _need_cuda(out, x, alpha, weight, bias)
    _contig("out", out); _contig("x", x)
    width = weight.numel()
    assert alpha.numel() == 1 and bias.numel() == width and alpha.dtype == weight.dtype == bias.dtype
    assert x.dtype in (torch.float32, weight.dtype) and out.dtype in (torch.float32, weight.dtype) and out.numel() == x.numel()
    call("nhv_dyntanh", dtype_code(weight), int(x.dtype == torch.float32), int(out.dtype == torch.float32), out.data_ptr(),
         x.data_ptr(), alpha.data_ptr(), weight.data_ptr(), bias.data_ptr(), x.numel() // width, width, stream_ptr())


def embed_dyntanh(out, table, ids, alpha, weight, bias) -> None:
    """out [T, width] float32 = tanh(alpha * table[ids]) * weight + bias: the looked-up rows through a Dynamic Tanh norm,
    as the start of a residual stream kept in 32-bit."""
    _need_cuda(out, table, ids, alpha, weight, bias)
    _contig("out", out); _contig("table", table)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and out.shape[1] == table.shape[1] == weight.numel()
    assert alpha.dtype == weight.dtype == bias.dtype == table.dtype
    call("nhv_embed_dyntanh", dtype_code(table), out.data_ptr(), table.data_ptr(), ids.data_ptr(), alpha.data_ptr(),
         weight.data_ptr(), bias.data_ptr(), ids.numel(), table.shape[1], table.shape[0], stream_ptr())


def dyntanh_stream(out, stream, pre, addend=None, post=None, rows=None, write_stream: bool = True) -> None:
    """The Dynamic Tanh norm over a float32 residual stream [T, width], with the add of the sub-block before it:
    s = stream[src] + (tanh(post.alpha * addend[src]) * post.w + post.b, if there is an addend), written back to the
    stream unless ``rows`` gathers; out[r] = tanh(pre.alpha * s) * pre.w + pre.b rounded once; src = rows[r] or r.
    ``pre`` / ``post``: (alpha, weight, bias) tensors in the storage type."""
    tensors = [*pre, *(post or ())]       # post None: the addend is added as it is
    _need_cuda(out, stream, addend, rows, *tensors)
    _contig("out", out); _contig("stream", stream)
    width = stream.shape[-1]
    assert stream.dtype == torch.float32 and all(t.dtype == out.dtype for t in tensors)
    assert pre[0].numel() == 1 and pre[1].numel() == pre[2].numel() == width
    if addend is not None:
        _contig("addend", addend)
        assert addend.shape == stream.shape and addend.dtype == out.dtype
        assert post is None or (post[0].numel() == 1 and post[1].numel() == post[2].numel() == width)
    n_rows = rows.numel() if rows is not None else stream.numel() // width
    assert out.numel() == n_rows * width and (rows is None or rows.dtype == torch.int32)
    pp = post if addend is not None and post is not None else (None, None, None)
    call("nhv_dyntanh_stream", dtype_code(out), out.data_ptr(), stream.data_ptr(), _ptr(addend), _ptr(pp[0]), _ptr(pp[1]),
         _ptr(pp[2]), pre[0].data_ptr(), pre[1].data_ptr(), pre[2].data_ptr(), _ptr(rows), n_rows, width,
         int(bool(write_stream and addend is not None and rows is None)), stream_ptr())


def causal_filter_add(out1, out2, x, w1, w2, state, batch) -> None:
    """out1 [T, C] = x + (causal filter over time of x with w1 [C, K], no bias, no activation); out2 likewise with w2
    (both None: one filter).  ``state`` [slots, (K - 1) * C] float32 holds each request's last K - 1 inputs, serves both
    filters and is moved on."""
    _need_cuda(out1, out2, x, w1, w2, state)
    C, K = w1.shape
    assert x.dim() == 2 and x.shape[1] == C and x.is_contiguous() and out1.shape == x.shape and out1.is_contiguous()
    assert x.dtype == w1.dtype == out1.dtype and w1.is_contiguous() and (out2 is None) == (w2 is None)
    assert out2 is None or (out2.shape == x.shape and out2.is_contiguous() and out2.dtype == x.dtype
                            and w2.shape == w1.shape and w2.dtype == w1.dtype and w2.is_contiguous())
    assert K == 1 or (state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1)
    call("nhv_causal_filter_add", dtype_code(x), out1.data_ptr(), _ptr(out2), C, x.data_ptr(), C, w1.data_ptr(), _ptr(w2),
         _ptr(state) if K > 1 else None, state.stride(0) if K > 1 else 0, batch.cu_q.data_ptr(), batch.q_start.data_ptr(),
         batch.state_slots.data_ptr(), batch.n_seqs, x.shape[0], C, K, stream_ptr())


def latent_rope_store(kv, q, q_lat, pages, slot_mapping, positions, cos_sin, rotary_dim: int, H: int, dn: int, dr: int,
                      rank: int, eps: float, weight) -> None:
    """For attention over one latent vector per token.  kv [T, rank + dr] (a view with unit column stride): the first
    ``rank`` elements normed (unit root mean square, times ``weight`` [rank]) and the last dr rotated go to the token's
    row of ``pages`` [pages, 1, 1, page_size, row >= rank + dr] (None: nothing is stored).  q [T, H * (dn + dr)]: every
    head's last dr elements, rotated, go to q_lat [T, H * (rank + dr)] behind the head's first ``rank`` places."""
    _need_cuda(kv, q, q_lat, pages, slot_mapping, positions, cos_sin, weight)
    T = kv.shape[0]
    assert kv.stride(1) == 1 and kv.shape[1] == rank + dr and q.stride(1) == 1 and q.shape == (T, H * (dn + dr))
    assert q_lat.stride(1) == 1 and q_lat.shape == (T, H * (rank + dr)) and kv.dtype == q.dtype == q_lat.dtype == weight.dtype
    assert weight.is_contiguous() and weight.numel() == rank
    if pages is not None:
        _contig("pages", pages)
        n_pages, planes, heads, page_size, row = pages.shape
        assert planes == 1 and heads == 1 and row >= rank + dr and pages.dtype == kv.dtype
        assert slot_mapping.dtype == torch.int32 and slot_mapping.numel() >= T
    else:
        n_pages, page_size, row = 0, 0, rank + dr
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] == rotary_dim
        assert positions.dtype == torch.int32
    call("nhv_latent_rope_store", dtype_code(kv), kv.data_ptr(), kv.stride(0), q.data_ptr(), q.stride(0), q_lat.data_ptr(),
         q_lat.stride(0), _ptr(pages), _ptr(slot_mapping), _ptr(positions), _ptr(cos_sin), int(rotary_dim),
         0 if cos_sin is None else cos_sin.shape[0], T, H, dn, dr, rank, row, page_size, n_pages, float(eps),
         weight.data_ptr(), stream_ptr())


def linear_heads(out, x, weight) -> None:
    """One product per head: out[:, h, :] = x[:, h, :] @ weight[h]^T for x [T, H, K], weight [H, N, K] (contiguous),
    out [T, H, N]; x and out may be views into wider rows (heads a fixed step apart, unit stride inside a head).
    float32 runs the fixed-order CUDA-core product; bfloat16 the library's batched product."""
    _need_cuda(out, x, weight)
    _contig("weight", weight)
    T, H, K = x.shape
    N = weight.shape[1]
    assert weight.shape == (H, N, K) and out.shape == (T, H, N) and x.dtype == weight.dtype == out.dtype
    assert x.stride(2) == 1 and out.stride(2) == 1
    if x.dtype == torch.bfloat16 and T > LINEAR_HEADS_SIMT_ROWS:
        library.LAUNCHES += 1
        torch.bmm(x.transpose(0, 1), weight.transpose(1, 2), out=out.transpose(0, 1))
        return
    call("nhv_gemm_nt_simt_batched", dtype_code(x), out.data_ptr(), x.data_ptr(), weight.data_ptr(), T, N, K, x.stride(0),
         K, out.stride(0), 0, H, x.stride(1), N * K, out.stride(1), stream_ptr())


LINEAR_HEADS_SIMT_ROWS = 0          # tokens up to which the per-head products in bfloat16 run on the CUDA cores


def general_delta(o, proj, aw, a_bias, w2, w0, state, batch, H: int, d: int, decay_floor: float) -> None:
    """The generalised delta rule over the step's tokens.  proj [T, >= 3 H d] (r, k, v in the storage type), aw
    [T, H d + rank] float32 (the removal rate's projection, then the decay's inner projection), a_bias / w0 [H d] and
    w2 [H d, rank] in the storage type, state [slots, H d d] float32 -> o [T, H d] float32 (before its norm and gate).
    The decay per key channel is exp(-decay_floor * sigmoid(w2 tanh(inner) + w0)); tanh(inner) takes the storage type
    as the operand of the product with w2, whose sums are float32."""
    _need_cuda(o, proj, aw, a_bias, w2, w0, state)
    T, n = proj.shape[0], H * d
    rank = w2.shape[1]
    assert proj.stride(1) == 1 and proj.shape[1] >= 3 * n and aw.dtype == torch.float32 and aw.stride(1) == 1
    assert aw.shape == (T, n + rank) and o.dtype == state.dtype == torch.float32 and o.is_contiguous() and o.shape == (T, n)
    assert a_bias.dtype == w2.dtype == w0.dtype == proj.dtype and w2.is_contiguous() and w2.shape == (n, rank)
    assert a_bias.numel() == n and w0.numel() == n and state.stride(1) == 1
    # the decay's second projection as a product of its own: tanh of the inner projection in the storage type, 32-bit sums
    inner = torch.empty(T, rank, dtype=proj.dtype, device=proj.device)
    call("nhv_general_delta_tanh", dtype_code(proj), inner.data_ptr(), aw.data_ptr() + 4 * n, aw.stride(0), T, rank,
         stream_ptr())
    dec = torch.empty(T, n, dtype=torch.float32, device=proj.device)
    linear_f32(dec, inner, w2)
    scratch = torch.empty(T * (6 * n + 2 * H), dtype=torch.float32, device=proj.device)
    vec, v32, sc = scratch.data_ptr(), scratch.data_ptr() + 4 * 5 * T * n, scratch.data_ptr() + 4 * 6 * T * n
    call("nhv_general_delta", dtype_code(proj), o.data_ptr(), proj.data_ptr(), proj.stride(0), aw.data_ptr(), aw.stride(0),
         a_bias.data_ptr(), dec.data_ptr(), w0.data_ptr(), state.data_ptr(), state.stride(0), vec, sc, v32,
         batch.cu_q.data_ptr(), batch.q_start.data_ptr(), batch.state_slots.data_ptr(), batch.n_seqs, T, H, d,
         float(decay_floor), stream_ptr())


def sigmoid_mul_heads(out, x, gate, group: int, x_head: int | None = None) -> None:
    """out[t, c] = x[t, c] * sigmoid(gate[t, c // group]): one gate per head of ``group`` columns, in 32-bit.
    ``x_head``: the distance between two heads in a row of x, where x holds padded heads (x [T, heads * x_head])."""
    _need_cuda(out, x, gate)
    heads = out.shape[1] // group
    assert out.dim() == 2 and out.dtype == x.dtype == gate.dtype and out.shape[1] % group == 0
    assert x.shape == ((out.shape[0], heads * x_head) if x_head else out.shape)
    assert gate.shape == (out.shape[0], heads) and out.stride(1) == x.stride(1) == gate.stride(1) == 1
    call("nhv_sigmoid_mul_heads", dtype_code(out), out.data_ptr(), out.stride(0), x.data_ptr(), x.stride(0), gate.data_ptr(),
         gate.stride(0), out.shape[0], out.shape[1], int(group), int(x_head or group), stream_ptr())


LATENT_TILE = 64        # rows of a temporary page of expanded keys and values


def latent_expand(pages, tables, batch, q, q_lat, ukv, H: int, dn: int, dr: int, dv: int, rank: int, D: int):
    """Attention over one latent per token, prepared for the tensor-core kernels: the latents of the step's requests
    (all their tokens in the cache) are expanded by ``ukv`` [H dn + H dv, rank] into a key [dn | rotated part dr | 0]
    and a value [dv | 0] per head, padded to D elements, in temporary pages of 64 tokens; the queries likewise.
    Returns (queries [T, H D], temporary pages [n, 2, H, 64, D], their block tables [requests, pages])."""
    _need_cuda(pages, q, q_lat, ukv)
    T, row = q.shape[0], pages.shape[-1]
    plan = getattr(batch, "_latent_rows", None)
    if plan is None or plan[3] != batch.host_kv_len:        # every such layer of the step uses the same rows
        counts = [-(-n // LATENT_TILE) for n in batch.host_kv_len]
        first, width = [0], max(counts)
        for c in counts:
            first.append(first[-1] + c)
        table = [[first[s] + i if i < counts[s] else -1 for i in range(width)] for s in range(len(counts))]
        plan = (torch.tensor([f * LATENT_TILE for f in first[:-1]], dtype=torch.int32).to(q.device, non_blocking=True),
                torch.tensor(table, dtype=torch.int32).to(q.device, non_blocking=True), first[-1], list(batch.host_kv_len))
        batch._latent_rows = plan
    row0, tmp_table, n_tmp = plan[:3]
    rows = n_tmp * LATENT_TILE
    lat = torch.empty(rows, rank, dtype=q.dtype, device=q.device)
    kr = torch.empty(rows, max(dr, 1), dtype=q.dtype, device=q.device)
    call("nhv_latent_gather", dtype_code(q), lat.data_ptr(), kr.data_ptr(), pages.data_ptr(), tables.block_tables.data_ptr(),
         tables.block_tables.stride(0), batch.kv_len.data_ptr(), row0.data_ptr(), batch.n_seqs, batch.max_kv_len, rank, dr,
         row, pages.shape[3], pages.shape[0], stream_ptr())
    kv = torch.empty(rows, ukv.shape[0], dtype=q.dtype, device=q.device)
    linear(kv, lat, ukv)
    tmp = torch.empty(n_tmp, 2, H, LATENT_TILE, D, dtype=q.dtype, device=q.device)
    qp = torch.empty(T, H * D, dtype=q.dtype, device=q.device)
    call("nhv_latent_assemble", dtype_code(q), tmp.data_ptr(), qp.data_ptr(), kv.data_ptr(), kr.data_ptr(), q.data_ptr(),
         q.stride(0), q_lat.data_ptr(), q_lat.stride(0), rows, T, H, dn, dr, dv, rank, D, stream_ptr())
    return qp, tmp, tmp_table


LATENTS_ON_TENSOR_CORES = True      # tests switch it off to compare with the CUDA-core kernel at the same shapes


def latent_attention(out, q_lat, pages, tables, batch, H: int, rank: int, row: int, scale: float, sinks=None) -> None:
    """Attention of the step's tokens over one latent per token: pages with one plane whose rows [row] are the key of
    every head and whose leading ``rank`` elements are the value of every head; q_lat [T, H row] -> out [T, H rank].
    ``sinks`` [H] float32: exp(sink) joins each head's softmax denominator once.  bfloat16 with rows and latents in
    steps of 8 runs on the tensor cores, a token's keys shared between blocks and merged (scratch: one partial result
    per token, head and piece); float32 and other sizes run the CUDA-core kernel."""
    _need_cuda(out, q_lat, pages, sinks)
    T = q_lat.shape[0]
    if not (LATENTS_ON_TENSOR_CORES and q_lat.dtype == torch.bfloat16 and pages.shape[1] == 1 and pages.shape[2] == 1
            and pages.shape[-1] == row and library.load_library().nhv_latent_decode_supports(H, rank, row)):
        attention_sink_simt(out, q_lat, pages, tables.block_tables, batch.cu_q, batch.kv_len, batch.n_seqs, batch.n_tokens,
                            H, 1, row, rank, scale, sinks)
        return
    _contig("kv_pages", pages)
    assert q_lat.shape == (T, H * row) and out.shape == (T, H * rank) and out.dtype == pages.dtype == torch.bfloat16
    assert q_lat.stride(1) == 1 and out.stride(1) == 1 and sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == H)
    tiles = -(-batch.max_kv_len // 64)
    pieces = max(1, min(tiles, 64, 2 * 148 // (T * -(-H // 16))))      # two rounds of blocks over the 148 SMs at most
    part = torch.empty(T * H * pieces * (rank + 2), dtype=torch.float32, device=out.device)
    call("nhv_latent_decode", out.data_ptr(), out.stride(0), q_lat.data_ptr(), q_lat.stride(0), pages.data_ptr(),
         tables.block_tables.data_ptr(), tables.block_tables.stride(0), batch.cu_q.data_ptr(), batch.kv_len.data_ptr(),
         batch.n_seqs, T, H, rank, row, pages.shape[3], pages.shape[0], float(scale), _ptr(sinks), pieces,
         part.data_ptr(), part.data_ptr() + 4 * T * H * pieces * rank, stream_ptr())


def gelu_tanh(x) -> None:
    """x = 0.5 x (1 + tanh(sqrt(2 / pi) (x + 0.044715 x^3))) in place."""
    _need_cuda(x)
    _contig("x", x)
    call("nhv_gelu_tanh", dtype_code(x), x.data_ptr(), x.numel(), stream_ptr())


def postnorm_stream(stream, rounded, terms, weight, scale, eps: float, side_eps: float | None = None) -> None:
    """A sub-block's output normed and added onto a float32 residual stream [T, width], in place:
    y = sum over ``terms`` ((tensor, coef, side weight or None), one or two) of coef * tensor, a term with a side weight
    first divided by its own root mean square and multiplied by that weight; stream += y / rms(y) * weight (* scale, a
    vector per channel, if given).  ``rounded`` (optional, storage type): receives the new stream rounded once, what the
    next sub-block reads.  All sums and norms are 32-bit."""
    tensors = [t for t, _, _ in terms] + [w for _, _, w in terms]
    _need_cuda(stream, rounded, weight, scale, *tensors)
    _contig("stream", stream)
    width = stream.shape[-1]
    if not 1 <= len(terms) <= 2:
        raise KernelError("the output norm adds one or two terms")
    (a, ca, wa), (b, cb, wb) = terms[0], (terms[1] if len(terms) == 2 else (None, 0.0, None))
    assert stream.dtype == torch.float32 and weight.numel() == width and weight.dtype == a.dtype
    for t in (a, b):
        assert t is None or (t.shape == stream.shape and t.is_contiguous() and t.dtype == a.dtype)
    for w in (wa, wb, scale):
        assert w is None or (w.numel() == width and w.dtype == a.dtype and w.is_contiguous())
    assert rounded is None or (rounded.shape == stream.shape and rounded.dtype == a.dtype and rounded.is_contiguous())
    if wa is None and wb is not None:
        raise KernelError("a side norm on the second term only is not offered")
    call("nhv_postnorm_stream", dtype_code(a), stream.data_ptr(), _ptr(rounded), a.data_ptr(), _ptr(wa), float(ca), _ptr(b),
         _ptr(wb), float(cb), weight.data_ptr(), _ptr(scale), stream.numel() // width, width, float(eps),
         float(eps if side_eps is None else side_eps), stream_ptr())


def stream_round(out, stream) -> None:
    """out (storage type) = the float32 stream rounded once."""
    _need_cuda(out, stream)
    _contig("out", out); _contig("stream", stream)
    assert stream.dtype == torch.float32 and out.numel() == stream.numel()
    call("nhv_stream_round", dtype_code(out), out.data_ptr(), stream.data_ptr(), stream.numel(), stream_ptr())


def token_shift_mix(out, x, mu, state, batch) -> None:
    """out [n, T, C]: out[s, t] = x[t] + (x[t - 1] - x[t]) * mu[s] for mu [n, C] (one contiguous plane per mix, so that
    each is a product's operand as it lies); the token before a request's first is zero, the one before this step's
    portion is the request's ``state`` [slots, C] float32, which is moved on."""
    _need_cuda(out, x, mu, state)
    _contig("out", out); _contig("x", x); _contig("mu", mu)
    T, C = x.shape
    n = mu.shape[0]
    assert out.shape == (n, T, C) and mu.shape == (n, C) and out.dtype == x.dtype == mu.dtype
    assert state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and state.shape[1] >= C
    call("nhv_token_shift_mix", dtype_code(x), out.data_ptr(), x.data_ptr(), mu.data_ptr(), state.data_ptr(), state.stride(0),
         batch.cu_q.data_ptr(), batch.q_start.data_ptr(), batch.state_slots.data_ptr(), batch.n_seqs, T, C, n, stream_ptr())


def decay_lowrank(w, inner, w2, w0) -> None:
    """w [T, n] float32 = exp(-exp(w0 + tanh(inner) @ w2^T)) for inner [T, rank] float32 (a view with unit column
    stride), w2 [n, rank] and w0 [n] in the storage type: a decay per token and channel from the sums of its inner
    projection, tanh and both exponentials in 32-bit."""
    _need_cuda(w, inner, w2, w0)
    _contig("w", w); _contig("w2", w2); _contig("w0", w0)
    T, rank = inner.shape
    n = w2.shape[0]
    assert w.dtype == inner.dtype == torch.float32 and inner.stride(1) == 1 and w.shape == (T, n)
    assert w2.shape == (n, rank) and w0.numel() == n and w2.dtype == w0.dtype
    call("nhv_decay_lowrank", dtype_code(w2), w.data_ptr(), inner.data_ptr(), inner.stride(0), w2.data_ptr(), w0.data_ptr(),
         T, n, rank, stream_ptr())


def decay_scan(o, r, k, v, state, batch, H: int, dk: int, dv: int, decay_tokens=None, decay_heads=None, bonus=None,
               silu: bool = False, read_after: bool = False) -> None:
    """A linear recurrence with a matrix state per head over the step's tokens: S <- diag(w) S + k v^T, with
    o = (S_before + diag(bonus) k v^T)^T r (``read_after`` False; no bonus: ones) or o = S_after^T r (True).
    r, k [T, H dk] and v [T, H dv]: views into one projection output (same row stride, unit column stride, storage type),
    through SiLU if ``silu``.  The decay w: ``decay_tokens`` [T, H dk] float32 or ``decay_heads`` [H] float32.
    state [slots, H dv dk] float32 -> o [T, H dv] float32."""
    _need_cuda(o, r, k, v, state, decay_tokens, decay_heads, bonus)
    T = r.shape[0]
    assert r.shape == k.shape == (T, H * dk) and v.shape == (T, H * dv) and r.dtype == k.dtype == v.dtype
    assert r.stride(1) == k.stride(1) == v.stride(1) == 1 and r.stride(0) == k.stride(0) == v.stride(0)
    assert o.dtype == state.dtype == torch.float32 and o.is_contiguous() and o.shape == (T, H * dv)
    assert state.dim() == 2 and state.stride(1) == 1 and state.shape[1] >= H * dk * dv
    assert (decay_tokens is None) != (decay_heads is None)
    assert decay_tokens is None or (decay_tokens.dtype == torch.float32 and decay_tokens.is_contiguous()
                                    and decay_tokens.shape == (T, H * dk))
    assert decay_heads is None or (decay_heads.dtype == torch.float32 and decay_heads.numel() == H)
    assert bonus is None or (bonus.dtype == r.dtype and bonus.is_contiguous() and bonus.numel() == H * dk)
    call("nhv_decay_scan", dtype_code(r), o.data_ptr(), r.data_ptr(), k.data_ptr(), v.data_ptr(), r.stride(0),
         _ptr(decay_tokens), _ptr(decay_heads), _ptr(bonus), state.data_ptr(), state.stride(0), batch.cu_q.data_ptr(),
         batch.q_start.data_ptr(), batch.state_slots.data_ptr(), batch.n_seqs, T, H, dk, dv, int(bool(silu)),
         int(bool(read_after)), stream_ptr())


def relu_squared(x) -> None:
    """x = max(x, 0) ** 2 in place."""
    _need_cuda(x)
    _contig("x", x)
    call("nhv_relu_squared", dtype_code(x), x.data_ptr(), x.numel(), stream_ptr())


def scale_softcap(logits, scale: float, cap: float | None) -> None:
    """float32 logits in place: times ``scale``, then (``cap`` given) cap * tanh(logits / cap)."""
    _need_cuda(logits)
    _contig("logits", logits)
    assert logits.dtype == torch.float32
    call("nhv_scale_softcap", logits.data_ptr(), float(scale), float(cap or 0.0), logits.numel(), stream_ptr())


def sigmoid_mul(out, x, gate) -> None:
    """out = x * sigmoid(gate), elementwise in 32-bit; each a [T, width] view with unit column stride."""
    _need_cuda(out, x, gate)
    assert out.shape == x.shape == gate.shape and out.dim() == 2 and out.dtype == x.dtype == gate.dtype
    assert out.stride(1) == x.stride(1) == gate.stride(1) == 1
    call("nhv_sigmoid_mul", dtype_code(out), out.data_ptr(), out.stride(0), x.data_ptr(), x.stride(0), gate.data_ptr(),
         gate.stride(0), x.shape[0], x.shape[1], stream_ptr())


def add_row_bias(x, bias) -> None:
    """x [T, width] += bias [width], in place (the sum in 32-bit)."""
    _need_cuda(x, bias)
    _contig("x", x)
    assert bias.dtype == x.dtype and bias.is_contiguous() and x.shape[-1] == bias.numel()
    call("nhv_add_row_bias", dtype_code(x), x.data_ptr(), bias.data_ptr(), x.numel() // bias.numel(), bias.numel(), stream_ptr())


def clamped_glu(out, gate_up, limit: float, alpha: float) -> None:
    """out = g * sigmoid(alpha * g) * (u + 1) with g = min(gate, limit) and u = clamp(up, -limit, limit), for gate_up
    [n, 2 * inter] with the gate in the first half of each row."""
    _need_cuda(out, gate_up)
    _contig("out", out); _contig("gate_up", gate_up)
    inter = gate_up.shape[-1] // 2
    assert gate_up.shape[-1] == 2 * inter and out.shape[-1] == inter and out.dtype == gate_up.dtype
    call("nhv_clamped_glu", dtype_code(out), out.data_ptr(), gate_up.data_ptr(), out.numel() // inter, inter, float(limit),
         float(alpha), stream_ptr())


MLSTM_COLUMN_BLOCK = 16     # columns of the memory that one block of the scan carries (ML_COLS of csrc/mlstm.cu)
MLSTM_LANES = 0             # lanes per column of the memory: 0 is the kernel's choice; tests set 8 or 16


def mlstm_state_floats(H: int, d: int, dv: int) -> int:
    """Floats that one request's mLSTM state takes: S [H, dv, d], then per (head, block of columns) the normaliser's d
    rows and the running maximum (every column block of the scan carries its own copy of them)."""
    return H * dv * d + H * -(-dv // MLSTM_COLUMN_BLOCK) * (d + 1)


def mlstm_scan(y, proj, gates, gate_bias, cap: float, state, batch, H: int, d: int, dv: int) -> None:
    """The mLSTM recurrence over the step's tokens.  proj [T, >= 2*H*d + H*dv] (q, k, v per head; a view with unit
    column stride), gates [T, 2*H] float32 (input then forget gates, before bias and cap), gate_bias [2*H] float32,
    state [slots, mlstm_state_floats] float32 -> y [T, H*dv] float32 (before its norm and gate)."""
    _need_cuda(y, proj, gates, gate_bias, state)
    T = proj.shape[0]
    assert proj.stride(1) == 1 and proj.shape[1] >= 2 * H * d + H * dv
    assert y.dtype == gates.dtype == gate_bias.dtype == state.dtype == torch.float32
    assert y.is_contiguous() and y.shape == (T, H * dv) and gates.stride(1) == 1 and gates.shape == (T, 2 * H)
    assert gate_bias.numel() == 2 * H and state.dim() == 2 and state.stride(1) == 1
    assert state.shape[1] >= mlstm_state_floats(H, d, dv)
    call("nhv_mlstm_scan", dtype_code(proj), y.data_ptr(), proj.data_ptr(), proj.stride(0), gates.data_ptr(), gates.stride(0),
         gate_bias.data_ptr(), float(cap), state.data_ptr(), state.stride(0), batch.cu_q.data_ptr(), batch.q_start.data_ptr(),
         batch.state_slots.data_ptr(), batch.n_seqs, T, H, d, dv, MLSTM_LANES, stream_ptr())


def moe_route(ids, weights, logits, correction, n_outputs: int, n_groups: int, keep: int, scores: str = "softmax",
              renorm: bool = True) -> None:
    """The router's choice per token.  logits [T, >= n_outputs] float32 (a view with unit column stride; further columns
    are not read), correction [n_outputs] float32 or None -> ids [T, top] int32 and weights [T, top] float32.
    Scores are the softmax over all outputs; the choice is by score + correction among the outputs of the ``keep`` best
    of ``n_groups`` groups of neighbours (a group's score: its largest choice score); the weights are the chosen scores
    divided by their sum (+ 1e-20).  ``scores`` "sigmoid": each output's score is the sigmoid of its logit;
    ``renorm`` False: the weights are the chosen scores as they are."""
    assert scores in ("softmax", "sigmoid")
    _need_cuda(ids, weights, logits, correction)
    T, top = ids.shape
    assert ids.dtype == torch.int32 and weights.dtype == logits.dtype == torch.float32 and weights.shape == ids.shape
    assert ids.is_contiguous() and weights.is_contiguous() and logits.stride(1) == 1 and logits.shape[0] == T
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == n_outputs)
    call("nhv_moe_route", ids.data_ptr(), weights.data_ptr(), logits.data_ptr(), logits.stride(0), _ptr(correction), T,
         n_outputs, n_groups, keep, top, int(scores == "sigmoid"), int(bool(renorm)), stream_ptr())


MOE_TILE_SIMT = 16      # rows of one expert that a block of the CUDA-core products takes (MG_BM of csrc/moe.cu)


def moe_sorted_rows(n_slots: int, n_experts: int, tile: int) -> int:
    """Rows of the by-expert ordering of ``n_slots`` (token, choice) slots: each expert's run is padded to whole tiles."""
    rows = n_slots + min(n_slots, n_experts) * (tile - 1)
    return -(-rows // tile) * tile


def moe_align(ids, n_experts: int, tile: int):
    """Order the slots of ids [T, top] by expert (choices >= n_experts, identity experts, take no row).  Returns
    (sorted_slots [rows] int32: slot of each row or -1, slot_pos [T * top] int32: row of each slot or -1,
    tile_expert [rows / tile] int32: expert of each tile or -1)."""
    _need_cuda(ids)
    n_slots = ids.numel()
    rows = moe_sorted_rows(n_slots, n_experts, tile)
    buf = torch.empty(rows + n_slots + rows // tile, dtype=torch.int32, device=ids.device)
    sorted_slots, slot_pos, tile_expert = buf[:rows], buf[rows:rows + n_slots], buf[rows + n_slots:]
    call("nhv_moe_align", ids.data_ptr(), n_slots, n_experts, tile, sorted_slots.data_ptr(), slot_pos.data_ptr(),
         tile_expert.data_ptr(), stream_ptr())
    return sorted_slots, slot_pos, tile_expert


def moe_experts_simt(act, y, x, gate, up, down, sorted_slots, tile_expert, top: int, limit: float, alpha: float,
                     up_shift: float = 1.0, row_scale=None) -> None:
    """The experts' two products over the ordered rows on the CUDA cores, for any storage type and size, in a fixed order
    of summation: act [rows, ff] = glu(x[token] gate[e]^T, x[token] up[e]^T), y [rows, width] = act down[e]^T, with
    gate / up [E, ff, width] and down [E, width, ff]."""
    _need_cuda(act, y, x, gate, up, down, sorted_slots, tile_expert)
    for name, t in (("act", act), ("y", y), ("x", x), ("gate", gate), ("up", up), ("down", down)):
        _contig(name, t)
    E, ff, width = gate.shape
    assert up.shape == gate.shape and down.shape == (E, width, ff) and x.shape[1] == width
    assert act.shape == (sorted_slots.numel(), ff) and y.shape == (sorted_slots.numel(), width)
    assert act.dtype == y.dtype == x.dtype == gate.dtype == up.dtype == down.dtype
    tiles = tile_expert.numel()
    assert tiles * MOE_TILE_SIMT == sorted_slots.numel()
    call("nhv_moe_gemm_simt", dtype_code(x), 1, act.data_ptr(), x.data_ptr(), width, gate.data_ptr(), up.data_ptr(),
         sorted_slots.data_ptr(), tile_expert.data_ptr(), tiles, top, ff, width, float(limit), float(alpha), float(up_shift),
         _ptr(row_scale), stream_ptr())
    call("nhv_moe_gemm_simt", dtype_code(x), 0, y.data_ptr(), act.data_ptr(), ff, down.data_ptr(), None,
         sorted_slots.data_ptr(), tile_expert.data_ptr(), tiles, top, width, ff, 0.0, 0.0, 0.0, None, stream_ptr())


MOE_ON_TENSOR_CORES = True      # tests switch it off to compare with the CUDA-core products at the same shapes
MOE_TILE = 0                    # rows per tile of the mma.sync products: 0 chooses by the step; tests set 16, 64, 128
MOE_TCGEN05 = None              # the tcgen05 products: None where an expert sees many rows; tests set True (always) or False
MOE_TCGEN05_TILE = 128          # rows per tile of the tcgen05 products (ROWS of csrc/moe_tcgen05.cu)


def moe_experts(x, gate, up, down, ids, limit: float, alpha: float, up_shift: float = 1.0, row_scale=None):
    """Every chosen expert's output for every token: orders the slots of ids [T, top] by expert and runs the experts' two
    products over that order: bfloat16 with sizes in steps of 8 on the tensor cores (tcgen05 with tiles of 128 rows
    where an expert sees about a hundred rows or more; mma.sync with tiles of 64 rows below that and of 16 where it
    sees few and the products stream the weights), everything else on the CUDA cores.
    The experts' unit is g' sigmoid(alpha g') (u' + up_shift) with g' = min(g, limit), u' = clamp(u, -limit, limit)
    (limit inf, alpha 1, up_shift 0: silu(g) u).  ``row_scale`` [T, top] float32: a factor on each chosen expert's input.
    Returns (y [rows, width], one row per slot that chose a real expert, and slot_pos [T * top] int32, the row of each
    slot or -1)."""
    E, ff, width = gate.shape
    assert row_scale is None or (row_scale.dtype == torch.float32 and row_scale.is_contiguous() and row_scale.numel() == ids.numel())
    top = ids.shape[1]
    mma = MOE_ON_TENSOR_CORES and x.dtype == torch.bfloat16 and width % 8 == 0 and ff % 8 == 0
    tile = MOE_TILE_SIMT
    if mma:
        tile = MOE_TILE or (128 if ids.numel() >= 192 * E else 64 if ids.numel() >= 24 * E else 16)
    if mma and (MOE_TCGEN05 or (MOE_TCGEN05 is None and not MOE_TILE and ids.numel() >= 96 * E)):
        return _moe_experts_tcgen05(x, gate, up, down, ids, limit, alpha, up_shift, row_scale)
    sorted_slots, slot_pos, tile_expert = moe_align(ids, E, tile)
    rows = sorted_slots.numel()
    act = torch.empty(rows, ff, dtype=x.dtype, device=x.device)
    y = torch.empty(rows, width, dtype=x.dtype, device=x.device)
    if not mma:
        moe_experts_simt(act, y, x, gate, up, down, sorted_slots, tile_expert, top, limit, alpha, up_shift, row_scale)
        return y, slot_pos
    _need_cuda(x, gate, up, down, ids)
    for name, t in (("x", x), ("gate", gate), ("up", up), ("down", down)):
        _contig(name, t)
    assert up.shape == gate.shape and down.shape == (E, width, ff) and x.shape[1] == width
    assert gate.dtype == up.dtype == down.dtype == torch.bfloat16
    tiles = tile_expert.numel()
    call("nhv_moe_gemm_mma", tile, 1, act.data_ptr(), x.data_ptr(), width, gate.data_ptr(), up.data_ptr(),
         sorted_slots.data_ptr(), tile_expert.data_ptr(), tiles, top, ff, width, float(limit), float(alpha), float(up_shift),
         _ptr(row_scale), stream_ptr())
    call("nhv_moe_gemm_mma", tile, 0, y.data_ptr(), act.data_ptr(), ff, down.data_ptr(), None,
         sorted_slots.data_ptr(), tile_expert.data_ptr(), tiles, top, width, ff, 0.0, 0.0, 0.0, None, stream_ptr())
    return y, slot_pos


def _moe_experts_tcgen05(x, gate, up, down, ids, limit: float, alpha: float, up_shift: float = 1.0, row_scale=None):
    """``moe_experts`` for prompts in bfloat16: tiles of 128 rows per expert, the tokens' rows gathered into that order
    (so that a tile is one TMA box), both products with tcgen05.mma and tensor-memory accumulators."""
    _need_cuda(x, gate, up, down, ids)
    for name, t in (("x", x), ("gate", gate), ("up", up), ("down", down)):
        _contig(name, t)
    E, ff, width = gate.shape
    top = ids.shape[1]
    assert up.shape == gate.shape and down.shape == (E, width, ff) and x.shape[1] == width
    assert x.dtype == gate.dtype == up.dtype == down.dtype == torch.bfloat16
    sorted_slots, slot_pos, tile_expert = moe_align(ids, E, MOE_TCGEN05_TILE)
    rows, tiles = sorted_slots.numel(), tile_expert.numel()
    xs = torch.empty(rows, width, dtype=x.dtype, device=x.device)
    act = torch.empty(rows, ff, dtype=x.dtype, device=x.device)
    y = torch.empty(rows, width, dtype=x.dtype, device=x.device)
    call("nhv_moe_gather_rows", xs.data_ptr(), x.data_ptr(), sorted_slots.data_ptr(), rows, top, width, stream_ptr())
    call("nhv_moe_gemm_tcgen05", 1, act.data_ptr(), xs.data_ptr(), gate.data_ptr(), up.data_ptr(), E, sorted_slots.data_ptr(),
         tile_expert.data_ptr(), tiles, ff, width, float(limit), float(alpha), float(up_shift), _ptr(row_scale), stream_ptr())
    call("nhv_moe_gemm_tcgen05", 0, y.data_ptr(), act.data_ptr(), down.data_ptr(), None, E, sorted_slots.data_ptr(),
         tile_expert.data_ptr(), tiles, width, ff, 0.0, 0.0, 0.0, None, stream_ptr())
    return y, slot_pos


def moe_combine(out, y, x, ids, weights, slot_pos, n_experts: int, shared=None, shared_gate=None) -> None:
    """out[t] = sum over the token's choices of weight * (the expert's row of y, or x[t] itself for an identity expert)
    (+ sigmoid(shared_gate[t]) * shared[t]; a shared term without a gate counts fully).  ``shared_gate``: a float32
    column view (one number per token).  ``weights`` None: every choice counts fully."""
    _need_cuda(out, y, x, ids, weights, slot_pos, shared, shared_gate)
    _contig("out", out); _contig("y", y); _contig("x", x)
    T, width = x.shape
    top = ids.shape[1]
    assert out.shape == x.shape and y.shape[1] == width and out.dtype == y.dtype == x.dtype
    assert shared is None or (shared.shape == x.shape and shared.dtype == x.dtype and shared.is_contiguous())
    assert shared_gate is None or (shared is not None and shared_gate.dtype == torch.float32 and shared_gate.shape[0] == T)
    call("nhv_moe_combine", dtype_code(out), out.data_ptr(), y.data_ptr(), x.data_ptr(), _ptr(shared), _ptr(shared_gate),
         0 if shared_gate is None else shared_gate.stride(0), ids.data_ptr(), _ptr(weights), slot_pos.data_ptr(), T, top,
         n_experts, width, stream_ptr())


def rope_norm_store(qkv, q_out, kv_pages, slot_mapping, positions, cos_sin, rotary_dim: int, nq: int, nkv: int, dk: int,
                    dv: int, eps: float | None, bias=None, values_from_keys: bool = False, q_weight=None,
                    k_weight=None, norm_first: bool = False, interleaved: bool = False) -> None:
    """qkv [T, nq*dk + nkv*dk + nkv*dv] -> q_out [T, nq*dk] (rotated, then scaled to unit root mean square; eps None:
    no norm) and K / V rows in kv_pages [pages, 2, nkv, page_size, row] at slot_mapping.  kv_pages None: queries only.
    ``bias`` (one element per query and key column of qkv, in its type) is added in 32-bit before the rotation.
    ``values_from_keys``: the stored values are the key heads as projected (bias added, not rotated); qkv then ends
    with the keys (it may have further columns that this op does not read) and dv == dk.  ``q_weight`` / ``k_weight``
    [dk]: the normed query / key heads times this weight (one weight for all heads of a kind).  ``norm_first``: the
    norm and its weight come before the rotation.  ``interleaved``: element 2i turns with element 2i + 1 instead of
    element i with element i + rotary_dim / 2 (the table is the same)."""
    _need_cuda(qkv, q_out, kv_pages, slot_mapping, positions, cos_sin, bias, q_weight, k_weight)
    for hw in (q_weight, k_weight):
        assert hw is None or (hw.dtype == qkv.dtype and hw.is_contiguous() and hw.numel() == dk and eps is not None)
    assert bias is None or (bias.dtype == qkv.dtype and bias.is_contiguous() and bias.numel() == nq * dk + nkv * dk)
    assert qkv.stride(-1) == 1 and q_out.stride(-1) == 1 and qkv.dim() == 2 and q_out.dim() == 2
    n_tokens = qkv.shape[0]
    if kv_pages is not None:
        _contig("kv_pages", kv_pages)
        n_pages, two, h, page_size, row = kv_pages.shape
        assert two == 2 and h == nkv and row >= max(dk, dv) and kv_pages.dtype == qkv.dtype
        assert slot_mapping.dtype == torch.int32 and slot_mapping.numel() >= n_tokens
    else:
        n_pages, page_size, row = 0, 0, max(dk, dv)
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] == rotary_dim
        assert positions.dtype == torch.int32
    call("nhv_rope_norm_store", dtype_code(qkv), qkv.data_ptr(), qkv.stride(0), q_out.data_ptr(), q_out.stride(0),
         _ptr(kv_pages), _ptr(slot_mapping), _ptr(positions), _ptr(cos_sin), int(rotary_dim),
         0 if cos_sin is None else cos_sin.shape[0], n_tokens, nq, nkv, dk, dv, row, page_size, n_pages,
         -1.0 if eps is None else float(eps), _ptr(bias), int(bool(values_from_keys)), _ptr(q_weight), _ptr(k_weight),
         int(bool(norm_first)), int(bool(interleaved)), stream_ptr())


def attention_sink_simt(out, q, kv_pages, block_table, cu_q, kv_len, n_seqs: int, n_tokens: int, nq: int, nkv: int,
                        dk: int, dv: int, scale: float, sinks=None, window: int = 0, chunk: int = 0, slopes=None,
                        keep_first: int = 0) -> None:
    """Causal attention of this step's tokens over the pages with key heads of dk and value heads of dv elements:
    q [T, nq*dk] -> out [T, nq*dv].  ``sinks`` [nq] float32: a term exp(sink) in each head's softmax denominator.
    ``window`` > 0: the last ``window`` keys only; ``chunk`` > 0: only the keys of the query's own chunk of ``chunk``
    positions, counted from position 0 of the request.  ``slopes`` [nq] float32: head h's score loses slopes[h] times
    the distance between query and key.  Pages with one plane ([pages, 1, nkv, page_size, row]): a row is the key and
    its leading dv elements are the value."""
    _need_cuda(out, q, kv_pages, block_table, cu_q, kv_len, sinks, slopes)
    _contig("kv_pages", kv_pages)
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and out.dtype == q.dtype == kv_pages.dtype
    n_pages, planes, h, page_size, row = kv_pages.shape
    assert planes in (1, 2) and h == nkv and row >= max(dk, dv) and (planes == 2 or dv <= dk)
    assert block_table.dtype == torch.int32 and block_table.stride(-1) == 1
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == nq)
    assert slopes is None or (slopes.dtype == torch.float32 and slopes.numel() == nq)
    call("nhv_attention_simt_ex", dtype_code(q), q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0),
         kv_pages.data_ptr(), block_table.data_ptr(), block_table.stride(0), cu_q.data_ptr(), kv_len.data_ptr(),
         n_seqs, n_tokens, nq, nkv, dk, dv, row, page_size, n_pages, int(window), int(chunk), float(scale), _ptr(sinks),
         _ptr(slopes), planes, int(keep_first), stream_ptr())


SINK_ATTENTION_ON_TENSOR_CORES = True     # tests switch it off to compare with the CUDA-core kernel at the same shapes


def attention_sink(out, q, kv_pages, tables, batch, nq: int, nkv: int, dk: int, dv: int, scale: float, sinks=None,
                   window: int = 0, chunk: int = 0, slopes=None, keep_first: int = 0) -> None:
    """Attention of the step's tokens over the cache for layers with a sink and / or value heads of another size
    than their key heads: picks the kernel for the dtype and sizes.  bfloat16 with key and value heads of one size
    (in steps of 16) runs on the tensor cores like ``attention``; float32 and unequal head sizes on the CUDA cores."""
    if (SINK_ATTENTION_ON_TENSOR_CORES and q.dtype == torch.bfloat16 and dk == dv and kv_pages.shape[-1] == dk
            and kv_pages.shape[1] == 2 and attention_mma.supports(dk, nq, nkv, batch.n_seqs)):
        attention_tensor_core(out, q, kv_pages, tables.block_tables, batch.cu_q, batch.kv_len, batch.n_seqs,
                              batch.n_prefill_tokens, batch.n_prefill_seqs, batch.n_decode_seqs, batch.max_kv_len,
                              nq, nkv, dk, scale, window, sinks, chunk, slopes, keep_first)
        return
    attention_sink_simt(out, q, kv_pages, tables.block_tables, batch.cu_q, batch.kv_len, batch.n_seqs, batch.n_tokens,
                        nq, nkv, dk, dv, scale, sinks, window, chunk, slopes, keep_first)


def linear_f32(out, x, weight) -> None:
    """out[M,N] float32 = x[M,K] @ weight[N,K]^T with the 32-bit sums kept (no rounding to the storage type on the
    way): small projections whose results enter a recurrence or a softmax, and heads that return exact logits.
    float32 operands run the fixed-order kernel; bfloat16 operands one warp per output for few outputs, else the
    library product with a float32 result."""
    _need_cuda(out, x, weight)
    _contig("out", out); _contig("weight", weight)
    assert x.dim() == 2 and x.stride(1) == 1 and x.dtype == weight.dtype and out.dtype == torch.float32
    M, K = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == K and out.shape == (M, N)
    if x.dtype == torch.float32:
        call("nhv_gemm_nt_simt", F32, out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, N, K, x.stride(0), K, N, 0,
             stream_ptr())
    elif M * N <= LINEAR_F32_ROWS_LIMIT and K % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 \
            and weight.data_ptr() % 16 == 0:
        call("nhv_gemm_rows_f32", out.data_ptr(), N, x.data_ptr(), x.stride(0), weight.data_ptr(), K, M, N, K, stream_ptr())
    elif x.is_contiguous() and M * N > LINEAR_F32_ROWS_LIMIT:
        library.LAUNCHES += 1
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
    else:
        call("nhv_gemm_nt_simt", BF16, out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, N, K, x.stride(0), K, N, 1,
             stream_ptr())


LINEAR_F32_ROWS_LIMIT = 1 << 13     # outputs up to which a bfloat16 product with float32 sums runs one warp per output


def to_f32(out, x) -> None:
    _need_cuda(out, x)
    _contig("out", out); _contig("x", x)
    assert out.dtype == torch.float32 and out.numel() == x.numel()
    call("nhv_to_f32", dtype_code(x), out.data_ptr(), x.data_ptr(), x.numel(), stream_ptr())


def qk_norm_rope_store(qkv, q_out, kv_pages, slot_mapping, positions, q_weight, k_weight, cos_sin, rotary_dim: int,
                       nq: int, nkv: int, head_dim: int, eps: float, weight_offset: float = 0.0) -> None:
    """qkv [T, (nq+2nkv)*d] -> q_out [T, nq*d] (normed, rotated) and K/V rows in kv_pages
    [pages, 2, nkv, page_size, d] at slot_mapping.  kv_pages None: queries only."""
    _need_cuda(qkv, q_out, kv_pages, slot_mapping, positions, q_weight, k_weight, cos_sin)
    assert qkv.stride(-1) == 1 and q_out.stride(-1) == 1 and qkv.dim() == 2 and q_out.dim() == 2
    n_tokens = qkv.shape[0]
    if kv_pages is not None:
        _contig("kv_pages", kv_pages)
        n_pages, two, h, page_size, d = kv_pages.shape
        assert two == 2 and h == nkv and d == head_dim and kv_pages.dtype == qkv.dtype
        assert slot_mapping.dtype == torch.int32 and slot_mapping.numel() >= n_tokens
    else:
        n_pages, page_size = 0, 0
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] == rotary_dim
        assert positions.dtype == torch.int32
    call("nhv_qk_norm_rope_store", dtype_code(qkv), qkv.data_ptr(), qkv.stride(0), q_out.data_ptr(), q_out.stride(0),
         _ptr(kv_pages), _ptr(slot_mapping), _ptr(positions), _ptr(q_weight), _ptr(k_weight), _ptr(cos_sin),
         int(rotary_dim), 0 if cos_sin is None else cos_sin.shape[0], n_tokens, nq, nkv, head_dim, page_size, n_pages,
         float(eps), float(weight_offset), stream_ptr())


def attention_simt(out, q, kv_pages, block_table, cu_q, kv_len, n_seqs: int, n_tokens: int, nq: int, nkv: int,
                   head_dim: int, scale: float, window: int = 0) -> None:
    """Causal attention of this step's tokens over the pages: q [T, nq*d] -> out [T, nq*d]."""
    _need_cuda(out, q, kv_pages, block_table, cu_q, kv_len)
    _contig("kv_pages", kv_pages)
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and out.dtype == q.dtype == kv_pages.dtype
    n_pages, two, h, page_size, d = kv_pages.shape
    assert two == 2 and h == nkv and d == head_dim
    assert block_table.dtype == torch.int32 and block_table.stride(-1) == 1
    assert cu_q.dtype == torch.int32 and kv_len.dtype == torch.int32
    call("nhv_attention_simt", dtype_code(q), q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0),
         kv_pages.data_ptr(), block_table.data_ptr(), block_table.stride(0), cu_q.data_ptr(), kv_len.data_ptr(),
         n_seqs, n_tokens, nq, nkv, head_dim, page_size, n_pages, int(window), float(scale), stream_ptr())


def attention(out, q, kv_pages, tables, batch, nq: int, nkv: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Attention of the step's tokens over the cache: picks the kernel for the dtype and sizes.
    bfloat16 with a head size in steps of 16 runs on the tensor cores; everything else (float32, other
    head sizes, groups of more than 64 heads, more than 512 requests in the step) on the CUDA cores."""
    if q.dtype == torch.bfloat16 and attention_mma.supports(head_dim, nq, nkv, batch.n_seqs):
        attention_tensor_core(out, q, kv_pages, tables.block_tables, batch.cu_q, batch.kv_len, batch.n_seqs,
                              batch.n_prefill_tokens, batch.n_prefill_seqs, batch.n_decode_seqs, batch.max_kv_len,
                              nq, nkv, head_dim, scale, window)
    else:
        attention_simt(out, q, kv_pages, tables.block_tables, batch.cu_q, batch.kv_len, batch.n_seqs, batch.n_tokens,
                       nq, nkv, head_dim, scale, window)


FUSE_DECODE_QK = True             # tests switch it off to compare with the two-kernel form
USE_TMA_DECODE = True             # tests switch it off to reach the mma.sync decode kernel at the same shapes

_decode_scratch: dict = {}


def _tma_decode_scratch(device, head_dim: int, blocks: int):
    """Partial results of the decode kernel's split requests: two slots per block, kept for the life of the
    process (every launch writes a slot before any block reads it)."""
    key = (device, head_dim)
    st = _decode_scratch.get(key)
    if st is None:
        st = _decode_scratch[key] = (torch.empty(blocks * 2 * 16 * head_dim, dtype=torch.float32, device=device),
                                     torch.empty(blocks * 2 * 16 * 2, dtype=torch.float32, device=device))
    return st


def _attention_decode_tma(out, q, qkv, kv_pages, block_table, batch_cu_q, batch_kv_len, n_seqs: int, nq: int, nkv: int,
                          head_dim: int, scale: float, window: int, q_weight=None, k_weight=None, cos_sin=None,
                          positions=None, slot_mapping=None, rotary_dim: int = 0, eps: float = 0.0,
                          weight_offset: float = 0.0, store: bool = False, sinks=None, chunk: int = 0,
                          keep_first: int = 0) -> None:
    launch, blocks = attention_decode.get(head_dim)
    n_pages, two, h, page_size, d = kv_pages.shape
    group = nq // nkv
    head_blocks = nkv * -(-group // 16)
    part_o, part_ml = _tma_decode_scratch(out.device, head_dim, blocks)
    counters = _decode_counters(out.device, n_seqs * head_blocks)
    library.LAUNCHES += 1
    launch(_ptr(q), 0 if q is None else q.stride(0), _ptr(qkv), 0 if qkv is None else qkv.stride(0), out.data_ptr(),
           out.stride(0), kv_pages.data_ptr(), block_table.data_ptr(), block_table.stride(0), batch_cu_q.data_ptr(),
           batch_kv_len.data_ptr(), n_seqs, nq, nkv, page_size, n_pages, int(window), int(chunk), float(scale), part_o.data_ptr(),
           part_ml.data_ptr(), counters.data_ptr(), _ptr(q_weight), _ptr(k_weight), _ptr(cos_sin), _ptr(positions),
           _ptr(slot_mapping), int(rotary_dim), 0 if cos_sin is None else cos_sin.shape[0], 1 if store else 0, float(eps),
           float(weight_offset), _ptr(sinks), int(keep_first), stream_ptr())


def attention_decode_fused(out, qkv, kv_pages, tables, batch, nq: int, nkv: int, head_dim: int, scale: float,
                           window: int, q_weight, k_weight, cos_sin, rotary_dim: int, eps: float,
                           weight_offset: float, store: bool, chunk: int = 0) -> bool:
    """A step of single tokens only, in bfloat16: attention straight from the projection's output.  The decode
    kernel norms and rotates the new query and key heads itself and stores the new keys and values (what
    ``qk_norm_rope_store`` does otherwise, in a launch of its own).  Returns False, having done nothing, when
    the step or the shapes do not allow it."""
    if not (FUSE_DECODE_QK and qkv.dtype == torch.bfloat16 and batch.n_prefill_seqs == 0 and batch.n_decode_seqs > 0
            and attention_mma.supports(head_dim, nq, nkv, batch.n_seqs)):
        return False
    if qkv.stride(0) % 8 or qkv.data_ptr() % 16:
        return False
    vec = head_dim // 32
    if head_dim % 32 or (cos_sin is not None and (rotary_dim <= 0 or rotary_dim % (2 * vec))):
        return False
    _need_cuda(out, qkv, kv_pages, q_weight, k_weight, cos_sin)
    _contig("kv_pages", kv_pages)
    n_pages, two, h, page_size, d = kv_pages.shape
    assert two == 2 and h == nkv and d == head_dim and kv_pages.dtype == qkv.dtype and out.stride(-1) == 1
    block_table = tables.block_tables
    assert block_table.dtype == torch.int32 and block_table.stride(-1) == 1
    n_seqs = batch.n_seqs
    if USE_TMA_DECODE and attention_decode.supports(head_dim, nq, nkv, page_size, n_seqs):
        _attention_decode_tma(out, None, qkv, kv_pages, block_table, batch.cu_q, batch.kv_len, n_seqs, nq, nkv, head_dim,
                              scale, window, q_weight, k_weight, cos_sin, batch.positions, tables.slot_mapping, rotary_dim,
                              eps, weight_offset, store, chunk=chunk)
        return True
    launch_fused = attention_mma.get(head_dim)[2]
    if launch_fused is None:
        return False
    tile = attention_mma.get(head_dim)[1]
    group = nq // nkv
    rows, head_blocks = min(group, 16), nkv * -(-group // 16)
    max_pieces = -(-batch.max_kv_len // tile) + 1
    scratch_o = torch.empty(n_seqs * head_blocks * max_pieces * rows * head_dim, dtype=torch.float32, device=qkv.device)
    scratch_ml = torch.empty(n_seqs * head_blocks * max_pieces * rows * 2, dtype=torch.float32, device=qkv.device)
    counters = _decode_counters(qkv.device, n_seqs * head_blocks)
    library.LAUNCHES += 1
    launch_fused(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), kv_pages.data_ptr(), block_table.data_ptr(),
                 block_table.stride(0), batch.cu_q.data_ptr(), batch.kv_len.data_ptr(), n_seqs, nq, nkv, page_size,
                 n_pages, int(window), int(chunk), float(scale), scratch_o.data_ptr(), scratch_ml.data_ptr(), counters.data_ptr(),
                 max_pieces, _ptr(q_weight), _ptr(k_weight), _ptr(cos_sin), batch.positions.data_ptr(),
                 tables.slot_mapping.data_ptr(), int(rotary_dim), 0 if cos_sin is None else cos_sin.shape[0],
                 1 if store else 0, float(eps), float(weight_offset), stream_ptr())
    return True


USE_TCGEN05_ATTENTION = True      # tests switch it off to reach the mma.sync prompt kernel at the same shapes


def attention_tcgen05_error(head_dim: int) -> int:
    """The error word of the tcgen05 attention kernel's bounded waits (0 = none)."""
    return attention_tcgen05.get(head_dim)[1]()


def attention_tensor_core(out, q, kv_pages, block_table, cu_q, kv_len, n_seqs: int, n_prefill_tokens: int,
                          n_prefill_seqs: int, n_decode_seqs: int, max_kv_len: int, nq: int, nkv: int, head_dim: int,
                          scale: float, window: int = 0, sinks=None, chunk: int = 0, slopes=None, keep_first: int = 0) -> None:
    """bfloat16 attention on the tensor cores.  Prompt portions go to the tcgen05 kernel, requests with
    one new token to the kernel that streams the cache with TMA, each where its shape is supported; what
    neither takes runs in the mma.sync kernel, whose single-token path shares a request's tiles between
    blocks and merges them (scratch: one partial result per piece of a request and head block).
    ``sinks`` [nq] float32: exp(sink) joins each head's softmax denominator once (where the head's sum is final).
    ``slopes`` [nq] float32: head h's score loses slopes[h] times the distance between query and key; the tcgen05 and
    the mma.sync kernels take them, the TMA kernel for single tokens does not, so those run in the mma.sync kernel.
    ``keep_first`` > 0 (with a window): the keys at positions below it stay visible; in every kernel their tiles come
    before the window's."""
    _need_cuda(out, q, kv_pages, block_table, cu_q, kv_len, sinks, slopes)
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == nq and sinks.is_contiguous())
    assert slopes is None or (slopes.dtype == torch.float32 and slopes.numel() == nq and slopes.is_contiguous())
    _contig("kv_pages", kv_pages)
    assert q.dtype == out.dtype == kv_pages.dtype == torch.bfloat16 and q.stride(-1) == 1 and out.stride(-1) == 1
    n_pages, two, h, page_size, d = kv_pages.shape
    assert two == 2 and h == nkv and d == head_dim
    assert block_table.dtype == torch.int32 and block_table.stride(-1) == 1
    launch, tile = attention_mma.get(head_dim)[:2]
    if (n_prefill_tokens > 0 and USE_TCGEN05_ATTENTION and (slopes is None or scale > 0)
            and attention_tcgen05.supports(head_dim, nq, nkv, page_size)):
        # prompt portions on the 5th-generation tensor cores; single tokens stay with the split kernel below
        library.LAUNCHES += 1
        attention_tcgen05.get(head_dim)[0](
            q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kv_pages.data_ptr(), block_table.data_ptr(),
            block_table.stride(0), cu_q.data_ptr(), kv_len.data_ptr(), n_seqs, n_prefill_tokens, n_prefill_seqs,
            nq, nkv, page_size, n_pages, int(window), int(chunk), float(scale), _ptr(sinks), _ptr(slopes), int(keep_first),
            stream_ptr())
        if n_decode_seqs == 0:
            return
        n_prefill_tokens = n_prefill_seqs = 0
    if (n_decode_seqs > 0 and slopes is None and USE_TMA_DECODE
            and attention_decode.supports(head_dim, nq, nkv, page_size, n_seqs)):
        # single tokens: the kernel that streams the cache with TMA; what is left for the launch below are the
        # prompt portions (if the tcgen05 kernel did not take them)
        _attention_decode_tma(out, q, None, kv_pages, block_table, cu_q, kv_len, n_seqs, nq, nkv, head_dim, scale, window,
                              sinks=sinks, chunk=chunk, keep_first=keep_first)
        if n_prefill_tokens == 0:
            return
        n_decode_seqs = 0
    scratch_o = scratch_ml = counters = None
    max_pieces = blocks = 0
    if n_decode_seqs > 0:
        # scratch for requests whose tiles are shared between blocks: one partial result per piece, and a
        # zeroed arrival counter per (request, head block) that the kernel leaves zeroed
        group = nq // nkv
        rows, head_blocks = min(group, 16), nkv * -(-group // 16)
        max_pieces = -(-max_kv_len // tile) + 1
        blocks = 3 * _sm_count(q.device)
        scratch_o = torch.empty(n_seqs * head_blocks * max_pieces * rows * head_dim, dtype=torch.float32, device=q.device)
        scratch_ml = torch.empty(n_seqs * head_blocks * max_pieces * rows * 2, dtype=torch.float32, device=q.device)
        counters = _decode_counters(q.device, n_seqs * head_blocks)
    library.LAUNCHES += 1
    launch(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kv_pages.data_ptr(), block_table.data_ptr(),
           block_table.stride(0), cu_q.data_ptr(), kv_len.data_ptr(), n_seqs, n_prefill_tokens, n_prefill_seqs,
           n_decode_seqs, nq, nkv, page_size, n_pages, int(window), int(chunk), float(scale), _ptr(scratch_o), _ptr(scratch_ml),
           _ptr(counters), max_pieces, blocks, _ptr(sinks), _ptr(slopes), int(keep_first), stream_ptr())


_sm_counts: dict = {}
_counter_buffers: dict = {}


def _sm_count(device) -> int:
    if device not in _sm_counts:
        _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_counts[device]


def _decode_counters(device, n: int) -> torch.Tensor:
    """Zeroed ints that outlive the step (the decode kernel returns them to zero)."""
    buf = _counter_buffers.get(device)
    if buf is None or buf.numel() < n:
        buf = _counter_buffers[device] = torch.zeros(max(n, 16384), dtype=torch.int32, device=device)
    return buf


def linear(out, x, weight) -> None:
    """out[M,N] = x[M,K] @ weight[N,K]^T.  out may be float32 while x and weight are bfloat16."""
    _need_cuda(out, x, weight)
    _contig("out", out); _contig("weight", weight)
    assert x.dim() == 2 and weight.dim() == 2 and x.stride(1) == 1 and x.dtype == weight.dtype
    M, K = x.shape
    N = weight.shape[0]
    assert weight.shape[1] == K and out.shape == (M, N)
    if x.dtype == torch.float32:
        assert out.dtype == torch.float32
        call("nhv_gemm_nt_simt", F32, out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, N, K, x.stride(0), K, N, 0,
             stream_ptr())
    elif small_m_ok(x, weight):
        _small_m(out, x, weight, M, N, K, int(out.dtype == torch.float32), 0)
    elif out.dtype == torch.float32:
        # the product is rounded to bfloat16 and then widened, as the reference's head does
        # (nanovllm/layers/embed_head.py:61, nanovllm/layers/sampler.py:12)
        tmp = torch.empty(M, N, dtype=x.dtype, device=x.device)
        torch.mm(x, weight.t(), out=tmp)
        to_f32(out, tmp)
    else:
        torch.mm(x, weight.t(), out=out)


SMALL_M = 8     # up to this many tokens the weight-streaming kernel runs instead of the library product
                # (measured on B200: it is ahead up to 8 tokens, the library from 9 on; the kernel itself takes 16)


def small_m_ok(x, weight) -> bool:
    return (x.dtype == torch.bfloat16 and x.shape[0] <= SMALL_M and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def swiglu_first_half(act, x, gate_up_weight) -> bool:
    """act[M, I] = silu(x Wg^T) * (x Wu^T) in one kernel when the batch is small enough for the
    weight-streaming kernel (gate_up_weight [2 I, K], gate rows first).  Returns False if it did not run."""
    if not small_m_ok(x, gate_up_weight):
        return False
    _need_cuda(act, x, gate_up_weight)
    _contig("act", act); _contig("gate_up_weight", gate_up_weight)
    M, K = x.shape
    inter = gate_up_weight.shape[0] // 2
    assert act.shape == (M, inter) and act.dtype == torch.bfloat16 and gate_up_weight.shape[1] == K
    _small_m(act, x, gate_up_weight, M, inter, K, 2, inter)
    return True


_stream_k_state: dict = {}
STREAM_K_COUNTERS = 8192


def _small_m(out, x, weight, M: int, N: int, K: int, mode: int, up_row_offset: int) -> None:
    """The weight-streaming product for up to 16 tokens: the persistent TMA kernel, one block per SM, with
    its scratch (partial sums of tiles that two blocks share, and the tiles' arrival counters)."""
    dev = x.device
    st = _stream_k_state.get(dev)
    if st is None:
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        st = _stream_k_state[dev] = (sms, torch.zeros(sms * 2 * 64 * 16, dtype=torch.float32, device=dev),
                                     torch.zeros(STREAM_K_COUNTERS, dtype=torch.int32, device=dev))
    sms, scratch, counters = st
    tiles = -(-N // (32 if mode == 2 else 64))
    slab = _slabs.get(weight.data_ptr())
    if slab is not None and slab[0]() is weight and slab[2] == mode and M <= SLAB_MAX_M:
        _slab_product(out, x, slab[1], M, N, K, mode, sms)
        return
    if tiles > STREAM_K_COUNTERS:
        call("nhv_gemm_small_m", out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, N, K, x.stride(0), N, mode,
             up_row_offset, stream_ptr())
        return
    call("nhv_gemm_stream_k", out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, N, K, x.stride(0), N, mode,
         up_row_offset, scratch.data_ptr(), counters.data_ptr(), STREAM_K_COUNTERS, sms, stream_ptr())


def _slab_product(out, x, copy, M: int, N: int, K: int, mode: int, sms: int) -> None:
    """The product from the per-SM copy, with a hint for the one after it.  A decode step runs the same products in
    the same order every time, so each remembers which copy was read right after its own last time; its blocks then
    ask the first bytes of that copy into L2 as they send for their own last stage, and the next product's ring
    fills from L2 instead of HBM (measured on B200 over the four products of an 8B-sized layer: 72.1 -> 70.1 us).
    Only a hint, and only between copies that were made together (``new_slab_family``: one model's copies live and
    die together, so a captured launch never names memory that has been given back); a copy that is gone or unknown
    gets none."""
    global _slab_last
    key = copy.data_ptr()
    family = _slab_family.get(key)
    if (_slab_last is not None and _slab_last != key and SLAB_HINT_BYTES and family is not None
            and _slab_family.get(_slab_last) == family):
        _slab_after[_slab_last] = (weakref.ref(copy), key, copy.numel() * copy.element_size())
    _slab_last = key
    hint = _slab_after.get(key)
    nxt = hint[0]() if hint is not None else None
    if nxt is not None and nxt.data_ptr() == hint[1] and nxt.numel() * nxt.element_size() == hint[2] and SLAB_HINT_BYTES:
        blocks = min(sms, _slab_blocks.get(hint[1], 0))
        if blocks > 0:
            call("nhv_gemm_slab_hint", out.data_ptr(), x.data_ptr(), key, M, N, K, x.stride(0), N, mode, sms, hint[1],
                 hint[2] // blocks, SLAB_HINT_BYTES, blocks, stream_ptr())
            return
    call("nhv_gemm_slab", out.data_ptr(), x.data_ptr(), key, M, N, K, x.stride(0), N, mode, sms, stream_ptr())


# of the next product's copy, per block, asked into L2 ahead (0: no hints; NHV_SLAB_HINT_BYTES overrides it)
SLAB_HINT_BYTES = int(os.environ.get("NHV_SLAB_HINT_BYTES", "65536"))
_slab_after: dict = {}  # data pointer of a copy -> (weak reference to the copy read after it last time, its pointer, its bytes)
_slab_blocks: dict = {} # data pointer of a copy -> the blocks that share it
_slab_family: dict = {} # data pointer of a copy -> the family it was made in
_family = 0


def new_slab_family() -> None:
    """The copies made from here on belong together (a model's: the runner says so before it makes them)."""
    global _family
    _family += 1


_slab_last = None       # data pointer of the copy that the last product read
SLAB_MAX_M = 8          # tokens that csrc/gemm_slab.cu takes
_slabs: dict = {}       # data pointer of a weight matrix -> (weak reference to it, its copy for gemm_slab.cu, mode)


def slab_copy_bytes(weight: torch.Tensor, mode: int) -> int:
    n, k = weight.shape
    geo = slab_geometry(n // 2 if mode == 2 else n, k, mode, _sm_count(weight.device))
    return geo["blocks"] * geo["slab_bytes"]


def can_stream_slabs(weight: torch.Tensor, mode: int) -> bool:
    return (weight.is_cuda and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.shape[1] % 8 == 0
            and weight.shape[0] >= (2 if mode == 2 else 1))


def prepare_streaming(weight: torch.Tensor, mode: int) -> int:
    """Keep a second copy of ``weight`` laid out for ``csrc/gemm_slab.cu`` (``slab_weight``); products of up to 8
    tokens with this matrix in this mode then read the copy: one share of rows per SM, every stage of the kernel's
    ring one contiguous copy of up to 32 KB, no sums across blocks.  Measured on B200 for the four matrices of an
    8B-sized layer: 73 us, against 87 us for the stream-K kernel on the row-major matrix (64 pieces of 512 bytes a
    row apart per stage, and a fix-up of shared tiles at the end of every launch).  The copy lives as long as the
    matrix.  Returns the bytes it takes (0 if the matrix cannot be streamed this way)."""
    if not can_stream_slabs(weight, mode):
        return 0
    key = weight.data_ptr()
    old = _slabs.get(key)
    if old is not None and old[0]() is weight and old[2] == mode:
        return 0
    copy = slab_weight(weight, mode, _sm_count(weight.device))
    n = weight.shape[0] // 2 if mode == 2 else weight.shape[0]
    _slab_blocks[copy.data_ptr()] = slab_geometry(n, weight.shape[1], mode, _sm_count(weight.device))["blocks"]
    _slab_family[copy.data_ptr()] = _family
    _slabs[key] = (weakref.ref(weight), copy, mode)
    weakref.finalize(weight, _drop_slab, key, copy.data_ptr())
    return copy.numel() * copy.element_size()


def _drop_slab(key: int, copy_ptr: int) -> None:
    entry = _slabs.get(key)
    if entry is not None and entry[1].data_ptr() == copy_ptr:
        del _slabs[key]
    _slab_blocks.pop(copy_ptr, None)
    _slab_after.pop(copy_ptr, None)
    _slab_family.pop(copy_ptr, None)


def slab_geometry(N: int, K: int, mode: int, sms: int) -> dict:
    """How ``csrc/gemm_slab.cu`` cuts a matrix with N result columns and K columns on a device with ``sms`` SMs."""
    import ctypes
    blocks, rpb, nb, ks = (ctypes.c_int() for _ in range(4))
    slab_bytes = ctypes.c_longlong()
    call("nhv_gemm_slab_geometry", N, K, mode, sms, ctypes.addressof(blocks), ctypes.addressof(rpb), ctypes.addressof(nb),
         ctypes.addressof(ks), ctypes.addressof(slab_bytes))
    return dict(blocks=blocks.value, rpb=rpb.value, nb=nb.value, ks=ks.value, slab_bytes=slab_bytes.value)


def slab_weight(weight: torch.Tensor, mode: int, sms: int) -> torch.Tensor:
    """The copy of a weight matrix [N, K] (mode 2: [gate rows; up rows]) that ``linear_slab`` reads: one share of
    rows per block, walked in sub-tiles of up to 64 rows over stages of nb * 64 columns; the bytes of a stage lie
    together, box by box (64 columns), row by row (128 bytes; mode 2: a sub-tile's gate rows, then its up rows), the
    16-byte chunks of row r of a box exchanged by c ^ (r & 7).  Rows and columns beyond the matrix are zeros."""
    assert weight.dtype == torch.bfloat16 and weight.dim() == 2
    rows, K = weight.shape
    N = rows // 2 if mode == 2 else rows
    geo = slab_geometry(N, K, mode, sms)
    G, r, nb, ks = geo["blocks"], geo["rpb"], geo["nb"], geo["ks"]
    th = 32 if mode == 2 else 64
    k_pad = ks * nb * 64

    def padded(part):                                    # [N, K] -> [G, r, ks, nb, 8 chunks, 8 elements]
        w = torch.zeros(G * r, k_pad, dtype=weight.dtype, device=weight.device)
        w[:N, :K] = part
        return w.view(G, r, ks, nb, 8, 8)

    kinds = [padded(weight[:N]), padded(weight[N:])] if mode == 2 else [padded(weight)]
    chunk = torch.arange(8, device=weight.device)
    pieces = []
    for t0 in range(0, r, th):
        h = min(th, r - t0)
        sub = torch.cat([kind[:, t0:t0 + h] for kind in kinds], 1)                           # [G, rows of the box, ks, nb, 8, 8]
        rows_t = sub.shape[1]
        src = chunk[None, :] ^ (torch.arange(rows_t, device=weight.device)[:, None] & 7)     # [rows, 8]: where chunk c' comes from
        sub = torch.gather(sub, 4, src[None, :, None, None, :, None].expand(G, rows_t, ks, nb, 8, 8))
        pieces.append(sub.permute(0, 2, 3, 1, 4, 5).reshape(G, -1))                          # [G, ks, nb, rows, 64]
    out = torch.cat(pieces, 1).contiguous()
    assert out.shape[1] * 2 == geo["slab_bytes"], (out.shape, geo)
    return out.view(-1)


def linear_slab(out, x, slabs, N: int, mode: int, sms: int) -> None:
    """out [M, N] = x [M, K] @ W^T for up to 8 tokens from the copy made by ``slab_weight`` (mode 2: silu(gate) * up)."""
    _need_cuda(out, x, slabs)
    M, K = x.shape
    call("nhv_gemm_slab", out.data_ptr(), x.data_ptr(), slabs.data_ptr(), M, N, K, x.stride(0), out.stride(0), mode, sms,
         stream_ptr())


def slab_error() -> int:
    """0 unless a bounded wait inside the slab product ever ran out (synchronises the device)."""
    from .library import load_library
    return load_library().nhv_gemm_slab_error()


_tcgen05_state: dict = {}


def linear_tcgen05(out, x, weight, mode: int = 0, up_row_offset: int = 0) -> None:
    """out = x @ weight^T for 1 to 128 tokens with tcgen05.mma and tensor-memory accumulators
    (csrc/gemm_tcgen05.cu).  mode 0: out bfloat16; 1: out float32 through bfloat16; 2: weight = [gate; up] rows,
    out = silu(gate) * up.  Not on the default path: measured on B200 at the 8B layer sizes the library product is
    still 1.2 to 5 times faster for 32 to 128 tokens; the kernel is kept tested and callable."""
    _need_cuda(out, x, weight)
    _contig("out", out); _contig("weight", weight)
    assert x.dtype == weight.dtype == torch.bfloat16 and x.stride(1) == 1
    M, K = x.shape
    N = out.shape[1]
    dev = x.device
    st = _tcgen05_state.get(dev)
    if st is None:
        sms = _sm_count(dev)
        st = _tcgen05_state[dev] = (sms, torch.zeros(sms * 2 * 128 * 128, dtype=torch.float32, device=dev),
                                    torch.zeros(STREAM_K_COUNTERS, dtype=torch.int32, device=dev))
    sms, scratch, counters = st
    call("nhv_gemm_tcgen05", out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, N, K, x.stride(0), N, mode, up_row_offset,
         scratch.data_ptr(), counters.data_ptr(), STREAM_K_COUNTERS, sms, stream_ptr())


def tcgen05_error() -> int:
    """0 unless a bounded wait inside the tcgen05 product ever ran out (synchronises the device)."""
    from .library import load_library
    return load_library().nhv_gemm_tcgen05_error()


def linear_stream_k(out, x, weight, mode: int = 0, up_row_offset: int = 0) -> None:
    """The weight-streaming product for 1 to 16 tokens, whatever `SMALL_M` says (tests, experiments).
    mode 0: out bfloat16; out float32 selects mode 1; mode 2: weight = [gate; up], out = silu(gate) * up."""
    _need_cuda(out, x, weight)
    _contig("out", out); _contig("weight", weight)
    M, K = x.shape
    if mode == 0 and out.dtype == torch.float32:
        mode = 1
    _small_m(out, x, weight, M, out.shape[1], K, mode, up_row_offset)


def stream_k_error() -> int:
    """0 unless a bounded wait inside the streaming product ever ran out (synchronises the device)."""
    from .library import load_library
    return load_library().nhv_gemm_stream_k_error()


def linear_simt(out, x, weight) -> None:
    """The fixed-order CUDA-core product for any storage type (tests, and sizes a fast kernel refuses)."""
    _need_cuda(out, x, weight)
    M, K = x.shape
    N = weight.shape[0]
    call("nhv_gemm_nt_simt", dtype_code(x), out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, N, K, x.stride(0), K,
         N, int(out.dtype == torch.float32 and x.dtype != torch.float32), stream_ptr())


# ---------------------------------------------------------------- bounded waits that ran out
# Kernels that wait on mbarriers bound their waits; one that runs out sets its file's error word and the kernel
# leaves with whatever it has, so the step's results are not valid.  The words reach the host with the step's
# tokens: the sampler folds them into one more int behind the tokens (``sample`` below), and callers that read
# logits instead ask ``take_wait_errors`` once per step.
ERROR_WORD_SLOTS = 16
_wait_error_sources: list = []          # (name, function giving the word's device address, function that reads and clears it)
_error_word_arrays: dict = {}           # device -> (int64 tensor [ERROR_WORD_SLOTS] of addresses, sources filled in)


def register_wait_error_source(name: str, address_fn, take_fn) -> None:
    if all(n != name for n, _, _ in _wait_error_sources):
        if len(_wait_error_sources) >= ERROR_WORD_SLOTS:
            raise KernelError("more kernels with error words than the step's health word has bits")
        _wait_error_sources.append((name, address_fn, take_fn))


def _register_library_sources() -> None:
    import ctypes
    from .library import load_library
    lib = load_library()
    for name in ("gemm_slab", "gemm_stream_k", "gemm_tcgen05", "moe_tcgen05"):
        word = getattr(lib, f"nhv_{name}_error_word")
        word.restype, word.argtypes = ctypes.c_void_p, []
        take = getattr(lib, f"nhv_{name}_error")
        take.restype, take.argtypes = ctypes.c_int, []
        register_wait_error_source(name, word, take)


def error_word_array(device) -> torch.Tensor:
    """Device array of the addresses of all error words known so far (zeros where there is none yet).  The
    array's own address never changes, so a captured step sees words registered after its capture too."""
    _register_library_sources()
    device = torch.device(device)
    entry = _error_word_arrays.get(device)
    if entry is None:
        entry = _error_word_arrays[device] = [torch.zeros(ERROR_WORD_SLOTS, dtype=torch.int64, device=device), 0]
    arr, filled = entry
    if filled < len(_wait_error_sources):
        with torch.cuda.device(device):
            addresses = [fn() or 0 for _, fn, _ in _wait_error_sources[filled:]]
        arr[filled:len(_wait_error_sources)] = torch.tensor(addresses, dtype=torch.int64)
        entry[1] = len(_wait_error_sources)
    return arr


def take_wait_errors() -> list[tuple[str, int]]:
    """(kernel, code) of every bounded wait that ran out since the last call; the words are cleared.
    Synchronises the device."""
    _register_library_sources()
    out = []
    for name, _, take in _wait_error_sources:
        code = take()
        if code != 0:
            out.append((name, code))
    return out


def raise_wait_errors() -> None:
    """Raise ``KernelError`` naming the kernels whose bounded waits ran out, if any did."""
    bad = take_wait_errors()
    if bad:
        raise KernelError("a bounded wait ran out in " + ", ".join(f"{n} (code {c})" for n, c in bad) +
                          ": the kernel gave up and left, and the results of the step are not valid")


def sample(out, logits, temperatures, seeds, positions) -> None:
    """out[r] = the token chosen from logits[r] (float32): argmax if temperatures[r] == 0, else the
    exponential race with noise keyed by (seeds[r], positions[r]).  ``out`` may have one element more than
    ``logits`` has rows: it receives the step's health word (bit i set: the i-th registered error word of a
    kernel with bounded waits is not zero; 0 means that all is well), which the host reads with the tokens."""
    _need_cuda(out, logits, temperatures, seeds, positions)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert temperatures.dtype == torch.float32 and seeds.dtype == torch.int64 and positions.dtype == torch.int32
    rows = logits.shape[0]
    st = _sampler_scratch.get(logits.device)
    if st is None or st[0].numel() < rows:
        # where the blocks that share a row meet: zero, and left zero by every launch
        n = max(rows, 512)
        if st is not None:
            _sampler_retired.append(st)      # a captured step may still point at the smaller ones
        st = _sampler_scratch[logits.device] = (torch.zeros(n, dtype=torch.int64, device=logits.device),
                                                torch.zeros(n, dtype=torch.int32, device=logits.device))
    words = status = None
    if out.numel() == rows + 1:
        words, status = error_word_array(logits.device).data_ptr(), out.data_ptr() + 4 * rows
    else:
        assert out.numel() == rows
    call("nhv_sample", out.data_ptr(), logits.data_ptr(), logits.stride(0), temperatures.data_ptr(), seeds.data_ptr(),
         positions.data_ptr(), rows, logits.shape[1], st[0].data_ptr(), st[1].data_ptr(), words, ERROR_WORD_SLOTS, status,
         stream_ptr())


_sampler_scratch: dict = {}
_sampler_retired: list = []
