"""Python faces of the CUDA kernels: one function per entry point.

Each function checks what the kernel cannot (device, layout, element type), passes
raw pointers and the current CUDA stream, and turns a non-zero status into an
exception.  Nothing here computes: without a CUDA device or the compiled
extension the functions raise; there is no other implementation to fall back to.
The parts of a model call these through the module (`ops.rmsnorm(...)`), so a test
can put a stand-in in a function's place.

`launches` counts the kernel launches issued through this module (a captured CUDA
graph replays its launches without passing here; the engine adds those itself).
"""
from __future__ import annotations

import functools

import ctypes
from ctypes import c_float, c_void_p

import torch

from .build import KernelBuildError, load_family

launches = 0

_F32, _BF16 = 0, 1
_sms = None


def sm_count() -> int:
    """Multiprocessors of the current CUDA device (148 on a B200); every launch plan below is sized from it.
    Without a device (the plans are also exercised on the host) the B200's number stands in."""
    global _sms
    if _sms is None:
        _sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count \
            if torch.cuda.is_available() else 148
    return _sms
_STATUS = {1: "element type not supported", 2: "size not supported", 3: "pointer or stride not aligned",
           4: "size beyond the entry point's fixed scratch", 5: "device set-up failed"}


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"element type {t.dtype} not supported (float32 or bfloat16)")


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the engine's kernels run on a CUDA device only; got a tensor on " + str(t.device))


def _ptr(t) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream of the current device (it changes under a graph capture, so it is looked up at every
    launch; the raw lookup costs a fraction of a microsecond where the Stream object costs fifteen)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(status: int, what: str) -> None:
    global launches
    if status == 0:
        launches += 1
        return
    if status >= 1000:
        raise KernelError(f"{what}: CUDA launch failed with error {status - 1000}")
    raise KernelError(f"{what}: {_STATUS.get(status, 'status ' + str(status))}")


def _int32(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")
    return t


def embed_gather(ids: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor,
                 pos_table: torch.Tensor | None = None, positions: torch.Tensor | None = None) -> torch.Tensor:
    """out[n, :] = float(table[ids[n], :]) * scale (+ float(pos_table[positions[n], :]) with a table of learned
    position rows); `out` is the float32 residual stream."""
    _need_cuda(ids, table, out, pos_table, positions)
    n, (V, H) = ids.shape[0], table.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape == (n, H) and table.is_contiguous()
    P = 0
    if pos_table is not None:
        P = pos_table.shape[0]
        assert pos_table.shape == (P, H) and pos_table.is_contiguous() and pos_table.dtype == table.dtype
        assert positions is not None and positions.shape[0] == n
        positions = _int32(positions, "positions")
    lib = load_family("embedding")
    _check(lib.wllm_embed_gather_pos(_ptr(_int32(ids, "ids")), _ptr(table), _dt(table), c_float(scale), _ptr(out),
                                     n, H, V, _ptr(pos_table), _ptr(positions if pos_table is not None else None), P,
                                     _stream()), "embed_gather")
    return out


def patch_tokens(ids: torch.Tensor, dst: torch.Tensor, sampled: torch.Tensor, src: torch.Tensor) -> None:
    """ids[dst[i]] = sampled[src[i]] on the device: tokens that the previous step sampled and the host has
    not read yet become inputs of this step."""
    _need_cuda(ids, dst, sampled, src)
    n = dst.shape[0]
    assert src.shape[0] == n
    lib = load_family("embedding")
    _check(lib.wllm_patch_tokens(_ptr(_int32(ids, "ids")), _ptr(_int32(dst, "dst")), _ptr(_int32(sampled, "sampled")),
                                 _ptr(_int32(src, "src")), n, _stream()), "patch_tokens")


def rmsnorm(resid: torch.Tensor, delta, weight, eps: float, offset: float, out: torch.Tensor,
            rows=None, delta_splits: int = 0, center: bool = False) -> torch.Tensor:
    """Fold `delta` into the residual (when given), then norm: see csrc/norm.cu.  With `delta_splits` = S > 0,
    `delta` is [S, n, H] float32 partial sums that are added in order.  `center`: the row's mean is taken off
    first (a layer norm without a bias).  `weight` None: nothing is normed, `out` is the residual's rows rounded to
    its element type."""
    _need_cuda(resid, delta, weight, out, rows)
    H = resid.shape[1]
    n = rows.shape[0] if rows is not None else resid.shape[0]
    assert resid.dtype == torch.float32 and resid.is_contiguous() and out.is_contiguous() and out.shape == (n, H)
    assert weight is None or (weight.shape == (H,) and weight.is_contiguous())
    split_stride = 0
    if delta is not None:
        assert delta.is_contiguous()
        if delta_splits:
            assert delta.shape == (delta_splits,) + tuple(resid.shape) and delta.dtype == torch.float32
            split_stride = resid.numel()
        else:
            assert delta.shape == resid.shape
    lib = load_family("norm")
    _check(lib.wllm_norm(_ptr(resid), _ptr(delta), _dt(delta) if delta is not None else _F32, max(1, delta_splits),
                         ctypes.c_longlong(split_stride), _ptr(weight), _dt(weight) if weight is not None else _F32, c_float(eps), c_float(offset),
                         1 if center else 0, _ptr(out), _dt(out), _ptr(_int32(rows, "rows") if rows is not None else None),
                         n, H, _stream()), "norm")
    return out


def _branch_args(branch, n: int, H: int):
    """(tensor, parts) of a branch output as the kernels take it: pointer, element type, parts, stride between parts."""
    t, parts = branch
    assert t.is_contiguous() and t.shape[-2:] == (n, H)
    if parts:
        assert t.dtype == torch.float32 and t.shape[0] == parts
    return _ptr(t), _dt(t), max(1, parts), ctypes.c_longlong(n * H if parts else 0)


def branch_norm(a, weight_a: torch.Tensor, out: torch.Tensor, eps: float, center: bool = False, factor: float = 1.0,
                b=None, weight_b: torch.Tensor | None = None, offset: float = 0.0) -> torch.Tensor:
    """out[n, H] (float32) = factor * (norm(a) * (offset + weight_a) [+ norm(b) * (offset + weight_b)]) for branch outputs
    that are not part of the residual yet.  `a`, `b`: (tensor [n, H] or float32 partial sums [S, n, H], S or 0), as ops.project returns
    them.  `center`: layer norm without a bias, else root mean square (csrc/norm.cu)."""
    n, H = out.shape
    _need_cuda(a[0], weight_a, out, b[0] if b is not None else None, weight_b)
    assert out.dtype == torch.float32 and out.is_contiguous() and weight_a.shape == (H,) and weight_a.is_contiguous()
    pa = _branch_args(a, n, H)
    if b is not None:
        assert weight_b is not None and weight_b.shape == (H,) and weight_b.dtype == weight_a.dtype and weight_b.is_contiguous()
        pb = _branch_args(b, n, H)
    else:
        pb = (_ptr(None), _F32, 1, ctypes.c_longlong(0))
    lib = load_family("norm")
    _check(lib.wllm_branch_norm_offset(*pa, _ptr(weight_a), *pb, _ptr(weight_b), _dt(weight_a), c_float(eps), 1 if center else 0,
                                       c_float(factor), c_float(offset), _ptr(out), n, H, _stream()), "branch_norm")
    return out


def sandwich_norm(resid: torch.Tensor, a, out: torch.Tensor, post_weight: torch.Tensor, post_center: bool, post_eps: float,
                  weight, offset: float, center: bool, eps: float, rows=None, gain_a=None, b=None, gain_b=None,
                  inner_eps: float = 0.0, factor: float = 1.0, post_offset: float = 0.0) -> torch.Tensor:
    """One kernel for a block that norms behind its sublayers too (csrc/norm.cu):
        u = a, or factor * (rms(a) * gain_a + rms(b) * gain_b) when gain_a is given;
        resid += norm(u) * (post_offset + post_weight)  (post_center: with the mean taken off);
        out = norm(resid) * (offset + weight), or, with `weight` None, resid as it is (rounded to out's type).
    `a`, `b`: (tensor [n, H] or float32 partial sums [S, n, H], S or 0).  With `rows` the residual is read at those rows
    and left as it is."""
    N, H = resid.shape
    n = rows.shape[0] if rows is not None else N
    _need_cuda(resid, a[0], out, post_weight, weight, rows, gain_a, gain_b, b[0] if b is not None else None)
    assert resid.dtype == torch.float32 and resid.is_contiguous() and out.is_contiguous() and out.shape == (n, H)
    gains = [g for g in (post_weight, weight, gain_a, gain_b) if g is not None]
    assert all(g.shape == (H,) and g.is_contiguous() and g.dtype == post_weight.dtype for g in gains)
    pa = _branch_args(a, N, H)
    pb = _branch_args(b, N, H) if b is not None else (_ptr(None), _F32, 1, ctypes.c_longlong(0))
    lib = load_family("norm")
    _check(lib.wllm_sandwich_norm_offset(_ptr(resid), *pa, _ptr(gain_a), *pb, _ptr(gain_b), c_float(inner_eps), c_float(factor),
                                         _ptr(post_weight), c_float(post_offset), 1 if post_center else 0, c_float(post_eps),
                                         _ptr(weight), c_float(offset), 1 if center else 0, c_float(eps), _dt(post_weight),
                                         _ptr(out), _dt(out), _ptr(_int32(rows, "rows") if rows is not None else None), n, H,
                                         _stream()), "sandwich_norm")
    return out

def hyper_norm(src: torch.Tensor, dst: torch.Tensor, S: int, branch, prev_mix, prev_out, in_w, gain: torch.Tensor, eps: float,
               out: torch.Tensor, rows=None) -> torch.Tensor:
    """A residual of S streams and the norm in front of a sublayer (csrc/hyper_connections.cu).  `src`: the streams
    [S, n, H] float32, or one [n, H] that every stream is read from; `dst`: where the streams are written [S, n, H] (may be
    `src`).  `branch`: None, or (tensor [n, H] | float32 partial sums [P, n, H], P or 0), the output of the sublayer before,
    which joins the streams first: x_t <- sum_s prev_mix[s, t] x_s + prev_out[t] y.  Then out = rmsnorm(sum_s in_w[s] x_s)
    * gain (in_w None: the plain sum).  With `rows` the streams are read at those rows and left as they are."""
    _need_cuda(src, dst, gain, out, rows, prev_mix, prev_out, in_w, branch[0] if branch is not None else None)
    n, H = dst.shape[1], dst.shape[2]
    assert dst.shape[0] == S and dst.dtype == torch.float32 == src.dtype and dst.is_contiguous() and src.is_contiguous()
    assert tuple(src.shape) in ((S, n, H), (n, H)) and gain.shape == (H,) and gain.dtype == torch.float32 and gain.is_contiguous()
    n_out = rows.shape[0] if rows is not None else n
    assert out.shape == (n_out, H) and out.is_contiguous()
    for t, shape in ((prev_mix, (S, S)), (prev_out, (S,)), (in_w, (S,))):
        assert t is None or (t.dtype == torch.float32 and tuple(t.shape) == shape and t.is_contiguous())
    if branch is not None:
        assert prev_mix is not None and prev_out is not None
        pb = _branch_args(branch, n, H)
    else:
        pb = (_ptr(None), _F32, 1, ctypes.c_longlong(0))
    lib = load_family("hyper_connections")
    _check(lib.wllm_hyper_norm(_ptr(src), ctypes.c_longlong(n * H if src.dim() == 3 else 0), _ptr(dst), ctypes.c_longlong(n * H),
                               S, *pb, _ptr(prev_mix), _ptr(prev_out), _ptr(in_w), _ptr(gain), c_float(eps), _ptr(out), _dt(out),
                               _ptr(_int32(rows, "rows") if rows is not None else None), n_out, H, _stream()), "hyper_norm")
    return out


def rope_kv_write(qkv: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor, slots, inv_freq: torch.Tensor,
                  k_pages, v_pages, nq: int, nkv: int, hd: int, rot_dim: int, page_size: int, in_splits: int = 0,
                  pairing: str = "half", vd: int | None = None, unit_norm_eps: float | None = None) -> None:
    """Rotate the q and k heads of the fused rows `qkv` [n, (nq+2nkv)*hd] (or [S, n, ...] float32 partial sums
    when in_splits = S > 0); rotated q goes to `q_out` [n, nq*hd], rotated k and v to the pages.
    pairing 'half': element j turns with j + rot_dim/2; 'interleaved': 2j with 2j + 1.
    `vd`: size of a value head when it is not hd (the row is then nq*hd | nkv*hd | nkv*vd, and may be the first
    columns of a wider fused row).  `unit_norm_eps`: every rotated q and k head is divided by its root mean
    square, y / sqrt(mean(y^2) + eps)."""
    if pairing not in ("half", "interleaved"):
        raise KernelError(f"rotary pairing {pairing!r} not supported (half, interleaved)")
    _need_cuda(qkv, q_out, positions, slots, inv_freq, k_pages, v_pages)
    vd = hd if vd is None else vd
    width = (nq + nkv) * hd + nkv * vd          # nkv = 0: a row of query heads alone (nothing goes to the pages)
    assert nkv > 0 or slots is None
    if in_splits:
        assert qkv.dim() == 3 and qkv.shape[0] == in_splits and qkv.stride(2) == 1 and qkv.dtype == torch.float32
        n, row_stride, split_stride = qkv.shape[1], qkv.stride(1), qkv.stride(0)
    else:
        assert qkv.dim() == 2 and qkv.stride(1) == 1
        n, row_stride, split_stride = qkv.shape[0], qkv.stride(0), 0
    assert qkv.shape[-1] == width and q_out.shape == (n, nq * hd) and q_out.stride(1) == 1
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dim // 2 and inv_freq.is_contiguous()
    if slots is not None:
        assert k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == q_out.dtype == v_pages.dtype
    lib = load_family("rope_cache")
    _check(lib.wllm_rope_kv_write_general(_ptr(qkv), _dt(qkv), row_stride, max(1, in_splits), ctypes.c_longlong(split_stride),
                                          _ptr(q_out), _dt(q_out), q_out.stride(0), _ptr(_int32(positions, "positions")),
                                          _ptr(_int32(slots, "slots") if slots is not None else None), _ptr(inv_freq),
                                          _ptr(k_pages), _ptr(v_pages), n, nq, nkv, hd, rot_dim, page_size,
                                          1 if pairing == "interleaved" else 0, vd, 0 if unit_norm_eps is None else 1,
                                          c_float(unit_norm_eps or 0.0), _stream()),
           "rope_kv_write")


def rope_row_norm_kv_write(qkv: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor, slots, inv_freq: torch.Tensor,
                           k_pages, v_pages, nq: int, nkv: int, hd: int, rot_dim: int, page_size: int, q_gain: torch.Tensor,
                           k_gain: torch.Tensor, eps: float, q_count: int, k_count: int, in_splits: int = 0,
                           pairing: str = "half", vd: int | None = None, bias: torch.Tensor | None = None,
                           v_first: torch.Tensor | None = None, blend: torch.Tensor | None = None, mix: str | None = None) -> None:
    """As rope_kv_write, with the token's query row and key row normed as wholes (all heads at once) in front of the
    turn: q <- q / sqrt(mean(q^2) + eps) * q_gain over the nq * hd query elements, the same for k with k_gain
    (csrc/rope_cache.cu).  `q_count`, `k_count`: the elements that count for the means (heads held in steps of 8
    elements carry zeros behind them).  `bias`: one float32 row [(nq + nkv) * hd + nkv * vd] added to the projections' sums
    in front of the norms.  `mix` 'first': the token's values are also left in `v_first` [n, nkv * vd] float32; 'later': the
    values that are cached are (1 - blend[0]) v + blend[0] v_first."""
    if pairing not in ("half", "interleaved"):
        raise KernelError(f"rotary pairing {pairing!r} not supported (half, interleaved)")
    _need_cuda(qkv, q_out, positions, slots, inv_freq, k_pages, v_pages, q_gain, k_gain)
    vd = hd if vd is None else vd
    width = (nq + nkv) * hd + nkv * vd
    ptr, dt, row_stride, nparts, part_stride, n = _fused_args(qkv, in_splits)
    assert qkv.shape[-1] >= width and q_out.shape == (n, nq * hd) and q_out.stride(1) == 1
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dim // 2 and inv_freq.is_contiguous()
    assert q_gain.shape == (nq * hd,) and k_gain.shape == (nkv * hd,) and q_gain.dtype == k_gain.dtype
    assert q_gain.is_contiguous() and k_gain.is_contiguous()
    if slots is not None:
        assert k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == q_out.dtype == v_pages.dtype
    if mix not in (None, "first", "later"):
        raise KernelError(f"value mixing {mix!r}: 'first' or 'later'")
    _need_cuda(bias, v_first, blend)
    assert bias is None or (bias.dtype == torch.float32 and bias.shape == (width,) and bias.is_contiguous())
    if mix is not None:
        assert v_first.dtype == torch.float32 and v_first.shape == (n, nkv * vd) and v_first.is_contiguous()
        assert mix == "first" or (blend.dtype == torch.float32 and blend.numel() == 1)
    lib = load_family("rope_cache")
    _check(lib.wllm_rope_row_norm_kv_write(ptr, dt, row_stride, nparts, part_stride, _ptr(q_out), _dt(q_out), q_out.stride(0),
                                           _ptr(_int32(positions, "positions")),
                                           _ptr(_int32(slots, "slots") if slots is not None else None), _ptr(inv_freq),
                                           _ptr(k_pages), _ptr(v_pages), n, nq, nkv, hd, rot_dim, page_size,
                                           1 if pairing == "interleaved" else 0, vd, _ptr(q_gain), _ptr(k_gain), _dt(q_gain),
                                           q_count, k_count, c_float(eps), _ptr(bias), _ptr(v_first if mix is not None else None),
                                           _ptr(blend if mix == "later" else None), {None: 0, "first": 1, "later": 2}[mix],
                                           _stream()), "rope_row_norm_kv_write")


def latent_prepare(fused: torch.Tensor, parts: int, positions: torch.Tensor, slots, inv_freq: torch.Tensor, gain: torch.Tensor,
                   eps: float, pages: torch.Tensor, page_size: int, q_plain: torch.Tensor, q_mapped: torch.Tensor, heads: int,
                   dim: int, rot: int, rot_dims: int, rank: int, hd: int, pairing: str = "half", q_rank: int = 0,
                   q_gain: torch.Tensor | None = None, cq_out: torch.Tensor | None = None) -> None:
    """From the fused projection row [heads * (dim + rot) | rank + rot] of every token (csrc/latent_attention.cu): the
    cache row [rms(latent columns) * gain | the rot columns behind them, turned | zeros] into `pages` at `slots`; the
    queries' plain parts into `q_plain` [n, heads * dim] (None: they are read where they are); their turned parts into
    columns rank .. of every head of `q_mapped` [n, heads * hd].  Norm and turn are 32-bit, from the projection's partial sums where it left them.
    With `q_rank` > 0 the row is [q_rank | rank] instead (queries that pass a latent row of their own; nothing turns): those
    columns, normed with `q_gain` [q_rank], go to `cq_out` [n, q_rank] for the product that makes the queries."""
    if pairing not in ("half", "interleaved"):
        raise KernelError(f"rotary pairing {pairing!r} not supported (half, interleaved)")
    _need_cuda(fused, positions, slots, inv_freq, gain, pages, q_plain, q_mapped)
    ptr, dt, row_stride, nparts, part_stride, n = _fused_args(fused, parts)
    assert fused.shape[-1] >= (q_rank if q_rank else heads * (dim + rot)) + rank + rot and hd >= rank + rot
    _need_cuda(q_gain, cq_out)
    if q_rank:
        assert rot == 0 and q_gain.shape == (q_rank,) and q_gain.is_contiguous() and q_gain.dtype == gain.dtype
        assert cq_out.shape == (n, q_rank) and cq_out.is_contiguous() and cq_out.dtype == q_mapped.dtype
    assert q_mapped.shape == (n, heads * hd) and q_mapped.is_contiguous()
    assert q_plain is None or (q_plain.shape == (n, heads * dim) and q_plain.is_contiguous() and q_plain.dtype == q_mapped.dtype)
    assert q_mapped.dtype == pages.dtype and pages.is_contiguous() and pages.shape[-1] == hd and pages.shape[-3] == 1
    assert gain.shape == (rank,) and gain.is_contiguous()
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dims // 2 and inv_freq.is_contiguous()
    lib = load_family("latent_attention")
    _check(lib.wllm_latent_prepare(ptr, dt, row_stride, nparts, part_stride, _ptr(_int32(positions, "positions")),
                                   _ptr(_int32(slots, "slots") if slots is not None else None), _ptr(inv_freq), _ptr(gain),
                                   _dt(gain), c_float(eps), _ptr(pages), page_size, _ptr(q_plain), _ptr(q_mapped), _dt(q_mapped),
                                   n, heads, dim, rot, rot_dims, 1 if pairing == "interleaved" else 0, rank, hd, q_rank,
                                   _ptr(q_gain if q_rank else None), _ptr(cq_out if q_rank else None), _stream()),
           "latent_prepare")


HEAD_LINEAR_BATCHED_ROWS = 32     # bfloat16 steps of this many tokens or more: the heads' maps are one batched matrix product


def head_linear(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """y[t, h, :] = x[t, h, :] @ w[h]^T for every head h.  x [n, heads, K] and y [n, heads, N] may be views (free row and
    head strides, unit inner stride); w [heads, N, K] contiguous.  32-bit accumulation.  float32: every output is one
    ascending chain over K (csrc/latent_attention.cu); bfloat16 steps of few tokens: a warp an output, the matrices read
    once; bfloat16 steps of more tokens: a batched product of the vendor's matrix library, as `linear` uses it."""
    _need_cuda(x, w, y)
    n, heads, K = x.shape
    N = w.shape[1]
    assert w.shape == (heads, N, K) and w.is_contiguous() and y.shape == (n, heads, N)
    assert x.stride(2) == 1 and y.stride(2) == 1 and x.dtype == w.dtype == y.dtype
    if x.dtype == torch.bfloat16 and n >= HEAD_LINEAR_BATCHED_ROWS:
        # one strided batched product of the vendor's matrix library, 32-bit accumulation, written in place: [heads, n, K] x [heads, K, N]
        global launches
        launches += 1
        torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=y.transpose(0, 1))
        return y
    lib = load_family("latent_attention")
    if x.dtype == torch.bfloat16 and K % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) % 8 == 0 and x.data_ptr() % 16 == 0:
        _check(lib.wllm_head_linear_few(_ptr(x), x.stride(0), x.stride(1), _ptr(w), _ptr(y), y.stride(0), y.stride(1), n, heads, N, K,
                                        _stream()), f"head_linear_few({n}x{heads}x{N}x{K})")
        return y
    _check(lib.wllm_head_linear(_ptr(x), x.stride(0), x.stride(1), _ptr(w), _ptr(y), y.stride(0), y.stride(1), _dt(x), n, heads,
                                N, K, _stream()), f"head_linear({n}x{heads}x{N}x{K})")
    return y


SIMT_CHUNK = 64    # keys per chunk of the one-warp-per-row attention (csrc/attention_simt.cu)


def latent_mma_ok(heads: int, rank: int, row: int, page_size: int) -> bool:
    """Sizes that the tensor-core attention over latent rows is built for (one build per row and value size)."""
    return heads > 0 and rank % 32 == 0 and 32 <= rank <= 512 and row % 8 == 0 and rank <= row <= 832 and \
        page_size > 0 and page_size & (page_size - 1) == 0


LATENT_TILE = 32    # keys per tile of the tensor-core attention over latent rows (csrc/latent_attention_mma.cu)


@functools.lru_cache(maxsize=4096)
def latent_split_plan(requests: int, heads: int, max_ctx: int, window: int) -> tuple:
    """(split_tiles, max_splits) for a step of single tokens: every token's tiles of keys are cut into splits of
    split_tiles tiles, a CTA each, so that the step fills the SMs about once (two CTAs fit an SM); (0, 1): no cut."""
    most = -(-max(1, max_ctx) // LATENT_TILE)
    tiles = most if window == 0 else min(most, -(-abs(window) // LATENT_TILE) + 1)
    if heads > 64 or tiles <= 1:
        return 0, 1
    split_tiles = max(1, -(-tiles * requests // (2 * sm_count())), -(-tiles // 64))
    max_splits = -(-tiles // split_tiles)
    return (split_tiles, max_splits) if max_splits > 1 else (0, 1)


def latent_mma_scratch_floats(requests: int, heads: int, rank: int, max_splits: int) -> int:
    return requests * max_splits * heads * (rank + 2)


def latent_attention_mma(q: torch.Tensor, out: torch.Tensor, pages: torch.Tensor, req_q_start: torch.Tensor,
                         req_q_len: torch.Tensor, req_ctx_len: torch.Tensor, block_table: torch.Tensor, max_q_len: int,
                         heads: int, rank: int, row: int, page_size: int, window: int, scale: float,
                         skip_single: bool = False, split_tiles: int = 0, max_splits: int = 1,
                         scratch: torch.Tensor | None = None) -> torch.Tensor:
    """bfloat16 attention of every request's new tokens over its cached latent rows (csrc/latent_attention_mma.cu).
    q: [n, heads * row]; pages: [pool pages, 1, page_size, row], a row's first `rank` elements being its value;
    out: [n, heads * rank].  `window` as for `paged_attention_simt`.  split_tiles > 0 (see latent_split_plan; `scratch`
    float32 of latent_mma_scratch_floats): the keys of requests that bring one token are cut into splits that a second
    kernel merges in order."""
    _need_cuda(q, out, pages, req_q_start, req_q_len, req_ctx_len, block_table, scratch)
    assert q.dtype == torch.bfloat16 == out.dtype == pages.dtype and q.stride(1) == 1 and out.stride(1) == 1
    assert pages.is_contiguous() and pages.shape[-1] == row and pages.shape[-2] == page_size and block_table.dim() == 2
    assert q.shape[1] == heads * row and out.shape[1] == heads * rank and latent_mma_ok(heads, rank, row, page_size)
    if split_tiles > 0:
        assert scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous()
        assert scratch.numel() >= latent_mma_scratch_floats(req_q_len.shape[0], heads, rank, max_splits)
    lib = load_family("latent_attention_mma", {"LATENT_ROW": row, "LATENT_RANK": rank})
    _check(lib.wllm_latent_attention_mma(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(pages),
                                         _ptr(_int32(req_q_start, "req_q_start")), _ptr(_int32(req_q_len, "req_q_len")),
                                         _ptr(_int32(req_ctx_len, "req_ctx_len")), _ptr(_int32(block_table, "block_table")),
                                         block_table.shape[1], req_q_len.shape[0], max_q_len, heads, page_size, window,
                                         c_float(scale), 1 if skip_single else 0, split_tiles, max_splits,
                                         _ptr(scratch) if split_tiles > 0 else None, _stream()),
           f"latent_attention_mma(row={row}, rank={rank}, heads={heads})")
    if split_tiles > 0 and max_splits > 1:
        global launches
        launches += 1    # the merge kernel
    return out


def simt_chunks(max_ctx: int, window: int, keep: int = 0) -> int:
    """Upper bound of the chunks of 64 keys that a row of a step touches, from the longest context of the
    step (and the window, if the layer has one, with the first keys it keeps behind it)."""
    most = -(-max(1, max_ctx) // SIMT_CHUNK)
    if window < 0:          # a mask of blocks of -window positions: a row sees no further back than its block's start
        return min(most, -(window // SIMT_CHUNK) + 1)
    return min(most, -(-window // SIMT_CHUNK) + 1 + -(-keep // SIMT_CHUNK)) if window > 0 else most


def paged_attention_simt(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                         token_req: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor,
                         nq: int, nkv: int, hd: int, page_size: int, window: int, scale: float,
                         scratch: torch.Tensor | None = None, max_chunks: int = 0, vd: int | None = None,
                         sinks: torch.Tensor | None = None, cap: float = 0.0, keep: int = 0,
                         values_in_keys: bool = False, slopes: torch.Tensor | None = None) -> torch.Tensor:
    """q: [n, nq*hd] view (row stride free); pages: [num_pages, nkv, page_size, hd]; out: [n, nq*hd].
    `window` > 0: a row sees itself and the window - 1 keys before it; < 0: the earlier keys of its own block of -window
    positions (blocks counted from position 0); 0: every earlier key.  `values_in_keys`: a token's value is the first vd
    elements of its key's row (`v_pages` is `k_pages`).
    `vd`: size of a value head when it is not hd (value pages [.., vd], out [n, nq*vd]); `sinks`: float32 [nq], one
    more term e^(sink) in every row's softmax denominator.  `cap` > 0: scores become cap * tanh(score / cap);
    `keep` > 0 (with a window): the sequence's first `keep` keys stay visible behind the window.  `slopes`: float32 [nq]; the
    score of key j from position p loses slopes[head] * (p - j), after the scale and the cap.
    With `scratch` (float32, n * nq * max_chunks * (hd + 2) floats) and max_chunks = simt_chunks(...) > 1 every
    (row, chunk of 64 keys) gets a warp of its own and a second kernel merges them; the result is the same,
    bit for bit, as without."""
    _need_cuda(q, out, k_pages, v_pages, token_req, positions, block_table, scratch, sinks)
    n = q.shape[0]
    vd = hd if vd is None else vd
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_pages.dtype == v_pages.dtype
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and block_table.dim() == 2
    assert k_pages.shape[-1] == hd and v_pages.shape[-1] == (hd if values_in_keys else vd)
    assert not values_in_keys or (v_pages.data_ptr() == k_pages.data_ptr() and vd <= hd)
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.shape == (nq,) and sinks.is_contiguous())
    assert slopes is None or (slopes.is_cuda and slopes.dtype == torch.float32 and slopes.shape == (nq,) and slopes.is_contiguous())
    if scratch is not None:
        assert scratch.dtype == torch.float32 and scratch.is_contiguous() and max_chunks >= 1
        assert scratch.numel() >= n * nq * max_chunks * (vd + 2)
    lib = load_family("attention_simt")
    _check(lib.wllm_paged_attention_simt_strided(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages),
                                                 _dt(q), _ptr(_int32(token_req, "token_req")),
                                                 _ptr(_int32(positions, "positions")), _ptr(_int32(block_table, "block_table")),
                                                 block_table.shape[1], n, nq, nkv, hd, page_size, window, c_float(scale),
                                                 _ptr(scratch), max_chunks if scratch is not None else 0, vd, _ptr(sinks),
                                                 c_float(cap), keep, hd if values_in_keys else 0, _ptr(slopes), _stream()),
           f"paged_attention_simt(head_dim={hd}/{vd}, heads={nq}/{nkv})")
    if scratch is not None and max_chunks > 1:
        global launches
        launches += 1    # the merge kernel
    return out


def paged_attention_simt_tiled(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                               req_q_start: torch.Tensor, req_q_len: torch.Tensor, req_ctx_len: torch.Tensor,
                               block_table: torch.Tensor, max_q_len: int, nq: int, nkv: int, hd: int, page_size: int,
                               window: int, scale: float, vd: int | None = None,
                               sinks: torch.Tensor | None = None, cap: float = 0.0, keep: int = 0,
                               values_in_keys: bool = False, slopes: torch.Tensor | None = None) -> torch.Tensor:
    """The same attention as `paged_attention_simt`, bit for bit, for steps that bring portions of prompts: a CTA
    takes 32 rows of one (request, key/value head) and reads every tile of keys and values once for all of them
    (csrc/attention_simt.cu, tiled).  Head sizes up to 256; requests are given by their start, length and context."""
    _need_cuda(q, out, k_pages, v_pages, req_q_start, req_q_len, req_ctx_len, block_table, sinks)
    vd = hd if vd is None else vd
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_pages.dtype == v_pages.dtype
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and block_table.dim() == 2
    assert k_pages.shape[-1] == hd and v_pages.shape[-1] == (hd if values_in_keys else vd)
    assert not values_in_keys or (v_pages.data_ptr() == k_pages.data_ptr() and vd <= hd)
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.shape == (nq,) and sinks.is_contiguous())
    assert slopes is None or (slopes.is_cuda and slopes.dtype == torch.float32 and slopes.shape == (nq,) and slopes.is_contiguous())
    lib = load_family("attention_simt")
    _check(lib.wllm_paged_attention_simt_tiled_strided(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages),
                                                       _ptr(v_pages), _dt(q), _ptr(_int32(req_q_start, "req_q_start")),
                                                       _ptr(_int32(req_q_len, "req_q_len")),
                                                       _ptr(_int32(req_ctx_len, "req_ctx_len")),
                                                       _ptr(_int32(block_table, "block_table")), block_table.shape[1],
                                                       req_q_len.shape[0], max_q_len, nq, nkv, hd, page_size, window,
                                                       c_float(scale), vd, _ptr(sinks), c_float(cap), keep,
                                                       hd if values_in_keys else 0, _ptr(slopes), _stream()),
           f"paged_attention_simt_tiled(head_dim={hd}/{vd}, heads={nq}/{nkv})")
    return out


def _indexed(device) -> torch.device:
    device = torch.device(device)
    if device.index is None and device.type == "cuda":
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def _status_word(device) -> torch.Tensor:
    """One int32 per device that stays 0 unless a kernel's bounded wait ran out (see tc_gemm_status)."""
    device = _indexed(device)
    status = _tc_status.get(device)
    if status is None:
        with torch.inference_mode(False):      # whoever asks first: the word is written in place from any mode later
            status = torch.zeros(1, dtype=torch.int32, device=device)
        _tc_status[device] = status
    return status


def mma_head_dim_ok(hd: int) -> bool:
    """Head sizes the tensor-core attention kernels are built for (one build per size)."""
    return hd % 16 == 0 and 16 <= hd <= 256


def attention_mma_scratch_floats(requests: int, nq: int, hd: int, max_splits: int) -> int:
    return requests * nq * max_splits * (hd + 2)


@functools.lru_cache(maxsize=4096)
def decode_split_plan(heads: int, max_ctx: int, tile: int) -> tuple:
    """(split_keys, max_splits) for the decode attention of `heads` (request, key/value head) pairs with up to
    max_ctx keys each.  Every pair is cut into parts of split_keys keys (whole tiles, at least 128) plus a
    shorter rest, one CTA a part, and the CTAs start longest first (the rests last).  Two part sizes are
    weighed by when their last CTA ends on 148 SMs: equal parts, one an SM at most; and parts of the SMs'
    even share of all keys, whose short rests run on the SMs that the whole parts leave free."""
    heads = max(1, heads)
    per_cta = 2 * tile                                          # a CTA costs about two tiles beside its keys

    def up(keys):
        return max(128, -(-keys // tile) * tile)

    def finish(keys):
        splits = -(-max_ctx // keys)
        rest, whole = max_ctx - (splits - 1) * keys, (splits - 1) * heads
        if whole + heads <= sm_count():
            return (keys if splits > 1 else rest) + per_cta
        if whole < sm_count():
            return max(keys + per_cta, -(-heads // (sm_count() - whole)) * (rest + per_cta))
        return -(-(whole + heads) // sm_count()) * (keys + per_cta)
    equal = up(-(-max_ctx // max(1, sm_count() // heads)))
    share = min(up(max_ctx), up(-(-max_ctx * heads // sm_count())))
    keys = min((equal, share), key=lambda k: (finish(k), -k))
    return keys, -(-max_ctx // keys)


def attention_mma_decode(q, out, k_pages, v_pages, req_q_start, req_q_len, req_ctx_len, block_table, nq: int, nkv: int,
                         hd: int, page_size: int, window: int, scale: float, split_keys: int, max_splits: int,
                         scratch: torch.Tensor, sinks: torch.Tensor | None = None, cap: float = 0.0, keep: int = 0,
                         slopes: torch.Tensor | None = None) -> None:
    """bfloat16 attention of the requests that bring one token (csrc/attention_mma.cu, decode).
    `sinks`: float32 [nq], one more term e^sink of every row's softmax denominator.  `cap` > 0: scores become
    cap * tanh(score / cap); `keep` > 0 (with a window): the sequence's first `keep` keys stay visible behind the window.
    `slopes`: float32 [nq]; the score of key j from position p loses slopes[head] * (p - j), after the scale and the cap."""
    _need_cuda(q, out, k_pages, v_pages, req_q_start, req_q_len, req_ctx_len, block_table, scratch, sinks, slopes)
    assert slopes is None or (slopes.dtype == torch.float32 and slopes.shape == (nq,) and slopes.is_contiguous())
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.shape == (nq,) and sinks.is_contiguous())
    assert q.dtype == torch.bfloat16 == out.dtype == k_pages.dtype and q.stride(1) == 1 and out.stride(1) == 1
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and scratch.dtype == torch.float32
    R = req_q_len.shape[0]
    assert scratch.numel() >= attention_mma_scratch_floats(R, nq, hd, max_splits)
    lib = load_family("attention_mma", {"HEAD_DIM": hd})
    _check(lib.wllm_attention_mma_decode_biased(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages),
                                               ctypes.c_longlong(k_pages.shape[0]),
                                               _ptr(_int32(req_q_start, "req_q_start")), _ptr(_int32(req_q_len, "req_q_len")),
                                               _ptr(_int32(req_ctx_len, "req_ctx_len")),
                                               _ptr(_int32(block_table, "block_table")), block_table.shape[1], R, nq, nkv,
                                               page_size, window, c_float(scale), split_keys, max_splits, _ptr(scratch),
                                               _ptr(_status_word(q.device)), _ptr(sinks), c_float(cap), keep, _ptr(slopes), _stream()),
           f"attention_mma_decode(head_dim={hd}, heads={nq}/{nkv})")
    global launches
    launches += 1 if max_splits > 1 else 0    # the merge kernel


def attention_prefill_halves_floats(requests: int, max_q_len: int, nq: int, nkv: int, hd: int) -> int:
    """Floats of the `halves` buffer of a prefill launch that shares heavy tiles between two CTAs."""
    tiles = -(-(max_q_len * (nq // nkv)) // 128)
    return tiles * nkv * requests * 2 * 128 * (hd + 4)


def prefill_share_plan(q_lens, ctx_lens, nq: int, nkv: int, hd: int, skip_single: bool) -> int:
    """`split_above` for attention_mma_prefill, from the step's request lengths on the host.  A prompt processed
    from its start gives its 128-row tiles 1, 2, ... tiles of keys to walk, and a grid of at most one CTA an
    SM then ends with its heaviest tile.  Such a grid is launched with two CTAs a tile, and the tiles that are
    heavier than a fair share (a quarter above the mean per SM, at least 8) are halved.  0: no sharing."""
    if hd % 64 != 0:
        return 0
    rep = nq // nkv
    longest = max((n for n in q_lens if not (skip_single and n == 1)), default=0)
    if longest <= 0 or -(-(longest * rep) // 128) * nkv * len(q_lens) > sm_count():
        return 0
    work = heaviest = 0
    for q_len, ctx_len in zip(q_lens, ctx_lens):
        if q_len <= 0 or (skip_single and q_len == 1):
            continue
        pos0, rows = ctx_len - q_len, q_len * rep
        for first in range(0, rows, 128):
            walked = (pos0 + (min(rows, first + 128) - 1) // rep) // 64 + 1
            work += walked * nkv
            heaviest = max(heaviest, walked)
    fair = max(8, -(-5 * work // (4 * sm_count())))
    return fair if heaviest > fair else 0


def attention_mma_prefill(q, out, k_pages, v_pages, req_q_start, req_q_len, req_ctx_len, block_table, max_q_len: int,
                          nq: int, nkv: int, hd: int, page_size: int, window: int, scale: float,
                          skip_single: bool, split_above: int = 0, halves: torch.Tensor | None = None,
                          sinks: torch.Tensor | None = None, cap: float = 0.0, keep: int = 0,
                          slopes: torch.Tensor | None = None) -> None:
    """bfloat16 attention of the requests that bring several tokens (csrc/attention_mma.cu, prefill).
    split_above > 0 (head sizes in steps of 64): a tile of 128 rows that walks more than that many tiles of 64
    keys is computed by two CTAs, half of the keys each; `halves` (float32) holds their partial results.
    `cap`, `keep`, `slopes`: as for attention_mma_decode; with any of them the mma.sync kernel that walks a list of key tiles runs."""
    _need_cuda(q, out, k_pages, v_pages, req_q_start, req_q_len, req_ctx_len, block_table, halves, sinks, slopes)
    assert slopes is None or (slopes.dtype == torch.float32 and slopes.shape == (nq,) and slopes.is_contiguous())
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.shape == (nq,) and sinks.is_contiguous())
    if split_above > 0:
        assert hd % 64 == 0 and halves is not None and halves.dtype == torch.float32 and halves.is_contiguous()
        assert halves.numel() >= attention_prefill_halves_floats(req_q_len.shape[0], max_q_len, nq, nkv, hd)
    assert q.dtype == torch.bfloat16 == out.dtype == k_pages.dtype and q.stride(1) == 1 and out.stride(1) == 1
    assert k_pages.is_contiguous() and v_pages.is_contiguous()
    lib = load_family("attention_mma", {"HEAD_DIM": hd})
    _check(lib.wllm_attention_mma_prefill_biased(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pages), _ptr(v_pages),
                                                ctypes.c_longlong(k_pages.shape[0]),
                                                _ptr(_int32(req_q_start, "req_q_start")), _ptr(_int32(req_q_len, "req_q_len")),
                                                _ptr(_int32(req_ctx_len, "req_ctx_len")),
                                                _ptr(_int32(block_table, "block_table")), block_table.shape[1],
                                                req_q_len.shape[0], max_q_len, nq, nkv, page_size, window, c_float(scale),
                                                1 if skip_single else 0, split_above, _ptr(halves) if split_above > 0 else None,
                                                _ptr(_status_word(q.device)), _ptr(sinks), c_float(cap), keep, _ptr(slopes), _stream()),
           f"attention_mma_prefill(head_dim={hd}, heads={nq}/{nkv})")


ACTIVATIONS = {"gelu_tanh": 0, "silu": 1, "relu": 2, "capped_swish": 3}


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, act: str, limit: float = 0.0, slope: float = 0.0) -> torch.Tensor:
    """out[n, c] = act(gate_up[n, c]) * gate_up[n, I + c]; 'capped_swish' (with `limit` and `slope`):
    g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(slope * g) * (u + 1)."""
    _need_cuda(gate_up, out)
    n, two_i = gate_up.shape
    assert gate_up.is_contiguous() and out.is_contiguous() and out.shape == (n, two_i // 2) and out.dtype == gate_up.dtype
    code = ACTIVATIONS.get(act)
    if code is None:
        raise KernelError(f"activation {act!r} not supported ({', '.join(ACTIVATIONS)})")
    lib = load_family("activation")
    _check(lib.wllm_gated_act_params(_ptr(gate_up), _ptr(out), _dt(gate_up), code, n, two_i // 2, c_float(limit),
                                     c_float(slope), _stream()), "gated_act")
    return out


def tanh_cap(x: torch.Tensor, cap: float, scale: float = 1.0) -> torch.Tensor:
    """x <- cap * tanh(x * scale / cap), in place on a contiguous 32-bit tensor."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous() and cap > 0
    lib = load_family("activation")
    _check(lib.wllm_scale_tanh_cap(_ptr(x), ctypes.c_longlong(x.numel()), c_float(cap), c_float(scale), _stream()), "tanh_cap")
    return x


def scale_rows(x: torch.Tensor, scale: float) -> torch.Tensor:
    """x <- x * scale, in place on a contiguous 32-bit tensor."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    lib = load_family("activation")
    _check(lib.wllm_scale_tanh_cap(_ptr(x), ctypes.c_longlong(x.numel()), c_float(0.0), c_float(scale), _stream()), "scale_rows")
    return x


UNIT_ACTIVATIONS = {"relu_squared": 0}


def unit_act(x: torch.Tensor, out: torch.Tensor, act: str) -> torch.Tensor:
    """out = act(x) elementwise for a feed-forward without a gate; 'relu_squared': max(x, 0)^2, 32-bit, rounded once."""
    _need_cuda(x, out)
    assert x.is_contiguous() and out.is_contiguous() and out.shape == x.shape and out.dtype == x.dtype
    code = UNIT_ACTIVATIONS.get(act)
    if code is None:
        raise KernelError(f"activation {act!r} not supported ({', '.join(UNIT_ACTIVATIONS)})")
    lib = load_family("activation")
    _check(lib.wllm_unit_act(_ptr(x), _ptr(out), _dt(x), code, ctypes.c_longlong(x.numel()), _stream()), "unit_act")
    return out


def sigmoid_gate(x: torch.Tensor, fused: torch.Tensor, parts: int, col0: int) -> torch.Tensor:
    """x[n, c] *= sigmoid(gate[n, c]) in place, the gate being columns col0 .. col0 + x.shape[1] of the fused projection
    `fused` [n, W] (or float32 partial sums [parts, n, W], added in order)."""
    _need_cuda(x, fused)
    n, width = x.shape
    ptr, dt, row_stride, nparts, part_stride, rows = _fused_args(fused, parts)
    assert rows == n and x.stride(1) == 1 and col0 + width <= fused.shape[-1]
    lib = load_family("activation")
    item = 4 if fused.dtype == torch.float32 else 2
    _check(lib.wllm_sigmoid_gate(_ptr(x), _dt(x), x.stride(0), c_void_p(fused.data_ptr() + col0 * item), dt, row_stride, nparts,
                                 part_stride, n, width, _stream()), "sigmoid_gate")
    return x


TOKEN_GATE_ACTIVATIONS = {"gelu_tanh": 0}


def token_gate(z: torch.Tensor, parts: int, token_ids: torch.Tensor, table: torch.Tensor, act: str, out: torch.Tensor) -> torch.Tensor:
    """out[n, c] = act(z[n, c]) * table[token_ids[n], c]: a projection of the residual gates the token's own table row.  `z` is
    [n, dim] (or float32 partial sums [parts, n, dim], added in order); the activation and the product are 32-bit, rounded once."""
    if act not in TOKEN_GATE_ACTIVATIONS:
        raise KernelError(f"activation {act!r} not supported ({', '.join(TOKEN_GATE_ACTIVATIONS)})")
    _need_cuda(z, token_ids, table, out)
    ptr, dt, row_stride, nparts, part_stride, n = _fused_args(z, parts)
    V, dim = table.shape
    assert table.is_contiguous() and out.shape == (n, dim) and out.is_contiguous() and out.dtype == table.dtype
    assert z.shape[-1] == dim and token_ids.shape[0] == n
    lib = load_family("activation")
    _check(lib.wllm_token_gate(ptr, dt, row_stride, nparts, part_stride, _ptr(_int32(token_ids, "token_ids")), _ptr(table), _dt(table),
                               V, _ptr(out), TOKEN_GATE_ACTIVATIONS[act], n, dim, _stream()), "token_gate")
    return out


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T in true 32-bit arithmetic (csrc/gemm_f32.cu)."""
    _need_cuda(a, w, out)
    assert a.dtype == torch.float32 and w.dtype == torch.float32 and a.stride(1) == 1 and w.stride(1) == 1
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    assert out.stride(1) == 1 and out.shape == (M, N) and out.dtype == torch.float32
    lib = load_family("gemm_f32")
    lib.wllm_gemm_f32_scratch_floats.restype = ctypes.c_longlong
    need = lib.wllm_gemm_f32_scratch_floats(M, N, K)       # partial sums of the few-rows kernel when K has several segments
    scratch = torch.empty(need, dtype=torch.float32, device=a.device) if need else None
    _check(lib.wllm_gemm_f32(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, N, K, _ptr(scratch),
                             ctypes.c_longlong(need), _stream()), "gemm_f32")
    if need:
        global launches
        launches += 1        # the kernel that adds the partial sums
    return out


def fma_peak_tflops(device, iters: int = 20000) -> float:
    """TFLOP/s of a loop of independent 32-bit fused multiply-adds on every SM (csrc/gemm_f32.cu): what the
    32-bit products are measured against, at the clock the device runs such a loop at."""
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    blocks = sms * 8
    out = torch.empty(blocks * 256, dtype=torch.float32, device=device)
    lib = load_family("gemm_f32")
    best = 0.0
    with torch.cuda.device(device):
        for _ in range(4):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            _check(lib.wllm_fma_loop(_ptr(out), blocks, iters, _stream()), "fma_loop")
            end.record()
            torch.cuda.synchronize()
            best = max(best, blocks * 256 * 8 * 2.0 * iters / (start.elapsed_time(end) * 1e-3) / 1e12)
    return best


_TC_EPILOGUES = {"bf16": 0, "f32": 1, "gelu_tanh": 2, "silu": 3, "relu": 4, "capped_swish": 5, "relu_squared": 6}
_TC_GATED = (2, 3, 4, 5)
_tc_status: dict = {}


def tc_gemm_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Shapes the tensor-memory GEMM takes: bfloat16, unit inner strides, K and pitches in steps of 8."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and w.dim() == 2
            and a.stride(1) == 1 and w.stride(1) == 1 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


@functools.lru_cache(maxsize=4096)
def tile_plan(M: int, N: int, K: int, gated: bool = False, may_split: bool = True) -> tuple:
    """(half_rows, parts).  More than 128 rows: see _pair_plan.  At most 128 rows, the product is bound by streaming W: the W tile of a
    stage is two halves of `half_rows` rows, and K is cut into `parts` (at most 16: whoever reads the partial
    sums loads that many at once).  Chosen so that tiles x parts fill the SMs evenly: the cost of a choice is
    the bytes of W that the busiest CTA streams, plus a fixed price per tile and a little per part."""
    if M > 128:
        return _pair_plan(M, N, K, gated), 1
    least = 48 if M <= 32 else (32 if M <= 64 else 16)     # a stage must hold the 128 rows the tensor core reads at A
    kblocks = -(-K // 64)
    cols = N // 2 if gated else N
    best = None
    for half in (128, 112, 96, 80, 64, 48, 32, 16):
        if half < least:
            continue
        tiles = -(-cols // (half if gated else 2 * half))
        wanted = max(1, min(kblocks, sm_count() // tiles, 16)) if may_split else 1
        per = -(-kblocks // wanted)
        parts = -(-kblocks // per)
        waves = -(-(tiles * parts) // sm_count())
        cost = waves * (per * half + 192) * (1.0 + 0.004 * parts)
        if best is None or cost < best[0]:
            best = (cost, half, parts)
    return best[1], best[2]


@functools.lru_cache(maxsize=1)
def resident_pairs() -> int:
    """Pairs of CTAs of the two-CTA product that the device holds at once (74 on 148 SMs)."""
    return max(1, int(load_family("gemm_bf16_tc").wllm_gemm_bf16_tc_resident_pairs()))


def _pair_plan(M: int, N: int, K: int, gated: bool) -> int:
    """half_rows for a product of more than 128 rows, on pairs of CTAs with tiles of 256 rows by 2 * half columns.
    The pairs walk the tiles in rounds; what a round costs was fitted to measurements at 2,048 rows: a block of K
    takes time in proportion to the bytes a CTA loads for it (its 128 rows of A and `half` rows of W: wider tiles
    do more arithmetic per byte from the L2), and a tile's drain is hidden behind the next tile's products except
    with wide tiles (half > 128: one accumulator), where it is paid every round.  Narrower halves than 128 were
    measured too (no faster a block), so they only win where they save a round; with a gate the tile is the two
    halves of 128."""
    if gated:
        return 128
    pairs, kblocks, tiles_m = resident_pairs(), -(-K // 64), -(-M // 256)
    best = None
    for half in (128, 112, 96, 80, 64, 144, 160, 176, 192, 208, 224, 240, 256):
        rounds = -(-(tiles_m * -(-N // (2 * half))) // pairs)
        block_us, drain_us = 0.0017 * (128 + max(half, 128)), 1.0 + 3.0 * max(half, 128) / 128
        cost = rounds * kblocks * block_us + (rounds if half > 128 else 1) * drain_us
        if best is None or cost < best[0] * 0.97:          # another width must pay by 3 %
            best = (cost, half)
    return best[1]


@functools.lru_cache(maxsize=4096)
def product_plan(M: int, N: int, K: int) -> tuple:
    """(half_rows, parts) for a projection whose reader adds partial sums: up to 128 rows tile_plan's choice; above,
    pairs of CTAs, and K is cut into parts as long as the tiles leave at least half of the pairs idle (a prompt of
    256 tokens has 8 tiles of its down projection for 74 pairs): as many parts as fit, of at least 4 blocks of K."""
    if M <= 128:
        return tile_plan(M, N, K)
    half = _pair_plan(M, N, K, False)
    pairs, kblocks = resident_pairs(), -(-K // 64)
    tiles = -(-M // 256) * -(-N // (2 * half))
    wanted = min(pairs // tiles, kblocks // 4, 16)
    if wanted < 2:
        return half, 1
    per = -(-kblocks // wanted)
    return half, -(-kblocks // per)


def split_plan(M: int, N: int, K: int) -> int:
    """Parts to cut K into so that a product of few rows still gives every SM a share of the weights."""
    return product_plan(M, N, K)[1]


def gemm_bf16_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, epilogue: str = "bf16",
                 max_ctas: int | None = None, k_splits: int = 1, half_rows: int | None = None, checked: bool = False,
                 limit: float = 0.0, slope: float = 0.0) -> torch.Tensor:
    """out = a @ w^T on tcgen05 tensor cores (csrc/gemm_bf16_tc.cu).  epilogue 'bf16' | 'f32' (32-bit out) |
    'gelu_tanh' | 'silu' | 'relu' (w = [gate; up] stacked: out[M, N/2] = act(a gate^T) * (a up^T)) | 'capped_swish' (the
    clamped gated unit of gated_act, with its `limit` and `slope`) | 'relu_squared' (no gate: out[M, N] = max(a w^T, 0)^2).
    k_splits > 1 ('f32' only) cuts K into parts; `out` is then [k_splits, M, N] partial sums.
    half_rows: the tile of products of at most 128 rows (see tile_plan, which chooses it when None)."""
    _need_cuda(a, w, out)
    if not checked and not tc_gemm_ok(a, w):        # `checked`: the caller has asked tc_gemm_ok already
        raise KernelError("gemm_bf16_tc: bfloat16 operands with K and row pitches in steps of 8 elements, 16-byte "
                          f"aligned; got a{tuple(a.shape)} stride {a.stride()} w{tuple(w.shape)} stride {w.stride()}")
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K
    code = _TC_EPILOGUES[epilogue]
    cols = N // 2 if code in _TC_GATED else N
    shape = (M, cols) if k_splits == 1 else (k_splits, M, cols)
    if out is None:
        out = torch.empty(shape, dtype=torch.float32 if code == 1 else torch.bfloat16, device=a.device)
    assert out.shape == shape and out.stride(-1) == 1 and out.dtype == (torch.float32 if code == 1 else torch.bfloat16)
    assert k_splits == 1 or (code == 1 and out.is_contiguous())
    status = _status_word(a.device)
    if max_ctas is None:
        max_ctas = sm_count()
    lib = load_family("gemm_bf16_tc")
    if half_rows is None:
        half_rows = tile_plan(M, N, K, code in _TC_GATED, k_splits > 1)[0]
    _check(lib.wllm_gemm_bf16_tc_params(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(-2), M, N, K, code,
                                        k_splits, half_rows, _ptr(status), max_ctas, c_float(limit), c_float(slope), _stream()),
           f"gemm_bf16_tc({M}x{N}x{K}, {epilogue}, {k_splits} parts)")
    return out


GAVE_UP = {11: "GEMM producer", 12: "GEMM tensor-core issue", 13: "GEMM epilogue", 21: "decode attention",
           22: "prefill attention (mma)", 23: "prefill attention loads", 24: "prefill attention tensor-core issue",
           25: "prefill attention softmax"}


def tc_gemm_status(device) -> int:
    """0, or the code of a role of the tensor-memory GEMM or attention kernels that gave up waiting
    (synchronises; the engine reads the same word with every step's sampled ids instead)."""
    status = _tc_status.get(_indexed(device))
    return 0 if status is None else int(status.item())


def reset_kernel_status(device) -> None:
    status = _tc_status.get(_indexed(device))
    if status is not None:
        status.zero_()


TC_MIN_ROWS = 65   # fewer rows outside project(): the vendor's library (see linear())


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, f32_out: bool = False) -> torch.Tensor:
    """a @ w^T.

    float32 operands: this engine's own FMA kernel (no reduced-precision matrix mode can reach it).
    bfloat16 operands: the tcgen05 / tensor-memory kernel of csrc/gemm_bf16_tc.cu when the shapes allow
    (K and pitches in steps of 8) and the step has more than a handful of rows (steps of few rows go
    through project() instead); otherwise the vendor's matrix library with 32-bit accumulation, which is where the reference engine sends every projection
    (src/wllm/models/llama.py:95-98).  `f32_out` asks for 32-bit results from bfloat16 operands (logits).
    """
    if a.dtype == torch.float32:
        return gemm_f32(a, w, out)
    _need_cuda(a, w)
    if tc_gemm_ok(a, w) and (a.shape[0] >= TC_MIN_ROWS or f32_out):
        return gemm_bf16_tc(a, w, out, "f32" if f32_out else "bf16", checked=True)
    global launches
    launches += 1
    r = torch.matmul(a, w.t(), out=out) if out is not None and not f32_out else torch.matmul(a, w.t())
    return r.float() if f32_out else r


def project(a: torch.Tensor, w: torch.Tensor, buffer) -> tuple:
    """a @ w^T for a layer's projections whose reader can add partial sums itself (the norm and the rotary
    kernels do).  Returns (tensor, parts).  parts = 0: `tensor` is the plain product [n, N] in the operands'
    type.  parts = S > 0 (bfloat16 steps whose tiles alone would leave most SMs idle: up to 128 rows, which are
    bound by streaming the weights, and short prompts): `tensor` is [S, n, N] float32 partial sums over S parts of
    K, left by a split-K run of the tensor-memory GEMM in which every SM takes a share.  `buffer(name, shape, dtype)` supplies the output."""
    n, N = a.shape[0], w.shape[0]
    if a.dtype == torch.bfloat16 and tc_gemm_ok(a, w):
        half, parts = product_plan(n, N, a.shape[1])
        if n <= 128 or parts > 1:
            out = buffer("parts", (parts, n, N), torch.float32)
            gemm_bf16_tc(a, w, out if parts > 1 else out[0], "f32", k_splits=parts, half_rows=half, checked=True)
            return out, parts
    return linear(a, w, buffer("product", (n, N), a.dtype)), 0


def gated_linear(a: torch.Tensor, w_gate_up: torch.Tensor, act: str, out: torch.Tensor, scratch, limit: float = 0.0,
                 slope: float = 0.0) -> torch.Tensor:
    """out[n, I] = act(a @ gate^T) * (a @ up^T) with w_gate_up = [gate; up] ('capped_swish': the clamped unit of
    gated_act, with its `limit` and `slope`).  bfloat16 with enough rows: one
    tensor-memory GEMM whose epilogue applies the activation; otherwise product, then activation kernel
    (`scratch(shape, dtype)` supplies the [n, 2I] intermediate)."""
    if a.dtype == torch.bfloat16 and tc_gemm_ok(a, w_gate_up):
        return gemm_bf16_tc(a, w_gate_up, out, act, checked=True, limit=limit, slope=slope)
    gu = linear(a, w_gate_up, scratch((a.shape[0], w_gate_up.shape[0]), a.dtype))
    return gated_act(gu, out, act, limit, slope)


def unit_linear(a: torch.Tensor, w_up: torch.Tensor, act: str, out: torch.Tensor, scratch) -> torch.Tensor:
    """out[n, I] = act(a @ up^T) for a feed-forward without a gate ('relu_squared').  bfloat16: one tensor-memory GEMM
    whose epilogue applies the activation on the 32-bit sums; otherwise product, then activation kernel
    (`scratch(shape, dtype)` supplies the [n, I] intermediate)."""
    if act not in UNIT_ACTIVATIONS:
        raise KernelError(f"activation {act!r} not supported ({', '.join(UNIT_ACTIVATIONS)})")
    if a.dtype == torch.bfloat16 and tc_gemm_ok(a, w_up):
        return gemm_bf16_tc(a, w_up, out, act, checked=True)
    h = linear(a, w_up, scratch((a.shape[0], w_up.shape[0]), a.dtype))
    return unit_act(h, out, act)


def _fused_args(fused, parts: int):
    """A fused projection [n, W] (or float32 partial sums [S, n, W]) as the kernels take it."""
    if parts:
        assert fused.dim() == 3 and fused.shape[0] == parts and fused.stride(2) == 1 and fused.dtype == torch.float32
        return _ptr(fused), _dt(fused), fused.stride(1), parts, ctypes.c_longlong(fused.stride(0)), fused.shape[1]
    assert fused.dim() == 2 and fused.stride(1) == 1
    return _ptr(fused), _dt(fused), fused.stride(0), 1, ctypes.c_longlong(0), fused.shape[0]


def linattn_prepare(fused, parts: int, q_off: int, k_off: int, v_off: int, heads: int, dim: int, vdim: int,
                    positions: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_scale: float = 1.0,
                    k_scale: float = 1.0, inv_freq: torch.Tensor | None = None, rot_dim: int = 0, low_off: int = -1,
                    w2: torch.Tensor | None = None, b2: torch.Tensor | None = None, tau: float = 1.0,
                    decay: torch.Tensor | None = None) -> None:
    """The 32-bit inputs of the decayed-state recurrence from a fused projection row (csrc/linear_attention.cu):
    q [n, heads*dim] and k, turned by the rotary angle of their position over the first rot_dim elements of a head
    and scaled; v [n, heads*vdim]; and, with `low_off` >= 0, the decay per key channel
    sigmoid(w2 @ low + b2)^(1/tau), where `low` are the rank = w2.shape[1] columns of the row from `low_off`."""
    _need_cuda(fused, positions, q, k, v, inv_freq, w2, b2, decay)
    ptr, dt, row_stride, nparts, part_stride, n = _fused_args(fused, parts)
    for t, width in ((q, heads * dim), (k, heads * dim), (v, heads * vdim)):
        assert t.dtype == torch.float32 and t.is_contiguous() and t.shape == (n, width)
    rank = 0
    if low_off >= 0:
        rank = w2.shape[1]
        assert w2.shape == (heads * dim, rank) and w2.is_contiguous() and b2.shape == (heads * dim,) and b2.dtype == w2.dtype
        assert decay.dtype == torch.float32 and decay.is_contiguous() and decay.shape == (n, heads * dim)
    if rot_dim:
        assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dim // 2 and inv_freq.is_contiguous()
    lib = load_family("linear_attention")
    _check(lib.wllm_linattn_prepare(ptr, dt, row_stride, nparts, part_stride, q_off, k_off, v_off, low_off, n, heads, dim,
                                    vdim, rank, _ptr(_int32(positions, "positions")), _ptr(inv_freq), rot_dim,
                                    c_float(q_scale), c_float(k_scale), _ptr(w2), _ptr(b2), _dt(w2) if w2 is not None else _F32,
                                    c_float(tau), _ptr(q), _ptr(k), _ptr(v), _ptr(decay), _stream()), "linattn_prepare")


LINATTN_SEGMENT_FROM = 128     # portions of at least this many tokens may be cut into segments that run side by side
LINATTN_MIN_SEGMENT = 32


def linattn_segment_plan(max_q_len: int, requests_multi: int, heads: int, vdim: int) -> tuple:
    """(seg_len, max_seg) for the recurrence over a step whose longest portion has max_q_len tokens; (0, 1): every
    request is walked in one go.  A walk is sequential in its tokens, and heads x tiles of 64 value columns x requests
    walks seldom fill the device; a long portion is therefore cut into segments that run side by side and are walked
    twice (csrc/linear_attention.cu), as many as the device holds at once (two CTAs an SM), of at least
    LINATTN_MIN_SEGMENT tokens."""
    if max_q_len < LINATTN_SEGMENT_FROM:
        return 0, 1
    walks = max(1, requests_multi) * heads * -(-vdim // 64)
    wanted = (2 * sm_count()) // walks
    if wanted < 3:            # two segments walked twice are no shorter than one walk
        return 0, 1
    seg_len = max(LINATTN_MIN_SEGMENT, -(-(-(-max_q_len // wanted)) // 8) * 8)
    max_seg = -(-max_q_len // seg_len)
    return (seg_len, max_seg) if max_seg > 2 else (0, 1)


def linattn_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay, head_decay, state: torch.Tensor,
                 out: torch.Tensor, req_q_start: torch.Tensor, req_q_len: torch.Tensor, req_slot: torch.Tensor, heads: int,
                 dim: int, vdim: int, seg_len: int = 0, max_seg: int = 1, seg_state: torch.Tensor | None = None,
                 seg_decay: torch.Tensor | None = None) -> torch.Tensor:
    """S <- diag(a_t) S + k_t v_t^T, o_t = S^T q_t over every request's tokens of the step, from and to the
    request's row of `state` [slots, heads, dim, vdim] (float32).  `decay` [n, heads*dim] per key channel, or None
    with `head_decay` [heads].  With seg_len > 0 and max_seg > 1 (linattn_segment_plan) portions are cut into segments
    of seg_len tokens that run side by side; seg_state (requests * max_seg * heads * dim * vdim floats) and seg_decay
    (requests * max_seg * heads * dim) are their scratch."""
    _need_cuda(q, k, v, decay, head_decay, state, out, req_q_start, req_q_len, req_slot, seg_state, seg_decay)
    R = req_q_len.shape[0]
    if seg_len > 0 and max_seg > 1:
        assert seg_state.dtype == seg_decay.dtype == torch.float32 and seg_state.is_contiguous() and seg_decay.is_contiguous()
        assert seg_state.numel() >= R * max_seg * heads * dim * vdim and seg_decay.numel() >= R * max_seg * heads * dim
        global launches
        launches += 2         # the segments' first walk and the kernel that chains their states
    n = q.shape[0]
    assert all(t.dtype == torch.float32 and t.is_contiguous() for t in (q, k, v, state, out))
    assert q.shape == k.shape == (n, heads * dim) and v.shape == out.shape == (n, heads * vdim)
    assert state.shape[1:] == (heads, dim, vdim)
    if decay is not None:
        assert decay.dtype == torch.float32 and decay.is_contiguous() and decay.shape == q.shape
    else:
        assert head_decay.dtype == torch.float32 and head_decay.shape == (heads,) and head_decay.is_contiguous()
    lib = load_family("linear_attention")
    _check(lib.wllm_linattn_scan(_ptr(q), _ptr(k), _ptr(v), _ptr(decay), _ptr(head_decay), _ptr(state), _ptr(out),
                                 _ptr(_int32(req_q_start, "req_q_start")), _ptr(_int32(req_q_len, "req_q_len")),
                                 _ptr(_int32(req_slot, "req_slot")), R, heads, dim, vdim, seg_len, max_seg,
                                 _ptr(seg_state), _ptr(seg_decay), _stream()),
           f"linattn_scan(heads={heads}, dim={dim}, vdim={vdim})")
    return out


def head_gate_norm(o: torch.Tensor, fused, parts: int, gate_off: int, weight, eps: float, out: torch.Tensor, heads: int,
                   vdim: int) -> torch.Tensor:
    """out[n, heads*vdim] = o / sqrt(mean over a head of o^2 + eps) [* weight[vdim]] * silu(gate), the gate being the
    columns of the fused projection row from `gate_off`; 32-bit inside, rounded once to out's element type."""
    _need_cuda(o, fused, weight, out)
    ptr, dt, row_stride, nparts, part_stride, n = _fused_args(fused, parts)
    assert o.dtype == torch.float32 and o.is_contiguous() and o.shape == (n, heads * vdim) == out.shape and out.is_contiguous()
    assert weight is None or (weight.shape == (vdim,) and weight.is_contiguous())
    lib = load_family("linear_attention")
    _check(lib.wllm_head_gate_norm(_ptr(o), ptr, dt, row_stride, nparts, part_stride, gate_off, _ptr(weight),
                                   _dt(weight) if weight is not None else _F32, c_float(eps), _ptr(out), _dt(out), n, heads,
                                   vdim, _stream()), "head_gate_norm")
    return out


def delta_prepare(fused, parts: int, offsets: dict, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, conv_q, conv_k,
                  conv_v, a_log, dt_bias, token_req, req_q_start, req_slot, conv_state, unit_eps: float, q_scale: float, q, k, v,
                  beta, decay) -> None:
    """What enters the gated delta rule, from the fused projection [n, W] (or float32 partial sums [parts, n, W]) whose columns
    `offsets` names (q, k, v, b, a): q, k [n, kv_heads, dim] and v [n, heads, vdim] through their short convolutions (taps
    [channels, taps], the last tap the token's own; the inputs before a portion's start come from `conv_state`
    [slots, taps - 1, channels]) and SiLU, q and k divided by sqrt(sum(x^2) + unit_eps) per head (q also times q_scale),
    beta = sigmoid(b) and decay = exp(-exp(a_log) softplus(a + dt_bias)) [n, heads]; all 32-bit (csrc/delta_rule.cu)."""
    _need_cuda(fused, conv_q, conv_k, conv_v, a_log, dt_bias, token_req, req_q_start, req_slot, conv_state, q, k, v, beta, decay)
    ptr, dt, row_stride, nparts, part_stride, n = _fused_args(fused, parts)
    C = 2 * kv_heads * dim + heads * vdim
    assert conv_q.shape == conv_k.shape == (kv_heads * dim, taps) and conv_v.shape == (heads * vdim, taps)
    assert conv_q.dtype == conv_k.dtype == conv_v.dtype == a_log.dtype == dt_bias.dtype
    assert all(t.is_contiguous() for t in (conv_q, conv_k, conv_v, a_log, dt_bias, q, k, v, beta, decay))
    assert a_log.shape == dt_bias.shape == (heads,)
    assert q.shape == k.shape == (n, kv_heads * dim) and v.shape == (n, heads * vdim) and beta.shape == decay.shape == (n, heads)
    assert all(t.dtype == torch.float32 for t in (q, k, v, beta, decay))
    assert taps == 1 or (conv_state.dtype == torch.float32 and conv_state.is_contiguous() and conv_state.shape[1:] == (taps - 1, C))
    lib = load_family("delta_rule")
    _check(lib.wllm_delta_prepare(ptr, dt, row_stride, nparts, part_stride, offsets["q"], offsets["k"], offsets["v"], offsets["b"],
                                  offsets["a"], n, heads, kv_heads, dim, vdim, taps, _ptr(conv_q), _ptr(conv_k), _ptr(conv_v),
                                  _ptr(a_log), _ptr(dt_bias), _dt(conv_q), _ptr(_int32(token_req, "token_req")),
                                  _ptr(_int32(req_q_start, "req_q_start")), _ptr(_int32(req_slot, "req_slot")),
                                  _ptr(conv_state if taps > 1 else None), c_float(unit_eps), c_float(q_scale), _ptr(q), _ptr(k), _ptr(v),
                                  _ptr(beta), _ptr(decay), _stream()), "delta_prepare")


def delta_conv_update(fused, parts: int, offsets: dict, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, req_q_start,
                      req_q_len, req_slot, conv_state) -> None:
    """The last taps - 1 inputs of the short convolutions, per request, after this step's tokens: conv_state[slot] becomes the
    tail of (what it held, the step's q | k | v columns of `fused`).  Requests that bring no token are passed by."""
    if taps <= 1:
        return
    _need_cuda(fused, req_q_start, req_q_len, req_slot, conv_state)
    ptr, dt, row_stride, nparts, part_stride, _ = _fused_args(fused, parts)
    lib = load_family("delta_rule")
    _check(lib.wllm_delta_conv_update(ptr, dt, row_stride, nparts, part_stride, offsets["q"], offsets["k"], offsets["v"], heads,
                                      kv_heads, dim, vdim, taps, _ptr(_int32(req_q_start, "req_q_start")),
                                      _ptr(_int32(req_q_len, "req_q_len")), _ptr(_int32(req_slot, "req_slot")), req_q_len.shape[0],
                                      _ptr(conv_state), _stream()), "delta_conv_update")


def delta_scan(q, k, v, beta, decay, state, out, req_q_start, req_q_len, req_slot, heads: int, kv_heads: int, dim: int, vdim: int):
    """The gated delta rule over every request's tokens of the step, in order, from and to its state slot:
    S <- decay S; u = beta (v - S^T k); S <- S + k u^T; out = S^T q.  q, k [n, kv_heads * dim], v, out [n, heads * vdim],
    beta, decay [n, heads], state [slots, heads, dim, vdim], all float32 (csrc/delta_rule.cu)."""
    _need_cuda(q, k, v, beta, decay, state, out, req_q_start, req_q_len, req_slot)
    n = q.shape[0]
    assert all(t.dtype == torch.float32 and t.is_contiguous() for t in (q, k, v, beta, decay, state, out))
    assert q.shape == k.shape == (n, kv_heads * dim) and v.shape == out.shape == (n, heads * vdim) and beta.shape == decay.shape == (n, heads)
    assert state.shape[1:] == (heads, dim, vdim)
    lib = load_family("delta_rule")
    _check(lib.wllm_delta_scan(_ptr(q), _ptr(k), _ptr(v), _ptr(beta), _ptr(decay), _ptr(state), _ptr(out),
                               _ptr(_int32(req_q_start, "req_q_start")), _ptr(_int32(req_q_len, "req_q_len")),
                               _ptr(_int32(req_slot, "req_slot")), req_q_len.shape[0], heads, kv_heads, dim, vdim, _stream()),
           f"delta_scan(heads={heads}/{kv_heads}, dim={dim}/{vdim})")
    return out


def moe_route(x: torch.Tensor, w_router: torch.Tensor, w_gate, chosen: torch.Tensor, weights: torch.Tensor, gate_out,
              groups: int = 1, groups_kept: int = 1, scores: str = "softmax") -> None:
    """The router of routed experts (csrc/moe.cu): scores = softmax(w_router x) in 32-bit over all E experts (`scores`
    'sigmoid': sigmoid(w_router x) expert by expert, not normalised; without groups the choice is made on the logits, whose order
    the sigmoid keeps, so that large logits that all round to a score of 1 do not tie), the choice
    limited to the `groups_kept` best of `groups` groups of neighbouring experts; chosen [n, top] (descending score) and
    weights [n, top] (the scores as they are).  With `w_gate` [H], gate_out[n] = sigmoid(w_gate . x)."""
    _need_cuda(x, w_router, w_gate, chosen, weights, gate_out)
    n, H = x.shape
    E, top = w_router.shape[0], chosen.shape[1]
    assert x.is_contiguous() and w_router.dtype == torch.float32 and w_router.shape == (E, H) and w_router.is_contiguous()
    assert chosen.shape == weights.shape == (n, top) and chosen.dtype == torch.int32 and weights.dtype == torch.float32
    assert chosen.is_contiguous() and weights.is_contiguous()
    if w_gate is not None:
        assert w_gate.dtype == torch.float32 and w_gate.shape == (H,) and w_gate.is_contiguous()
        assert gate_out.dtype == torch.float32 and gate_out.shape == (n,) and gate_out.is_contiguous()
    if scores not in ("softmax", "sigmoid"):
        raise KernelError(f"router scores {scores!r}: 'softmax' or 'sigmoid'")
    lib = load_family("moe")
    _check(lib.wllm_moe_route(_ptr(x), _dt(x), _ptr(w_router), _ptr(w_gate), _ptr(chosen), _ptr(weights), _ptr(gate_out), n, H, E,
                              top, groups, groups_kept, 1 if scores == "sigmoid" else 0, _stream()), f"moe_route(experts={E}, top={top}, groups={groups}/{groups_kept})")


MOE_TILE_ROWS = 128      # rows of a row tile of the experts' products on the tensor-memory kernel


def moe_row_tiles(pairs: int, experts: int) -> int:
    """Most row tiles (MOE_TILE_ROWS rows of one expert each) that `pairs` sorted rows of `experts` experts can make."""
    return -(-pairs // MOE_TILE_ROWS) + experts


MOE_PLAN_SEGMENTS = 8     # warps an expert that scan a long list of pairs (csrc/moe.cu)


def moe_plan(chosen: torch.Tensor, count: torch.Tensor, offset: torch.Tensor, order: torch.Tensor, place: torch.Tensor,
             tiles: torch.Tensor | None = None, scratch: torch.Tensor | None = None) -> None:
    """The (token, rank) pairs of `chosen` [n, top] sorted by expert, stably: count [E], offset [E + 1], order [pairs] (sorted
    row -> pair), place [pairs] (pair -> sorted row).  `tiles` (int32, 1 + 3 * moe_row_tiles(pairs, E)): the table of row
    tiles for gemm_bf16_tc_grouped: their number, then (expert, first sorted row, rows) a tile.  `scratch` (int32,
    MOE_PLAN_SEGMENTS * E): with it a long list is scanned by several warps an expert; the result is the same."""
    _need_cuda(chosen, count, offset, order, place, tiles, scratch)
    pairs, E = chosen.numel(), count.shape[0]
    assert offset.shape == (E + 1,) and order.shape == place.shape == (pairs,)
    for t in (chosen, count, offset, order, place):
        assert t.dtype == torch.int32 and t.is_contiguous()
    assert tiles is None or (tiles.dtype == torch.int32 and tiles.is_contiguous() and tiles.numel() >= 1 + 3 * moe_row_tiles(pairs, E))
    lib = load_family("moe")
    assert scratch is None or (scratch.dtype == torch.int32 and scratch.is_contiguous() and scratch.numel() >= MOE_PLAN_SEGMENTS * E)
    _check(lib.wllm_moe_plan_tiles(_ptr(chosen), pairs, E, _ptr(count), _ptr(offset), _ptr(order), _ptr(place), _ptr(tiles),
                                   MOE_TILE_ROWS, _ptr(scratch), _stream()), "moe_plan")
    global launches
    launches += 1


def moe_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, offset: torch.Tensor, order: torch.Tensor, top: int,
                gated: bool, limit: float = 0.0, slope: float = 0.0, unit: str | None = None,
                row_weights: torch.Tensor | None = None) -> torch.Tensor:
    """The experts' products over rows sorted by expert.  gated: a [n, K] holds the tokens' rows (sorted row r reads row
    order[r] // top), w [E, 2N, K] = [gate; up] per expert, out [pairs, N] = the clamped gated unit, in the operands' type.
    `unit` 'relu_squared' (not gated): a [n, K] holds the tokens' rows too, w [E, N, K], out [pairs, N] = relu(s (w a))^2 in the
    operands' type, s = row_weights[pair] (float32 [pairs] in pair order; None: 1).
    Otherwise a [pairs, K] holds sorted rows, w [E, N, K], out [pairs, N] float32.  32-bit accumulation."""
    _need_cuda(a, w, out, offset, order, row_weights)
    if unit not in (None, "relu_squared") or (unit is not None and gated):
        raise KernelError(f"expert unit {unit!r}: None or 'relu_squared', and not gated")
    E, pairs, K = w.shape[0], order.shape[0], a.shape[1]
    N = w.shape[1] // 2 if gated else w.shape[1]
    gathers = gated or unit is not None
    assert a.dtype == w.dtype and a.stride(1) == 1 and w.is_contiguous() and w.shape[2] == K and out.is_contiguous()
    assert out.shape == (pairs, N) and out.dtype == (a.dtype if gathers else torch.float32) and offset.shape == (E + 1,)
    assert gathers or a.shape[0] == pairs
    assert row_weights is None or (unit is not None and row_weights.dtype == torch.float32 and row_weights.numel() == pairs and row_weights.is_contiguous())
    lib = load_family("moe")
    _check(lib.wllm_moe_grouped_unit(_ptr(a), a.stride(0), _ptr(w), _ptr(out), _dt(a), 1 if gated else (2 if unit else 0), pairs, N, K,
                                     _ptr(_int32(offset, "offset")), _ptr(_int32(order, "order")), E, top, c_float(limit), c_float(slope),
                                     _ptr(row_weights), _stream()), f"moe_grouped({pairs}x{N}x{K}, {E} experts)")
    return out


def moe_gather(x: torch.Tensor, order: torch.Tensor, top: int, out: torch.Tensor, row_weights: torch.Tensor | None = None) -> torch.Tensor:
    """out[r] = x[order[r] // top]: the tokens' bfloat16 rows in the order of the sorted pairs; with `row_weights` (float32
    [pairs], pair order) every row is multiplied by its pair's weight, in 32-bit, rounded once."""
    _need_cuda(x, order, out, row_weights)
    pairs, K = out.shape
    assert x.dtype == out.dtype == torch.bfloat16 and x.stride(1) == 1 and out.is_contiguous() and x.shape[1] == K and order.shape == (pairs,)
    assert row_weights is None or (row_weights.dtype == torch.float32 and row_weights.numel() == pairs and row_weights.is_contiguous())
    lib = load_family("moe")
    _check(lib.wllm_moe_gather_scaled(_ptr(x), x.stride(0), _ptr(_int32(order, "order")), top, _ptr(out), pairs, K, _ptr(row_weights),
                                      _stream()), "moe_gather")
    return out


def tc_grouped_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Shapes the grouped tensor-memory product takes: bfloat16, rows of A contiguous, K in steps of 8."""
    return (a.dtype == torch.bfloat16 == w.dtype and a.dim() == 2 and w.dim() == 3 and a.is_contiguous() and w.is_contiguous()
            and a.shape[1] == w.shape[2] and a.shape[1] % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_bf16_tc_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tiles: torch.Tensor, gated: bool, limit: float = 0.0,
                         slope: float = 0.0, unit: str | None = None) -> torch.Tensor:
    """The experts' products on tcgen05 tensor cores (csrc/gemm_bf16_tc.cu, grouped): a [rows, K] bfloat16 rows sorted by
    expert, w [E, N, K] (or, gated, [E, 2N, K] = [gate; up]: out = the clamped gated unit, bfloat16 [rows, N]; else out float32
    [rows, N]; `unit` 'relu_squared': out = relu(a w^T)^2, bfloat16), `tiles` the table of row tiles that moe_plan left on the device."""
    _need_cuda(a, w, out, tiles)
    if not tc_grouped_ok(a, w):
        raise KernelError("gemm_bf16_tc_grouped: contiguous bfloat16 operands with K in steps of 8")
    rows, K = a.shape
    E = w.shape[0]
    N = w.shape[1] // 2 if gated else w.shape[1]
    if unit not in (None, "relu_squared") or (unit is not None and gated):
        raise KernelError(f"expert unit {unit!r}: None or 'relu_squared', and not gated")
    assert out.shape == (rows, N) and out.is_contiguous() and out.dtype == (torch.bfloat16 if gated or unit else torch.float32)
    assert tiles.dtype == torch.int32 and tiles.numel() >= 1 + 3 * moe_row_tiles(rows, E)
    lib = load_family("gemm_bf16_tc")
    _check(lib.wllm_gemm_bf16_tc_grouped(_ptr(a), K, _ptr(w), K, _ptr(out), N, rows, N, K, E, 5 if gated else (6 if unit else 1), _ptr(tiles),
                                         moe_row_tiles(rows, E), _ptr(_status_word(a.device)), sm_count(), c_float(limit),
                                         c_float(slope), _stream()), f"gemm_bf16_tc_grouped({rows}x{N}x{K}, {E} experts)")
    return out


def moe_combine(y: torch.Tensor, place: torch.Tensor, weights: torch.Tensor, shared, gate, out: torch.Tensor) -> torch.Tensor:
    """out[t] = sum over ranks k, in order, of weights[t, k] * y[place[t * top + k]]  (+ gate[t] * shared[t]; `shared`:
    None or (tensor [n, H] | float32 partial sums [P, n, H], P or 0)).  `weights` None: the outputs are added as they are."""
    _need_cuda(y, place, weights, gate, out, shared[0] if shared is not None else None)
    n, H = out.shape
    top = place.shape[0] // max(n, 1)
    assert y.dtype == torch.float32 == out.dtype and y.is_contiguous() and out.is_contiguous() and y.shape[1] == H
    assert place.shape == (n * top,) and (weights is None or (weights.shape == (n, top) and weights.dtype == torch.float32 and weights.is_contiguous()))
    ps = _branch_args(shared, n, H) if shared is not None else (_ptr(None), _F32, 1, ctypes.c_longlong(0))
    lib = load_family("moe")
    _check(lib.wllm_moe_combine(_ptr(y), _ptr(_int32(place, "place")), _ptr(weights), top, *ps, _ptr(gate), _ptr(out), n, H,
                                _stream()), "moe_combine")
    return out


__all__ = ["KernelError", "KernelBuildError", "embed_gather", "rmsnorm", "rope_kv_write", "paged_attention_simt",
           "paged_attention_simt_tiled",
           "attention_mma_decode", "attention_mma_prefill", "mma_head_dim_ok", "gemm_bf16_tc", "tc_gemm_ok",
           "tc_gemm_status",
           "gated_act", "gemm_f32", "linear", "project", "gated_linear", "split_plan", "branch_norm", "linattn_prepare",
           "linattn_scan", "head_gate_norm", "sandwich_norm"]
