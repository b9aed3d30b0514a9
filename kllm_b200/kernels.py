"""Python faces of the CUDA kernels: each takes torch tensors on a CUDA device,
checks what the kernel assumes, and launches on torch's current stream.

The libraries are compiled and loaded on first use (``csrc/build.py``).  There is
no CPU or library fallback here: a tensor that is not on a CUDA device is an error.
``launches`` counts the kernels launched through this module (a captured CUDA
graph replays its launches without passing through here; the graph runner adds
its own count).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .csrc.build import load_library

launches = 0

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel operand is not on a CUDA device (there is no CPU path)")


def _check(lib, name: str, rc: int):
    global launches
    if rc != 0:
        fn = getattr(lib, "kllm_last_error_" + name)
        fn.restype = ctypes.c_char_p
        raise KernelError(f"{name}: {fn().decode(errors='replace')} (code {rc})")
    launches += 1


def _i32(t: Optional[torch.Tensor], what: str):
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{what} must be a contiguous int32 tensor")


def embed(out_x: torch.Tensor, table: torch.Tensor, ids: torch.Tensor,
          last_token: Optional[torch.Tensor] = None) -> None:
    """out_x[t,:] = float32(table[ids[t],:]); out_x float32 [n, d].  With ``last_token``
    (int32, one entry per request slot) an id -(s + 1) means last_token[s], the token
    that ``sample`` stored there."""
    _cuda(out_x, table, ids, last_token)
    _i32(ids, "ids"); _i32(last_token, "last_token")
    n, d = out_x.shape
    if out_x.dtype != torch.float32 or not out_x.is_contiguous() or not table.is_contiguous():
        raise KernelError("embed: residual stream must be contiguous float32")
    if table.shape[1] != d or ids.numel() != n:
        raise KernelError("embed: shapes do not agree")
    lib = load_library("embedding")
    rc = lib.kllm_embed(_p(out_x), _p(table), _p(ids), _p(last_token), n, d, table.shape[0], dtype_code(table.dtype),
                        _stream())
    _check(lib, "embedding", rc)


def gather_rows(out: torch.Tensor, src: torch.Tensor, rows: torch.Tensor) -> None:
    """out[r,:] = src[rows[r],:] for contiguous 2-D tensors of one dtype."""
    _cuda(out, src, rows)
    _i32(rows, "rows")
    if out.dtype != src.dtype or not out.is_contiguous() or not src.is_contiguous() or out.shape[1] != src.shape[1]:
        raise KernelError("gather_rows: operands do not agree")
    lib = load_library("embedding")
    rc = lib.kllm_gather_rows(_p(out), _p(src), _p(rows), rows.numel(),
                              ctypes.c_int64(src.shape[1] * src.element_size()), _stream())
    _check(lib, "embedding", rc)


def add_rmsnorm(x: torch.Tensor, res: Optional[torch.Tensor], out: torch.Tensor, gain: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """x (+)= res in float32, out = rmsnorm(x) * gain.

    ``rows`` given: out[r] comes from row rows[r] of x (+ res) and x is not written.
    """
    _cuda(x, res, out, gain, rows)
    _i32(rows, "rows")
    d = x.shape[1]
    if x.dtype != torch.float32 or gain.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("add_rmsnorm: x and gain must be float32, contiguous")
    if res is not None and (res.dtype not in (out.dtype, torch.float32) or not res.is_contiguous()
                            or res.shape != x.shape):
        raise KernelError("add_rmsnorm: res must match x in shape and be float32 or of out's dtype")
    if gain.numel() != d or out.shape[1] != d:
        raise KernelError("add_rmsnorm: widths do not agree")
    n_rows = out.shape[0]
    if rows is None and n_rows != x.shape[0]:
        raise KernelError("add_rmsnorm: row counts do not agree")
    if rows is not None and rows.numel() != n_rows:
        raise KernelError("add_rmsnorm: rows and out do not agree")
    lib = load_library("norm")
    rc = lib.kllm_add_rmsnorm(_p(x), _p(res), _p(out), _p(gain), _p(rows), n_rows, d,
                              ctypes.c_float(eps), dtype_code(out.dtype),
                              dtype_code(res.dtype if res is not None else out.dtype), _stream())
    _check(lib, "norm", rc)


def rope_append(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cos_sin: Optional[torch.Tensor],
                positions: torch.Tensor, token_req: torch.Tensor, block_table: Optional[torch.Tensor],
                kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor],
                n_heads: int, n_kv: int, head_dim: int) -> None:
    """Rotate q in place; write rotated k and v into the paged cache.

    q, k, v are 2-D views (rows may be strided, the last dim is dense); caches are
    [pages, n_kv, page_size, head_dim].  With kcache None only q is rotated; with
    cos_sin None nothing is rotated and k, v are only stored.
    """
    _cuda(q, k, v, cos_sin, positions, token_req, block_table, kcache, vcache)
    _i32(positions, "positions"); _i32(token_req, "token_req"); _i32(block_table, "block_table")
    for t in (q, k, v):
        if t.stride(1) != 1:
            raise KernelError("rope_append: q, k, v rows must be dense")
    if cos_sin is not None and (cos_sin.dtype != torch.float32 or not cos_sin.is_contiguous()):
        raise KernelError("rope_append: the cos/sin table must be contiguous float32")
    n = q.shape[0]
    rot = cos_sin.shape[1] if cos_sin is not None else 0
    if kcache is not None:
        if kcache.shape != vcache.shape or kcache.shape[1] != n_kv or kcache.shape[3] != head_dim \
                or not kcache.is_contiguous() or not vcache.is_contiguous() or kcache.dtype != q.dtype:
            raise KernelError("rope_append: cache layout must be [pages, n_kv, page_size, head_dim] in q's dtype")
        page_size, max_blocks = kcache.shape[2], block_table.shape[1]
    else:
        page_size, max_blocks = 1, 0
    lib = load_library("rope")
    rc = lib.kllm_rope_append(_p(q), ctypes.c_int64(q.stride(0)), _p(k), ctypes.c_int64(k.stride(0)),
                              _p(v), ctypes.c_int64(v.stride(0)), _p(cos_sin), _p(positions),
                              _p(token_req), _p(block_table), max_blocks, _p(kcache), _p(vcache),
                              n, n_heads, n_kv, head_dim, rot, page_size, dtype_code(q.dtype), _stream())
    _check(lib, "rope", rc)


def attention_generic(out: torch.Tensor, q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                      positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor,
                      n_heads: int, n_kv: int, head_dim: int, window: int, scale: float) -> None:
    """Causal GQA attention of every new token over its request's cached keys."""
    _cuda(out, q, kcache, vcache, positions, token_req, block_table)
    _i32(positions, "positions"); _i32(token_req, "token_req"); _i32(block_table, "block_table")
    if q.stride(1) != 1 or not out.is_contiguous() or out.dtype != q.dtype or kcache.dtype != q.dtype:
        raise KernelError("attention: operands must share a dtype; out contiguous, q rows dense")
    if not kcache.is_contiguous() or not vcache.is_contiguous() or kcache.shape[1] != n_kv or kcache.shape[3] != head_dim:
        raise KernelError("attention: cache layout must be [pages, n_kv, page_size, head_dim]")
    n = q.shape[0]
    lib = load_library("attention_generic")
    rc = lib.kllm_attention_generic(_p(out), _p(q), ctypes.c_int64(q.stride(0)), _p(kcache), _p(vcache),
                                    _p(positions), _p(token_req), _p(block_table), block_table.shape[1],
                                    n, n_heads, n_kv, head_dim, kcache.shape[2], int(window or 0),
                                    ctypes.c_float(scale), dtype_code(q.dtype), _stream())
    _check(lib, "attention_generic", rc)


SIMT_CHUNK = 256      # keys per CTA when a decoding token's context is cut (attention_simt)


def attention_simt(out: torch.Tensor, q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, ctx,
                   block_table: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, window: int,
                   scale: float, score_slopes: Optional[torch.Tensor] = None) -> None:
    """Causal GQA attention of the step's tokens on the CUDA cores, float32 arithmetic
    (csrc/attention_simt.cu): the attention of the float32 path.  The requests that bring
    one token each at the head of the batch (decoding requests, which the scheduler puts
    first) have their contexts cut into chunks of SIMT_CHUNK keys, one CTA each, merged in
    chunk order; the portions after them run as tiles of up to 64 (token, head) rows.
    ``score_slopes`` (float32 [n_heads]): slope[h] * (key position - query position) is added
    to the scaled scores of head h."""
    _cuda(out, q, kcache, vcache, block_table, score_slopes)
    if score_slopes is not None and (score_slopes.dtype != torch.float32 or not score_slopes.is_contiguous()
                                     or score_slopes.numel() != n_heads):
        raise KernelError("attention: score slopes must be a contiguous float32 tensor, one per head")
    _i32(block_table, "block_table"); _i32(ctx.q_start, "q_start"); _i32(ctx.start_pos, "start_pos")
    if q.stride(1) != 1 or not out.is_contiguous() or out.dtype != q.dtype or kcache.dtype != q.dtype:
        raise KernelError("attention: operands must share a dtype; out contiguous, q rows dense")
    if not kcache.is_contiguous() or not vcache.is_contiguous() or kcache.shape[1] != n_kv or kcache.shape[3] != head_dim:
        raise KernelError("attention: cache layout must be [pages, n_kv, page_size, head_dim]")
    group = n_heads // max(1, n_kv)
    lib = load_library("attention_simt")
    n_req = ctx.n_requests
    singles = n_req if ctx.all_single else 0
    if not ctx.all_single and ctx.host_n_new:
        while singles < n_req and ctx.host_n_new[singles] == 1:
            singles += 1
    bound = ctx.split_bound or ctx.max_ctx
    if window:
        bound = min(bound, int(window))
    splits = max(1, -(-bound // SIMT_CHUNK))
    common = (n_heads, n_kv, head_dim, kcache.shape[2], int(window or 0), ctypes.c_float(scale))
    first = 0
    global launches
    if singles and splits > 1:
        part_o = torch.empty((singles * n_heads, splits, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((singles * n_heads, splits, 2), dtype=torch.float32, device=q.device)
        rc = lib.kllm_attention_simt(_p(out), _p(part_o), _p(part_ml), _p(q), ctypes.c_int64(q.stride(0)), _p(kcache),
                                     _p(vcache), _p(ctx.q_start), _p(ctx.start_pos), _p(block_table),
                                     block_table.shape[1], singles, singles, *common, 1, SIMT_CHUNK, splits,
                                     _p(score_slopes), dtype_code(q.dtype), _stream())
        _check(lib, "attention_simt", rc)
        rc = lib.kllm_attention_simt_merge(_p(out), _p(part_o), _p(part_ml), _p(ctx.positions), singles, n_heads,
                                           head_dim, int(window or 0), SIMT_CHUNK, splits, dtype_code(q.dtype), _stream())
        _check(lib, "attention_simt", rc)
        first = singles
    if first < n_req:
        qt = max(1, 64 // group)
        rest = ctx.n_tokens - first
        rc = lib.kllm_attention_simt(_p(out), None, None, _p(q), ctypes.c_int64(q.stride(0)), _p(kcache), _p(vcache),
                                     _p(ctx.q_start[first:]), _p(ctx.start_pos[first:]), _p(block_table[first:]),
                                     block_table.shape[1], n_req - first, rest // qt + (n_req - first), *common, qt, 0, 1,
                                     _p(score_slopes), dtype_code(q.dtype), _stream())
        _check(lib, "attention_simt", rc)


def simt_fits(q: torch.Tensor, n_heads: int, n_kv: int, head_dim: int) -> bool:
    """Whether ``attention_simt`` takes these operands: head size a multiple of 4 up to
    256, at most 64 heads per kv head, rows aligned to four elements."""
    quad = 4 * q.element_size()
    return (head_dim % 4 == 0 and 0 < head_dim <= 256 and n_heads // max(1, n_kv) <= 64
            and q.data_ptr() % quad == 0 and q.stride(0) % 4 == 0)


TC_HEAD_DIMS = tuple(range(16, 129, 16))     # head sizes of the tensor-core attention library
TCGEN05_HEAD_DIMS = (64, 128)                # head sizes of the tcgen05 prefill attention
PREFETCH_L2 = os.environ.get("KLLM_B200_PREFETCH", "1") != "0"   # kernels warm L2 for the kernel after them
# ... with at most this much of the next matrix: what is asked for beyond a fraction of the
# 126 MB of L2 pushes out lines that are still needed and is read from HBM twice
PREFETCH_L2_BYTES = int(float(os.environ.get("KLLM_B200_PREFETCH_MB", "24")) * 2 ** 20)
USE_TCGEN05 = os.environ.get("KLLM_B200_TCGEN05", "1") != "0"
_sm_count = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current device (148 on a B200)."""
    dev = torch.cuda.current_device()
    if dev not in _sm_count:
        _sm_count[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _sm_count[dev]


def decode_splits(n_tokens: int, n_kv: int, ctx_bound: int) -> int:
    """Into how many key ranges the decode kernel cuts a token's context.

    A CTA takes one (token, kv head, range); two CTAs fit an SM.  The ranges are
    whole 64-key tiles, as many as fill the SMs in ONE wave (a second wave of short
    CTAs would double the kernel's time), at most 16, all the same length.  When one
    range per token would be long, two are used even if that spills into a second
    wave: long CTAs hide it."""
    slots = 2 * sm_count()
    tiles = max(1, -(-ctx_bound // 64))
    base = max(1, n_tokens * n_kv)
    splits = max(1, min(slots // base, tiles, 16))
    if splits == 1 and tiles >= 16:
        splits = 2
    per = -(-tiles // splits)
    return -(-tiles // per)


def attention(out: torch.Tensor, q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, ctx,
              block_table: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, window: int,
              scale: float, score_slopes: Optional[torch.Tensor] = None) -> None:
    """Causal GQA attention of the step's tokens over the paged cache, by the
    kernel that fits: bfloat16 with a head size in TC_HEAD_DIMS runs on tensor cores
    (the decode form when every request brings one token, else the prefill form: on
    tcgen05 for head sizes 64 and 128, on mma.sync for the other multiples of 16);
    float32 and other head sizes run on the CUDA cores (``attention_simt``; head sizes
    that are no multiple of 4 and groups wider than 64 the one-warp-per-row kernel).  A mixed
    step whose first requests bring one token each (the scheduler puts decoding requests
    first) is cut in two: those tokens take the decode form, which spreads a long context
    over many CTAs, the portions after them the prefill form, in which a single token
    would walk its whole context with one CTA of 128 rows, 127 of them idle.
    ``score_slopes`` (a bias on the scores that is linear in the distance, per head) is
    taken by the CUDA-core kernel only; the tensor-core kernels have no such argument."""
    group = n_heads // max(1, n_kv)
    if score_slopes is not None:
        if not simt_fits(q, n_heads, n_kv, head_dim):
            raise KernelError("attention: a bias on the scores needs a head size that is a multiple of 4 up to 256, "
                              "at most 64 heads per kv head and rows aligned to four elements")
        return attention_simt(out, q, kcache, vcache, ctx, block_table, n_heads, n_kv, head_dim, window, scale,
                              score_slopes)
    tc = q.dtype == torch.bfloat16 and head_dim in TC_HEAD_DIMS
    if tc and ctx.all_single and group <= 16:
        return attention_decode(out, q, kcache, vcache, ctx.positions, ctx.token_req, block_table, n_heads,
                                n_kv, head_dim, window, scale,
                                decode_splits(ctx.n_tokens, n_kv, ctx.split_bound or ctx.max_ctx))
    singles = 0
    if tc and group <= 16 and ctx.host_n_new:
        while singles < ctx.n_requests and ctx.host_n_new[singles] == 1:
            singles += 1
    if 0 < singles < ctx.n_requests:
        # token t of the first `singles` is request t: no token-to-request table needed
        attention_decode(out[:singles], q[:singles], kcache, vcache, ctx.positions[:singles], None,
                         block_table[:singles], n_heads, n_kv, head_dim, window, scale,
                         decode_splits(singles, n_kv, ctx.max_ctx))
    q_start, start_pos, table, n_req = ctx.q_start, ctx.start_pos, block_table, ctx.n_requests
    if 0 < singles < ctx.n_requests:
        q_start, start_pos, table, n_req = q_start[singles:], start_pos[singles:], block_table[singles:], n_req - singles
    if tc and USE_TCGEN05 and head_dim in TCGEN05_HEAD_DIMS and group <= 128:
        return attention_prefill_tcgen05(out, q, kcache, vcache, q_start, start_pos, table,
                                         n_req, n_heads, n_kv, head_dim, window, scale,
                                         probabilities=tcgen05_form(head_dim, group, n_kv, ctx.n_tokens - singles,
                                                                    n_req, ctx.max_ctx))
    if tc and group <= 64:
        return attention_prefill(out, q, kcache, vcache, q_start, start_pos, table,
                                 n_req, n_heads, n_kv, head_dim, window, scale)
    if simt_fits(q, n_heads, n_kv, head_dim):
        return attention_simt(out, q, kcache, vcache, ctx, block_table, n_heads, n_kv, head_dim, window, scale)
    return attention_generic(out, q, kcache, vcache, ctx.positions, ctx.token_req, block_table, n_heads, n_kv,
                             head_dim, window, scale)


def _check_attention(out, q, kcache, vcache, block_table, n_kv, head_dim):
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16:
        raise KernelError("tensor-core attention takes bfloat16 operands")
    if q.stride(1) != 1 or not out.is_contiguous() or not kcache.is_contiguous() or not vcache.is_contiguous():
        raise KernelError("attention: out and caches contiguous, q rows dense")
    if kcache.shape[1] != n_kv or kcache.shape[3] != head_dim or kcache.shape != vcache.shape:
        raise KernelError("attention: cache layout must be [pages, n_kv, page_size, head_dim]")
    _i32(block_table, "block_table")


def attention_decode(out, q, kcache, vcache, positions, token_req, block_table, n_heads, n_kv, head_dim,
                     window, scale, num_splits: int) -> None:
    """Tensor-core decode attention: every token attends on its own, its keys cut
    into ``num_splits`` ranges that are merged in a fixed order."""
    _cuda(out, q, kcache, vcache, positions, token_req, block_table)
    _check_attention(out, q, kcache, vcache, block_table, n_kv, head_dim)
    _i32(positions, "positions"); _i32(token_req, "token_req")
    n = q.shape[0]
    part_o = part_ml = None
    if num_splits > 1:
        part_o = torch.empty((n, n_heads, num_splits, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, n_heads, num_splits, 2), dtype=torch.float32, device=q.device)
    lib = load_library("attention_tc", {"KLLM_HD": head_dim})
    rc = lib.kllm_attention_decode(_p(out), _p(part_o), _p(part_ml), _p(q), ctypes.c_int64(q.stride(0)),
                                   _p(kcache), _p(vcache), _p(positions), _p(token_req), _p(block_table),
                                   block_table.shape[1], n, n_heads, n_kv, head_dim, kcache.shape[2],
                                   int(window or 0), ctypes.c_float(scale), int(num_splits), _stream())
    _check(lib, "attention_tc", rc)
    global launches
    if num_splits > 1:
        launches += 1       # the combine kernel


def attention_decode_fused(out, q, k_new, v_new, cos_sin, kcache, vcache, positions, token_req, block_table,
                           counters, n_heads, n_kv, head_dim, window, scale, num_splits: int,
                           prefetch: Optional[torch.Tensor] = None) -> None:
    """Decode attention of one token per request with the rotary encoding, the cache
    write and the merge of the key ranges inside the kernel.  q, k_new, v_new are the
    step's unrotated projections; ``counters`` is an all-zero int32 tensor of at least
    n_tokens * n_kv elements that the kernel leaves all zero.  ``token_req`` may be None:
    token t then belongs to request t, and the kernel reads its block-table row without
    waiting for that look-up.  ``prefetch``: a contiguous tensor that a later kernel
    streams; it is requested into L2 once this kernel's own copies are on their way."""
    _cuda(out, q, k_new, v_new, cos_sin, kcache, vcache, positions, token_req, block_table, counters)
    _check_attention(out, q, kcache, vcache, block_table, n_kv, head_dim)
    _i32(positions, "positions"); _i32(token_req, "token_req"); _i32(counters, "counters")
    n = q.shape[0]
    if k_new.stride(1) != 1 or v_new.stride(1) != 1 or k_new.dtype != q.dtype or v_new.dtype != q.dtype:
        raise KernelError("attention (fused): k and v must be bfloat16 with dense rows")
    if cos_sin.dtype != torch.float32 or not cos_sin.is_contiguous() or cos_sin.shape[1] != head_dim:
        raise KernelError("attention (fused): the cos/sin table must be float32 [positions, head_dim]")
    if counters.numel() < n * n_kv:
        raise KernelError("attention (fused): too few counters")
    part_o = part_ml = None
    if num_splits > 1:
        part_o = torch.empty((n, n_heads, num_splits, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, n_heads, num_splits, 2), dtype=torch.float32, device=q.device)
    lib = load_library("attention_tc", {"KLLM_HD": head_dim})
    rc = lib.kllm_attention_decode_fused(
        _p(out), _p(part_o), _p(part_ml), _p(counters), _p(q), ctypes.c_int64(q.stride(0)), _p(k_new),
        ctypes.c_int64(k_new.stride(0)), _p(v_new), ctypes.c_int64(v_new.stride(0)), _p(cos_sin), _p(kcache),
        _p(vcache), _p(positions), _p(token_req), _p(block_table), block_table.shape[1], n, n_heads, n_kv,
        head_dim, kcache.shape[2], int(window or 0), ctypes.c_float(scale), int(num_splits),
        *_prefetch_args(prefetch), _stream())
    _check(lib, "attention_tc", rc)


def attention_prefill(out, q, kcache, vcache, q_start, start_pos, block_table, n_requests, n_heads, n_kv,
                      head_dim, window, scale) -> None:
    """Tensor-core attention of portions: request s brings rows q_start[s]..q_start[s+1]
    that start at cache position start_pos[s]."""
    _cuda(out, q, kcache, vcache, q_start, start_pos, block_table)
    _check_attention(out, q, kcache, vcache, block_table, n_kv, head_dim)
    _i32(q_start, "q_start"); _i32(start_pos, "start_pos")
    lib = load_library("attention_tc", {"KLLM_HD": head_dim})
    rc = lib.kllm_attention_prefill(_p(out), _p(q), ctypes.c_int64(q.stride(0)), _p(kcache), _p(vcache),
                                    _p(q_start), _p(start_pos), _p(block_table), block_table.shape[1],
                                    q.shape[0], int(n_requests), n_heads, n_kv, head_dim, kcache.shape[2],
                                    int(window or 0), ctypes.c_float(scale), _stream())
    _check(lib, "attention_tc", rc)


def tcgen05_form(head_dim: int, group: int, n_kv: int, n_tokens: int, n_requests: int, max_ctx: int) -> str:
    """Which of the two tcgen05 attention kernels a step of portions takes ("smem" / "tmem",
    see ``attention_prefill_tcgen05``), from measurements (profiles/attn_prefill_tc5_forms.md):
    head size 128 always keeps its probabilities in tensor memory.  At head size 64 that form
    (four CTAs per SM) wins when the step is many short chains of tiles or several waves of
    CTAs, and loses to the other (two CTAs per SM, two score buffers) when one long prompt's
    longest chain is the whole kernel: all CTAs resident at once and more than 16 key tiles."""
    if head_dim != 64:
        return "tmem"
    ctas = (n_tokens // max(1, 128 // group) + n_requests) * n_kv
    tiles = -(-max_ctx // 64)
    return "tmem" if tiles <= 16 or ctas >= 6 * sm_count() else "smem"


def attention_prefill_tcgen05(out, q, kcache, vcache, q_start, start_pos, block_table, n_requests, n_heads, n_kv,
                              head_dim, window, scale, probabilities: Optional[str] = None) -> None:
    """Attention of portions on tcgen05 tensor cores with TMEM accumulators (head size
    64 or 128); same contract as ``attention_prefill``.  Two kernels, which differ in where
    the probabilities wait for the second product: ``probabilities="smem"``
    (csrc/attention_tcgen05.cu: two score buffers in tensor memory, P through shared
    memory, two CTAs of head size 64 per SM) or ``"tmem"`` (csrc/attention_tcgen05_ptmem.cu:
    P written over the scores in tensor memory and read from there, half the tensor memory
    and shared memory per CTA, four / two CTAs per SM).  Default (no step shape known): tmem
    for head size 128 (1.3 to 1.6 times faster), smem for head size 64; ``attention`` picks
    by the step's shape (``tcgen05_form``)."""
    _cuda(out, q, kcache, vcache, q_start, start_pos, block_table)
    _check_attention(out, q, kcache, vcache, block_table, n_kv, head_dim)
    _i32(q_start, "q_start"); _i32(start_pos, "start_pos")
    probabilities = probabilities or ("tmem" if head_dim == 128 else "smem")
    if probabilities not in ("smem", "tmem"):
        raise KernelError("attention (tcgen05): probabilities wait in 'smem' or in 'tmem'")
    name = "attention_tcgen05" + ("_ptmem" if probabilities == "tmem" else "")
    lib = load_library(name, {"KLLM_HD": head_dim})
    fn = lib.kllm_attention_prefill_tcgen05_ptmem if probabilities == "tmem" else lib.kllm_attention_prefill_tcgen05
    rc = fn(_p(out), _p(q), ctypes.c_int64(q.stride(0)), _p(kcache), _p(vcache), _p(q_start), _p(start_pos),
            _p(block_table), block_table.shape[1], q.shape[0], int(n_requests), n_heads, n_kv, head_dim,
            kcache.shape[2], int(window or 0), ctypes.c_float(scale), _p(status_word(q.device)), _stream())
    _check(lib, name, rc)


_status_words = {}      # device index -> int32 tensor that kernels set when a bounded wait runs out


def status_word(device) -> torch.Tensor:
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _status_words:
        _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _status_words[idx]


def check_status(device) -> None:
    """Raise if a kernel reported that a bounded wait (on an mbarrier) ran out; its
    results are then not valid.  Synchronises the device."""
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        raise KernelError(f"a kernel gave up waiting on an mbarrier (wait number {code} in its source); "
                          "its results are not valid")


TIMELINE_TAGS = {200: "attn_decode_fused", 201: "attn_decode_fused (merging CTA)"}
for _pro, _pn in ((0, "x"), (1, "norm")):
    for _epi, _en in ((0, "bf16"), (1, "f32"), (2, "add"), (3, "swiglu")):
        TIMELINE_TAGS[100 + _pro * 10 + _epi] = f"skinny_gemm {_pn}->{_en}"


def timeline():
    """Rows of the kernels' timeline tables, oldest first (only in a process started with
    KLLM_B200_TIMELINE=1, which loads the instrumented builds): a list of dicts with the
    library, the kernel, and per recorded CTA (first, middle, last of the grid) the
    nanosecond timer at the kernel's marks; see the TL_END lines in csrc for what the
    marks of a kernel mean.  Synchronises the device."""
    import numpy as np
    from .csrc.build import loaded_libraries
    torch.cuda.synchronize()
    rows = []
    for variant, lib in loaded_libraries().items():
        name = variant.split("-")[0]
        fn = getattr(lib, "kllm_timeline_" + name, None) if "KLLM_TIMELINE" in variant else None
        if fn is None:
            continue
        buf = np.zeros((512, 3, 9), dtype=np.uint64)
        if fn(buf.ctypes.data_as(ctypes.c_void_p)) != 0:
            raise KernelError(f"timeline of {variant} could not be read")
        for slot in range(512):
            ctas = [buf[slot, c, :8].astype(np.int64) for c in range(3) if buf[slot, c, 0] > 0]
            if ctas:
                tags = sorted({int(buf[slot, c, 8]) for c in range(3) if buf[slot, c, 0] > 0})
                rows.append({"library": variant, "kernel": " / ".join(TIMELINE_TAGS.get(t, str(t)) for t in tags),
                             "start": int(min(c[0] for c in ctas)), "end": int(max(c.max() for c in ctas)),
                             "marks": ctas})
    rows.sort(key=lambda r: r["start"])
    return rows


def silu_mul(out: torch.Tensor, gate: torch.Tensor, up: torch.Tensor) -> None:
    """out = silu(gate) * up; 2-D operands with dense rows (strided rows allowed);
    gate and up share a dtype, float32 or out's."""
    _cuda(out, gate, up)
    for t in (out, gate, up):
        if t.stride(1) != 1:
            raise KernelError("silu_mul: operands must have dense rows")
    if gate.dtype != up.dtype or gate.dtype not in (out.dtype, torch.float32):
        raise KernelError("silu_mul: gate and up must share a dtype, float32 or out's")
    n, f = out.shape
    lib = load_library("activation")
    rc = lib.kllm_silu_mul(_p(out), ctypes.c_int64(out.stride(0)), _p(gate), ctypes.c_int64(gate.stride(0)),
                           _p(up), ctypes.c_int64(up.stride(0)), n, f, dtype_code(out.dtype),
                           dtype_code(gate.dtype), _stream())
    _check(lib, "activation", rc)


def sample(out: torch.Tensor, logits: torch.Tensor, temperature: Optional[torch.Tensor],
           uniform: Optional[torch.Tensor], last_token: Optional[torch.Tensor] = None,
           slots: Optional[torch.Tensor] = None, host_out: Optional[torch.Tensor] = None) -> None:
    """out[r] = argmax (temperature[r] <= 0) or the inverse CDF of softmax(z/T) at uniform[r];
    with ``last_token`` and ``slots`` (int32 [rows]) also last_token[slots[r]] = out[r];
    with ``host_out`` (pinned host int32 [rows]) the kernel also writes the choices there itself."""
    _cuda(out, logits, temperature, uniform, last_token, slots)
    if host_out is not None and (host_out.is_cuda or not host_out.is_pinned() or host_out.dtype != torch.int32
                                 or not host_out.is_contiguous() or host_out.numel() < logits.shape[0]):
        raise KernelError("sample: host_out must be a pinned, contiguous int32 host tensor of [rows]")
    _i32(out, "out"); _i32(last_token, "last_token"); _i32(slots, "slots")
    if (last_token is None) != (slots is None) or (slots is not None and slots.numel() != logits.shape[0]):
        raise KernelError("sample: last_token and slots [rows] go together")
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with dense rows")
    for t in (temperature, uniform):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != logits.shape[0]):
            raise KernelError("sample: temperature and uniform must be float32 [rows]")
    lib = load_library("sampling")
    rc = lib.kllm_sample(_p(out), _p(logits), ctypes.c_int64(logits.stride(0)), logits.shape[0],
                         logits.shape[1], _p(temperature), _p(uniform), _p(last_token), _p(slots), _p(host_out), _stream())
    _check(lib, "sampling", rc)


SKINNY_MAX_ROWS = 16
_PRO = {"bf16": 0, "norm": 1}
_EPI = {"bf16": 0, "f32": 1, "add": 2, "swiglu": 3}


SKINNY_F32_MAX_ROWS = 8
SKINNY_F32_MAX_WIDTH = 220 * 1024 // (8 * 4) // 128 * 128      # 8 float32 rows in shared memory


def skinny_fits(n: int, k: int, dtype: torch.dtype, sliced: bool = False) -> bool:
    """Whether the weight-streaming product takes n rows of width k in this dtype
    (bfloat16: csrc/skinny_gemm.cu, up to 16 rows; float32: csrc/skinny_gemm_f32.cu, up to
    8 rows, width a multiple of 128).  ``sliced``: the caller adds into a float32 matrix
    from rows of the weights' dtype, where a width too long for shared memory is taken
    slice by slice."""
    if dtype == torch.float32:
        return 1 <= n <= SKINNY_F32_MAX_ROWS and k >= 128 and k % 128 == 0 and (sliced or k <= SKINNY_F32_MAX_WIDTH)
    if dtype != torch.bfloat16 or not (1 <= n <= SKINNY_MAX_ROWS) or k < 32 or k % 32:
        return False
    return sliced or k <= _skinny_max_width(n)


def _skinny_max_width(n: int) -> int:
    """Largest width (a multiple of 32) whose X rows, the 16 warps' partial tiles and the
    norm's gain fit the 227 KB of shared memory (smem_bytes in csrc/skinny_gemm.cu)."""
    nt = 1 if n <= 8 else 2
    room = 227 * 1024 - 16 * 16 * 8 * nt * 4
    k = room // (8 * nt * 2 + 4) // 32 * 32
    while 8 * nt * (k + (32 if (k * 2) % 128 == 0 else 0)) * 2 + k * 4 > room:
        k -= 32
    return k


def _prefetch_args(t: Optional[torch.Tensor]):
    if t is None or not PREFETCH_L2:
        return None, ctypes.c_int64(0)
    if not t.is_contiguous():
        raise KernelError("prefetch: the tensor to bring into L2 must be contiguous")
    return _p(t), ctypes.c_int64(min(t.numel() * t.element_size(), PREFETCH_L2_BYTES) // 16 * 16)


def skinny_gemm(weight: torch.Tensor, *, x: Optional[torch.Tensor] = None, x_f32: Optional[torch.Tensor] = None,
                gain: Optional[torch.Tensor] = None, eps: float = 0.0, rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None, weight_up: Optional[torch.Tensor] = None, epilogue: str = "bf16",
                out: Optional[torch.Tensor] = None, prefetch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = X @ weight^T for at most 16 rows, the weights streamed once (csrc/skinny_gemm.cu
    for bfloat16 weights, csrc/skinny_gemm_f32.cu for float32 weights: true float32 FMAs,
    at most 8 rows).

    X is either ``x`` ([n, K] in the weights' dtype) or rmsnorm(``x_f32``) * ``gain`` computed
    inside the kernel (rows ``rows`` of x_f32 when given).  ``epilogue``: "store" stores y
    [n, N] in the weights' dtype ("bf16" / "f32" name the dtype); "add" adds y into the
    float32 ``out``; "swiglu" takes ``weight`` as gate and ``weight_up`` as up matrix and
    stores silu(gate) * up [n, N] in the weights' dtype.
    ``prefetch``: a contiguous tensor that a later kernel will stream (the next weight
    matrix); the kernel asks for it to be brought into L2 before its own work.
    A width K too long for shared memory is taken in column slices, one launch each, when
    X is bfloat16 and the epilogue is "add" (the slices' sums meet in ``out``, always in
    the same order).
    """
    _cuda(weight, x, x_f32, gain, rows, weight_up, out, prefetch)
    N, K = weight.shape
    if epilogue == "store":
        epilogue = "f32" if weight.dtype == torch.float32 else "bf16"
    if weight.dtype == torch.float32:
        return _skinny_gemm_f32(weight, x, x_f32, gain, eps, rows, n_rows, weight_up, epilogue, out)
    if weight.dtype != torch.bfloat16 or weight.stride(1) != 1 or weight.stride(0) % 8:
        raise KernelError("skinny_gemm: the weight must be bfloat16 with dense rows at a stride that is a multiple of 8")
    if weight_up is not None and weight_up.stride() != weight.stride():
        raise KernelError("skinny_gemm: the up matrix must be laid out like the gate matrix")
    if x is not None and epilogue == "add" and out is not None and K % 32 == 0 and 1 <= x.shape[0] <= SKINNY_MAX_ROWS \
            and K > _skinny_max_width(x.shape[0]):
        widest = _skinny_max_width(x.shape[0])
        parts = -(-K // widest)
        width = -(-K // parts // 32) * 32
        for lo in range(0, K, width):
            hi = min(K, lo + width)
            skinny_gemm(weight[:, lo:hi], x=x[:, lo:hi], epilogue="add", out=out,
                        prefetch=prefetch if hi == K else None)
        return out
    if x is not None:
        pro, n = 0, x.shape[0]
        if x.dtype != torch.bfloat16 or x.stride(1) != 1 or x.shape[1] != K:
            raise KernelError("skinny_gemm: x must be bfloat16 [n, K] with dense rows")
    else:
        pro = 1
        _i32(rows, "rows")
        n = rows.numel() if rows is not None else x_f32.shape[0]
        if n_rows is not None:
            n = n_rows
        if x_f32.dtype != torch.float32 or not x_f32.is_contiguous() or x_f32.shape[1] != K \
                or gain.dtype != torch.float32 or gain.numel() != K:
            raise KernelError("skinny_gemm: x_f32 [rows, K] and gain [K] must be contiguous float32")
    if not skinny_fits(n, K, torch.bfloat16):
        raise KernelError(f"skinny_gemm: {n} rows of width {K} are not supported")
    epi = _EPI[epilogue]
    if epilogue == "swiglu" and (weight_up is None or weight_up.shape != weight.shape
                                 or weight_up.dtype != torch.bfloat16):
        raise KernelError("skinny_gemm: swiglu needs an up matrix like the gate matrix")
    if out is None:
        if epilogue == "add":
            raise KernelError("skinny_gemm: 'add' needs the matrix to add into")
        out = torch.empty((n, N), dtype=torch.float32 if epilogue == "f32" else torch.bfloat16, device=weight.device)
    want = torch.float32 if epilogue in ("f32", "add") else torch.bfloat16
    if out.dtype != want or out.stride(1) != 1 or out.shape[0] < n or out.shape[1] != N:
        raise KernelError("skinny_gemm: out has the wrong dtype or shape")
    lib = load_library("skinny_gemm")
    y16 = out if want == torch.bfloat16 else None
    y32 = out if want == torch.float32 else None
    rc = lib.kllm_skinny_gemm(_p(weight), _p(weight_up), ctypes.c_int64(weight.stride(0)), N, K, n, _p(x),
                              ctypes.c_int64(x.stride(0) if x is not None else 0), _p(x_f32), _p(gain), _p(rows),
                              ctypes.c_float(eps), _p(y16), _p(y32), ctypes.c_int64(out.stride(0)), pro, epi,
                              *_prefetch_args(prefetch), _stream())
    _check(lib, "skinny_gemm", rc)
    return out


def _skinny_gemm_f32(weight, x, x_f32, gain, eps, rows, n_rows, weight_up, epilogue, out):
    """The float32 form of ``skinny_gemm`` (same arguments; no prefetch hint)."""
    N, K = weight.shape
    if weight.stride(1) != 1 or weight.stride(0) % 4:
        raise KernelError("skinny_gemm: float32 weights need dense rows at a stride that is a multiple of 4")
    if epilogue not in ("f32", "add", "swiglu"):
        raise KernelError(f"skinny_gemm: float32 weights have no epilogue {epilogue!r}")
    if x is not None:
        n = x.shape[0]
        if x.dtype != torch.float32 or x.stride(1) != 1 or x.shape[1] != K:
            raise KernelError("skinny_gemm: x must be float32 [n, K] with dense rows")
        if epilogue == "add" and out is not None and K > SKINNY_F32_MAX_WIDTH and K % 128 == 0 and n <= SKINNY_F32_MAX_ROWS:
            parts = -(-K // SKINNY_F32_MAX_WIDTH)
            width = -(-K // parts // 128) * 128
            for lo in range(0, K, width):
                hi = min(K, lo + width)
                _skinny_gemm_f32(weight[:, lo:hi], x[:, lo:hi], None, None, 0.0, None, None, None, "add", out)
            return out
        src, pro, stride = x, 0, x.stride(0)
    else:
        _i32(rows, "rows")
        n = n_rows if n_rows is not None else (rows.numel() if rows is not None else x_f32.shape[0])
        if x_f32.dtype != torch.float32 or not x_f32.is_contiguous() or x_f32.shape[1] != K \
                or gain.dtype != torch.float32 or gain.numel() != K:
            raise KernelError("skinny_gemm: x_f32 [rows, K] and gain [K] must be contiguous float32")
        src, pro, stride = x_f32, 1, K
    if not skinny_fits(n, K, torch.float32):
        raise KernelError(f"skinny_gemm: {n} float32 rows of width {K} are not supported")
    if epilogue == "swiglu" and (weight_up is None or weight_up.shape != weight.shape or weight_up.dtype != torch.float32
                                 or weight_up.stride() != weight.stride()):
        raise KernelError("skinny_gemm: swiglu needs an up matrix like the gate matrix")
    if out is None:
        if epilogue == "add":
            raise KernelError("skinny_gemm: 'add' needs the matrix to add into")
        out = torch.empty((n, N), dtype=torch.float32, device=weight.device)
    if out.dtype != torch.float32 or out.stride(1) != 1 or out.shape[0] < n or out.shape[1] != N:
        raise KernelError("skinny_gemm: out has the wrong dtype or shape")
    lib = load_library("skinny_gemm_f32")
    rc = lib.kllm_skinny_gemm_f32(_p(weight), _p(weight_up), ctypes.c_int64(weight.stride(0)), N, K, n, _p(src),
                                  ctypes.c_int64(stride), _p(gain), _p(rows), ctypes.c_float(eps), _p(out),
                                  ctypes.c_int64(out.stride(0)), pro, {"f32": 0, "add": 1, "swiglu": 2}[epilogue], _stream())
    _check(lib, "skinny_gemm_f32", rc)
    return out


def linear_add(acc: torch.Tensor, x: torch.Tensor, weight: torch.Tensor) -> None:
    """acc += x @ weight^T through the vendor GEMM library, acc float32 (the residual
    stream), the sum formed in float32 inside the product's epilogue: what the reference
    does in a kernel of its own after cublasSgemm (backend/model.cu:97-110)."""
    _cuda(acc, x, weight)
    if torch.backends.cuda.matmul.allow_tf32:
        raise KernelError("TF32 matmul mode is on; the float32 path must stay true 32-bit")
    if acc.dtype != torch.float32 or not acc.is_contiguous():
        raise KernelError("linear_add: the matrix added into must be contiguous float32")
    if x.dtype == torch.float32:
        torch.addmm(acc, x, weight.t(), out=acc)
    else:
        torch.addmm(acc, x, weight.t(), out_dtype=torch.float32, out=acc)


def _gemm_args(x, weight, weight_up, out, epilogue):
    return (_p(x), ctypes.c_int64(x.stride(0)), _p(weight), ctypes.c_int64(weight.stride(0)), _p(weight_up),
            x.shape[0], weight.shape[0], x.shape[1], _p(out), ctypes.c_int64(out.stride(0)), _EPI[epilogue])


def gemm_fits(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "bf16",
              weight_up: Optional[torch.Tensor] = None) -> bool:
    """Whether ``gemm`` takes these operands (bfloat16, dense rows, k and the row strides
    multiples of 8, 16-byte aligned addresses)."""
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or x.dim() != 2 or weight.dim() != 2:
        return False
    if x.stride(1) != 1 or weight.stride(1) != 1 or out.stride(1) != 1 or x.shape[1] != weight.shape[1]:
        return False
    if weight_up is not None and (weight_up.dtype != torch.bfloat16 or weight_up.shape != weight.shape
                                  or weight_up.stride() != weight.stride()):
        return False
    lib = load_library("gemm_tcgen05")
    return bool(lib.kllm_gemm_tcgen05_fits(*_gemm_args(x, weight, weight_up, out, epilogue)))


def gemm_pays(n: int, N: int, epilogue: str = "bf16", least: int = 75) -> bool:
    """Whether ``gemm``'s tiles of 128 rows x 256 accumulator columns would keep the
    tensor cores of all SMs busy for at least ``least`` percent of the product's time
    (full tiles over waves x SMs); below that the library product adapts its tiling
    better.  Same arithmetic as kllm_gemm_tcgen05_efficiency, without loading the library."""
    if not USE_TCGEN05 or n <= 0 or N <= 0:
        return False
    sms = sm_count()
    nout = 128 if epilogue == "swiglu" else 256
    tiles = -(-n // 128) * -(-N // nout)
    waves = -(-tiles // sms)
    return 100.0 * (n / 128.0) * (N / float(nout)) / (waves * sms) >= least


def gemm(x: torch.Tensor, weight: torch.Tensor, *, epilogue: str = "bf16", out: Optional[torch.Tensor] = None,
         weight_up: Optional[torch.Tensor] = None, bn: int = 0) -> torch.Tensor:
    """y = x @ weight^T on the tcgen05 tensor cores (csrc/gemm_tcgen05.cu), x bfloat16
    [n, K], weight bfloat16 [N, K].

    ``epilogue``: "bf16" / "f32" store y [n, N]; "add" adds y into the float32 ``out``;
    "swiglu" takes ``weight`` as gate and ``weight_up`` as up matrix and stores
    silu(gate) * up as bfloat16 [n, N].  ``bn``: accumulator width of a tile (0 = chosen
    by the tile count).
    """
    _cuda(x, weight, weight_up, out)
    n, N = x.shape[0], weight.shape[0]
    want = torch.float32 if epilogue in ("f32", "add") else torch.bfloat16
    if out is None:
        if epilogue == "add":
            raise KernelError("gemm: 'add' needs the matrix to add into")
        out = torch.empty((n, N), dtype=want, device=x.device)
    if out.dtype != want or out.shape[0] != n or out.shape[1] != N:
        raise KernelError("gemm: out has the wrong dtype or shape")
    if epilogue == "swiglu" and weight_up is None:
        raise KernelError("gemm: swiglu needs an up matrix like the gate matrix")
    if not gemm_fits(x, weight, out, epilogue, weight_up):
        raise KernelError(f"gemm: operands {tuple(x.shape)} x {tuple(weight.shape)} (strides {x.stride()}, "
                          f"{weight.stride()}, out {out.stride()}) are not supported")
    lib = load_library("gemm_tcgen05")
    rc = lib.kllm_gemm_tcgen05(*_gemm_args(x, weight, weight_up, out, epilogue), int(bn), _p(status_word(x.device)),
                               _stream())
    _check(lib, "gemm_tcgen05", rc)
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """y = x @ weight^T through the vendor GEMM library (cuBLAS, via torch.mm), as
    the reference does for every projection (backend/model.cu:496-503).

    float32 operands run as true float32 (the reduced-precision TF32 mode stays
    off); bfloat16 operands accumulate in float32.
    """
    _cuda(x, weight)
    if torch.backends.cuda.matmul.allow_tf32:
        raise KernelError("TF32 matmul mode is on; the float32 path must stay true 32-bit")
    if out_dtype is not None and out_dtype != x.dtype:
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    if out is not None:
        return torch.mm(x, weight.t(), out=out)
    return torch.mm(x, weight.t())
