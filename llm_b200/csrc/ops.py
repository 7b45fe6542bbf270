"""Python faces of the kernels: each takes torch tensors on the GPU, checks what
the kernel assumes, and calls the C entry point on the current stream.  There is
no other implementation behind them: without the library, or with a tensor that is
not on a CUDA device, they raise.
"""
from __future__ import annotations

import ctypes
import functools
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import load, load_tensor

_F32, _BF16 = 0, 1


class KernelError(RuntimeError):
    pass


class PartialSum:
    """The result of a split-K product that has not been summed yet: float32
    [splits, rows, cols] in the shared scratch buffer.  The kernels that take one sum it on
    the fly, in the order of the splits.  It lives in one buffer per device and is valid only
    until the next product runs: consume it first."""

    def __init__(self, buf: torch.Tensor, splits: int, rows: int, cols: int, dtype: torch.dtype):
        self.buf, self.splits, self.rows, self.cols, self.dtype = buf, splits, rows, cols, dtype

    @property
    def split_stride(self) -> int:
        return self.rows * self.cols


def _split_args(x):
    """(direct pointer, partials pointer, splits, split stride) of a tensor, a PartialSum or None."""
    if isinstance(x, PartialSum):
        return c_void_p(0), c_void_p(x.buf.data_ptr()), c_int(x.splits), c_longlong(x.split_stride)
    return _ptr(x), c_void_p(0), c_int(0), c_longlong(0)


def _kind(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def _ptr(t, name="tensor"):
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device (there is no CPU path)")
    return c_void_p(t.data_ptr())


_STREAM = None


def set_stream(handle) -> None:
    """Fix the CUDA stream that the kernels launch on (a raw handle), or None to go back to
    asking torch for its current stream at every launch, which costs several microseconds."""
    global _STREAM
    _STREAM = handle


def _stream():
    if _STREAM is not None:
        return c_void_p(_STREAM)
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_LAUNCHES = 0


def launch_count() -> int:
    """Kernel launches issued through this module so far (graph replays included)."""
    return _LAUNCHES


def count_launches(n: int) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def _check(code: int, tensor: bool = False) -> None:
    """Count a launch; raise with the text of the library that reported an error."""
    global _LAUNCHES
    _LAUNCHES += 1
    if code != 0:
        msg = (load_tensor() if tensor else load()).llmk_last_error().decode("utf-8", "replace")
        raise KernelError(f"kernel call failed ({code}): {msg}")


def _check_t(code: int) -> None:
    _check(code, tensor=True)


def _rows_contig(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be 2-D with unit stride in its last dimension")


def embedding(resid: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, n_tokens: int,
              status: torch.Tensor) -> None:
    """resid[:n_tokens] (float32) = table[ids]; an id outside the table sets status[0]."""
    assert resid.dtype == torch.float32 and ids.dtype == torch.int32 and status.dtype == torch.int32
    assert resid.is_contiguous() and table.is_contiguous()
    vocab, hidden = table.shape
    _check(load().llmk_embedding(_ptr(resid), _ptr(table), _ptr(ids), c_int(n_tokens), c_int(hidden),
                                 c_int(vocab), c_int(_kind(table.dtype)), _ptr(status), _stream()))


def add_rmsnorm(resid: torch.Tensor, delta, gamma: torch.Tensor, out, rows: int, eps: float) -> None:
    """resid[:rows] += delta (a tensor or a PartialSum, if given); out[:rows] = rmsnorm(resid) * gamma
    (if out given)."""
    assert resid.dtype == torch.float32 and gamma.dtype == torch.float32 and resid.is_contiguous()
    hidden = resid.shape[-1]
    ref = out if out is not None else delta
    if ref is None:
        return
    if isinstance(delta, PartialSum):
        assert delta.cols == hidden and delta.rows == rows
    elif delta is not None:
        assert delta.is_contiguous() and delta.shape[-1] == hidden
    if out is not None:
        assert out.is_contiguous() and out.shape[-1] == hidden
        if delta is not None:
            assert delta.dtype == out.dtype
    d, parts, splits, stride = _split_args(delta)
    _check(load().llmk_add_rmsnorm(_ptr(resid), d, parts, splits, stride, _ptr(gamma), _ptr(out), c_int(rows),
                                   c_int(hidden), c_float(eps), c_int(_kind(ref.dtype)), _stream()))


def gather_rows(out: torch.Tensor, resid: torch.Tensor, delta, rows: torch.Tensor, n_rows: int) -> None:
    """out[r] = resid[rows[r]] (+ delta[rows[r]], a tensor or a PartialSum), float32."""
    assert out.dtype == torch.float32 and resid.dtype == torch.float32 and rows.dtype == torch.int32
    kind = _kind(delta.dtype) if delta is not None else _F32
    d, parts, splits, stride = _split_args(delta)
    _check(load().llmk_gather_rows(_ptr(out), _ptr(resid), d, parts, splits, stride, _ptr(rows), c_int(n_rows),
                                   c_int(resid.shape[-1]), c_int(kind), _stream()))


def cast_rows(out: torch.Tensor, rows_f32: torch.Tensor, n_rows: int) -> None:
    """out[:n_rows] = rows_f32[:n_rows] rounded to out's dtype (float32 or bfloat16)."""
    assert rows_f32.dtype == torch.float32 and out.is_contiguous() and rows_f32.is_contiguous()
    assert out.shape[-1] == rows_f32.shape[-1]
    _check(load().llmk_cast_rows(_ptr(out), _ptr(rows_f32), c_longlong(n_rows * out.shape[-1]), c_int(_kind(out.dtype)),
                                 _stream()))


def add_bias(x: torch.Tensor, bias: torch.Tensor, rows: int) -> None:
    """x[:rows] += bias (float32 [cols]), in place."""
    _rows_contig(x, "x")
    assert bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == x.shape[1]
    _check(load().llmk_add_bias(_ptr(x), c_longlong(x.stride(0)), _ptr(bias), c_int(rows), c_int(x.shape[1]),
                                c_int(_kind(x.dtype)), _stream()))


def silu_mul(out: torch.Tensor, gate_up, rows: int) -> None:
    """out[:rows, :I] = silu(gate_up[:, :I]) * gate_up[:, I:]; gate_up a tensor or a PartialSum."""
    inter = out.shape[-1]
    assert out.is_contiguous() and out.dtype == gate_up.dtype
    if isinstance(gate_up, PartialSum):
        assert gate_up.cols == 2 * inter and gate_up.rows == rows
    else:
        assert gate_up.shape[-1] == 2 * inter and gate_up.is_contiguous()
    d, parts, splits, stride = _split_args(gate_up)
    _check(load().llmk_silu_mul(_ptr(out), d, parts, splits, stride, c_int(rows), c_int(inter),
                                c_int(_kind(out.dtype)), _stream()))


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int) -> None:
    """out[:rows] = a[:rows] @ w.T with float32 accumulation on the CUDA cores."""
    _rows_contig(a, "a"); _rows_contig(w, "w"); _rows_contig(out, "out")
    n, k = w.shape
    assert a.shape[1] == k and out.shape[1] == n and a.dtype == w.dtype
    _check(load().llmk_gemm_simt(_ptr(a), _ptr(w), _ptr(out), c_int(rows), c_int(n), c_int(k),
                                 c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                                 c_int(_kind(a.dtype)), c_int(_kind(out.dtype)), _stream()))


def rope_kv_write(qkv, cos, sin, positions: torch.Tensor, slot_map: torch.Tensor,
                  k_pages, v_pages, n_tokens: int, n_heads: int, n_kv: int,
                  head_dim: int, q_out=None) -> torch.Tensor:
    """Rotate q and k by the tables, store k and v at slot_map in the pages.  qkv is a tensor
    [T, >= (n_heads + 2 n_kv) head_dim] (q is then rotated in place unless q_out is given) or a
    PartialSum of that shape (q_out is then required).  Returns the tensor that holds rotated q."""
    assert positions.dtype == torch.int32 and slot_map.dtype == torch.int32
    if isinstance(qkv, PartialSum):
        assert q_out is not None and qkv.cols >= (n_heads + 2 * n_kv) * head_dim
        src_stride = qkv.cols
    else:
        _rows_contig(qkv, "qkv")
        assert qkv.shape[1] >= (n_heads + 2 * n_kv) * head_dim
        src_stride = qkv.stride(0)
        if q_out is None:
            q_out = qkv
    _rows_contig(q_out, "q_out")
    assert q_out.dtype == qkv.dtype
    if n_kv:
        assert k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == qkv.dtype
        assert k_pages.shape[3] == head_dim and k_pages.shape[1] == n_kv
    page = k_pages.shape[2] if k_pages is not None else 1
    if cos is not None:
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32
        assert cos.shape[1] == head_dim // 2 and cos.is_contiguous() and sin.is_contiguous()
    d, parts, splits, stride = _split_args(qkv)
    _check(load().llmk_rope_kv_write(d, parts, splits, stride, c_longlong(src_stride), _ptr(q_out),
                                     c_longlong(q_out.stride(0)), _ptr(cos), _ptr(sin),
                                     _ptr(positions), _ptr(slot_map), _ptr(k_pages), _ptr(v_pages),
                                     c_int(n_tokens), c_int(n_heads), c_int(n_kv), c_int(head_dim),
                                     c_int(page), c_int(_kind(qkv.dtype)), _stream()))
    return q_out


def paged_attention_generic(out: torch.Tensor, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                            block_table: torch.Tensor, token_entry: torch.Tensor, positions: torch.Tensor,
                            n_tokens: int, n_heads: int, n_kv: int, head_dim: int, window: int,
                            scale: float) -> None:
    """out[t, h*HS:(h+1)*HS] = causal (windowed) attention of q[t, h] over its request's pages."""
    _rows_contig(out, "out"); _rows_contig(q, "q")
    assert block_table.dim() == 2 and block_table.is_contiguous() and block_table.dtype == torch.int32
    assert token_entry.dtype == torch.int32 and positions.dtype == torch.int32
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and q.dtype == k_pages.dtype == out.dtype
    _check(load().llmk_paged_attention_generic(
        _ptr(out), c_longlong(out.stride(0)), _ptr(q), c_longlong(q.stride(0)), _ptr(k_pages), _ptr(v_pages),
        _ptr(block_table), c_int(block_table.shape[1]), _ptr(token_entry), _ptr(positions), c_int(n_tokens),
        c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(k_pages.shape[2]), c_int(window or 0),
        c_float(scale), c_int(_kind(q.dtype)), _stream()))


def feed_tokens(token_ids: torch.Tensor, sampled: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, n: int) -> None:
    """token_ids[dst[i]] = sampled[src[i]] for i < n, all int32 on the device."""
    assert token_ids.dtype == sampled.dtype == dst.dtype == src.dtype == torch.int32
    _check(load().llmk_feed_tokens(_ptr(token_ids), _ptr(sampled), _ptr(dst), _ptr(src), c_int(n), _stream()))


def sample_rows(out: torch.Tensor, logits: torch.Tensor, rows: int, temperature=None, uniform=None) -> None:
    """out[r] = argmax of logits[r] (ties to the lowest id) where temperature[r] <= 0 or no
    temperatures are given, else the inverse-CDF draw of softmax(logits[r] / temperature[r])
    at uniform[r]."""
    _rows_contig(logits, "logits")
    assert logits.dtype == torch.float32 and out.dtype == torch.int32
    if temperature is not None:
        assert temperature.dtype == torch.float32 and uniform is not None and uniform.dtype == torch.float32
    _check(load().llmk_sample_rows(_ptr(out), _ptr(logits), c_longlong(logits.stride(0)), c_int(rows),
                                   c_int(logits.shape[1]), _ptr(temperature), _ptr(uniform), _stream()))


_ATTN_PARTIALS = {}
_ATTN_PARTIALS_RETIRED = []      # outgrown buffers stay alive: captured graphs may still hold their addresses


def _attn_partials(device, n_floats: int) -> torch.Tensor:
    """Scratch of the decode attention; zeroed, because its first words are arrival counters
    that the kernel expects to be zero and leaves zero."""
    buf = _ATTN_PARTIALS.get(device)
    if buf is None or buf.numel() < n_floats:
        if buf is not None:
            _ATTN_PARTIALS_RETIRED.append(buf)
        buf = torch.zeros(max(n_floats, 1 << 20), dtype=torch.float32, device=device)
        _ATTN_PARTIALS[device] = buf
    return buf


def decode_splits(n_entries: int, n_kv: int, max_keys: int, sms: int = 0) -> int:
    """How many ranges the keys of one request are cut into.  Up to 2,048 keys: ranges of about
    128 keys (one tile of 32 per warp of a CTA) while the batch is small and the kernel bound by
    latency, fewer and longer ones as (requests x kv heads) grows, so that about 256 CTAs run; at
    most 16, and clusters of 7 or 8 CTAs measured slower than 6 longer ranges.  Beyond that the
    kernel is bound by bytes: as many ranges of at least 256 keys as fill the SMs with two CTAs
    each in one wave, at most 64.  sms: the device's SM count, if the caller has it."""
    pairs = max(1, n_entries * n_kv)
    if max_keys > 2048:
        return max(1, min(64, (2 * (sms or sm_count())) // pairs, max_keys // 256))
    s = max(1, min(16, _ceil_div(max_keys, 128), 256 // pairs))
    return 6 if s in (7, 8) else s


def paged_attention_decode(out: torch.Tensor, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                           block_table: torch.Tensor, kv_lens: torch.Tensor, n_entries: int, n_heads: int,
                           n_kv: int, head_dim: int, window: int, scale: float, splits=None, max_keys: int = 0) -> None:
    """One query token per entry (row e of q), attending to its request's kv_lens[e] keys.
    max_keys: an upper bound of kv_lens, if the host knows one below the table's width."""
    _rows_contig(out, "out"); _rows_contig(q, "q")
    assert block_table.dim() == 2 and block_table.is_contiguous() and block_table.dtype == torch.int32
    assert kv_lens.dtype == torch.int32 and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert q.dtype == k_pages.dtype == out.dtype
    page = k_pages.shape[2]
    if splits is None:
        splits = decode_splits(n_entries, n_kv, max_keys or block_table.shape[1] * page)
    buf = _attn_partials(q.device, _decode_scratch_floats(n_entries, n_heads, head_dim, splits))
    args = (_ptr(out), c_longlong(out.stride(0)), _ptr(q), c_longlong(q.stride(0)), _ptr(k_pages), _ptr(v_pages),
            _ptr(block_table), c_int(block_table.shape[1]), _ptr(kv_lens), c_int(n_entries), c_int(n_heads),
            c_int(n_kv), c_int(head_dim), c_int(page), c_int(window or 0), c_float(scale), c_int(splits),
            c_void_p(buf.data_ptr()), c_int(_kind(q.dtype)))
    # bfloat16 with a head size of 64 or 128 and pages of a power of two: the query heads of a
    # group as rows of warp-level MMAs (tensor-core library); everything else on the CUDA cores
    if (q.dtype == torch.bfloat16 and head_dim in (64, 128) and page & (page - 1) == 0
            and q.stride(0) % 2 == 0 and q.data_ptr() % 4 == 0):
        _check_t(load_tensor().llmk_paged_attention_decode_mma(*args, c_int(max_keys), _stream()))
    else:
        _check(load().llmk_paged_attention_decode(*args, _stream()))


def _decode_scratch_floats(n_entries: int, n_heads: int, head_dim: int, splits: int) -> int:
    lib = load()
    lib.llmk_paged_attention_decode_scratch.restype = c_longlong
    return int(lib.llmk_paged_attention_decode_scratch(c_int(n_entries), c_int(n_heads), c_int(head_dim), c_int(splits)))


def decode_attention_fused_supported(qkv, cos, sin, head_dim: int, page_size: int = 16) -> bool:
    """Whether one kernel can rotate, store and attend for a decode step: bfloat16, head size 64
    or 128, pages of a power of two, rows that start on 16-byte boundaries."""
    if qkv.dtype != torch.bfloat16 or page_size & (page_size - 1):
        return False
    d, parts, _, stride = _split_args(qkv)
    src_stride = qkv.cols if isinstance(qkv, PartialSum) else qkv.stride(0)
    return bool(load_tensor().llmk_decode_attention_fused_supported(d, parts, stride, c_longlong(src_stride), _ptr(cos),
                                                             _ptr(sin), c_int(head_dim), c_int(_BF16)))


def decode_attention_fused(out: torch.Tensor, qkv, cos, sin, k_pages: torch.Tensor, v_pages: torch.Tensor,
                           block_table: torch.Tensor, kv_lens: torch.Tensor, n_entries: int, n_heads: int,
                           n_kv: int, head_dim: int, window: int, scale: float, write_kv: bool = True,
                           splits=None, max_keys: int = 0) -> None:
    """One new token per entry: row e of qkv (a tensor or a PartialSum) holds its q, k and v
    heads (q alone if not write_kv).  q and k are rotated at position kv_lens[e] - 1, k and v are
    stored there in the entry's pages, and the token attends to its request's kv_lens[e] keys."""
    _rows_contig(out, "out")
    assert block_table.dim() == 2 and block_table.is_contiguous() and block_table.dtype == torch.int32
    assert kv_lens.dtype == torch.int32 and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert qkv.dtype == k_pages.dtype == out.dtype == torch.bfloat16
    page = k_pages.shape[2]
    if splits is None:
        splits = decode_splits(n_entries, n_kv, max_keys or block_table.shape[1] * page)
    lib = load_tensor()
    buf = _attn_partials(out.device, _decode_scratch_floats(n_entries, n_heads, head_dim, splits))
    d, parts, qkv_splits, stride = _split_args(qkv)
    src_stride = qkv.cols if isinstance(qkv, PartialSum) else qkv.stride(0)
    if isinstance(qkv, PartialSum):
        assert qkv.rows == n_entries
    _check_t(lib.llmk_decode_attention_fused(
        _ptr(out), c_longlong(out.stride(0)), d, parts, qkv_splits, stride, c_longlong(src_stride), _ptr(cos),
        _ptr(sin), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), c_int(block_table.shape[1]), _ptr(kv_lens),
        c_int(n_entries), c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(page), c_int(window or 0),
        c_float(scale), c_int(splits), c_int(int(write_kv)), c_void_p(buf.data_ptr()), c_int(max_keys), _stream()))


def attention_tc_supported(dtype, n_heads: int, n_kv: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 attention takes these sizes (bfloat16, head size 64 or 128, pages
    of 16 to 128 tokens, at most 128 query heads per kv head)."""
    if dtype != torch.bfloat16:
        return False
    return bool(load_tensor().llmk_attention_tc_supported(c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(page_size)))


def attention_tc(out: torch.Tensor, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                 block_table: torch.Tensor, cu_tokens: torch.Tensor, kv_lens: torch.Tensor, n_tokens: int,
                 n_entries: int, n_heads: int, n_kv: int, head_dim: int, window: int, scale: float) -> None:
    """Flash attention on the tensor cores for entries of any length: rows of entry e are
    cu_tokens[e] .. cu_tokens[e+1], its keys (new tokens included) number kv_lens[e]."""
    _rows_contig(out, "out"); _rows_contig(q, "q")
    assert q.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert block_table.dim() == 2 and block_table.is_contiguous() and block_table.dtype == torch.int32
    assert cu_tokens.dtype == torch.int32 and kv_lens.dtype == torch.int32
    assert k_pages.is_contiguous() and v_pages.is_contiguous()
    _check_t(load_tensor().llmk_attention_tc(
        _ptr(out), c_longlong(out.stride(0)), _ptr(q), c_longlong(q.stride(0)), _ptr(k_pages), _ptr(v_pages),
        c_int(k_pages.shape[0]), _ptr(block_table), c_int(block_table.shape[1]), _ptr(cu_tokens), _ptr(kv_lens),
        c_int(n_tokens), c_int(n_entries), c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(k_pages.shape[2]),
        c_int(window or 0), c_float(scale), _stream()))


def attention_tc_take_error() -> int:
    """The code the tensor-core attention left when one of its bounded waits gave up (0 = none)."""
    return int(load_tensor().llmk_attention_tc_take_error())


def paged_attention(out, qkv, k_pages, v_pages, group, ctx, n_heads: int, n_kv: int, head_dim: int,
                    window: int, scale: float) -> None:
    """Attention of the step's tokens over their requests' pages; q is the first
    n_heads * head_dim columns of qkv.  Chooses the kernel for the batch: in bfloat16 the
    split-key decode kernel when every entry brings one token and the tcgen05 kernel otherwise,
    where it takes the sizes; the general kernel for float32 and for all other sizes (head sizes
    off the 16-grid among them)."""
    if ctx.decode_only and qkv.dtype == torch.bfloat16 and head_dim % 16 == 0:
        max_keys = min(ctx.kv_bucket or 1 << 30, group.block_table.shape[1] * k_pages.shape[2])
        if window:
            max_keys = min(max_keys, window)
        paged_attention_decode(out, qkv, k_pages, v_pages, group.block_table, ctx.kv_lens, ctx.n_entries,
                               n_heads, n_kv, head_dim, window, scale,
                               splits=decode_splits(ctx.n_entries, n_kv, max_keys), max_keys=max_keys)
        return
    if attention_tc_supported(qkv.dtype, n_heads, n_kv, head_dim, k_pages.shape[2]) and qkv.stride(0) % 8 == 0:
        attention_tc(out, qkv, k_pages, v_pages, group.block_table, ctx.cu_tokens, ctx.kv_lens, ctx.n_tokens,
                     ctx.n_entries, n_heads, n_kv, head_dim, window, scale)
        return
    paged_attention_generic(out, qkv, k_pages, v_pages, group.block_table, ctx.token_entry, ctx.positions,
                            ctx.n_tokens, n_heads, n_kv, head_dim, window, scale)


FUSE_DECODE_ATTENTION = True


def rope_store_attend(out, qkv, cos, sin, k_pages, v_pages, group, ctx, n_heads: int, n_kv: int, head_dim: int,
                      window: int, scale: float, write_kv: bool, q_rot) -> None:
    """The three steps between the QKV product and the output projection: rotate q and k by the
    tables, store k and v in the pages (if write_kv), attend.  qkv is a tensor or a PartialSum;
    q_rot() gives a buffer for rotated queries when they cannot stay where they are.  A decode
    step in bfloat16 with a head size of 64 or 128 runs as one kernel, everything else as the
    rotate-and-store kernel followed by the attention kernel that fits the batch."""
    if (FUSE_DECODE_ATTENTION and ctx.decode_only and ctx.n_tokens == ctx.n_entries
            and decode_attention_fused_supported(qkv, cos, sin, head_dim, k_pages.shape[2])):
        max_keys = min(ctx.kv_bucket or 1 << 30, group.block_table.shape[1] * k_pages.shape[2])
        if window:
            max_keys = min(max_keys, window)
        decode_attention_fused(out, qkv, cos, sin, k_pages, v_pages, group.block_table, ctx.kv_lens, ctx.n_entries,
                               n_heads, n_kv, head_dim, window, scale, write_kv=write_kv,
                               splits=decode_splits(ctx.n_entries, n_kv, max_keys), max_keys=max_keys)
        return
    q = rope_kv_write(qkv, cos, sin, ctx.positions, group.slot_map, k_pages, v_pages, ctx.n_tokens, n_heads,
                      n_kv if write_kv else 0, head_dim, q_out=q_rot() if isinstance(qkv, PartialSum) else None)
    paged_attention(out, q, k_pages, v_pages, group, ctx, n_heads, n_kv, head_dim, window, scale)


# ---- tensor-core product ------------------------------------------------------------

_PARTIALS = {}      # device -> float32 scratch for split-K partial sums
_PARTIAL_BYTES = 64 << 20


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


@functools.lru_cache(maxsize=None)
def sm_count() -> int:
    """Streaming multiprocessors of the current device (the planners size grids and rounds by it)."""
    return max(1, int(load().llmk_device_sm_count()))


PERSISTENT_GEMM = True
PAIR_GEMM = True


def plan_gemm(M: int, N: int, K: int, fused_reduce: bool = False, cta_limit: int = 0):
    """cta_limit > 0 (swapped mode only): at most so many CTAs, for a product that should leave
    SMs to the kernel after it."""
    return _plan_gemm(M, N, K, fused_reduce, PERSISTENT_GEMM, PAIR_GEMM, sm_count(), cta_limit)


@functools.lru_cache(maxsize=4096)
def _plan_gemm(M: int, N: int, K: int, fused_reduce: bool, persistent: bool, pair: bool = False, _SMS: int = 148,
               cta_limit: int = 0):
    """(swap, tile, splits, k-blocks per split, mode) for the tensor-core product; mode 0 = one
    CTA per tile, 1 = the splits of a tile sum on chip in a cluster, 2 = persistent CTAs, 3 =
    persistent pairs of CTAs on tiles of 256 rows.

    Up to 128 rows the weights take the 128-row side of the MMA and the rows become its N
    (16 to 128); above that the rows take the 128-row side and the tile is 128 or 256 weight
    rows wide.  K (in blocks of 64) is split over CTAs when there are too few tiles to keep
    all SMs streaming; where the shape allows it the splits of a tile form a cluster and sum
    their results in shared memory, else they write float32 partial results for a later sum.
    The estimate, in microseconds, for more than 128 rows: a fixed cost plus waves of tiles times
    k-blocks times a k-block's time, fitted to timings of the products of the 1.1B and 7B shapes
    at 129 to 4,096 rows; plus the sum of the partial results where K is split."""
    kb = _ceil_div(K, 64)
    if M < NORMAL_MODE_FROM_ROWS:
        return _plan_swapped(M, N, kb, fused_reduce, _SMS, cta_limit)
    if M <= 128:
        return _plan_few_rows(M, N, kb, fused_reduce, _SMS, cta_limit)
    best = None
    for tile in (256, 224, 192, 160, 128):
        tiles = _ceil_div(M, 128) * _ceil_div(N, tile)
        # us per k-block of one CTA: bound by the bytes that it brings into shared memory
        t_kb = (128 + tile) * 128 / 114e3
        for s in range(1, min(kb, 32) + 1):
            per = _ceil_div(kb, s)
            if _ceil_div(kb, per) != s:
                continue
            if s > 1 and s * M * N * 4 > _PARTIAL_BYTES:
                break
            mode = 0
            waves = _ceil_div(tiles * s, _SMS)
            cost = waves * (per * t_kb + 0.8) + 7.2
            if persistent and s == 1 and tiles > _SMS:
                # more than one wave of tiles: one CTA per SM walks over them and drains one
                # accumulator while the next tile's products run
                mode = 2
                cost = waves * per * t_kb + 12.3
            if s > 1:
                traffic = (2 * s + 1) * M * N * 4 / 3.3e6             # partials written and read back, us
                cost += traffic + (0.8 if fused_reduce else 3.3)
            if best is None or cost < best[0] - 1e-9:
                best = (cost, False, tile, s, per, mode)
        if pair:
            # pairs of CTAs on tiles of 256 rows bring a third fewer bytes into shared memory per
            # product: a k-block takes what its MMAs take (with the gaps measured) or, on narrow
            # tiles, the latency of the ring
            t_kb = max(0.31 + 0.0004 * (tile - 128), 1.43 * 256 * tile * 64 * 2 / 2 / 15.2e6)
            waves = _ceil_div(_ceil_div(M, 256) * _ceil_div(N, tile), _SMS // 2)
            cost = waves * kb * t_kb + 8.6
            if cost < best[0] - 1e-9:
                best = (cost, False, tile, 1, kb, 3)
    return best[1:]


# From this many rows on (up to 128) the rows take the 128-row side of the MMA like a prompt's, one
# CTA per tile of 128 weight rows with the SM and a ring of 192 KB to itself, instead of the
# swapped mode's two CTAs per SM with rings half that size.  Measured on the four products of the
# 1.1B shape with the kernel that sums the partial results behind them (us, swapped -> normal):
# 32 rows 9.2 -> 8.5, 7.5 -> 6.7, 15.0 -> 10.6, 9.5 -> 10.2; 64 rows 11.4 -> 9.8, 9.3 -> 7.7, 17.9 ->
# 11.1, 11.6 -> 11.0; 128 rows 15.2 -> 10.7, 13.2 -> 9.1, 27.5 -> 11.8, 16.1 -> 12.6; at 16 rows and
# fewer the swapped mode is ahead (7.9 against 8.2, 8.0 against 10.0).  Whole decode steps: 24 requests
# 1.066 -> 1.055 ms, 31 requests 1.099 -> 1.087 ms, 64 requests 1.31 -> 1.20 ms; 17 requests the same.
NORMAL_MODE_FROM_ROWS = 24


def _plan_few_rows(M: int, N: int, kb: int, fused_reduce: bool, _SMS: int, cta_limit: int = 0):
    """The normal mode for 32 to 128 rows: tiles of 128 or 256 weight rows, one per CTA, K split
    over CTAs while there are too few tiles to draw the memory's bandwidth.  The estimate, in
    microseconds: a CTA's ring holds 192 KB in flight against a latency of about 1.5 us, of which
    the weights are a half (tiles of 128) or two thirds (of 256); the CTAs of a round share the
    measured 6.5 TB/s; a round costs a microsecond beside its bytes, the launch 1.6; partial
    results are written and read back where K is split.  Checked against timings of the products
    of the 1.1B, 7B and 8B shapes at 32, 64 and 128 rows."""
    best = None
    for tile in (128, 256):
        tiles = _ceil_div(N, tile)
        per_cta = 0.128e6 * tile / (128 + tile)                   # bytes of weights per microsecond that one CTA can draw
        for s in range(1, min(kb, 16) + 1):
            per = _ceil_div(kb, s)
            if _ceil_div(kb, per) != s:
                continue
            if s > 1 and (s * M * N * 4 > _PARTIAL_BYTES or (cta_limit and tiles * s > cta_limit)):
                break
            cta_bytes, left, cost = tile * per * 128, tiles * s, 1.6
            while left > 0:
                r = min(left, _SMS)
                cost += cta_bytes * r / min(6.5e6, r * per_cta) + 1.0
                left -= r
            if s > 1:
                cost += 2 * s * M * N * 4 / 7e6 + (0.5 * _ceil_div(s, 4) if fused_reduce else 3.0)
            if best is None or cost < best[0] - 1e-9:
                best = (cost, False, tile, s, per, 0)
    return best[1:]


_SWAPPED_STAGES = {16: 6, 32: 5, 64: 4, 128: 3}      # as stages_for() in gemm_tc.cu


def _plan_swapped(M: int, N: int, kb: int, fused_reduce: bool, _SMS: int, cta_limit: int = 0):
    """The swapped mode (up to 128 rows): a stream of weights.  Two CTAs share an SM, so up to 296
    run at a time.  A CTA alone is bound by what its ring keeps in flight (stages x stage bytes per
    memory latency of about 2 us), the CTAs of one SM by its way to L2, all CTAs together by HBM;
    the constants were fitted to timings of the five products of the 1.1B shape at 16, 32, 64 and
    128 rows (the plans picked this way are within 1 % of the best measured ones in sum).  On-chip sums through a cluster measured
    slower at decode sizes than partial results plus a summing consumer (a cluster needs all its
    CTAs scheduled at once, which takes away the early start of the next product's weight loads);
    they stay an option of gemm_fast."""
    tile = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
    tiles = _ceil_div(N, 128)
    stage_bytes = (128 + tile) * 128
    t_mma = 128 * tile * 64 * 2 / 15.2e6
    best = None
    for s in range(1, min(kb, 32) + 1):
        per = _ceil_div(kb, s)
        if _ceil_div(kb, per) != s:
            continue
        if s > 1 and s * M * N * 4 > _PARTIAL_BYTES:
            break
        n_cta = tiles * s
        if cta_limit and s > 1 and n_cta > cta_limit:
            break
        rounds = _ceil_div(n_cta, 2 * _SMS)
        conc = n_cta if rounds == 1 else 2 * _SMS
        per_sm = min(2, _ceil_div(n_cta, _SMS))           # CTAs on the fullest SM: they share its tensor pipe and its way to L2
        t_kb = max(t_mma * per_sm, 2.3 / _SWAPPED_STAGES[tile], stage_bytes * conc / 8.0e6, stage_bytes * per_sm / 80e3)
        cost = rounds * per * t_kb + 1.8
        if s > 1:
            cost += s * M * N * 4 / 7e6                   # partial results written
            # and summed: by their consumer (four splits' loads in flight at a time, so every
            # further four splits cost it another trip to L2), or by a kernel of their own
            cost += 0.5 * _ceil_div(s, 4) + s * M * N * 4 / 7e6 if fused_reduce else 3.0
        if best is None or cost < best[0] - 1e-9:
            best = (cost, True, tile, s, per, 0)
    return best[1:]


def _partials(device) -> torch.Tensor:
    buf = _PARTIALS.get(device)
    if buf is None:
        buf = torch.empty(_PARTIAL_BYTES // 4, dtype=torch.float32, device=device)
        _PARTIALS[device] = buf
    return buf


def gemm_fast_available(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int) -> bool:
    """Whether the tcgen05 product takes this problem (bfloat16, rows of 16-byte multiples)."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    # the conditions of llmk_gemm_tc_supported, checked here: this runs before every product of a
    # step that is not replayed from a graph, and a call into the library costs microseconds
    n, k = w.shape
    return (rows > 0 and n > 0 and k > 0 and k % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and a.is_cuda and w.is_cuda)


def gemm_fast(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int, plan=None, allow_partial: bool = False,
              cta_limit: int = 0):
    """out[:rows] = a[:rows] @ w.T on the tensor cores (bfloat16 in, float32 accumulation).
    Returns out; or, with allow_partial and a split-K plan, a PartialSum that the caller hands to
    a kernel that sums it (out is then not written).  cta_limit: see plan_gemm."""
    _rows_contig(a, "a"); _rows_contig(w, "w"); _rows_contig(out, "out")
    n, k = w.shape
    assert a.shape[1] == k and out.shape[1] == n
    plan = plan or plan_gemm(rows, n, k, fused_reduce=allow_partial, cta_limit=cta_limit)
    swap, tile, splits, per = plan[:4]
    cluster = int(plan[4]) if len(plan) > 4 else 0
    lib = load_tensor()
    if splits == 1 or cluster:
        _check_t(lib.llmk_gemm_tc(_ptr(a), _ptr(w), _ptr(out), c_int(rows), c_int(n), c_int(k),
                                c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                                c_int(_kind(out.dtype)), c_int(int(swap)), c_int(tile), c_int(splits), c_int(per),
                                c_int(int(cluster)), c_int(0), _stream()))
        return out
    part = _partials(a.device)
    _check_t(lib.llmk_gemm_tc(_ptr(a), _ptr(w), _ptr(part), c_int(rows), c_int(n), c_int(k),
                            c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(n), c_int(_F32),
                            c_int(int(swap)), c_int(tile), c_int(splits), c_int(per), c_int(0), c_int(0), _stream()))
    if allow_partial:
        return PartialSum(part, splits, rows, n, out.dtype)
    assert out.is_contiguous()
    _check_t(lib.llmk_reduce_partials(_ptr(out), _ptr(part), c_longlong(rows * n), c_int(splits),
                                    c_int(_kind(out.dtype)), _stream()))
    return out


def gemm_swiglu_available(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int) -> bool:
    """Whether gemm_swiglu takes this problem: bfloat16 throughout, more rows than the swapped
    mode serves (there K is split over CTAs and the activation kernel sums the splits), an even
    number of weight rows."""
    return (rows > 128 and out.dtype == torch.bfloat16 and w.shape[0] % 16 == 0
            and gemm_fast_available(a, w, out, rows))


def gemm_swiglu(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int) -> None:
    """out[:rows] = silu(a @ gate.T) * (a @ up.T) for w = [gate; up] stacked along its rows
    ([2I, K]), out [rows, I] bfloat16.  One persistent tensor-core kernel: each tile multiplies by
    128 gate rows and their 128 up rows and applies the activation in its epilogue, so the
    product never reaches memory."""
    _rows_contig(a, "a"); _rows_contig(w, "w"); _rows_contig(out, "out")
    n, k = w.shape
    assert a.shape[1] == k and out.shape[1] == n // 2 and n % 2 == 0
    if not gemm_swiglu_available(a, w, out, rows):
        raise KernelError(f"gemm_swiglu does not take {rows} rows of {a.dtype} -> {out.dtype}")
    _check_t(load_tensor().llmk_gemm_tc(_ptr(a), _ptr(w), _ptr(out), c_int(rows), c_int(n), c_int(k),
                               c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                               c_int(_BF16), c_int(0), c_int(256), c_int(1), c_int(_ceil_div(k, 64)),
                               c_int(3 if PAIR_GEMM else 2), c_int(1), _stream()))


FUSE_PROMPT_ROPE = True


def _qkv_rope_tile(rows: int, n: int, k: int, head_dim: int) -> int:
    """The tile width (whole heads, up to 256 columns) with the fewest rounds of pair tiles, by
    the pair kernel's terms of plan_gemm."""
    best = None
    _SMS = sm_count()
    for tile in range(head_dim, 257, head_dim):
        t_kb = max(0.31 + 0.0004 * (tile - 128), 1.43 * 256 * tile * 64 * 2 / 2 / 15.2e6)
        cost = _ceil_div(_ceil_div(rows, 256) * _ceil_div(n, tile), _SMS // 2) * t_kb
        if best is None or cost < best[0] - 1e-9:
            best = (cost, tile)
    return best[1]


def qkv_rope_store(x: torch.Tensor, w: torch.Tensor, q_out, rows: int, cos, sin, positions: torch.Tensor,
                   slot_map: torch.Tensor, k_pages, v_pages, n_heads: int, n_kv: int, head_dim: int):
    """The QKV projection of a prompt portion with rotation and cache store in its epilogue:
    x[:rows] @ w.T for w = [q heads; k heads; v heads] (n_kv of each; 0: query heads only), the
    query and key heads rotated by the tables at positions[t], queries written to q_out() [rows,
    n_heads * head_dim], keys and values to place slot_map[t] of the pages.  Returns the tensor
    of the queries; or None, having done nothing, where the kernel does not apply (float32, up to
    128 rows, whose product splits K instead, a head size other than 64 or 128): the caller then
    runs the product and rope_kv_write."""
    if (not FUSE_PROMPT_ROPE or not PAIR_GEMM or rows <= 128 or x.dtype != torch.bfloat16
            or w.dtype != torch.bfloat16 or head_dim not in (64, 128)):
        return None
    n, k = w.shape
    if n != (n_heads + 2 * n_kv) * head_dim:
        return None
    if cos is not None and (cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape[1] != head_dim // 2
                            or not cos.is_contiguous() or not sin.is_contiguous()):
        return None
    if n_kv and not (k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == torch.bfloat16
                     and k_pages.shape[1] == n_kv and k_pages.shape[3] == head_dim):
        return None
    lib = load_tensor()
    q = q_out()
    _rows_contig(x, "x"); _rows_contig(w, "w"); _rows_contig(q, "q_out")
    assert q.dtype == torch.bfloat16 and positions.dtype == torch.int32 and slot_map.dtype == torch.int32
    args = (_ptr(x), _ptr(w), c_int(rows), c_int(n), c_int(k), c_longlong(x.stride(0)), c_longlong(w.stride(0)))
    if not lib.llmk_gemm_tc_qkv_rope_supported(*args, _ptr(q), c_longlong(q.stride(0)), _ptr(cos), _ptr(sin),
                                               _ptr(k_pages) if n_kv else c_void_p(0),
                                               _ptr(v_pages) if n_kv else c_void_p(0), c_int(n_heads), c_int(n_kv),
                                               c_int(head_dim)):
        return None
    _check_t(lib.llmk_gemm_tc_qkv_rope(_ptr(x), _ptr(w), _ptr(q), c_int(rows), c_int(n), c_int(k),
                                       c_longlong(x.stride(0)), c_longlong(w.stride(0)), c_longlong(q.stride(0)),
                                       c_int(_qkv_rope_tile(rows, n, k, head_dim)), _ptr(cos), _ptr(sin),
                                       _ptr(positions), _ptr(slot_map), _ptr(k_pages) if n_kv else c_void_p(0),
                                       _ptr(v_pages) if n_kv else c_void_p(0), c_int(n_heads), c_int(n_kv),
                                       c_int(head_dim), c_int(k_pages.shape[2] if n_kv else 1), _stream()))
    return q


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch between the kernels of a step (on by default); set in both
    kernel libraries."""
    load().llmk_set_pdl(c_int(int(on)))
    load_tensor().llmk_set_pdl(c_int(int(on)))


def set_error_block(block) -> None:
    """Point the tensor-core kernels' error words at `block` (int32 [4] on the device: word 1 is
    the product's, word 2 the attention's), or back at the library's own words with None."""
    if block is not None:
        assert block.dtype == torch.int32 and block.numel() >= 4 and block.is_contiguous()
    load_tensor().llmk_set_error_block(_ptr(block))


_WAIT_NAMES = {1: "TMA producer", 2: "MMA issuer", 0: "epilogue"}
_ATTN_WAITS = {11: "the query tile", 12: "a key/value tile", 13: "the scores", 14: "the probabilities",
               15: "the output product", 16: "tile alignment"}


def describe_wait(word: int, code: int) -> str:
    """What a code in an error word (1: tensor-core product, 2: tensor-core attention) stands for."""
    if word == 1:
        kernel = {0: "one-tile", 1: "persistent", 2: "pair"}.get((code - 1) // 3, "unknown")
        return f"the tensor-core product ({kernel} kernel): its {_WAIT_NAMES[code % 3]} gave up a bounded wait (code {code})"
    if word == 2:
        return f"the tensor-core attention gave up a bounded wait for {_ATTN_WAITS.get(code, 'code ' + str(code))} (code {code})"
    return f"error word {word}: code {code}"


def gemm_tc_take_error() -> int:
    """The code a tensor-core kernel left when one of its bounded waits gave up (0 = none)."""
    return int(load_tensor().llmk_gemm_tc_take_error())
