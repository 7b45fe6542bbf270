"""The decode-attention entry point that allocates nothing, called through its exported C
symbol, against the ordinary entry point.

Some hosts of these kernels cannot call cudaMalloc (they gave all device memory to their own
arena, or cannot take the synchronisation an allocation may bring) and so cannot supply the
scratch buffers of llmk_paged_attention_decode.  llmk_paged_attention_decode_static keeps that
scratch in a fixed array inside the library.  This file runs last so that a run that stops at
the first failure has already run everything else; it passes alone in a fresh process too.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call_static(lib, out, q, kp, vp, bt, kv_lens, B, NH, NKV, HS, window, scale, splits, kind):
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.llmk_paged_attention_decode_static(
        c_void_p(out.data_ptr()), c_longlong(out.stride(0)), c_void_p(q.data_ptr()), c_longlong(q.stride(0)),
        c_void_p(kp.data_ptr()), c_void_p(vp.data_ptr()), c_void_p(bt.data_ptr()), c_int(bt.shape[1]),
        c_void_p(kv_lens.data_ptr()), c_int(B), c_int(NH), c_int(NKV), c_int(HS), c_int(kp.shape[2]), c_int(window),
        c_float(scale), c_int(splits), c_int(kind), stream)


@pytest.mark.parametrize("dtype,kind", [(torch.bfloat16, 1), (torch.float32, 0)])
def test_static_scratch_variant_matches_twice_in_a_row(dtype, kind):
    from llm_b200.csrc import ops
    from llm_b200.csrc.build import load
    lib = load()
    lib.llmk_paged_attention_decode_static.restype = c_int
    torch.manual_seed(21)
    NH, NKV, HS, page, splits = 8, 2, 64, 16, 6
    limit = 1e-2 if dtype == torch.bfloat16 else 2e-6       # the bounds the other kernel tests use
    for lens, window in (([5, 130, 64, 300], 0), ([300, 17, 1], 50)):     # two calls in a row share the scratch
        B = len(lens)
        W = -(-max(lens) // page)
        n_pages = B * W
        kp = torch.randn(n_pages, NKV, page, HS, device=DEV).to(dtype)
        vp = torch.randn(n_pages, NKV, page, HS, device=DEV).to(dtype)
        bt = torch.randperm(n_pages, device=DEV).to(torch.int32).view(B, W).contiguous()
        q = torch.randn(B, NH * HS, device=DEV).to(dtype)
        kv_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
        scale = 1.0 / math.sqrt(HS)
        want = torch.zeros(B, NH * HS, device=DEV, dtype=dtype)
        ops.paged_attention_decode(want, q, kp, vp, bt, kv_lens, B, NH, NKV, HS, window, scale, splits=splits)
        got = torch.full_like(want, float("nan"))
        rc = _call_static(lib, got, q, kp, vp, bt, kv_lens, B, NH, NKV, HS, window, scale, splits, kind)
        assert rc == 0, lib.llmk_last_error()
        torch.cuda.synchronize()
        err = float((got.double() - want.double()).abs().max() / want.double().abs().max())
        assert err <= limit, err
        # and against the formula itself: softmax(q K^T scale) V in float64 over each entry's own pages
        G = NH // NKV
        plain = torch.zeros(B, NH * HS, dtype=torch.float64)
        for b, n in enumerate(lens):
            lo = max(0, n - window) if window else 0
            pages = bt[b, :-(-n // page)].long().cpu()
            K = kp.double().cpu()[pages].permute(1, 0, 2, 3).reshape(NKV, -1, HS)[:, lo:n]
            V = vp.double().cpu()[pages].permute(1, 0, 2, 3).reshape(NKV, -1, HS)[:, lo:n]
            p = torch.softmax(torch.einsum("kgd,ktd->kgt", q[b].double().cpu().view(NKV, G, HS), K) * scale, dim=-1)
            plain[b] = torch.einsum("kgt,ktd->kgd", p, V).reshape(-1)
        assert float((got.double().cpu() - plain).abs().max() / plain.abs().max()) <= limit


def test_static_scratch_variant_refuses_what_does_not_fit():
    from llm_b200.csrc.build import load
    lib = load()
    lib.llmk_paged_attention_decode_static.restype = c_int
    B, NH, HS, splits = 64, 64, 256, 32            # 64*64*32*258 floats, far beyond the built-in 2^20
    t = torch.zeros(8, device=DEV)
    ti = torch.zeros(8, dtype=torch.int32, device=DEV)
    rc = lib.llmk_paged_attention_decode_static(
        c_void_p(t.data_ptr()), c_longlong(NH * HS), c_void_p(t.data_ptr()), c_longlong(NH * HS), c_void_p(t.data_ptr()),
        c_void_p(t.data_ptr()), c_void_p(ti.data_ptr()), c_int(1), c_void_p(ti.data_ptr()), c_int(B), c_int(NH), c_int(NH),
        c_int(HS), c_int(16), c_int(0), c_float(1.0), c_int(splits), c_int(0), c_void_p(0))
    assert rc < 0
    assert b"exceed" in lib.llmk_last_error()
    torch.cuda.synchronize()
