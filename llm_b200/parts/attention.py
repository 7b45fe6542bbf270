"""Grouped-query attention over the paged cache.

One product gives q, k and v (the reference fuses the three weights the same way,
model/modules/QKVLinear.h:20-33); q and k are rotated by the position part's table
and k, v are stored in the layer's pages (kernel/Gemm/QKVGemm.h:27-63); every query
head attends to the keys of kv head h // (NH/NKV) that are at or before its own
position and inside the window, if there is one
(kernel/attention/attention_NH_32_NKV_4_HS_64.h:169-172,228-232); then the output
projection (model/modules/Attention.h:19).  Sizes, window and scale are parameters.
"""
from __future__ import annotations

import math

import torch

from ..csrc import ops
from .base import CacheNeed, ParamInfo, Part, build_part, register_part
from .linear import FUSE_PARTIALS, linear


class PagedAttention(Part):
    role = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position=None,
                 window=None, scale=None, shares_cache: bool = False, bias: bool = False, prefix: str = "",
                 dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        if num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} heads do not divide into {num_kv_heads} kv heads")
        if head_dim <= 0 or head_dim > 256:
            raise ValueError(f"attention: head_dim {head_dim} must be 1 to 256")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.shares_cache = shares_cache          # reads another layer's pages: no k, v of its own
        self.position = build_part("position", position, dtype, device) if position is not None else None
        self.q_size = num_heads * head_dim
        self.kv_size = 0 if shares_cache else num_kv_heads * head_dim
        self.bias = bool(bias)        # q/k/v and o projections carry bias vectors (model/modules/Attention.h:16-19)
        self.w_qkv = None
        self.w_o = None
        self.b_qkv = None
        self.b_o = None

    def parameters(self):
        p = {self.name("q_proj.weight"): ParamInfo((self.q_size, self.hidden_size))}
        if not self.shares_cache:
            p[self.name("k_proj.weight")] = ParamInfo((self.kv_size, self.hidden_size))
            p[self.name("v_proj.weight")] = ParamInfo((self.kv_size, self.hidden_size))
        p[self.name("o_proj.weight")] = ParamInfo((self.hidden_size, self.q_size))
        if self.bias:
            p[self.name("q_proj.bias")] = ParamInfo((self.q_size,), kind="gain", init="normal")
            if not self.shares_cache:
                p[self.name("k_proj.bias")] = ParamInfo((self.kv_size,), kind="gain", init="normal")
                p[self.name("v_proj.bias")] = ParamInfo((self.kv_size,), kind="gain", init="normal")
            p[self.name("o_proj.bias")] = ParamInfo((self.hidden_size,), kind="gain", init="normal")
        return p

    def bind(self, tensors):
        parts = [tensors[self.name("q_proj.weight")]]
        if not self.shares_cache:
            parts += [tensors[self.name("k_proj.weight")], tensors[self.name("v_proj.weight")]]
        self.w_qkv = torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else parts[0].contiguous()
        self.w_o = tensors[self.name("o_proj.weight")].contiguous()
        if self.bias:
            names = ["q_proj.bias"] + ([] if self.shares_cache else ["k_proj.bias", "v_proj.bias"])
            self.b_qkv = torch.cat([tensors[self.name(n)] for n in names]).contiguous()
            self.b_o = tensors[self.name("o_proj.bias")].contiguous()

    def cache_need(self):
        if self.shares_cache:
            return None
        return CacheNeed("window" if self.window else "full", self.num_kv_heads, self.head_dim, self.window)

    def state_need(self):
        return None

    def children(self):
        return [self.position] if self.position is not None else []

    def _qkv_cta_limit(self, ctx, k_pages) -> int:
        """A decode step whose attention has to read several times the bytes of the QKV weights
        (many requests, long contexts) is bound by that reading, and the attention kernel asks for
        its keys and values before it waits for the product: a product on fewer CTAs leaves it SMs
        to start on.  Measured: 64 requests of 640 keys at TinyLlama sizes, 2 instead of 8 splits
        of K: 5 % off the step; about 30 requests of 1,200 keys at Llama-2-7B sizes: 2 % off; with
        8 requests (of 8,000 keys, Llama-3-8B sizes) or with a cache of under four times the
        weights' bytes the full grid is faster."""
        if not ctx.decode_only or self.w_qkv.dtype != torch.bfloat16 or ctx.n_entries < 24:
            return 0
        keys = min(ctx.kv_bucket or 0, self.window or (1 << 30))
        cache_bytes = 2 * ctx.n_entries * keys * k_pages.shape[1] * self.head_dim * k_pages.element_size()
        weight_bytes = self.w_qkv.numel() * self.w_qkv.element_size()
        if cache_bytes <= 4 * weight_bytes:
            return 0
        # from 32 rows on the product runs one CTA per SM (see ops.NORMAL_MODE_FROM_ROWS): half the SMs
        # then measured best (64 requests: 1.29 ms a step with a third, 1.20 ms with half or all)
        return ops.sm_count() // (2 if ctx.n_tokens >= ops.NORMAL_MODE_FROM_ROWS else 3)

    def forward(self, x: torch.Tensor, ctx, view) -> torch.Tensor:
        T = ctx.n_tokens
        ws = ctx.workspace
        width = self.q_size + 2 * self.kv_size
        cos = sin = None
        own_transform = None
        if self.position is not None:
            if hasattr(self.position, "tables"):
                cos, sin = self.position.tables()
            elif hasattr(self.position, "apply"):
                own_transform = self.position.apply
        k_pages, v_pages = view.k_pages, view.v_pages
        attn = ws.get("attn_out", T, self.q_size, self.dtype)
        if own_transform is not None:
            # a position part with a transform of its own: it runs on the summed projection, between
            # the product and the cache store; the kernels after it neither rotate nor sum
            qkv = linear(x, self.w_qkv, ws.get("qkv", T, width, self.dtype), T, bias=self.b_qkv)
            q_view = qkv[:, :self.q_size].view(T, self.num_heads, self.head_dim)
            k_view = (qkv[:, self.q_size:self.q_size + self.kv_size].view(T, -1, self.head_dim)
                      if self.kv_size else None)
            own_transform(q_view, k_view, ctx)
        elif self.bias:
            # biased projections: the product is summed and the bias added before rotation and store
            qkv = linear(x, self.w_qkv, ws.get("qkv", T, width, self.dtype), T, bias=self.b_qkv)
        else:
            # many rows: one kernel projects, rotates and stores; then the attention over the pages
            q = ops.qkv_rope_store(x, self.w_qkv, lambda: ws.get("q_rot", T, self.q_size, self.dtype), T, cos, sin,
                                   ctx.positions, view.group.slot_map, k_pages, v_pages, self.num_heads,
                                   0 if self.shares_cache else k_pages.shape[1], self.head_dim)
            if q is not None:
                ops.paged_attention(attn, q, k_pages, v_pages, view.group, ctx, self.num_heads, k_pages.shape[1],
                                    self.head_dim, self.window or 0, self.scale)
                return linear(attn, self.w_o, ws.get("mixer_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS)
            qkv = linear(x, self.w_qkv, ws.get("qkv", T, width, self.dtype), T, allow_partial=FUSE_PARTIALS,
                         cta_limit=self._qkv_cta_limit(ctx, k_pages))
        ops.rope_store_attend(attn, qkv, cos, sin, k_pages, v_pages, view.group, ctx, self.num_heads,
                              k_pages.shape[1], self.head_dim, self.window or 0, self.scale,
                              write_kv=not self.shares_cache,
                              q_rot=lambda: ws.get("q_rot", T, self.q_size, self.dtype))
        return linear(attn, self.w_o, ws.get("mixer_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS,
                      bias=self.b_o)


register_part("mixer", "attention", PagedAttention)
