"""Plain, slow implementation of the dense Llama decoder, for tests only.

Whole sequences, no cache, one function per part, float64 on the CPU.  It shares
no code with the engine: everything here is written from the formulas of the
reference project (zhan-wei-919/llm), cited by file:line next to each function.
The reference's own model code is CUDA-only and its attention kernel is locked to
one shape, so it cannot be imported or run on a CPU.  Two things pin this file to
it all the same: tests/test_cpu_golden.py compares the functions here with outputs
of the plain C++ loops that the reference ships inside its kernel tests
(tests/golden/, made by tests/golden/make_golden.py), and on a GPU
tests/test_reference_parity_gpu.py compares forward() with the logits of the
reference's own model at the one shape it runs.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def embedding(table: torch.Tensor, ids) -> torch.Tensor:
    """out[t, :] = table[ids[t], :]  (kernel/embedding/TokenEmbedding.h:12-17)."""
    return table.to(F64)[torch.as_tensor(ids, dtype=torch.long)]


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * gamma, eps inside the root
    (kernel/LayerNorm/RMSNorm.h:13-30,40-42)."""
    x = x.to(F64)
    ms = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    return x / torch.sqrt(ms + eps) * gamma.to(F64)


def rope_tables(positions, head_dim: int, theta: float):
    """cos/sin of pos * theta^(-2i/HS), i < HS/2; the inverse frequency is rounded to
    32-bit and the angle is their 32-bit product, as in the reference
    (kernel/embedding/RoPECache.h:15-20)."""
    half = head_dim // 2
    i = torch.arange(half, dtype=F64)
    inv = torch.pow(torch.tensor(float(theta), dtype=F64), -2.0 * i / head_dim).to(torch.float32)
    pos = torch.as_tensor(positions, dtype=torch.float32)
    ang = (pos[:, None] * inv[None, :]).to(F64)
    return torch.cos(ang), torch.sin(ang)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half on [T, heads, HS]: pairs (i, i+HS/2)
    (kernel/embedding/RoPE.h:22-32; kernel/Gemm/QKVGemm.h:47-53)."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def attention(q, k, v, window: int | None = None, scale: float | None = None):
    """Causal grouped-query attention over one whole sequence.

    q [T, NH, HS], k/v [T, NKV, HS]; query head h reads kv head h // (NH/NKV);
    key j is visible to query t iff max(0, t-window+1) <= j <= t
    (kernel/attention/attention_NH_32_NKV_4_HS_64.h:169-172,214-232,269-316).
    """
    T, NH, HS = q.shape
    NKV = k.shape[1]
    G = NH // NKV
    scale = 1.0 / math.sqrt(HS) if scale is None else scale
    out = torch.zeros(T, NH, HS, dtype=F64)
    t_idx = torch.arange(T)
    visible = t_idx[None, :] <= t_idx[:, None]
    if window is not None:
        visible &= t_idx[None, :] > (t_idx[:, None] - window)
    for h in range(NH):
        g = h // G
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return out


def project(x, w, name, bias=False):
    """x W^T (+ b): the bias is added to the sum before anything else happens to it, rotation
    included (model/modules/Linear.h:12-34; kernel/Gemm/QKVGemm.h:27-45)."""
    y = x @ w[name + ".weight"].to(F64).T
    return y + w[name + ".bias"].to(F64) if bias else y


def attention_part(n, w, prefix, cfg, positions):
    """q/k/v projections, RoPE on q and k, attention, output projection
    (model/modules/Attention.h:16-19; model/modules/QKVLinear.h:20-33)."""
    T = n.shape[0]
    NH, NKV, HS = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    q = project(n, w, prefix + ".q_proj", cfg.get("attention_bias")).view(T, NH, HS)
    k = project(n, w, prefix + ".k_proj", cfg.get("attention_bias")).view(T, NKV, HS)
    v = project(n, w, prefix + ".v_proj", cfg.get("attention_bias")).view(T, NKV, HS)
    cos, sin = rope_tables(positions, HS, cfg["rope_theta"])
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o = attention(q, k, v, window=cfg.get("sliding_window"))
    return project(o.reshape(T, NH * HS), w, prefix + ".o_proj", cfg.get("attention_bias"))


def silu(a: torch.Tensor) -> torch.Tensor:
    """a / (1 + exp(-a))  (kernel/activation/SwiGLU.h:31-33)."""
    return a / (1.0 + torch.exp(-a))


def swiglu_mlp(m, w, prefix, bias=False):
    """down( silu(gate(m)) * up(m) )  (model/modules/MLP.h:10-13)."""
    g = project(m, w, prefix + ".gate_proj", bias)
    u = project(m, w, prefix + ".up_proj", bias)
    return project(silu(g) * u, w, prefix + ".down_proj", bias)


def block(x, w, layer: int, cfg, positions):
    """Pre-norm block: x + attn(norm(x)), then + mlp(norm(.))
    (model/llm/tiny_llama.cpp:29-34)."""
    p = f"model.layers.{layer}"
    eps = cfg["rms_norm_eps"]
    n = rmsnorm(x, w[p + ".input_layernorm.weight"], eps)
    x = x + attention_part(n, w, p + ".self_attn", cfg, positions)
    m = rmsnorm(x, w[p + ".post_attention_layernorm.weight"], eps)
    return x + swiglu_mlp(m, w, p + ".mlp", cfg.get("mlp_bias"))


def normalise_config(cfg: dict) -> dict:
    cfg = dict(cfg)
    cfg.setdefault("num_key_value_heads", cfg["num_attention_heads"])
    if cfg.get("head_dim") is None:
        cfg["head_dim"] = cfg["hidden_size"] // cfg["num_attention_heads"]
    cfg.setdefault("rope_theta", 10000.0)
    cfg.setdefault("sliding_window", None)
    cfg.setdefault("tie_word_embeddings", False)
    return cfg


def forward(cfg: dict, w: dict, ids, rows=None) -> torch.Tensor:
    """Logits [T, V] (float64) of one whole sequence starting at position 0
    (model/llm/tiny_llama.cpp:53-62); with `rows`, only at those positions."""
    cfg = normalise_config(cfg)
    positions = list(range(len(ids)))
    x = embedding(w["model.embed_tokens.weight"], ids)
    for layer in range(cfg["num_hidden_layers"]):
        x = block(x, w, layer, cfg, positions)
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long)]
    x = rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return x @ head.to(F64).T


def argmax_lowest(row: torch.Tensor) -> int:
    """Greedy choice, ties to the smallest id (kernel/sampling/Argmax.h:20-26)."""
    best = row.max()
    return int(torch.nonzero(row == best)[0, 0])


def greedy_generate(cfg, w, prompt, max_new_tokens, eos_token_id=None):
    """Recompute the whole sequence for every new token; stop at eos or at the
    limit (runtime/Scheduler.h:258-260)."""
    ids = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        tok = argmax_lowest(forward(cfg, w, ids)[-1])
        ids.append(tok)
        out.append(tok)
        if eos_token_id is not None and tok == eos_token_id:
            break
    return out


# ---- sampling reference ---------------------------------------------------

_M64 = (1 << 64) - 1


def _mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform_for(seed: int, request_id: int, position: int) -> float:
    """The engine's counter-based uniform in [0, 1): three rounds of the splitmix64
    finaliser over (seed, request, position), top 24 bits.  The reference has no
    temperature sampling, so this documents the engine's own definition."""
    z = _mix64(seed & _M64)
    z = _mix64(z ^ (request_id & _M64))
    z = _mix64(z ^ (position & _M64))
    return (z >> 40) / float(1 << 24)


def sample_temperature(logits_row: torch.Tensor, temperature: float, u: float) -> int:
    """Inverse-CDF draw from softmax(logits / temperature): the first id whose
    cumulative probability exceeds u."""
    p = torch.softmax(logits_row.to(F64) / temperature, dim=-1)
    c = torch.cumsum(p, dim=-1)
    idx = int(torch.searchsorted(c, torch.tensor(u * float(c[-1]), dtype=F64), right=True))
    return min(idx, p.numel() - 1)
