"""Tiny configurations and helpers shared by the tests.  A and B are the two tiny
configurations of the benchmark definition; C adds a sliding window, tied embeddings
and plain multi-head attention.  They differ in every size and option."""
from __future__ import annotations

import os

import numpy as np
import torch

CONFIG_A = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=172,
                num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                vocab_size=256, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=128,
                tie_word_embeddings=False, hidden_act="silu")
CONFIG_B = dict(architectures=["LlamaForCausalLM"], hidden_size=96, intermediate_size=256,
                num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
                vocab_size=384, rms_norm_eps=1e-6, rope_theta=500000.0, max_position_embeddings=256,
                tie_word_embeddings=False, hidden_act="silu")
CONFIG_C = dict(architectures=["LlamaForCausalLM"], hidden_size=80, intermediate_size=100,
                num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=5, head_dim=48,
                vocab_size=301, rms_norm_eps=1e-4, rope_theta=1000.0, max_position_embeddings=192,
                tie_word_embeddings=True, sliding_window=37, hidden_act="silu")

# D and E have sizes that the tensor-core kernels take (head size 64 / 128, rows of 16-byte
# multiples), so the bfloat16 engine runs its tcgen05 products and attention on them.
CONFIG_D = dict(architectures=["LlamaForCausalLM"], hidden_size=128, intermediate_size=344,
                num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                vocab_size=520, rms_norm_eps=1e-5, rope_theta=20000.0, max_position_embeddings=512,
                tie_word_embeddings=False, hidden_act="silu")
CONFIG_E = dict(architectures=["LlamaForCausalLM"], hidden_size=96, intermediate_size=200,
                num_hidden_layers=3, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                vocab_size=333, rms_norm_eps=1e-6, rope_theta=300000.0, max_position_embeddings=400,
                tie_word_embeddings=False, sliding_window=150, hidden_act="silu")

# F and G: biases on the projections and head sizes off the 16-grid (80: whole 16-byte pieces per
# row; 100: none in bfloat16), which run on the general kernels in both precisions.
CONFIG_F = dict(architectures=["LlamaForCausalLM"], hidden_size=160, intermediate_size=208,
                num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=80,
                vocab_size=410, rms_norm_eps=1e-5, rope_theta=50000.0, max_position_embeddings=300,
                tie_word_embeddings=False, attention_bias=True, mlp_bias=True, hidden_act="silu")
CONFIG_G = dict(architectures=["LlamaForCausalLM"], hidden_size=96, intermediate_size=130,
                num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=3, head_dim=100,
                vocab_size=277, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=256,
                tie_word_embeddings=True, sliding_window=53, attention_bias=True, hidden_act="silu")

# H: room for a context of thousands of keys (the decode attention's many ranges, long tables of pages).
CONFIG_H = dict(architectures=["LlamaForCausalLM"], hidden_size=128, intermediate_size=200,
                num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                vocab_size=290, rms_norm_eps=1e-5, rope_theta=100000.0, max_position_embeddings=6144,
                tie_word_embeddings=False, hidden_act="silu")

CONFIGS = {"A": (CONFIG_A, 16), "B": (CONFIG_B, 8), "C": (CONFIG_C, 32),
           "D": (CONFIG_D, 16), "E": (CONFIG_E, 32), "F": (CONFIG_F, 16), "G": (CONFIG_G, 8),
           "H": (CONFIG_H, 16)}   # name -> (config, page size)


def make_model_dir(tmp_root, name: str, dtype: str, seed: int = 1234, peaked: bool = False) -> str:
    """A model folder of configuration `name` with seeded random weights.  peaked: the query and
    key projections are scaled so that the attention scores have a standard deviation of about 1.5
    instead of about 0.05 (more than that and bfloat16's own rounding of the scores, which grows with
    them, no longer fits the bound of these tests).  With the plain random weights every softmax is nearly uniform and the
    attention output is close to the mean of the values whatever keys are read; with peaked scores
    a few keys carry each row, so one wrong key, page or mask edge moves the logits by far more
    than the bfloat16 bound."""
    import math

    from llm_b200.weights.loader import write_random_model
    from llm_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    cfg, _ = CONFIGS[name]
    d = os.path.join(str(tmp_root), f"tiny_{name}_{dtype}" + ("_peaked" if peaked else ""))
    if not os.path.isdir(d):
        write_random_model(d, cfg, seed, dtype)
        if peaked:
            path = os.path.join(d, "model.safetensors")
            f = SafetensorsFile(path)
            tensors = {n: f.tensor(n).clone() for n in f.names()}
            f.close()
            factor = math.sqrt(1.5 / (0.0004 * cfg["hidden_size"]))
            for n, t in tensors.items():
                if n.endswith(("q_proj.weight", "k_proj.weight")):
                    tensors[n] = (t.float() * factor).to(t.dtype)
            write_safetensors(path, tensors, metadata={"format": "pt"})
    return d


def load_plain_weights(model_dir: str):
    from llm_b200.weights.safetensors_io import SafetensorsFile
    f = SafetensorsFile(os.path.join(model_dir, "model.safetensors"))
    return {n: f.tensor(n).clone() for n in f.names()}


def random_tokens(n: int, vocab: int, seed: int):
    rng = np.random.default_rng(seed)
    return [int(x) for x in rng.integers(0, vocab, size=n)]


def max_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """Largest absolute difference relative to the largest reference magnitude."""
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


# Normalised error bounds: the 32-bit path differs from the float64 plain implementation by
# rounding only; bfloat16 carries 8 bits of mantissa through every product.
TOL = {"float32": 2e-5, "bfloat16": 3e-2}
