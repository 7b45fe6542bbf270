"""The plain implementation against outputs of the reference's own CPU loops.

tests/golden/reference_loops.npz holds what the plain C++ oracles inside the reference's kernel
tests (rmsnorm_cpu, build_rope_tables / rope_cpu, silu_mul_cpu, the softmax-attention loop, the
projection + rotate-half loops) computed in float32 on seeded inputs; tests/golden/make_golden.py
made it.  The plain implementation works in float64, so the two agree to float32 rounding."""
import os

import numpy as np
import torch

import plain_llama as P

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_loops.npz"))


def t(name, *shape):
    return torch.from_numpy(GOLD[name].astype(np.float64)).reshape(*shape)


def close(got, want, tol):
    err = float((got - want).abs().max() / want.abs().max())
    assert err < tol, err


def test_rmsnorm_matches_the_reference_loop():
    x, g, want = t("rms_x", 7, 96), t("rms_g", 96), t("rms_out", 7, 96)
    close(P.rmsnorm(x, g, 1e-5), want, 2e-6)


def test_rope_tables_and_rotation_match_the_reference_loops():
    cos, sin = P.rope_tables(range(64), 32, 10000.0)
    # the reference forms 1 / powf(theta, 2i/HS) in float32; the plain table rounds the float64 power
    # once: the angles differ by an ulp of the frequency times the position
    assert float((cos - t("rope_cos", 64, 16)).abs().max()) < 2e-5
    assert float((sin - t("rope_sin", 64, 16)).abs().max()) < 2e-5
    x, want = t("rope_x", 6, 3, 32), t("rope_out", 6, 3, 32)
    got = P.apply_rope(x, t("rope_cos", 64, 16)[37:43], t("rope_sin", 64, 16)[37:43])
    close(got, want, 2e-6)
    cos6, sin6 = P.rope_tables(range(37, 43), 32, 10000.0)
    close(P.apply_rope(x, cos6, sin6), want, 3e-5)


def test_silu_mul_matches_the_reference_loop():
    gate, up, want = t("swiglu_gate", 301), t("swiglu_up", 301), t("swiglu_out", 301)
    close(P.silu(gate) * up, want, 2e-6)


def test_windowed_attention_matches_the_reference_loop():
    NH, NKV, HS, total, start, window = 6, 2, 16, 21, 19, 9
    q, k, v = t("attn_q", total, NH, HS), t("attn_k", start + total, NKV, HS), t("attn_v", start + total, NKV, HS)
    want = t("attn_out", total, NH, HS)
    # the plain implementation takes a whole sequence: the earlier tokens get zero queries, and the
    # rows of the new tokens are compared
    q_all = torch.cat([torch.zeros(start, NH, HS, dtype=torch.float64), q])
    got = P.attention(q_all, k, v, window=window)[start:]
    close(got, want, 5e-6)


def test_projection_and_rotation_match_the_reference_loops():
    K, NH, NKV, HS, M = 24, 3, 1, 8, 5
    QN, KN = NH * HS, NKV * HS
    x = t("qkv_input", M, K)
    qw, kw, vw = t("qkv_qw", QN, K), t("qkv_kw", KN, K), t("qkv_vw", KN, K)
    qb, kb, vb = t("qkv_qb", QN), t("qkv_kb", KN), t("qkv_vb", KN)
    positions = [0, 1, 17, 18, 301]
    cos, sin = P.rope_tables(positions, HS, 10000.0)
    for name, bias in (("qkv_out_bias", True), ("qkv_out_plain", False)):
        q = (x @ qw.T + (qb if bias else 0)).view(M, NH, HS)
        k = (x @ kw.T + (kb if bias else 0)).view(M, NKV, HS)
        v = x @ vw.T + (vb if bias else 0)
        q, k = P.apply_rope(q, cos, sin), P.apply_rope(k, cos, sin)
        rows = []
        half = HS // 2
        for tok in range(M):       # the loops' order: per token the pairs (i, i + HS/2) of q, then of k, then v
            for heads in (q[tok], k[tok]):
                rows.append(torch.stack([heads[:, :half], heads[:, half:]], dim=-1).reshape(-1))
            rows.append(v[tok])
        close(torch.cat(rows), t(name, M * (QN + 2 * KN)), 3e-5)


def _reference_tree():
    here = os.path.dirname(os.path.abspath(__file__))
    for cand in (os.environ.get("LLM_B200_REFERENCE"), "/root/reference", os.path.join(here, "..", "baseline", "_ref")):
        if cand and os.path.isfile(os.path.join(cand, "utils", "safetensor_loader.h")):
            return os.path.abspath(cand)
    return None


def test_written_safetensors_is_read_by_the_reference_index_reader(tmp_path):
    """A model.safetensors written here, read back by the reference's own index reader
    (utils/safetensor_loader.h:64-95, plain C++): names, dtypes, shapes and byte ranges agree, and
    the bytes at those ranges are the tensors'."""
    import shutil
    import subprocess

    import pytest

    from llm_b200.weights.safetensors_io import write_safetensors

    ref = _reference_tree()
    if ref is None or shutil.which("g++") is None:
        pytest.skip("no copy of the reference tree or no g++ here")
    g = torch.Generator().manual_seed(5)
    tensors = {
        "model.embed_tokens.weight": torch.randn(7, 5, generator=g).to(torch.bfloat16),
        "model.norm.weight": torch.randn(5, generator=g),
        "model.layers.0.mlp.up_proj.weight": torch.randn(3, 5, generator=g).to(torch.float16),
    }
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, tensors, metadata={"format": "pt"})
    src = tmp_path / "read_index.cpp"
    src.write_text('#include "utils/safetensor_loader.h"\n#include <cstdio>\n'
                   'int main(int argc, char **argv) {\n'
                   '  auto infos = weight_loader(argv[1]);\n'
                   '  for (auto &e : infos) {\n'
                   '    std::printf("%s %s %llu %llu", e.first.c_str(), dtype_name(e.second.d),\n'
                   '                (unsigned long long)e.second.start, (unsigned long long)e.second.end);\n'
                   '    for (int s : e.second.shape) std::printf(" %d", s);\n'
                   '    std::printf("\\n");\n'
                   '  }\n  return 0;\n}\n')
    exe = str(tmp_path / "read_index")
    subprocess.run(["g++", "-std=c++17", "-I", ref, "-I", "/usr/local/cuda/include", str(src), "-o", exe], check=True)
    out = subprocess.run([exe, path], check=True, capture_output=True, text=True).stdout
    seen = {}
    for line in out.strip().splitlines():
        name, dtype, start, end, *shape = line.split()
        seen[name] = (dtype, int(start), int(end), tuple(int(s) for s in shape))
    assert set(seen) == set(tensors)
    raw = open(path, "rb").read()
    data_start = 8 + int.from_bytes(raw[:8], "little")
    names = {torch.bfloat16: "bf16", torch.float32: "f32", torch.float16: "f16"}
    for name, tensor in tensors.items():
        dtype, start, end, shape = seen[name]
        assert dtype == names[tensor.dtype] and shape == tuple(tensor.shape)
        assert end - start == tensor.numel() * tensor.element_size()
        assert raw[data_start + start:data_start + end] == tensor.contiguous().view(torch.uint8).numpy().tobytes()
