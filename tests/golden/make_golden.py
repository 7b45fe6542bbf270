"""Makes tests/golden/reference_loops.npz: outputs of the plain CPU loops that the reference
project (zhan-wei-919/llm) ships inside its own kernel tests, on seeded inputs.

    python tests/golden/make_golden.py [/path/to/reference]

The reference's model code is CUDA-only, but its tests carry ordinary C++ oracles:
  rmsnorm_cpu                       kernel/LayerNorm/test/test_rmsnorm.cu:30-49
  build_rope_tables, rope_cpu       kernel/embedding/test/test_rope.cu:10-49
  silu_mul_cpu                      kernel/activation/test/test_swiglu.cu:17-24
  the softmax-attention loop        kernel/attention/test/test_gqattention_window.cu:192-214
  projection + rotate-half          runtime/test/test_qkv_linear.cu:107-114,151-181
This script copies those line ranges, at run time, out of the reference tree into a temporary
C++ file beside a driver of its own (the inputs, a main, the variables the excerpts expect),
compiles it with g++ for the CPU with T = float, runs it and stores inputs and outputs.  None
of the reference's text is kept here or in the output; tests/test_cpu_golden.py compares the
plain implementation (tests/plain_llama.py) with the stored vectors.
"""
from __future__ import annotations

import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "reference_loops.npz")


def excerpt(ref: str, path: str, first: int, last: int) -> str:
    with open(os.path.join(ref, path), encoding="utf-8") as f:
        lines = f.readlines()
    return "".join(lines[first - 1:last])


DRIVER = r"""
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdint>
#include <vector>

static uint64_t rng_state = 12345;
static float rnd() {                       // uniform in [-1, 1)
	rng_state = rng_state * 6364136223846793005ull + 1442695040888963407ull;
	return (float)((rng_state >> 40) / (double)(1 << 24)) * 2.0f - 1.0f;
}
static std::vector<float> values(size_t n, float scale = 1.0f) {
	std::vector<float> v(n);
	for (float &x : v) x = rnd() * scale;
	return v;
}
static void dump(const char *name, const std::vector<float> &v) {
	FILE *f = std::fopen(name, "wb");
	std::fwrite(v.data(), sizeof(float), v.size(), f);
	std::fclose(f);
}

// ---- excerpts of the reference's tests (T = float) ----
%(rmsnorm)s
%(rope)s
%(swiglu)s

// the attention loop reads these names
namespace attn {
constexpr int NH = 6, NKV = 2, HS = 16, QS = NH * HS, KS = NKV * HS;
constexpr int total = 21, start = 19, window_size = 9;
struct Stats {std::vector<float> want; void add(float, float w) {want.push_back(w);}};
static std::vector<float> run(const std::vector<float> &q, const std::vector<float> &k, const std::vector<float> &v) {
	Stats stats;
	std::vector<float> got(q.size(), 0.0f);
%(attention)s
	return stats.want;
}
}

// the projection + rotation loops read these names
namespace qkv {
constexpr int K = 24, NH = 3, NKV = 1, HS = 8, QN = NH * HS, KN = NKV * HS, M = 5;
%(projection)s
using T = float;
struct Stats {std::vector<float> want; void add(float, float w) {want.push_back(w);}};
static std::vector<float> run(const std::vector<float> &input, const std::vector<float> &qw, const std::vector<float> &kw,
                              const std::vector<float> &vw, const std::vector<float> &qb, const std::vector<float> &kb,
                              const std::vector<float> &vb, bool has_bias, const std::vector<int> &positions) {
	Stats stats;
	std::vector<int> destinations(M);
	for (int t = 0; t < M; ++t) destinations[t] = t;
	std::vector<float> got_q(M * QN, 0.0f), got_k(M * KN, 0.0f), got_v(M * KN, 0.0f);
%(qkv_loops)s
	return stats.want;
}
}

int main() {
	{	// RMSNorm: 7 rows of 96
		int BT = 7, C = 96;
		auto x = values((size_t)BT * C, 3.0f), g = values(C);
		for (float &w : g) w = 1.0f + 0.1f * w;
		std::vector<float> out((size_t)BT * C);
		rmsnorm_cpu<float>(out.data(), x.data(), g.data(), BT, C, 1e-5f);
		dump("rms_x.f32", x); dump("rms_g.f32", g); dump("rms_out.f32", out);
	}
	{	// RoPE tables and rotation: 6 tokens from position 37, 3 heads of 32
		int seq = 6, NH = 3, HS = 32, pos0 = 37;
		std::vector<float> cos_t, sin_t;
		build_rope_tables(cos_t, sin_t, 64, HS, 10000.0f);
		auto x = values((size_t)seq * NH * HS);
		std::vector<float> out(x.size());
		rope_cpu<float>(out.data(), x.data(), cos_t.data(), sin_t.data(), seq, NH, HS, pos0);
		dump("rope_cos.f32", cos_t); dump("rope_sin.f32", sin_t); dump("rope_x.f32", x); dump("rope_out.f32", out);
	}
	{	// SiLU(gate) * up
		int N = 301;
		auto gate = values(N, 6.0f), up = values(N, 2.0f);
		std::vector<float> out(N);
		silu_mul_cpu<float>(out.data(), gate.data(), up.data(), N);
		dump("swiglu_gate.f32", gate); dump("swiglu_up.f32", up); dump("swiglu_out.f32", out);
	}
	{	// windowed grouped-query attention of 21 new tokens after 19 earlier ones
		using namespace attn;
		int seq_len = start + total;
		auto q = values((size_t)total * QS, 2.0f), k = values((size_t)seq_len * KS, 2.0f), v = values((size_t)seq_len * KS);
		dump("attn_q.f32", q); dump("attn_k.f32", k); dump("attn_v.f32", v); dump("attn_out.f32", attn::run(q, k, v));
	}
	{	// projection with bias, rotate-half by position
		using namespace qkv;
		auto input = values((size_t)M * K), qw = values((size_t)QN * K, 0.3f), kw = values((size_t)KN * K, 0.3f), vw = values((size_t)KN * K, 0.3f);
		auto qb = values(QN, 0.2f), kb = values(KN, 0.2f), vb = values(KN, 0.2f);
		std::vector<int> positions = {0, 1, 17, 18, 301};
		dump("qkv_input.f32", input); dump("qkv_qw.f32", qw); dump("qkv_kw.f32", kw); dump("qkv_vw.f32", vw);
		dump("qkv_qb.f32", qb); dump("qkv_kb.f32", kb); dump("qkv_vb.f32", vb);
		dump("qkv_out_bias.f32", qkv::run(input, qw, kw, vw, qb, kb, vb, true, positions));
		dump("qkv_out_plain.f32", qkv::run(input, qw, kw, vw, qb, kb, vb, false, positions));
	}
	return 0;
}
"""


def main() -> int:
    ref = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    parts = {
        "rmsnorm": excerpt(ref, "kernel/LayerNorm/test/test_rmsnorm.cu", 30, 49),
        "rope": excerpt(ref, "kernel/embedding/test/test_rope.cu", 10, 49),
        "swiglu": excerpt(ref, "kernel/activation/test/test_swiglu.cu", 17, 24),
        "attention": excerpt(ref, "kernel/attention/test/test_gqattention_window.cu", 192, 214),
        "projection": excerpt(ref, "runtime/test/test_qkv_linear.cu", 107, 114),
        "qkv_loops": excerpt(ref, "runtime/test/test_qkv_linear.cu", 151, 181),
    }
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "loops.cpp")
        with open(src, "w", encoding="utf-8") as f:
            f.write(DRIVER % parts)
        exe = os.path.join(tmp, "loops")
        subprocess.run(["g++", "-O1", "-std=c++17", "-ffp-contract=off", src, "-o", exe], check=True)
        subprocess.run([exe], check=True, cwd=tmp)
        arrays = {n[:-4]: np.fromfile(os.path.join(tmp, n), dtype=np.float32)
                  for n in sorted(os.listdir(tmp)) if n.endswith(".f32")}
    np.savez_compressed(OUT, **arrays)
    print(f"wrote {OUT}: {', '.join(f'{k}[{v.size}]' for k, v in arrays.items())}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
