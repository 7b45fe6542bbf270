"""The parts are general: a toy mixer with per-request state of its own, a toy feed-forward
with routing, a toy position encoding and a toy block arrangement, all defined here, are
registered, built and stepped without a change to the package; a layer order that names a
layer twice and a layer that reads another layer's cache run through the same engine.  None of
this is a model of the reference or of anyone: the plain computations are written out below."""
import json
import math
import os

import pytest
import torch

from tiny import TOL, random_tokens

pytestmark = pytest.mark.gpu


# ---- a toy mixer with state: y_t = W * (mean of x_0..x_t) ---------------------------------
def _register_toy():
    from llm_b200.config.model_config import register_architecture
    from llm_b200.models.spec import LayerSpec, ModelSpec, PartSpec
    from llm_b200.parts.base import ParamInfo, Part, StateNeed, register_part
    from llm_b200.parts.linear import linear

    class RunningMeanMixer(Part):
        role = "mixer"

        def __init__(self, hidden_size, prefix="", dtype=None, device=None):
            super().__init__(prefix, dtype, device)
            self.hidden_size = hidden_size
            self.w = None

        def parameters(self):
            return {self.name("mix.weight"): ParamInfo((self.hidden_size, self.hidden_size))}

        def bind(self, tensors):
            self.w = tensors[self.name("mix.weight")].contiguous()

        def cache_need(self):
            return None

        def state_need(self):
            return StateNeed((self.hidden_size + 1,), torch.float32)     # running sum and count

        def is_graph_safe(self, ctx):
            return False                   # the loop below follows the step's host-side sizes

        def forward(self, x, ctx, view):
            T = ctx.n_tokens
            means = torch.empty((T, self.hidden_size), dtype=torch.float32, device=x.device)
            at = 0
            for n, slot in zip(ctx.host_entry_tokens.tolist(), ctx.host_state_slots.tolist()):
                st = view.state[slot]
                sums = st[:-1] + torch.cumsum(x[at:at + n].float(), dim=0)
                counts = st[-1] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                means[at:at + n] = sums / counts[:, None]
                st[:-1] = sums[-1]
                st[-1] = counts[-1]
                at += n
            out = ctx.workspace.get("toy_out", T, self.hidden_size, self.dtype)
            return linear(means.to(self.dtype).contiguous(), self.w, out, T)

    register_part("mixer", "running_mean", RunningMeanMixer)

    class ToyConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

    def build_spec(cfg):
        d = cfg.d
        H, V = d["hidden_size"], d["vocab_size"]
        norm = lambda p: PartSpec("rmsnorm", {"size": H, "eps": d["eps"]}, p)
        rope = PartSpec("rope", {"head_dim": d["head_dim"], "theta": 5000.0, "max_position": d["max_position"]})
        layers = []
        for i, kind in enumerate(d["mixers"]):
            p = f"toy.layers.{i}"
            if kind == "mean":
                mixer = PartSpec("running_mean", {"hidden_size": H}, p + ".mixer")
                cache_of = None
            else:
                shares = kind.startswith("share:")
                mixer = PartSpec("attention", {"hidden_size": H, "num_heads": d["heads"], "num_kv_heads": d["kv_heads"],
                                               "head_dim": d["head_dim"], "position": rope,
                                               "window": d.get("window") if kind == "window" else None,
                                               "shares_cache": shares}, p + ".attn")
                cache_of = int(kind.split(":")[1]) if shares else None
            ffn = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": d["inter"]}, p + ".ffn")
            layers.append(LayerSpec("prenorm", {"norm1": norm(p + ".n1"), "mixer": mixer, "norm2": norm(p + ".n2"),
                                                "ffn": ffn}, cache_of=cache_of))
        return ModelSpec(hidden_size=H, vocab_size=V, max_position=d["max_position"],
                         embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}, "toy.embed"),
                         layers=tuple(layers), order=tuple(d["order"]), final_norm=norm("toy.norm"),
                         head=PartSpec("lm_head", {"hidden_size": H, "vocab_size": V}, "toy.head"))

    register_architecture("ToyForTest", ToyConfig, build_spec)


TOY = dict(architectures=["ToyForTest"], hidden_size=48, vocab_size=97, eps=1e-5, head_dim=16, heads=3, kv_heads=1,
           inter=80, max_position=128, window=9,
           # layer 0: attention; 1: the toy mixer; 2: windowed attention; 3: attention that reads layer 0's cache
           mixers=["full", "mean", "window", "share:0"],
           order=[0, 1, 2, 3, 1, 0])           # layers 1 and 0 run twice


def plain_toy(cfg, w, ids):
    """Whole sequence, float64, no cache; every occurrence of a layer in the order keeps keys of
    its own, and the sharing layer attends over the keys of layer 0's latest earlier run."""
    import plain_llama as pl
    H, HS, NH, NKV = cfg["hidden_size"], cfg["head_dim"], cfg["heads"], cfg["kv_heads"]
    T = len(ids)
    f = lambda n: w[n].double()
    x = f("toy.embed.weight")[torch.tensor(ids)]
    cos, sin = pl.rope_tables(list(range(T)), HS, 5000.0)
    latest_kv = {}
    for li in cfg["order"]:
        p = f"toy.layers.{li}"
        kind = cfg["mixers"][li]
        n = pl.rmsnorm(x, f(p + ".n1.weight"), cfg["eps"])
        if kind == "mean":
            means = torch.cumsum(n, 0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]
            a = means @ f(p + ".mixer.mix.weight").T
        else:
            q = pl.apply_rope((n @ f(p + ".attn.q_proj.weight").T).view(T, NH, HS), cos, sin)
            if kind.startswith("share:"):
                k, v = latest_kv[int(kind.split(":")[1])]
            else:
                k = pl.apply_rope((n @ f(p + ".attn.k_proj.weight").T).view(T, NKV, HS), cos, sin)
                v = (n @ f(p + ".attn.v_proj.weight").T).view(T, NKV, HS)
                latest_kv[li] = (k, v)
            o = pl.attention(q, k, v, window=cfg["window"] if kind == "window" else None)
            a = o.reshape(T, NH * HS) @ f(p + ".attn.o_proj.weight").T
        x = x + a
        m = pl.rmsnorm(x, f(p + ".n2.weight"), cfg["eps"])
        x = x + pl.swiglu_mlp(m, {k_: v_ for k_, v_ in w.items()}, p + ".ffn")
    return pl.rmsnorm(x, f("toy.norm.weight"), cfg["eps"]) @ f("toy.head.weight").T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_repeated_layers_and_shared_cache(tmp_path, dtype):
    import replay
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine
    from llm_b200.weights.loader import write_random_model
    from tiny import load_plain_weights
    _register_toy()
    d = write_random_model(str(tmp_path / "toy"), TOY, 11, dtype)
    w = load_plain_weights(d)
    # ffn tensors follow the swiglu part's names under the toy prefix
    w_ffn = {k.replace(".ffn.", ".ffn."): v for k, v in w.items()}
    reqs = {f"t{i}": random_tokens(n, TOY["vocab_size"], 300 + i) for i, n in enumerate([4, 31, 19, 50])}
    ref = {rid: plain_toy(TOY, w_ffn, toks) for rid, toks in reqs.items()}
    eng = Engine(d, EngineOptions(dtype=dtype, kv_block_size=8, max_num_seqs=4, max_num_batched_tokens=64,
                                  num_kv_blocks=24, use_cuda_graphs=True))      # the toy mixer itself keeps its steps out of graphs
    model = eng.model
    assert len(model.state_needs) == 2                      # the toy layer runs twice: two states
    assert len(model.cache_instances) == 3                  # layer 0 twice, layer 2 once, none for the sharer
    assert sorted(set(model.group_keys)) == [("full", None), ("window", 9)]
    for what, steps in (("whole", replay.steps_whole(reqs)), ("portions", replay.steps_portions(reqs)),
                        ("tail", replay.steps_tail_decode(reqs, tail=6)), ("mixed", replay.steps_mixed(reqs))):
        got = replay.run_steps(eng, steps)
        for rid in reqs:
            err = float((got[rid].double() - ref[rid]).abs().max() / ref[rid].abs().max())
            assert err < TOL[dtype], (what, rid, err)
        eng.cache.check()


# ---- a toy feed-forward with routing, a toy position encoding, a toy block arrangement -------------
def _register_toy_routed():
    from llm_b200.config.model_config import register_architecture
    from llm_b200.models.spec import LayerSpec, ModelSpec, PartSpec
    from llm_b200.parts.base import ParamInfo, Part, ResidualStream, build_part, register_part
    from llm_b200.parts.position import RotaryEmbedding

    class TopOneExperts(Part):
        """Every token goes to the expert with the largest router logit (float32 logits) and gets
        that expert's W2 relu(W1 x), weighted by the softmax probability of its logit."""
        role = "ffn"

        def __init__(self, hidden_size, expert_size, num_experts, prefix="", dtype=None, device=None):
            super().__init__(prefix, dtype, device)
            self.h, self.i, self.e = hidden_size, expert_size, num_experts

        def parameters(self):
            p = {self.name("router.weight"): ParamInfo((self.e, self.h))}
            for k in range(self.e):
                p[self.name(f"experts.{k}.w1.weight")] = ParamInfo((self.i, self.h))
                p[self.name(f"experts.{k}.w2.weight")] = ParamInfo((self.h, self.i))
            return p

        def bind(self, tensors):
            self.router = tensors[self.name("router.weight")].float()
            self.w1 = [tensors[self.name(f"experts.{k}.w1.weight")] for k in range(self.e)]
            self.w2 = [tensors[self.name(f"experts.{k}.w2.weight")] for k in range(self.e)]

        def is_graph_safe(self, ctx):
            return False                   # which rows go to which expert is decided on the host

        def forward(self, x, ctx):
            T = ctx.n_tokens
            logits = x[:T].float() @ self.router.T                     # routing in float32
            prob, choice = torch.softmax(logits, -1).max(-1)
            out = ctx.workspace.get("toy_moe_out", T, self.h, self.dtype)
            for k in range(self.e):
                rows = torch.nonzero(choice == k).flatten()
                if rows.numel():
                    hdn = torch.relu(x[rows].float() @ self.w1[k].float().T)
                    out[rows] = ((hdn @ self.w2[k].float().T) * prob[rows, None]).to(self.dtype)
            return out

    register_part("ffn", "top_one_experts", TopOneExperts)

    class StretchedRotary(RotaryEmbedding):
        """Rotation angles of positions divided by a factor (another table behind the same interface)."""

        def __init__(self, head_dim, theta, max_position, factor, prefix="", dtype=None, device=None):
            super().__init__(head_dim, theta, max_position, prefix, dtype, device)
            self.factor = float(factor)

        def tables(self):
            if self._tables is None:
                half = self.head_dim // 2
                inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / self.head_dim)
                ang = torch.arange(self.max_position, dtype=torch.float64)[:, None] / self.factor * inv[None]
                self._tables = (torch.cos(ang).float().to(self.device).contiguous(), torch.sin(ang).float().to(self.device).contiguous())
            return self._tables

    register_part("position", "stretched_rope", StretchedRotary)

    class ParallelBlock:
        """x += mixer(norm(x)) + ffn(norm(x)): one norm feeds both, their sum is left pending."""
        role = "block"

        def __init__(self, part_specs, dtype, device):
            self.parts = {"norm1": build_part("norm", part_specs["norm1"], dtype, device),
                          "mixer": build_part("mixer", part_specs["mixer"], dtype, device),
                          "ffn": build_part("ffn", part_specs["ffn"], dtype, device)}
            self.mixer = self.parts["mixer"]

        def forward(self, stream: ResidualStream, ctx, view):
            n = self.parts["norm1"].forward(stream, ctx)
            a = self.parts["mixer"].forward(n, ctx, view)
            f = self.parts["ffn"].forward(n, ctx)
            T = ctx.n_tokens
            both = ctx.workspace.get("toy_parallel_sum", T, a.shape[1], a.dtype)
            torch.add(a[:T].float(), f[:T].float(), out=both) if a.dtype == torch.float32 else both.copy_((a[:T].float() + f[:T].float()).to(a.dtype))
            stream.pending = both

    register_part("block", "parallel", ParallelBlock)

    class Cfg:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

    def build_spec(cfg):
        d = cfg.d
        H, V = d["hidden_size"], d["vocab_size"]
        norm = lambda p: PartSpec("rmsnorm", {"size": H, "eps": d["eps"]}, p)
        pos = PartSpec("stretched_rope", {"head_dim": d["head_dim"], "theta": 777.0, "max_position": d["max_position"], "factor": d["factor"]})
        layers = []
        for i, kind in enumerate(d["blocks"]):
            p = f"toy.layers.{i}"
            mixer = PartSpec("attention", {"hidden_size": H, "num_heads": d["heads"], "num_kv_heads": d["kv_heads"],
                                           "head_dim": d["head_dim"], "position": pos}, p + ".attn")
            ffn = PartSpec("top_one_experts", {"hidden_size": H, "expert_size": d["expert_size"], "num_experts": d["experts"]}, p + ".moe")
            parts = {"norm1": norm(p + ".n1"), "mixer": mixer, "ffn": ffn}
            if kind == "prenorm":
                parts["norm2"] = norm(p + ".n2")
            layers.append(LayerSpec(kind, parts))
        return ModelSpec(hidden_size=H, vocab_size=V, max_position=d["max_position"],
                         embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}, "toy.embed"),
                         layers=tuple(layers), order=tuple(range(len(layers))), final_norm=norm("toy.norm"),
                         head=PartSpec("lm_head", {"hidden_size": H, "vocab_size": V, "tied_to": "toy.embed.weight"}, "toy.head"))

    register_architecture("ToyRoutedForTest", Cfg, build_spec)


TOY_ROUTED = dict(architectures=["ToyRoutedForTest"], hidden_size=64, vocab_size=131, eps=1e-6, head_dim=32, heads=2,
                  kv_heads=2, expert_size=40, experts=3, max_position=96, factor=2.5, blocks=["prenorm", "parallel", "prenorm"])


def plain_toy_routed(cfg, w, ids):
    import plain_llama as pl
    H, HS, NH, NKV = cfg["hidden_size"], cfg["head_dim"], cfg["heads"], cfg["kv_heads"]
    T = len(ids)
    f = lambda n: w[n].double()
    x = f("toy.embed.weight")[torch.tensor(ids)]
    half = HS // 2
    inv = torch.pow(torch.tensor(777.0, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / HS)
    ang = torch.arange(T, dtype=torch.float64)[:, None] / cfg["factor"] * inv[None]
    cos, sin = torch.cos(ang), torch.sin(ang)

    def attn(n, p):
        q = pl.apply_rope((n @ f(p + ".attn.q_proj.weight").T).view(T, NH, HS), cos, sin)
        k = pl.apply_rope((n @ f(p + ".attn.k_proj.weight").T).view(T, NKV, HS), cos, sin)
        v = (n @ f(p + ".attn.v_proj.weight").T).view(T, NKV, HS)
        return pl.attention(q, k, v).reshape(T, NH * HS) @ f(p + ".attn.o_proj.weight").T

    def moe(n, p, n_for_routing):
        logits = n_for_routing @ f(p + ".moe.router.weight").T
        prob, choice = torch.softmax(logits, -1).max(-1)
        out = torch.zeros(T, H, dtype=torch.float64)
        for t in range(T):
            k = int(choice[t])
            out[t] = (torch.relu(n[t] @ f(p + f".moe.experts.{k}.w1.weight").T) @ f(p + f".moe.experts.{k}.w2.weight").T) * prob[t]
        return out, choice

    choices = []
    for i, kind in enumerate(cfg["blocks"]):
        p = f"toy.layers.{i}"
        n = pl.rmsnorm(x, f(p + ".n1.weight"), cfg["eps"])
        if kind == "parallel":
            m, c = moe(n, p, n)
            x = x + attn(n, p) + m
        else:
            x = x + attn(n, p)
            n2 = pl.rmsnorm(x, f(p + ".n2.weight"), cfg["eps"])
            m, c = moe(n2, p, n2)
            x = x + m
        choices.append(c)
    return pl.rmsnorm(x, f("toy.norm.weight"), cfg["eps"]) @ f("toy.embed.weight").T, choices


def test_toy_routed_feed_forward_position_encoding_and_block():
    """A feed-forward with top-1 routing, rotation angles from another table and a block that runs
    mixer and feed-forward side by side, all defined in this file, run through the unchanged engine
    in 32-bit, however the tokens are cut.  (Routing is a hard choice, so this runs in 32-bit only:
    in bfloat16 a near-tie of two router logits could send a token to another expert.)"""
    import tempfile
    import replay
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine
    from llm_b200.weights.loader import write_random_model
    from tiny import load_plain_weights
    _register_toy_routed()
    with tempfile.TemporaryDirectory() as tmp:
        d = write_random_model(os.path.join(tmp, "toy_routed"), TOY_ROUTED, 5, "float32")
        w = load_plain_weights(d)
        reqs = {f"m{i}": random_tokens(n, TOY_ROUTED["vocab_size"], 500 + i) for i, n in enumerate([3, 40, 17, 66])}
        ref = {rid: plain_toy_routed(TOY_ROUTED, w, toks)[0] for rid, toks in reqs.items()}
        used = set()
        for toks in reqs.values():
            for c in plain_toy_routed(TOY_ROUTED, w, toks)[1]:
                used |= set(c.tolist())
        assert len(used) == TOY_ROUTED["experts"]                 # the random router spreads the tokens over all experts
        eng = Engine(d, EngineOptions(dtype="float32", kv_block_size=16, max_num_seqs=4, max_num_batched_tokens=96,
                                      num_kv_blocks=16, use_cuda_graphs=True))
        for what, steps in (("whole", replay.steps_whole(reqs)), ("portions", replay.steps_portions(reqs)),
                            ("mixed", replay.steps_mixed(reqs))):
            got = replay.run_steps(eng, steps)
            for rid in reqs:
                err = float((got[rid].double() - ref[rid]).abs().max() / ref[rid].abs().max())
                assert err < TOL["float32"], (what, rid, err)
            eng.cache.check()


# ---- a position encoding with a transform of its own, a head that owns everything after the last
# ---- layer (no final norm, capped logits), and a part that says it must not be captured in a graph
def _register_toy_positions_and_head():
    from llm_b200.config.model_config import register_architecture
    from llm_b200.csrc import ops
    from llm_b200.models.spec import LayerSpec, ModelSpec, PartSpec
    from llm_b200.parts.base import ParamInfo, Part, register_part
    from llm_b200.parts.linear import linear

    class PairwisePartialRotary(Part):
        """Rotates the first `rotary_dim` dims of every head in neighbouring pairs (2i, 2i+1) by
        pos * theta^(-2i/rotary_dim) and leaves the rest: neither a table for the built-in kernels
        nor their pairing, so it brings apply()."""
        role = "position"

        def __init__(self, rotary_dim, theta, prefix="", dtype=None, device=None):
            super().__init__(prefix, dtype, device)
            self.rotary_dim, self.theta = rotary_dim, float(theta)
            self.inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                                 -torch.arange(0, rotary_dim, 2, dtype=torch.float64) / rotary_dim).to(device)

        def apply(self, q, k, ctx):
            T = ctx.n_tokens
            pos = ctx.positions[:T].double()
            ang = pos[:, None] * self.inv[None]
            cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            for x in (q, k):
                if x is None:
                    continue
                a, b = x[:T, :, 0:self.rotary_dim:2].double(), x[:T, :, 1:self.rotary_dim:2].double()
                x[:T, :, 0:self.rotary_dim:2] = (a * cos - b * sin).to(x.dtype)
                x[:T, :, 1:self.rotary_dim:2] = (a * sin + b * cos).to(x.dtype)

    register_part("position", "pairwise_partial_rotary", PairwisePartialRotary)

    class CappedHead(Part):
        """logits = cap * tanh(rows W^T / cap) on the stream as the last layer left it: no norm."""
        role = "head"

        def __init__(self, hidden_size, vocab_size, cap, prefix="", dtype=None, device=None):
            super().__init__(prefix, dtype, device)
            self.h, self.v, self.cap = hidden_size, vocab_size, float(cap)

        def parameters(self):
            return {self.name("weight"): ParamInfo((self.v, self.h))}

        def bind(self, tensors):
            self.weight = tensors[self.name("weight")].contiguous()

        def logits(self, stream, ctx, final_norm, buffers):
            assert final_norm is None
            rows, cast, out = buffers
            R = ctx.n_logit_rows
            ops.gather_rows(rows, stream.resid, stream.pending, ctx.logit_rows, R)
            ops.cast_rows(cast, rows, R)
            linear(cast, self.weight, out, R)
            out[:R] = self.cap * torch.tanh(out[:R] / self.cap)
            return out

    register_part("head", "capped_head", CappedHead)

    class HostSizedFeedForward(Part):
        """relu(x W1^T) W2^T, computed entry by entry from the step's host-side sizes: a captured
        graph of one step would be wrong for a step that cuts the tokens differently, so it says so."""
        role = "ffn"

        def __init__(self, hidden_size, inner_size, prefix="", dtype=None, device=None):
            super().__init__(prefix, dtype, device)
            self.h, self.i = hidden_size, inner_size

        def parameters(self):
            return {self.name("w1.weight"): ParamInfo((self.i, self.h)), self.name("w2.weight"): ParamInfo((self.h, self.i))}

        def bind(self, tensors):
            self.w1, self.w2 = tensors[self.name("w1.weight")], tensors[self.name("w2.weight")]

        def is_graph_safe(self, ctx):
            return False

        def forward(self, x, ctx):
            out = ctx.workspace.get("toy_host_ffn", ctx.n_tokens, self.h, self.dtype)
            at = 0
            for n in ctx.host_entry_tokens.tolist():
                hid = torch.relu(x[at:at + n].float() @ self.w1.float().T)
                out[at:at + n] = (hid @ self.w2.float().T).to(self.dtype)
                at += n
            return out

    register_part("ffn", "host_sized", HostSizedFeedForward)

    class Cfg:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

    def build_spec(cfg):
        d = cfg.d
        H, V = d["hidden_size"], d["vocab_size"]
        norm = lambda p: PartSpec("rmsnorm", {"size": H, "eps": 1e-5}, p)
        pos = PartSpec("pairwise_partial_rotary", {"rotary_dim": d["rotary_dim"], "theta": 5000.0})
        layers = []
        for i in range(d["layers"]):
            p = f"toy.layers.{i}"
            mixer = PartSpec("attention", {"hidden_size": H, "num_heads": d["heads"], "num_kv_heads": d["kv_heads"],
                                           "head_dim": d["head_dim"], "position": pos}, p + ".attn")
            ffn = (PartSpec("host_sized", {"hidden_size": H, "inner_size": 2 * H}, p + ".ffn") if d["host_sized_ffn"]
                   else PartSpec("swiglu", {"hidden_size": H, "intermediate_size": 2 * H}, p + ".ffn"))
            layers.append(LayerSpec("prenorm", {"norm1": norm(p + ".n1"), "mixer": mixer, "norm2": norm(p + ".n2"), "ffn": ffn}))
        return ModelSpec(hidden_size=H, vocab_size=V, max_position=d["max_position"],
                         embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}, "toy.embed"),
                         layers=tuple(layers), order=tuple(range(len(layers))), final_norm=None,
                         head=PartSpec("capped_head", {"hidden_size": H, "vocab_size": V, "cap": d["cap"]}, "toy.head"))

    register_architecture("ToyPositionsHeadForTest", Cfg, build_spec)


TOY_POS = dict(architectures=["ToyPositionsHeadForTest"], hidden_size=128, vocab_size=203, head_dim=64, heads=4, kv_heads=2,
               rotary_dim=24, layers=2, max_position=320, cap=0.05, host_sized_ffn=False)


def plain_toy_positions(cfg, w, ids):
    import plain_llama as pl
    H, HS, NH, NKV, R = cfg["hidden_size"], cfg["head_dim"], cfg["heads"], cfg["kv_heads"], cfg["rotary_dim"]
    T = len(ids)
    f = lambda n: w[n].double()
    x = f("toy.embed.weight")[torch.tensor(ids)]
    inv = torch.pow(torch.tensor(5000.0, dtype=torch.float64), -torch.arange(0, R, 2, dtype=torch.float64) / R)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rotate(t):
        t = t.clone()
        a, b = t[:, :, 0:R:2].clone(), t[:, :, 1:R:2].clone()
        t[:, :, 0:R:2], t[:, :, 1:R:2] = a * cos - b * sin, a * sin + b * cos
        return t

    for i in range(cfg["layers"]):
        p = f"toy.layers.{i}"
        n = pl.rmsnorm(x, f(p + ".n1.weight"), 1e-5)
        q = rotate((n @ f(p + ".attn.q_proj.weight").T).view(T, NH, HS))
        k = rotate((n @ f(p + ".attn.k_proj.weight").T).view(T, NKV, HS))
        v = (n @ f(p + ".attn.v_proj.weight").T).view(T, NKV, HS)
        x = x + pl.attention(q, k, v).reshape(T, NH * HS) @ f(p + ".attn.o_proj.weight").T
        m = pl.rmsnorm(x, f(p + ".n2.weight"), 1e-5)
        if cfg["host_sized_ffn"]:
            x = x + torch.relu(m @ f(p + ".ffn.w1.weight").T) @ f(p + ".ffn.w2.weight").T
        else:
            x = x + (pl.silu(m @ f(p + ".ffn.gate_proj.weight").T) * (m @ f(p + ".ffn.up_proj.weight").T)) @ f(p + ".ffn.down_proj.weight").T
    return cfg["cap"] * torch.tanh((x @ f("toy.head.weight").T) / cfg["cap"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_position_transform_and_head_without_final_norm(dtype):
    """A position encoding that is no table for the built-in kernels (its own apply() between the
    projection and the cache store) and a head that does everything after the last layer itself
    (no final norm, capped logits), defined here, through the unchanged engine with CUDA graphs
    on: prompts in portions (the tensor-core attention in bfloat16) and decoded tokens."""
    import tempfile
    import replay
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine
    from llm_b200.weights.loader import write_random_model
    from tiny import load_plain_weights
    _register_toy_positions_and_head()
    with tempfile.TemporaryDirectory() as tmp:
        d = write_random_model(os.path.join(tmp, "toy_pos"), TOY_POS, 9, dtype)
        w = load_plain_weights(d)
        reqs = {f"p{i}": random_tokens(n, TOY_POS["vocab_size"], 800 + i) for i, n in enumerate([5, 150, 47, 290])}
        ref = {rid: plain_toy_positions(TOY_POS, w, toks) for rid, toks in reqs.items()}
        eng = Engine(d, EngineOptions(dtype=dtype, kv_block_size=16, max_num_seqs=4, max_num_batched_tokens=320,
                                      num_kv_blocks=40, use_cuda_graphs=True))
        for what, steps in (("whole", replay.steps_whole(reqs)), ("tail decode", replay.steps_tail_decode(reqs)),
                            ("mixed", replay.steps_mixed(reqs))):
            got = replay.run_steps(eng, steps)
            for rid in reqs:
                err = float((got[rid].double() - ref[rid]).abs().max() / ref[rid].abs().max())
                assert err < TOL[dtype], (what, rid, err)
        assert eng.counters["graph_replays"] > 0           # every part here is safe to capture
        eng.cache.check()


def test_a_part_that_is_not_graph_safe_turns_capture_off_by_itself():
    """The feed-forward of this model sizes its work from the step's host-side data and says so:
    with CUDA graphs on for the engine, no step is captured or replayed, and the logits are right
    however the tokens are cut (a replayed graph would repeat the first step's cut)."""
    import tempfile
    import replay
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine
    from llm_b200.weights.loader import write_random_model
    from tiny import load_plain_weights
    _register_toy_positions_and_head()
    cfg = dict(TOY_POS, host_sized_ffn=True)
    with tempfile.TemporaryDirectory() as tmp:
        d = write_random_model(os.path.join(tmp, "toy_host"), cfg, 10, "float32")
        w = load_plain_weights(d)
        reqs = {f"h{i}": random_tokens(n, cfg["vocab_size"], 900 + i) for i, n in enumerate([40, 9, 66])}
        ref = {rid: plain_toy_positions(cfg, w, toks) for rid, toks in reqs.items()}
        eng = Engine(d, EngineOptions(dtype="float32", kv_block_size=16, max_num_seqs=4, max_num_batched_tokens=96,
                                      num_kv_blocks=16, use_cuda_graphs=True))
        for steps in (replay.steps_tail_decode(reqs), replay.steps_mixed(reqs)):
            got = replay.run_steps(eng, steps)
            for rid in reqs:
                assert float((got[rid].double() - ref[rid]).abs().max() / ref[rid].abs().max()) < TOL["float32"]
        assert eng.counters["graph_captures"] == 0 and eng.counters["graph_replays"] == 0
