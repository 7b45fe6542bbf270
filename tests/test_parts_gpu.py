"""Each part of a layer alone, built through the registries from a PartSpec, against the
plain implementation's function for that part."""
import math

import numpy as np
import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def rel_err(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def make_ctx(entries, page, n_pages, table_width, max_rows=256):
    """A StepContext for [(start position, tokens, pages of the request)] with one cache group."""
    from llm_b200.engine.context import GroupView, StepContext, Workspace
    T = sum(n for _, n, _ in entries)
    B = len(entries)
    pos = np.concatenate([np.arange(s, s + n) for s, n, _ in entries]).astype(np.int32)
    ent = np.concatenate([np.full(n, i) for i, (_, n, _) in enumerate(entries)]).astype(np.int32)
    cu = np.concatenate([[0], np.cumsum([n for _, n, _ in entries])]).astype(np.int32)
    kv = np.array([s + n for s, n, _ in entries], dtype=np.int32)
    bt = np.zeros((B, table_width), dtype=np.int32)
    slot = np.zeros(T, dtype=np.int32)
    at = 0
    for i, (s, n, pages) in enumerate(entries):
        bt[i, :len(pages)] = pages
        for p in range(s, s + n):
            slot[at] = pages[p // page] * page + p % page
            at += 1
    dev = lambda a: torch.from_numpy(a).to(DEV)
    group = GroupView(page_size=page, block_table=dev(bt), slot_map=dev(slot))
    ctx = StepContext(n_tokens=T, n_entries=B, n_logit_rows=0, token_ids=dev(np.zeros(T, np.int32)), positions=dev(pos),
                      token_entry=dev(ent), cu_tokens=dev(cu), kv_lens=dev(kv), state_slots=dev(np.arange(B, dtype=np.int32)),
                      logit_rows=dev(np.zeros(1, np.int32)), status=torch.zeros(1, dtype=torch.int32, device=DEV),
                      host_entry_tokens=np.array([n for _, n, _ in entries], np.int32),
                      host_entry_start=np.array([s for s, _, _ in entries], np.int32),
                      host_state_slots=np.arange(B, dtype=np.int32), groups={0: group},
                      workspace=Workspace(max_rows, DEV))
    ctx.kv_bucket = (int(kv.max()) + 255) // 256 * 256
    return ctx, group


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from llm_b200.models.spec import PartSpec
    from llm_b200.parts.base import ResidualStream, build_part
    torch.manual_seed(0)
    norm = build_part("norm", PartSpec("rmsnorm", {"size": 136, "eps": 3e-4}, "n"), dtype, DEV)
    assert list(norm.parameters()) == ["n.weight"] and norm.parameters()["n.weight"].shape == (136,)
    gain = 1 + 0.2 * torch.randn(136, device=DEV)
    norm.bind({"n.weight": gain})
    ctx, _ = make_ctx([(0, 9, [0])], 16, 1, 1)
    resid = torch.randn(16, 136, device=DEV)
    pending = torch.randn(9, 136, device=DEV).to(dtype)
    want_resid = resid[:9].double() + pending.double()
    stream = ResidualStream(resid, 9)
    stream.pending = pending
    out = norm.forward(stream, ctx)
    assert stream.pending is None and rel_err(stream.resid[:9], want_resid) < 1e-6
    assert rel_err(out, pl.rmsnorm(want_resid.cpu(), gain.cpu(), 3e-4)) < (1e-5 if dtype == torch.float32 else 1e-2)


def test_position_part_tables_match_plain():
    from llm_b200.models.spec import PartSpec
    from llm_b200.parts.base import build_part
    for hs, theta, n in ((16, 10000.0, 128), (32, 500000.0, 256), (128, 1000.0, 64)):
        rope = build_part("position", PartSpec("rope", {"head_dim": hs, "theta": theta, "max_position": n}), None, DEV)
        cos, sin = rope.tables()
        pc, ps = pl.rope_tables(list(range(n)), hs, theta)
        assert cos.shape == (n, hs // 2)
        assert float((cos.double().cpu() - pc).abs().max()) < 1e-6 and float((sin.double().cpu() - ps).abs().max()) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("NH,NKV,HS,window", [(4, 2, 16, None), (3, 1, 32, 11), (4, 2, 64, None)])
def test_attention_part(dtype, NH, NKV, HS, window):
    """The mixer alone: a request prefilled in two portions beside another request's tokens."""
    from llm_b200.engine.context import LayerView
    from llm_b200.models.spec import PartSpec
    from llm_b200.parts.base import build_part
    torch.manual_seed(1)
    H, page = 72, 16
    rope = PartSpec("rope", {"head_dim": HS, "theta": 10000.0, "max_position": 128})
    part = build_part("mixer", PartSpec("attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": HS,
                                                      "position": rope, "window": window}, "a"), dtype, DEV)
    need = part.cache_need()
    assert need.kind == ("window" if window else "full") and need.num_kv_heads == NKV and need.head_dim == HS
    assert part.state_need() is None
    w = {n: (torch.randn(i.shape) / math.sqrt(i.shape[1])).to(dtype) for n, i in part.parameters().items()}
    assert set(w) == {"a.q_proj.weight", "a.k_proj.weight", "a.v_proj.weight", "a.o_proj.weight"}
    part.bind({n: t.to(DEV) for n, t in w.items()})
    xs = [torch.randn(n, H).to(dtype) for n in (40, 21)]
    cfg = dict(num_attention_heads=NH, num_key_value_heads=NKV, head_dim=HS, rope_theta=10000.0, sliding_window=window)
    refs = [pl.attention_part(x.double(), w, "a", cfg, list(range(len(x)))) for x in xs]
    kp = torch.zeros(8, NKV, page, HS, device=DEV, dtype=dtype)
    vp = torch.zeros_like(kp)
    pages = [[5, 2, 7], [1, 6]]
    got = [torch.zeros(len(x), H, dtype=torch.float64) for x in xs]
    for step in ([(0, 0, 25), (1, 0, 20)], [(0, 25, 15), (1, 20, 1)]):
        ctx, group = make_ctx([(s, n, pages[r]) for r, s, n in step], page, 8, 4)
        view = LayerView(group=group, k_pages=kp, v_pages=vp)
        x = torch.cat([xs[r][s:s + n] for r, s, n in step]).to(DEV).contiguous()
        y = part.forward(x, ctx, view)
        if not isinstance(y, torch.Tensor):                   # a split-K product still to be summed
            y = y.buf[:y.splits * y.rows * y.cols].view(y.splits, y.rows, y.cols).sum(0)
        at = 0
        for r, s, n in step:
            got[r][s:s + n] = y[at:at + n].double().cpu()
            at += n
    for r in range(2):
        assert rel_err(got[r], refs[r]) < (2e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,I", [(64, 172), (96, 256)])
def test_feed_forward_part(dtype, H, I):
    from llm_b200.models.spec import PartSpec
    from llm_b200.parts.base import build_part
    torch.manual_seed(2)
    part = build_part("ffn", PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I}, "m"), dtype, DEV)
    w = {n: (torch.randn(i.shape) / math.sqrt(i.shape[1])).to(dtype) for n, i in part.parameters().items()}
    part.bind({n: t.to(DEV) for n, t in w.items()})
    ctx, _ = make_ctx([(0, 13, [0])], 16, 1, 1)
    x = torch.randn(13, H).to(dtype)
    y = part.forward(x.to(DEV), ctx)
    if not isinstance(y, torch.Tensor):
        y = y.buf[:y.splits * y.rows * y.cols].view(y.splits, y.rows, y.cols).sum(0)
    assert rel_err(y, pl.swiglu_mlp(x.double(), w, "m")) < (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_head_and_block_parts(dtype):
    from llm_b200.engine.context import LayerView
    from llm_b200.models.spec import PartSpec
    from llm_b200.parts.base import ResidualStream, build_part, part_class
    torch.manual_seed(3)
    H, V, NH, NKV, HS, I, page = 64, 301, 4, 2, 16, 100, 16
    emb = build_part("embedding", PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}, "e"), dtype, DEV)
    head = build_part("head", PartSpec("lm_head", {"hidden_size": H, "vocab_size": V}, "h"), dtype, DEV)
    tied = build_part("head", PartSpec("lm_head", {"hidden_size": H, "vocab_size": V, "tied_to": "e.weight"}, "h"), dtype, DEV)
    assert tied.parameters() == {}
    table = (torch.randn(V, H) * 0.5).to(dtype)
    hw = (torch.randn(V, H) / 8).to(dtype)
    emb.bind({"e.weight": table.to(DEV)})
    head.bind({"h.weight": hw.to(DEV)})
    tied.bind({"e.weight": table.to(DEV)})
    ids = [5, 300, 0, 17, 17, 123, 9]
    ctx, group = make_ctx([(0, len(ids), [3])], page, 4, 1)
    ctx.token_ids[:len(ids)] = torch.tensor(ids, dtype=torch.int32, device=DEV)
    stream = ResidualStream(torch.zeros(16, H, device=DEV), len(ids))
    emb.forward(ctx, stream)
    assert torch.equal(stream.resid[:len(ids)].cpu(), pl.embedding(table, ids).float())
    rows = torch.randn(4, H).to(dtype)
    logits = torch.zeros(4, V, device=DEV)
    head.forward(rows.to(DEV), 4, logits)
    assert rel_err(logits, rows.double() @ hw.double().T) < (1e-5 if dtype == torch.float32 else 1e-2)
    tied.forward(rows.to(DEV), 4, logits)
    assert rel_err(logits, rows.double() @ table.double().T) < (1e-5 if dtype == torch.float32 else 1e-2)

    # one pre-norm block against the plain block
    rope = PartSpec("rope", {"head_dim": HS, "theta": 10000.0, "max_position": 64})
    norm = lambda p: PartSpec("rmsnorm", {"size": H, "eps": 1e-5}, p)
    specs = {"norm1": norm("model.layers.0.input_layernorm"), "norm2": norm("model.layers.0.post_attention_layernorm"),
             "mixer": PartSpec("attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": HS,
                                             "position": rope}, "model.layers.0.self_attn"),
             "ffn": PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I}, "model.layers.0.mlp")}
    block = part_class("block", "prenorm")(specs, dtype, DEV)
    w = {}
    for part in block.parts.values():
        for n, info in part.parameters().items():
            w[n] = (1 + 0.1 * torch.randn(info.shape)) if info.kind == "gain" else (torch.randn(info.shape) / math.sqrt(info.shape[1])).to(dtype)
    for part in block.parts.values():
        part.bind({n: t.to(DEV) for n, t in w.items()})
    x0 = torch.randn(len(ids), H)
    stream = ResidualStream(torch.zeros(16, H, device=DEV), len(ids))
    stream.resid[:len(ids)] = x0.to(DEV)
    view = LayerView(group=group, k_pages=torch.zeros(4, NKV, page, HS, device=DEV, dtype=dtype),
                     v_pages=torch.zeros(4, NKV, page, HS, device=DEV, dtype=dtype))
    block.forward(stream, ctx, view)
    pend = stream.pending
    if not isinstance(pend, torch.Tensor):
        pend = pend.buf[:pend.splits * pend.rows * pend.cols].view(pend.splits, pend.rows, pend.cols).sum(0)
    cfg = dict(num_attention_heads=NH, num_key_value_heads=NKV, head_dim=HS, rope_theta=10000.0, rms_norm_eps=1e-5,
               sliding_window=None)
    want = pl.block(x0.double(), w, 0, cfg, list(range(len(ids))))
    got = stream.resid[:len(ids)].double().cpu() + pend[:len(ids)].double().cpu()
    assert rel_err(got, want) < (1e-5 if dtype == torch.float32 else 2e-2)
