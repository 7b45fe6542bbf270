"""Each kernel alone against a plain float32/float64 torch reference of the same
operation, at sizes other than the engine's tiny models (odd widths, tails, several
head shapes)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 1e-5 if dtype == torch.float32 else 1.6e-2


def rel_err(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


@pytest.fixture(scope="module")
def ops():
    from llm_b200.csrc import ops as o
    return o


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_bad_id(ops, dtype):
    torch.manual_seed(0)
    table = torch.randn(301, 72, device=DEV).to(dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    resid = torch.full((8, 72), 7.0, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embedding(resid, table, ids, 5, status)
    assert torch.equal(resid[:5], table[ids.long()].float()) and float(resid[5:].min()) == 7.0
    assert int(status.item()) == 0
    ops.embedding(resid, table, torch.tensor([3, 301], dtype=torch.int32, device=DEV), 2, status)
    assert int(status.item()) == 1 and float(resid[1].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden,eps", [(7, 72, 1e-5), (7, 1000, 1e-6), (7, 2048, 1e-2), (7, 8961, 1e-5),
                                             # as many rows as a prompt step has
                                             (701, 2048, 1e-5), (650, 1000, 1e-5), (603, 4096, 1e-6), (600, 2056, 1e-5),
                                             (1200, 8, 1e-5), (640, 4104, 1e-5)])
def test_add_rmsnorm(ops, dtype, rows, hidden, eps):
    torch.manual_seed(1)
    resid = torch.randn(rows + 1, hidden, device=DEV) * 3
    delta = torch.randn(rows, hidden, device=DEV).to(dtype)
    gain = 1 + 0.1 * torch.randn(hidden, device=DEV)
    ref_resid = resid[:rows].double() + delta.double()
    ref = ref_resid / torch.sqrt((ref_resid ** 2).mean(-1, keepdim=True) + eps) * gain.double()
    keep = resid[rows].clone()
    out = torch.zeros(rows, hidden, device=DEV, dtype=dtype)
    ops.add_rmsnorm(resid, delta, gain, out, rows, eps)
    assert rel_err(resid[:rows], ref_resid) < 1e-6 and torch.equal(resid[rows], keep)
    assert rel_err(out, ref) < tol(dtype)
    # without a pending term the residual is left alone
    before = resid.clone()
    ops.add_rmsnorm(resid, None, gain, out, rows, eps)
    assert torch.equal(resid, before) and rel_err(out, ref) < tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gather_rows_and_silu_mul(ops, dtype):
    torch.manual_seed(2)
    resid = torch.randn(20, 130, device=DEV)
    delta = torch.randn(20, 130, device=DEV).to(dtype)
    rows = torch.tensor([19, 0, 7, 7], dtype=torch.int32, device=DEV)
    out = torch.zeros(4, 130, device=DEV)
    ops.gather_rows(out, resid, delta, rows, 4)
    assert rel_err(out, resid[rows.long()].double() + delta[rows.long()].double()) < 1e-6
    ops.gather_rows(out, resid, None, rows, 3)
    assert torch.equal(out[:3], resid[rows.long()[:3]])
    inter = 8961 if dtype == torch.float32 else 173
    gu = (torch.randn(5, 2 * inter, device=DEV) * 4).to(dtype)
    act = torch.zeros(5, inter, device=DEV, dtype=dtype)
    ops.silu_mul(act, gu, 5)
    g, u = gu[:, :inter].double(), gu[:, inter:].double()
    assert rel_err(act, g / (1 + torch.exp(-g)) * u) < tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 172, 64), (33, 65, 172), (130, 257, 96), (64, 64, 17), (3, 1000, 2048)])
def test_gemm_simt(ops, dtype, M, N, K):
    torch.manual_seed(3)
    a = torch.randn(M + 2, K, device=DEV).to(dtype)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(dtype)
    out = torch.full((M + 2, N), 5.0, device=DEV, dtype=dtype)
    ops.gemm_simt(a, w, out, M)
    ref = a[:M].double() @ w.double().T
    assert rel_err(out[:M], ref) < tol(dtype)
    assert float(out[M:].float().min()) == 5.0                  # rows beyond M untouched
    if dtype == torch.bfloat16:
        out32 = torch.zeros(M, N, device=DEV)
        ops.gemm_simt(a, w, out32, M)
        assert rel_err(out32, ref) < 1e-5                       # float32 output of a bfloat16 product


def test_gemm_simt_rows_do_not_depend_on_the_batch(ops):
    torch.manual_seed(4)
    a = torch.randn(150, 200, device=DEV)
    w = torch.randn(77, 200, device=DEV)
    full = torch.zeros(150, 77, device=DEV)
    ops.gemm_simt(a, w, full, 150)
    one = torch.zeros(1, 77, device=DEV)
    for r in (0, 63, 64, 149):
        ops.gemm_simt(a[r:r + 1].contiguous(), w, one, 1)
        assert torch.equal(one[0], full[r])


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 256, 512), (16, 2048, 2048), (17, 384, 192), (50, 1000, 320),
                                   (128, 128, 128), (100, 136, 72), (129, 256, 128), (300, 520, 264), (512, 2560, 2048)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tensor_core(ops, M, N, K, out_dtype):
    torch.manual_seed(5)
    a = torch.randn(M + 1, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    out = torch.full((M + 1, N), 3.0, device=DEV, dtype=out_dtype)
    assert ops.gemm_fast_available(a, w, out, M)
    ops.gemm_fast(a, w, out, M)
    torch.cuda.synchronize()
    assert ops.gemm_tc_take_error() == 0
    ref = a[:M].double() @ w.double().T
    assert rel_err(out[:M], ref) < (1e-5 if out_dtype == torch.float32 else 1e-2)
    assert float(out[M:].float().min()) == 3.0


@pytest.mark.parametrize("swap,tile,splits,cluster", [
    (True, 16, 1, False), (True, 16, 4, False), (True, 32, 2, False), (True, 64, 3, False), (True, 128, 1, False),
    (False, 128, 1, False), (False, 256, 1, False), (False, 256, 2, False), (False, 128, 5, False),
    (False, 160, 1, False), (False, 224, 2, False), (False, 96, 1, False), (False, 32, 1, False),
    (True, 16, 6, True), (True, 16, 2, True), (True, 32, 3, True), (True, 64, 3, True)])
def test_gemm_tensor_core_every_configuration(ops, swap, tile, splits, cluster):
    torch.manual_seed(6)
    M = {16: 9, 32: 30, 64: 64, 128: 77}[tile] if swap else 200
    N, K = 392, 5 * 64 + 24
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    out = torch.zeros(M, N, device=DEV)
    kb = -(-K // 64)
    per = -(-kb // splits)
    ops.gemm_fast(a, w, out, M, plan=(swap, tile, -(-kb // per), per, cluster))
    torch.cuda.synchronize()
    assert ops.gemm_tc_take_error() == 0
    assert rel_err(out, a.double() @ w.double().T) < 1e-5
    if cluster:
        out16 = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
        ops.gemm_fast(a, w, out16, M, plan=(swap, tile, -(-kb // per), per, cluster))
        assert rel_err(out16, a.double() @ w.double().T) < 1e-2


@pytest.mark.parametrize("M,N,K,tile,out_dtype", [
    (300, 520, 5 * 64 + 24, 32, torch.float32),       # 51 tiles, ragged edges on every side
    (2100, 1944, 3 * 64, 96, torch.bfloat16),         # 357 tiles: CTAs take two or three each
    (1300, 2072, 7 * 64 + 8, 256, torch.float32),     # widest tile, more k-blocks than stages
    (4099, 1160, 64, 160, torch.bfloat16),            # one k-block per tile: accumulators swap every block
    (129, 2500, 13 * 64, 224, torch.float32)])        # the second 128 rows hold one row only
@pytest.mark.parametrize("mode", [2, 3])
def test_gemm_tensor_core_persistent(ops, M, N, K, tile, out_dtype, mode):
    """One CTA per SM (mode 2), or a pair of CTAs on two SMs with one MMA for both (mode 3), walks
    over the tiles with two accumulators in tensor memory."""
    torch.manual_seed(8)
    a = torch.randn(M + 1, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    out = torch.full((M + 1, N), 3.0, device=DEV, dtype=out_dtype)
    kb = -(-K // 64)
    ops.gemm_fast(a, w, out, M, plan=(False, tile, 1, kb, mode))
    torch.cuda.synchronize()
    assert ops.gemm_tc_take_error() == 0
    ref = a[:M].double() @ w.double().T
    assert rel_err(out[:M], ref) < (1e-5 if out_dtype == torch.float32 else 1e-2)
    assert float(out[M:].float().min()) == 3.0
    # row by row, so that a tile that landed in another tile's place shows
    worst = ((out[:M].double() - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)).max()
    assert float(worst) < (1e-4 if out_dtype == torch.float32 else 3e-2)
    # a far-off element: one large entry in the last row and column must land exactly there
    a2 = torch.zeros(M, K, device=DEV, dtype=torch.bfloat16)
    w2 = torch.zeros(N, K, device=DEV, dtype=torch.bfloat16)
    a2[M - 1, K - 1] = 2.0
    w2[N - 1, K - 1] = 4.0
    out2 = torch.full((M, N), 1.0, device=DEV, dtype=out_dtype)
    ops.gemm_fast(a2, w2, out2, M, plan=(False, tile, 1, kb, mode))
    assert float(out2[M - 1, N - 1]) == 8.0 and float(out2.float().abs().sum()) == 8.0


@pytest.mark.parametrize("M,I,K", [
    (300, 272, 5 * 64 + 24),        # 9 tiles, a ragged last tile of gate rows that runs into the up rows
    (2100, 976, 3 * 64),            # 136 tiles
    (1300, 1048, 7 * 64 + 8),       # I no multiple of 16; more k-blocks than stages
    (2048, 5632, 256)])             # 704 tiles: CTAs take four or five each
@pytest.mark.parametrize("pair", [False, True])
def test_gemm_tensor_core_with_silu_epilogue(ops, M, I, K, pair, monkeypatch):
    """silu(gate) * up written by the product's epilogue: a tile takes 128 gate rows and their up
    rows; by one CTA, or by a pair of which one stages the gate rows and the other the up rows."""
    monkeypatch.setattr(ops, "PAIR_GEMM", pair)
    torch.manual_seed(9)
    a = torch.randn(M + 1, K, device=DEV).to(torch.bfloat16)
    gate = (torch.randn(I, K, device=DEV) / math.sqrt(K) * 3).to(torch.bfloat16)
    up = (torch.randn(I, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    w = torch.cat([gate, up]).contiguous()
    out = torch.full((M + 1, I), 3.0, device=DEV, dtype=torch.bfloat16)
    assert ops.gemm_swiglu_available(a, w, out, M)
    ops.gemm_swiglu(a, w, out, M)
    torch.cuda.synchronize()
    assert ops.gemm_tc_take_error() == 0
    g = a[:M].double() @ gate.double().T
    u = a[:M].double() @ up.double().T
    ref = g / (1 + torch.exp(-g)) * u
    assert rel_err(out[:M], ref) < 1e-2
    assert float(out[M:].float().min()) == 3.0 and float(out[M:].float().max()) == 3.0
    # one large gate and up in the last row and column land exactly there
    a2 = torch.zeros(M, K, device=DEV, dtype=torch.bfloat16)
    w2 = torch.zeros(2 * I, K, device=DEV, dtype=torch.bfloat16)
    a2[M - 1, K - 1] = 2.0
    w2[I - 1, K - 1] = 8.0          # gate = 16: silu(16) = 16 to bfloat16 precision
    w2[2 * I - 1, K - 1] = 0.5      # up = 1
    out2 = torch.full((M, I), 1.0, device=DEV, dtype=torch.bfloat16)
    ops.gemm_swiglu(a2, w2, out2, M)
    assert float(out2[M - 1, I - 1]) == 16.0 and float(out2.float().abs().sum()) == 16.0


def test_gemm_silu_epilogue_is_not_offered_for_few_rows_or_float32(ops):
    a = torch.zeros(8, 512, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(256, 512, device=DEV, dtype=torch.bfloat16)
    assert not ops.gemm_swiglu_available(a, w, torch.zeros(8, 128, device=DEV, dtype=torch.bfloat16), 8)
    a = torch.zeros(300, 512, device=DEV, dtype=torch.bfloat16)
    assert not ops.gemm_swiglu_available(a, w, torch.zeros(300, 128, device=DEV), 300)
    assert ops.gemm_swiglu_available(a, w, torch.zeros(300, 128, device=DEV, dtype=torch.bfloat16), 300)


def test_gemm_tensor_core_refuses_unaligned_rows(ops):
    a = torch.zeros(4, 172, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(64, 172, device=DEV, dtype=torch.bfloat16)
    assert not ops.gemm_fast_available(a, w, torch.zeros(4, 64, device=DEV, dtype=torch.bfloat16), 4)
    assert not ops.gemm_fast_available(a.float(), w.float(), torch.zeros(4, 64, device=DEV), 4)
    # the check made in Python agrees with the library's own
    from ctypes import c_int, c_longlong, c_void_p
    lib = ops.load_tensor()
    base = torch.zeros(16, 520, device=DEV, dtype=torch.bfloat16)
    for rows, k, col0, pitch_of in ((4, 512, 0, base), (4, 512, 8, base), (4, 512, 4, base), (4, 172, 0, base), (0, 512, 0, base)):
        a2 = pitch_of[:max(rows, 1), col0:col0 + k]
        w2 = torch.zeros(64, k, device=DEV, dtype=torch.bfloat16)
        lib_says = bool(lib.llmk_gemm_tc_supported(c_void_p(a2.data_ptr()), c_void_p(w2.data_ptr()), c_int(rows), c_int(64), c_int(k),
                                                    c_longlong(a2.stride(0)), c_longlong(w2.stride(0))))
        assert ops.gemm_fast_available(a2, w2, None, rows) == lib_says, (rows, k, col0)


def paged_reference(q, k, v, window, scale):
    """q [T, NH, HS], k/v [T, NKV, HS] of one sequence -> [T, NH*HS], float64."""
    T, NH, HS = q.shape
    G = NH // k.shape[1]
    out = torch.zeros(T, NH, HS, dtype=torch.float64)
    for t in range(T):
        lo = max(0, t - window + 1) if window else 0
        for h in range(NH):
            s = (k[lo:t + 1, h // G].double() @ q[t, h].double()) * scale
            out[t, h] = torch.softmax(s, 0) @ v[lo:t + 1, h // G].double()
    return out.reshape(T, NH * HS)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("NH,NKV,HS,page,window", [(4, 2, 16, 16, 0), (3, 1, 32, 8, 0), (6, 3, 48, 32, 19),
                                                   (8, 8, 64, 16, 40), (2, 1, 128, 64, 0), (5, 5, 256, 16, 0),
                                                   (2, 2, 80, 16, 0), (3, 1, 100, 8, 25), (4, 2, 6, 16, 0)])   # off the 16-grid
def test_rope_write_and_paged_attention(ops, dtype, NH, NKV, HS, page, window):
    """Two requests in one batch with reversed, interleaved pages: rope + cache write, then
    attention of a prompt portion beside a single decoded token."""
    torch.manual_seed(7)
    lens = [45, 70]
    n_pages = 24
    W = 12
    kp = torch.zeros(n_pages, NKV, page, HS, device=DEV, dtype=dtype)
    vp = torch.zeros_like(kp)
    half = HS // 2
    inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / HS)
    ang = torch.arange(128, dtype=torch.float64)[:, None] * inv[None]
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    need = [-(-n // page) for n in lens]
    pages = list(range(n_pages - 1, -1, -1))                       # reversed physical order
    tables = [[pages[2 * i + r] for i in range(need[r])] for r in range(2)] if 2 * max(need) <= n_pages else None
    if tables is None:
        pytest.skip("pool too small for this page size")
    bt = torch.zeros(2, W, dtype=torch.int32)
    for r in range(2):
        bt[r, :need[r]] = torch.tensor(tables[r], dtype=torch.int32)
    bt = bt.to(DEV)
    width = (NH + 2 * NKV) * HS
    seqs = [torch.randn(n, width) for n in lens]
    scale = 1.0 / math.sqrt(HS)
    refs = []
    for s in seqs:
        q = s[:, :NH * HS].reshape(-1, NH, HS).to(dtype).double()
        k = s[:, NH * HS:(NH + NKV) * HS].reshape(-1, NKV, HS).to(dtype).double()
        v = s[:, (NH + NKV) * HS:].reshape(-1, NKV, HS).to(dtype)
        c, sn = cos[:len(s)].double().cpu()[:, None], sin[:len(s)].double().cpu()[:, None]
        rot = lambda x: torch.cat([x[..., :half] * c - x[..., half:] * sn, x[..., :half] * sn + x[..., half:] * c], -1)
        refs.append(paged_reference(rot(q).to(dtype), rot(k).to(dtype), v, window, scale))

    # steps: request 0 in portions 30 + 15, request 1 in 69 + a single token beside request 0's second portion
    plan = [[(0, 0, 30), (1, 0, 69)], [(0, 30, 15), (1, 69, 1)]]
    got = [torch.zeros(n, NH * HS, dtype=torch.float64) for n in lens]
    for step in plan:
        rows = torch.cat([seqs[r][a:a + n] for r, a, n in step]).to(dtype).to(DEV).contiguous()
        pos = torch.cat([torch.arange(a, a + n) for r, a, n in step]).to(torch.int32)
        ent = torch.cat([torch.full((n,), i) for i, (r, a, n) in enumerate(step)]).to(torch.int32)
        slot = torch.tensor([tables[r][p // page] * page + p % page for r, a, n in step for p in range(a, a + n)],
                            dtype=torch.int32)
        T = rows.shape[0]
        ops.rope_kv_write(rows, cos, sin, pos.to(DEV), slot.to(DEV), kp, vp, T, NH, NKV, HS)
        out = torch.zeros(T, NH * HS, device=DEV, dtype=dtype)
        ops.paged_attention_generic(out, rows, kp, vp, bt, ent.to(DEV), pos.to(DEV), T, NH, NKV, HS, window, scale)
        at = 0
        for r, a, n in step:
            got[r][a:a + n] = out[at:at + n].double().cpu()
            at += n
    for r in range(2):
        assert rel_err(got[r], refs[r]) < (2e-6 if dtype == torch.float32 else 1.6e-2)


def test_attention_finds_a_far_key_and_respects_the_window_edge(ops):
    """One key far back gets a score that dominates: its value must come through, and must
    vanish exactly when the window no longer reaches it."""
    NH = NKV = 1
    HS, page, n = 32, 16, 300
    kp = torch.zeros(20, 1, page, HS, device=DEV)
    vp = torch.zeros_like(kp)
    torch.manual_seed(8)
    k = torch.randn(n, HS) * 0.1
    v = torch.randn(n, HS)
    far = 37
    k[far] = 0
    k[far, 0] = 50.0
    table = list(range(19, 0, -1))
    for p in range(n):
        kp[table[p // page], 0, p % page] = k[p].to(DEV)
        vp[table[p // page], 0, p % page] = v[p].to(DEV)
    bt = torch.tensor([table + [0]], dtype=torch.int32, device=DEV)
    q = torch.zeros(1, HS, device=DEV)
    q[0, 0] = 50.0
    out = torch.zeros(1, HS, device=DEV)
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    ent = torch.zeros(1, dtype=torch.int32, device=DEV)
    for window, sees in ((0, True), (n - far, True), (n - far - 1, False)):
        ops.paged_attention_generic(out, q, kp, vp, bt, ent, pos, 1, 1, 1, HS, window, 1.0)
        close = float((out[0].cpu() - v[far]).abs().max()) < 1e-4
        assert close == sees, (window, sees)


def _far_key_cache(n, far, HS, page, n_pages, seed):
    """A cache of n keys with small random keys and one key at `far` that a query (50, 0, ...)
    scores overwhelmingly; pages in reversed order."""
    torch.manual_seed(seed)
    k = (torch.randn(n, HS) * 0.1).to(torch.bfloat16)
    v = torch.randn(n, HS).to(torch.bfloat16)
    k[far] = 0
    k[far, 0] = 50.0
    kp = torch.zeros(n_pages, 1, page, HS, dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    table = list(range(n_pages - 1, n_pages - 1 - (-(-n // page)), -1))
    for p in range(n):
        kp[table[p // page], 0, p % page] = k[p]
        vp[table[p // page], 0, p % page] = v[p]
    bt = torch.tensor([table + [0] * (n_pages - len(table))], dtype=torch.int32, device=DEV)
    return k, v, kp.to(DEV), vp.to(DEV), bt


@pytest.mark.parametrize("HS,page", [(64, 16), (128, 32)])
@pytest.mark.parametrize("splits", [1, 4, 12])        # one range; ranges merged in a cluster; merged through the scratch
def test_decode_kernels_find_a_far_key_and_respect_the_window_edge(ops, HS, page, splits):
    """The bfloat16 decode kernels (queries given, and the fused kernel that rotates and stores):
    a key hundreds of positions back, in another range and another page than the query, must come
    through, and must vanish exactly when the window no longer reaches it; and when the newest key
    (the one that the fused kernel stores itself) dominates, its value comes through."""
    n, far, G = 700, 37, 2
    k, v, kp, vp, bt = _far_key_cache(n, far, HS, page, 48, 21)
    kv_lens = torch.tensor([n], dtype=torch.int32, device=DEV)
    q = torch.zeros(1, G * HS, device=DEV, dtype=torch.bfloat16)
    q[0, 0] = 50.0
    q[0, HS] = 50.0
    cos = torch.ones(n, HS // 2, device=DEV)
    sin = torch.zeros(n, HS // 2, device=DEV)
    for window, sees in ((0, True), (n - far, True), (n - far - 1, False)):
        out = torch.zeros(1, G * HS, device=DEV, dtype=torch.bfloat16)
        ops.paged_attention_decode(out, q, kp, vp, bt, kv_lens, 1, G, 1, HS, window, 1.0, splits=splits)
        for h in range(G):
            close = float((out[0, h * HS:(h + 1) * HS].float().cpu() - v[far].float()).abs().max()) < 2e-2
            assert close == sees, ("queries given", window, h)
        # the fused kernel: the row brings q, a small new key and a new value for position n - 1
        row = torch.zeros(1, (G + 2) * HS, device=DEV, dtype=torch.bfloat16)
        row[0, :G * HS] = q[0]
        row[0, G * HS:(G + 1) * HS] = k[n - 1].to(DEV)
        row[0, (G + 1) * HS:] = v[n - 1].to(DEV)
        kp2, vp2 = kp.clone(), vp.clone()
        slot_page, slot_off = int(bt[0, (n - 1) // page]), (n - 1) % page
        kp2[slot_page, 0, slot_off] = 0
        vp2[slot_page, 0, slot_off] = 0
        out2 = torch.zeros_like(out)
        ops.decode_attention_fused(out2, row, cos, sin, kp2, vp2, bt, kv_lens, 1, G, 1, HS, window, 1.0, splits=splits)
        for h in range(G):
            close = float((out2[0, h * HS:(h + 1) * HS].float().cpu() - v[far].float()).abs().max()) < 2e-2
            assert close == sees, ("fused", window, h)
        assert torch.equal(kp2, kp) and torch.equal(vp2, vp)           # the newest key and value landed in their place
    # the newest key dominates: only the fused kernel's own copy of it can give its value
    row = torch.zeros(1, (G + 2) * HS, device=DEV, dtype=torch.bfloat16)
    row[0, 0] = 50.0
    row[0, HS] = 50.0
    row[0, G * HS] = 60.0
    v_new = torch.randn(HS).to(torch.bfloat16)
    row[0, (G + 1) * HS:] = v_new.to(DEV)
    out3 = torch.zeros(1, G * HS, device=DEV, dtype=torch.bfloat16)
    ops.decode_attention_fused(out3, row, cos, sin, kp.clone(), vp.clone(), bt, kv_lens, 1, G, 1, HS, 0, 1.0, splits=splits)
    for h in range(G):
        assert float((out3[0, h * HS:(h + 1) * HS].float().cpu() - v_new.float()).abs().max()) < 2e-2


@pytest.mark.parametrize("HS,page", [(64, 16), (64, 32), (128, 64)])
def test_tensor_core_attention_finds_a_far_key_and_respects_the_window_edge(ops, HS, page):
    """The prompt kernel: 40 new tokens after 660 cached ones, every query scoring one far key
    overwhelmingly.  Each row must return that key's value exactly as long as its own window
    reaches the key."""
    n, far, G, T = 700, 37, 2, 40
    k, v, kp, vp, bt = _far_key_cache(n, far, HS, page, 48, 22)
    q = torch.zeros(T, G * HS, device=DEV, dtype=torch.bfloat16)
    q[:, 0] = 50.0
    q[:, HS] = 50.0
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    kv_lens = torch.tensor([n], dtype=torch.int32, device=DEV)
    first = n - T                                                  # position of the first new token
    for window in (0, n - far, first - far + 20, first - far):
        out = torch.zeros(T, G * HS, device=DEV, dtype=torch.bfloat16)
        ops.attention_tc(out, q, kp, vp, bt, cu, kv_lens, T, 1, G, 1, HS, window, 1.0)
        torch.cuda.synchronize()
        assert ops.attention_tc_take_error() == 0
        for t in range(T):
            sees = window == 0 or (first + t) - window + 1 <= far
            for h in range(G):
                close = float((out[t, h * HS:(h + 1) * HS].float().cpu() - v[far].float()).abs().max()) < 2e-2
                assert close == sees, (window, t, h)


def test_sampling_kernel(ops):
    import plain_llama
    torch.manual_seed(9)
    V = 1003
    logits = torch.randn(6, V, device=DEV) * 3
    logits[1, 3] = logits[1, 9] = 50.0          # a tie: the lowest id wins
    logits[2, V - 1] = 60.0                     # the last id
    out = torch.zeros(6, dtype=torch.int32, device=DEV)
    ops.sample_rows(out, logits, 6)
    want = [plain_llama.argmax_lowest(logits[r].cpu()) for r in range(6)]
    assert out.tolist() == want and want[1] == 3 and want[2] == V - 1
    temps = torch.tensor([0.8, 0.0, 1.5, 0.3, 1.0, 0.8], device=DEV)
    for trial in range(20):
        u = torch.rand(6)
        ops.sample_rows(out, logits, 6, temps, u.to(DEV))
        got = out.tolist()
        for r in range(6):
            if float(temps[r]) <= 0:
                assert got[r] == want[r]
                continue
            p = torch.softmax(logits[r].double().cpu() / float(temps[r]), -1)
            c = torch.cumsum(p, -1)
            ref = plain_llama.sample_temperature(logits[r].cpu(), float(temps[r]), float(u[r]))
            if got[r] != ref:       # only a draw that lands within rounding of a boundary may differ by one id
                lo = float(c[got[r] - 1]) if got[r] > 0 else 0.0
                assert abs(got[r] - ref) == 1 and min(abs(float(u[r]) - lo), abs(float(u[r]) - float(c[got[r]]))) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("NH,NKV,HS,page,window,splits", [(4, 2, 16, 16, 0, 3), (3, 1, 32, 8, 0, 1), (6, 3, 48, 32, 19, 4),
                                                          (32, 4, 64, 16, 0, 7), (2, 1, 128, 64, 100, 32), (12, 1, 256, 16, 0, 5),
                                                          (10, 10, 80, 16, 0, 2),
                                                          (8, 2, 64, 24, 0, 3)])     # pages of no power of two
def test_decode_attention_matches_the_general_kernel_and_plain(ops, dtype, NH, NKV, HS, page, window, splits):
    """Requests of very different lengths in one decode batch, pages in shuffled order."""
    torch.manual_seed(11)
    lens = [1, 2, 33, 257, 140]
    B = len(lens)
    W = -(-max(lens) // page) + 1
    n_pages = sum(-(-n // page) for n in lens) + 3
    perm = torch.randperm(n_pages).tolist()
    kp = torch.randn(n_pages, NKV, page, HS, device=DEV).to(dtype)
    vp = torch.randn(n_pages, NKV, page, HS, device=DEV).to(dtype)
    bt = torch.zeros(B, W, dtype=torch.int32)
    at = 0
    for b, n in enumerate(lens):
        k = -(-n // page)
        bt[b, :k] = torch.tensor(perm[at:at + k], dtype=torch.int32)
        at += k
    bt = bt.to(DEV)
    q = torch.randn(B, NH * HS + 8, device=DEV).to(dtype)       # a row pitch wider than the heads
    kv_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 0.7 / math.sqrt(HS)
    out = torch.zeros(B, NH * HS, device=DEV, dtype=dtype)
    ops.paged_attention_decode(out, q, kp, vp, bt, kv_lens, B, NH, NKV, HS, window, scale, splits=splits)
    ref = torch.zeros(B, NH * HS, dtype=torch.float64)
    G = NH // NKV
    for b, n in enumerate(lens):
        lo = max(0, n - window) if window else 0
        keys = [(int(bt[b, j // page]), j % page) for j in range(lo, n)]
        for h in range(NH):
            K = torch.stack([kp[pg, h // G, o].double().cpu() for pg, o in keys])
            V = torch.stack([vp[pg, h // G, o].double().cpu() for pg, o in keys])
            s = (K @ q[b, h * HS:(h + 1) * HS].double().cpu()) * scale
            ref[b, h * HS:(h + 1) * HS] = torch.softmax(s, 0) @ V
    assert rel_err(out, ref) < (2e-6 if dtype == torch.float32 else 1e-2)
    gen = torch.zeros_like(out)
    ent = torch.arange(B, dtype=torch.int32, device=DEV)
    ops.paged_attention_generic(gen, q, kp, vp, bt, ent, kv_lens - 1, B, NH, NKV, HS, window, scale)
    assert rel_err(out, gen.double()) < (2e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("partial", [False, True])
@pytest.mark.parametrize("NH,NKV,HS,page,window,splits,write_kv", [
    (32, 4, 64, 16, 0, 5, True),       # ranges merged in a cluster
    (8, 1, 64, 8, 0, 1, True),         # one range
    (40, 2, 64, 32, 100, 12, True),    # 20 heads per group: two passes; merge through the scratch
    (6, 3, 128, 16, 0, 3, True),
    (4, 2, 128, 64, 70, 2, False)])    # reads pages that it does not write
def test_decode_attention_fused_with_rotation_and_store(ops, partial, NH, NKV, HS, page, window, splits, write_kv):
    """One kernel for a decode step's rotation, cache store and attention gives what the
    rotate-and-store kernel followed by the decode attention gives, from a tensor and from
    unsummed split-K partial results; requests whose newest token is first or last in a page."""
    torch.manual_seed(13)
    dtype = torch.bfloat16
    lens = [1, page, page + 1, 257, 140, 2 * page]
    B = len(lens)
    W = -(-max(lens) // page) + 1
    n_pages = sum(-(-n // page) for n in lens) + 3
    perm = torch.randperm(n_pages).tolist()
    kp = torch.randn(n_pages, NKV, page, HS, device=DEV).to(dtype)
    vp = torch.randn(n_pages, NKV, page, HS, device=DEV).to(dtype)
    bt = torch.zeros(B, W, dtype=torch.int32)
    at = 0
    for b, n in enumerate(lens):
        k = -(-n // page)
        bt[b, :k] = torch.tensor(perm[at:at + k], dtype=torch.int32)
        at += k
    slot = torch.tensor([int(bt[b, (n - 1) // page]) * page + (n - 1) % page for b, n in enumerate(lens)],
                        dtype=torch.int32, device=DEV)
    bt = bt.to(DEV)
    kv_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    pos = kv_lens - 1
    width = (NH + (2 * NKV if write_kv else 0)) * HS
    qk_splits = 5
    parts = torch.randn(qk_splits, B, width, device=DEV)
    if partial:
        src = ops.PartialSum(parts.reshape(-1), qk_splits, B, width, dtype)
        plain_src = ops.PartialSum(parts.reshape(-1), qk_splits, B, width, dtype)
    else:
        src = parts.sum(0).to(dtype)
        plain_src = src.clone()
    cos = torch.cos(torch.rand(300, HS // 2, device=DEV) * 6)
    sin = torch.sqrt(1 - cos * cos)
    scale = 0.9 / math.sqrt(HS)
    # the two-kernel path
    kp1, vp1 = kp.clone(), vp.clone()
    q1 = torch.zeros(B, NH * HS, device=DEV, dtype=dtype)
    ops.rope_kv_write(plain_src, cos, sin, pos, slot, kp1, vp1, B, NH, NKV if write_kv else 0, HS, q_out=q1)
    out1 = torch.zeros(B, NH * HS, device=DEV, dtype=dtype)
    ops.paged_attention_decode(out1, q1, kp1, vp1, bt, kv_lens, B, NH, NKV, HS, window, scale, splits=splits)
    # the fused kernel
    kp2, vp2 = kp.clone(), vp.clone()
    out2 = torch.zeros(B, NH * HS, device=DEV, dtype=dtype)
    assert ops.decode_attention_fused_supported(src, cos, sin, HS)
    ops.decode_attention_fused(out2, src, cos, sin, kp2, vp2, bt, kv_lens, B, NH, NKV, HS, window, scale,
                               write_kv=write_kv, splits=splits)
    torch.cuda.synchronize()
    assert torch.equal(kp1, kp2) and torch.equal(vp1, vp2)          # the same values at the same places, nothing else touched
    if write_kv:
        assert not torch.equal(kp, kp2)
    assert rel_err(out2, out1.double()) < 2e-3
    # and against the plain formula on the stored pages
    ref = torch.zeros(B, NH * HS, dtype=torch.float64)
    G = NH // NKV
    for b, n in enumerate(lens):
        lo = max(0, n - window) if window else 0
        keys = [(int(bt[b, j // page]), j % page) for j in range(lo, n)]
        for h in range(NH):
            K = torch.stack([kp1[pg, h // G, o].double().cpu() for pg, o in keys])
            V = torch.stack([vp1[pg, h // G, o].double().cpu() for pg, o in keys])
            sc = (K @ q1[b, h * HS:(h + 1) * HS].double().cpu()) * scale
            ref[b, h * HS:(h + 1) * HS] = torch.softmax(sc, 0) @ V
    assert rel_err(out2, ref) < 1e-2


def _plain_decode_attention(q, kp, vp, bt, lens, NH, NKV, HS, page, window, scale):
    """softmax(q K^T scale) V per entry and head in float64 over the entry's own pages."""
    G = NH // NKV
    ref = torch.zeros(len(lens), NH * HS, dtype=torch.float64)
    kp64, vp64, bt_h = kp.double().cpu(), vp.double().cpu(), bt.cpu()
    for b, n in enumerate(lens):
        lo = max(0, n - window) if window else 0
        pages = bt_h[b, :-(-n // page)].long()
        K = kp64[pages].permute(1, 0, 2, 3).reshape(NKV, -1, HS)[:, lo:n]           # [NKV, keys, HS]
        V = vp64[pages].permute(1, 0, 2, 3).reshape(NKV, -1, HS)[:, lo:n]
        qb = q[b, :NH * HS].double().cpu().view(NKV, G, HS)
        p = torch.softmax(torch.einsum("kgd,ktd->kgt", qb, K) * scale, dim=-1)
        ref[b] = torch.einsum("kgt,ktd->kgd", p, V).reshape(-1)
    return ref


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("B,NH,NKV,HS,splits", [(80, 32, 4, 64, 1),      # 320 CTAs of one range each
                                                (40, 32, 4, 64, 2),      # two ranges, merged by the last CTA to arrive
                                                (41, 16, 8, 64, 3),      # three ranges, two heads per group
                                                (160, 8, 1, 128, 1)])    # the same choice at head size 128
def test_decode_attention_with_more_ctas_than_one_wave(ops, fused, B, NH, NKV, HS, splits):
    """A grid that does not fit the SMs at once with deep stages runs the one-stage variant of the
    MMA decode kernel (at head size 64 also held to 128 registers): requests of ragged lengths,
    pages in shuffled order, queries given and rotated-and-stored by the kernel itself, against
    the float64 formula."""
    torch.manual_seed(21)
    dtype, page, window = torch.bfloat16, 16, 0
    g = torch.Generator().manual_seed(B)
    lens = [int(x) for x in torch.randint(1, 300, (B,), generator=g)]
    lens[0], lens[1], lens[2] = 1, page, page + 1
    W = -(-max(lens) // page) + 1
    n_pages = sum(-(-n // page) for n in lens) + 5
    perm = torch.randperm(n_pages, generator=g).tolist()
    kp = torch.randn(n_pages, NKV, page, HS, device=DEV).to(dtype)
    vp = torch.randn(n_pages, NKV, page, HS, device=DEV).to(dtype)
    bt = torch.zeros(B, W, dtype=torch.int32)
    at = 0
    for b, n in enumerate(lens):
        k = -(-n // page)
        bt[b, :k] = torch.tensor(perm[at:at + k], dtype=torch.int32)
        at += k
    bt_d = bt.to(DEV)
    kv_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.3 / math.sqrt(HS)                  # scores wide enough that the far keys matter
    out = torch.zeros(B, NH * HS, device=DEV, dtype=dtype)
    assert splits * NKV * B > (2 if HS == 64 else 1) * torch.cuda.get_device_properties(0).multi_processor_count
    if not fused:
        q = torch.randn(B, NH * HS, device=DEV).to(dtype)
        ops.paged_attention_decode(out, q, kp, vp, bt_d, kv_lens, B, NH, NKV, HS, window, scale, splits=splits)
    else:
        qkv = torch.randn(B, (NH + 2 * NKV) * HS, device=DEV).to(dtype)
        cos = torch.cos(torch.rand(300, HS // 2, device=DEV) * 6)
        sin = torch.sqrt(1 - cos * cos)
        slot = torch.tensor([int(bt[b, (n - 1) // page]) * page + (n - 1) % page for b, n in enumerate(lens)],
                            dtype=torch.int32, device=DEV)
        kp1, vp1 = kp.clone(), vp.clone()
        q = torch.zeros(B, NH * HS, device=DEV, dtype=dtype)
        ops.rope_kv_write(qkv.clone(), cos, sin, kv_lens - 1, slot, kp1, vp1, B, NH, NKV, HS, q_out=q)
        ops.decode_attention_fused(out, qkv, cos, sin, kp, vp, bt_d, kv_lens, B, NH, NKV, HS, window, scale, splits=splits)
        torch.cuda.synchronize()
        assert torch.equal(kp, kp1) and torch.equal(vp, vp1)
    ref = _plain_decode_attention(q, kp, vp, bt, lens, NH, NKV, HS, page, window, scale)
    err = (out.double().cpu() - ref).abs().max(dim=1).values / ref.abs().max()
    assert float(err.max()) < 1e-2, f"entry {int(err.argmax())} of length {lens[int(err.argmax())]}: {float(err.max()):.3e}"


@pytest.mark.parametrize("B,NH,NKV,HS,longest,window,splits", [
    (1, 8, 2, 64, 9000, 0, None),        # the planner's choice for long ranges: 36 ranges of deep stages
    (1, 8, 1, 128, 20000, 0, 64),        # the most ranges the merge takes
    (3, 32, 4, 64, 5000, 0, None),       # 24 ranges, counter merge
    (2, 4, 4, 64, 4100, 3000, 7),        # seven long ranges: no cluster although it would fit one
    (40, 8, 8, 128, 2100, 0, None)])     # one long range per CTA
def test_decode_attention_over_long_contexts(ops, B, NH, NKV, HS, longest, window, splits):
    """Thousands of keys per request: many ranges merged through the scratch, deep stages, the
    bounded request of later tiles into L2; one far key per request made to stand out, so that a
    range lost or merged twice shows.  Against the float64 formula."""
    torch.manual_seed(5)
    dtype, page = torch.bfloat16, 16
    g = torch.Generator().manual_seed(B + longest)
    lens = [longest] + [int(x) for x in torch.randint(longest // 2, longest, (B - 1,), generator=g)]
    W = -(-longest // page)
    n_pages = sum(-(-n // page) for n in lens) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    kp = torch.randn(n_pages, NKV, page, HS, device=DEV).to(dtype)
    vp = torch.randn(n_pages, NKV, page, HS, device=DEV).to(dtype)
    bt = torch.zeros(B, W, dtype=torch.int32)
    at = 0
    for b, n in enumerate(lens):
        k = -(-n // page)
        bt[b, :k] = torch.tensor(perm[at:at + k], dtype=torch.int32)
        at += k
    q = torch.randn(B, NH * HS, device=DEV).to(dtype)
    # the far key: one position per request (inside the window) whose key is the first head's query, scaled
    for b, n in enumerate(lens):
        lo = max(0, n - window) if window else 0
        far = lo + (n - lo) // 7
        pg, off = int(bt[b, far // page]), far % page
        kp[pg, 0, off] = (q[b, :HS].float() * 1.5).to(dtype)      # score 12 or 17 against N(0, 1)
    scale = 1.0 / math.sqrt(HS)
    out = torch.zeros(B, NH * HS, device=DEV, dtype=dtype)
    kv_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    if splits is None:
        assert ops.decode_splits(B, NKV, W * page) > 16 or B * NKV >= 2 * ops.sm_count() // 2
    ops.paged_attention_decode(out, q, kp, vp, bt.to(DEV), kv_lens, B, NH, NKV, HS, window, scale, splits=splits)
    ref = _plain_decode_attention(q, kp, vp, bt, lens, NH, NKV, HS, page, window, scale)
    err = (out.double().cpu() - ref).abs().max(dim=1).values / ref.abs().max()
    assert float(err.max()) < 1e-2, f"entry {int(err.argmax())} of length {lens[int(err.argmax())]}: {float(err.max()):.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("HS,splits", [(64, 1), (64, 3), (128, 12), (48, 2)])
def test_decode_attention_with_an_entry_that_holds_no_keys(ops, dtype, HS, splits):
    """The C entry points take lengths from device memory: an entry of length 0 gets zeros (and
    holds nobody up), one whose length exceeds its table row is cut to the row."""
    torch.manual_seed(31)
    NH, NKV, page = 8, 2, 16
    lens = [0, 37, 0, 90, 1]
    given = [0, 37, -3, 90 + 1000, 1]               # what the kernel is told: 90 + 1000 is cut to the row's 96 keys
    W = 6
    n_pages = 5 * W
    kp = torch.randn(n_pages, NKV, page, HS, device=DEV).to(dtype)
    vp = torch.randn(n_pages, NKV, page, HS, device=DEV).to(dtype)
    bt = torch.randperm(n_pages)[:5 * W].view(5, W).to(torch.int32)
    lens[3] = W * page
    q = torch.randn(5, NH * HS, device=DEV).to(dtype)
    out = torch.full((5, NH * HS), 7.0, device=DEV, dtype=dtype)
    ops.paged_attention_decode(out, q, kp, vp, bt.to(DEV), torch.tensor(given, dtype=torch.int32, device=DEV), 5, NH, NKV,
                               HS, 0, 0.2, splits=splits)
    ref = _plain_decode_attention(q, kp, vp, bt, [max(n, 1) for n in lens], NH, NKV, HS, page, 0, 0.2)
    for e, n in enumerate(lens):
        if n == 0:
            assert float(out[e].abs().max()) == 0.0
        else:
            assert rel_err(out[e], ref[e]) < (2e-6 if dtype == torch.float32 else 1e-2)


def test_decode_attention_fused_refuses_other_sizes(ops):
    cos = torch.ones(8, 24, device=DEV)
    assert not ops.decode_attention_fused_supported(torch.zeros(2, 48 * 3, device=DEV, dtype=torch.bfloat16), cos, cos, 48)
    assert not ops.decode_attention_fused_supported(torch.zeros(2, 64 * 3, device=DEV), cos, cos, 64)
    odd = torch.zeros(2, 64 * 3 + 4, device=DEV, dtype=torch.bfloat16)
    assert not ops.decode_attention_fused_supported(odd, cos, cos, 64)
    ok = torch.zeros(2, 64 * 3, device=DEV, dtype=torch.bfloat16)
    assert ops.decode_attention_fused_supported(ok, cos, cos, 64, page_size=32)
    assert not ops.decode_attention_fused_supported(ok, cos, cos, 64, page_size=24)      # pages of no power of two


def test_consumers_sum_split_k_partials_themselves(ops):
    """add_rmsnorm, silu_mul, gather_rows and rope_kv_write given the float32 partial results
    of a split-K product give what they give for the summed tensor."""
    torch.manual_seed(12)
    rows, hidden, splits = 6, 200, 3
    parts = torch.randn(splits, rows, hidden, device=DEV)
    summed = parts.sum(0)
    ps = ops.PartialSum(parts.reshape(-1), splits, rows, hidden, torch.bfloat16)
    gain = 1 + 0.1 * torch.randn(hidden, device=DEV)
    r1 = torch.randn(rows, hidden, device=DEV)
    r2 = r1.clone()
    o1 = torch.zeros(rows, hidden, device=DEV, dtype=torch.bfloat16)
    o2 = torch.zeros_like(o1)
    ops.add_rmsnorm(r1, ps, gain, o1, rows, 1e-5)
    ref_resid = r2.double() + summed.double()
    assert rel_err(r1, ref_resid) < 1e-6
    ref = ref_resid / torch.sqrt((ref_resid ** 2).mean(-1, keepdim=True) + 1e-5) * gain.double()
    assert rel_err(o1, ref) < 1e-2
    # gather
    idx = torch.tensor([5, 0, 3], dtype=torch.int32, device=DEV)
    g = torch.zeros(3, hidden, device=DEV)
    ops.gather_rows(g, r2, ps, idx, 3)
    assert rel_err(g, (r2.double() + summed.double())[idx.long()]) < 1e-6
    # silu
    inter = hidden // 2
    act = torch.zeros(rows, inter, device=DEV, dtype=torch.bfloat16)
    ops.silu_mul(act, ps, rows)
    gg, uu = summed[:, :inter].double(), summed[:, inter:].double()
    assert rel_err(act, gg / (1 + torch.exp(-gg)) * uu) < 1e-2
    # rope + store: the partial source against the summed bf16 source
    NH, NKV, HS, page = 3, 1, 40, 8
    width = (NH + 2 * NKV) * HS
    assert width == hidden
    cos = torch.cos(torch.rand(16, HS // 2, device=DEV) * 6)
    sin = torch.sqrt(1 - cos * cos)
    pos = torch.arange(rows, dtype=torch.int32, device=DEV)
    slot = torch.tensor([8, 9, 10, 3, 4, 5], dtype=torch.int32, device=DEV)
    kp1 = torch.zeros(3, NKV, page, HS, device=DEV, dtype=torch.bfloat16); vp1 = torch.zeros_like(kp1)
    kp2 = torch.zeros_like(kp1); vp2 = torch.zeros_like(kp1)
    q1 = torch.zeros(rows, NH * HS, device=DEV, dtype=torch.bfloat16)
    ops.rope_kv_write(ps, cos, sin, pos, slot, kp1, vp1, rows, NH, NKV, HS, q_out=q1)
    src = summed.clone()          # float32 source through the same kernel, then compare in bf16 terms
    q2 = torch.zeros(rows, NH * HS, device=DEV)
    kp2f = torch.zeros(3, NKV, page, HS, device=DEV); vp2f = torch.zeros_like(kp2f)
    ops.rope_kv_write(src, cos, sin, pos, slot, kp2f, vp2f, rows, NH, NKV, HS, q_out=q2)
    assert rel_err(q1, q2) < 1e-2 and rel_err(kp1, kp2f) < 1e-2 and rel_err(vp1, vp2f) < 1e-2


@pytest.mark.parametrize("NH,NKV,HS,page,window", [(8, 1, 64, 16, 0), (32, 4, 64, 16, 0), (4, 2, 64, 32, 150), (3, 3, 64, 64, 0),
                                                   (6, 2, 64, 16, 37), (2, 1, 128, 16, 0), (8, 2, 128, 32, 200), (5, 1, 128, 128, 0)])
def test_tensor_core_attention_matches_the_general_kernel(ops, NH, NKV, HS, page, window):
    """A ragged batch: a long prompt portion that starts deep in its request, short portions,
    single tokens, shuffled pages; compared with the general kernel on the same cache and with
    the formula."""
    torch.manual_seed(13)
    # (keys already cached, new tokens) per entry
    plan = [(300, 150), (0, 37), (511, 1), (129, 1), (0, 1), (250, 6)]
    B = len(plan)
    total = [a + n for a, n in plan]
    W = -(-max(total) // page) + 1
    n_pages = sum(-(-t // page) for t in total) + 2
    perm = torch.randperm(n_pages).tolist()
    kp = (torch.randn(n_pages, NKV, page, HS, device=DEV)).to(torch.bfloat16)
    vp = (torch.randn(n_pages, NKV, page, HS, device=DEV)).to(torch.bfloat16)
    bt = torch.full((B, W), -1, dtype=torch.int32)
    at = 0
    for b, t in enumerate(total):
        k = -(-t // page)
        bt[b, :k] = torch.tensor(perm[at:at + k], dtype=torch.int32)
        at += k
    bt = bt.to(DEV)
    T = sum(n for _, n in plan)
    q = (torch.randn(T, NH * HS + 16, device=DEV) * 1.5).to(torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor([n for _, n in plan]).cumsum(0)), dtype=torch.int32, device=DEV)
    kv_lens = torch.tensor(total, dtype=torch.int32, device=DEV)
    pos = torch.cat([torch.arange(a, a + n) for a, n in plan]).to(torch.int32).to(DEV)
    ent = torch.cat([torch.full((n,), i) for i, (_, n) in enumerate(plan)]).to(torch.int32).to(DEV)
    scale = 1.0 / math.sqrt(HS)
    assert ops.attention_tc_supported(torch.bfloat16, NH, NKV, HS, page)
    out = torch.zeros(T, NH * HS, device=DEV, dtype=torch.bfloat16)
    ops.attention_tc(out, q, kp, vp, bt, cu, kv_lens, T, B, NH, NKV, HS, window, scale)
    torch.cuda.synchronize()
    assert ops.attention_tc_take_error() == 0
    ref = torch.zeros_like(out)
    ops.paged_attention_generic(ref, q, kp, vp, bt.clamp_min(0), ent, pos, T, NH, NKV, HS, window, scale)
    err_rows = (out.double() - ref.double()).abs().max(dim=1).values / ref.double().abs().max()
    bad = torch.nonzero(err_rows > 1.2e-2)
    assert bad.numel() == 0, f"first differing row {int(bad[0])} (entry {int(ent[int(bad[0])])}, pos {int(pos[int(bad[0])])}): {float(err_rows[int(bad[0])]):.3e}"
    # and against the formula itself, in float64 on the entries' own pages
    want = torch.zeros(T, NH * HS, dtype=torch.float64)
    G = NH // NKV
    row = 0
    for b, (a, n) in enumerate(plan):
        pages = bt[b, :-(-total[b] // page)].long().cpu()
        K = kp.double().cpu()[pages].permute(1, 0, 2, 3).reshape(NKV, -1, HS)[:, :total[b]]
        V = vp.double().cpu()[pages].permute(1, 0, 2, 3).reshape(NKV, -1, HS)[:, :total[b]]
        qb = q[row:row + n, :NH * HS].double().cpu().view(n, NKV, G, HS)
        sc = torch.einsum("nkgd,ktd->nkgt", qb, K) * scale
        p_new = torch.arange(a, a + n)[:, None]
        keys = torch.arange(total[b])[None, :]
        visible = (keys <= p_new) & ((keys > p_new - window) if window else torch.ones_like(keys, dtype=torch.bool))
        sc = sc.masked_fill(~visible[:, None, None, :], float("-inf"))
        want[row:row + n] = torch.einsum("nkgt,ktd->nkgd", torch.softmax(sc, -1), V).reshape(n, -1)
        row += n
    assert rel_err(out, want) < 1.2e-2


def test_tensor_core_attention_refuses_other_sizes(ops):
    assert not ops.attention_tc_supported(torch.bfloat16, 4, 2, 48, 16)
    assert not ops.attention_tc_supported(torch.bfloat16, 4, 2, 64, 8)
    assert not ops.attention_tc_supported(torch.float32, 4, 2, 64, 16)
    assert not ops.attention_tc_supported(torch.bfloat16, 256, 1, 64, 16)


@pytest.mark.parametrize("M,NH,NKV,HS,K,page", [
    (300, 5, 1, 64, 5 * 64 + 24, 16),     # 7 heads: the last tile is one head wide; a ragged last row tile
    (1111, 12, 4, 64, 3 * 64, 8),         # 20 heads; several tiles per pair
    (400, 3, 3, 128, 2 * 64 + 8, 16),     # head size 128: two 32-column pieces per half
    (260, 6, 0, 64, 64, 16)])             # query heads only (a layer that reads another layer's pages)
def test_qkv_projection_with_rotation_and_store_in_its_epilogue(ops, M, NH, NKV, HS, K, page):
    """The pair kernel's QKV epilogue against product, rotation and store written out in float32:
    positions and places are scattered, so a row that took another row's angle or page shows."""
    torch.manual_seed(12)
    N = (NH + 2 * NKV) * HS
    a = torch.randn(M + 1, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    max_pos = 2 * M
    inv = 1.0 / (10000.0 ** (torch.arange(0, HS, 2, dtype=torch.float64) / HS))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    g = torch.Generator().manual_seed(3)
    pos = torch.randperm(max_pos, generator=g)[:M].to(torch.int32)
    n_pages = -(-M // page) + 3
    slot = torch.randperm(n_pages * page, generator=g)[:M].to(torch.int32)
    kp = torch.full((n_pages, max(NKV, 1), page, HS), 7.0, device=DEV, dtype=torch.bfloat16)
    vp = torch.full((n_pages, max(NKV, 1), page, HS), 7.0, device=DEV, dtype=torch.bfloat16)
    q_buf = torch.full((M + 1, NH * HS), 3.0, device=DEV, dtype=torch.bfloat16)
    q = ops.qkv_rope_store(a, w, lambda: q_buf, M, cos, sin, pos.to(DEV), slot.to(DEV), kp if NKV else None,
                           vp if NKV else None, NH, NKV, HS)
    torch.cuda.synchronize()
    assert q is q_buf and ops.gemm_tc_take_error() == 0
    ref = (a[:M].double() @ w.double().T).cpu()

    def rotate(x):          # [M, heads, HS]
        c, s = ang[pos.long()].cos()[:, None, :], ang[pos.long()].sin()[:, None, :]
        x1, x2 = x[..., :HS // 2], x[..., HS // 2:]
        return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)

    q_ref = rotate(ref[:, :NH * HS].view(M, NH, HS)).reshape(M, NH * HS)
    assert rel_err(q[:M], q_ref) < 1e-2
    assert float(q_buf[M].float().min()) == 3.0 and float(q_buf[M].float().max()) == 3.0
    if NKV:
        k_ref = rotate(ref[:, NH * HS:(NH + NKV) * HS].view(M, NKV, HS))
        v_ref = ref[:, (NH + NKV) * HS:].view(M, NKV, HS)
        pg, off = (slot // page).long(), (slot % page).long()
        assert rel_err(kp.cpu()[pg, :, off], k_ref) < 1e-2
        assert rel_err(vp.cpu()[pg, :, off], v_ref) < 1e-2
        untouched = torch.ones(n_pages, page, dtype=torch.bool)
        untouched[pg, off] = False
        assert bool((kp.cpu().float().permute(0, 2, 1, 3)[untouched] == 7.0).all())
        assert bool((vp.cpu().float().permute(0, 2, 1, 3)[untouched] == 7.0).all())
    # without tables nothing is rotated
    q2 = ops.qkv_rope_store(a, w, lambda: q_buf, M, None, None, pos.to(DEV), slot.to(DEV), kp if NKV else None,
                            vp if NKV else None, NH, NKV, HS)
    assert rel_err(q2[:M], ref[:, :NH * HS]) < 1e-2


def test_qkv_epilogue_is_not_offered_for_few_rows_float32_or_other_head_sizes(ops):
    a = torch.zeros(300, 64, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(4 * 64, 64, device=DEV, dtype=torch.bfloat16)
    pos = torch.zeros(300, dtype=torch.int32, device=DEV)
    buf = lambda: torch.zeros(300, 4 * 64, device=DEV, dtype=torch.bfloat16)
    assert ops.qkv_rope_store(a, w, buf, 128, None, None, pos, pos, None, None, 4, 0, 64) is None
    assert ops.qkv_rope_store(a.float(), w.float(), buf, 300, None, None, pos, pos, None, None, 4, 0, 64) is None
    assert ops.qkv_rope_store(a, w, buf, 300, None, None, pos, pos, None, None, 8, 0, 32) is None
    assert ops.qkv_rope_store(a, w, buf, 300, None, None, pos, pos, None, None, 4, 0, 64) is not None
