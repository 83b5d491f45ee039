"""The tcgen05 matrix product alone, against a float64 product of the same bfloat16
numbers: all three forms (tokens on the 128-row side, with and without the fused
SwiGLU, and features on the 128-row side), sizes that are no multiples of any tile,
k cut into slices, and bias."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def randn(*shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).to(DEV)


def run(tokens, features, k, splits, with_bias, seed=0):
    from thintensor_b200.kernels import api

    x, w = randn(tokens, k, seed=seed), randn(features, k, seed=seed + 1)
    bias = torch.randn(features, device=DEV) if with_bias else None
    out = torch.full((splits, tokens, features), float("nan"), dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    api.gemm_tcgen05(x, w, bias, out, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait ran out"
    want = x.double() @ w.double().T + (bias.double() if with_bias else 0)
    got = out.double().sum(0)
    assert torch.isfinite(got).all()
    # float32 accumulation of exact bfloat16 products: the error grows like sqrt(k) * eps
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4 * k ** 0.5)


@pytest.mark.parametrize("tokens", [1, 8, 16, 17, 33, 64, 100, 128])
@pytest.mark.parametrize("features,k,splits", [(128, 64, 1), (311, 72, 1), (2048, 2048, 4), (200, 1000, 3), (128256 // 16, 256, 1)])
def test_features_on_m(tokens, features, k, splits):
    run(tokens, features, k, splits, with_bias=(tokens % 2 == 0))


@pytest.mark.parametrize("tokens", [129, 256, 300, 1000])
@pytest.mark.parametrize("features,k,splits", [(128, 64, 1), (311, 72, 1), (3072, 2048, 1), (200, 1000, 2), (2048, 8192, 4)])
def test_tokens_on_m(tokens, features, k, splits):
    run(tokens, features, k, splits, with_bias=(features % 2 == 1))


@pytest.mark.parametrize("tokens,features,k", [(2048, 3072, 2048), (1500, 2000, 1000), (3000, 1000, 136), (12345, 311, 72), (2048, 2048, 8192),
                                               (2500, 1100, 72), (6000, 2052, 200)])
def test_tokens_on_m_persistent(tokens, features, k):
    """Enough 128 x 256 tiles for the persistent kernel: tiles that hang over every edge,
    several tiles per CTA (two accumulators in turn), bias."""
    run(tokens, features, k, 1, with_bias=(k % 3 == 0), seed=7)


@pytest.mark.parametrize("tokens,features,k,splits", [
    (512, 2048, 2048, 4),        # 32 tiles x 4 slices of 8 k-blocks
    (512, 2048, 8192, 4),
    (1000, 2048, 4096, 4),       # 64 tiles x 4 = 256 work items: two per CTA, both accumulators
    (300, 2000, 2120, 4),        # 34 k-blocks in slices of 9, 9, 9, 7; the last block half empty; ragged edges
    (640, 520, 1096, 3),         # 18 k-blocks in slices of 6
    (200, 2048, 2368, 9),        # 37 k-blocks in 9 slices would leave the last one empty: the generic kernel writes its zeros
])
def test_tokens_on_m_persistent_sliced(tokens, features, k, splits):
    """The persistent kernel with k cut into slices: every slice in its own plane of the output,
    the bias in the first only."""
    run(tokens, features, k, splits, with_bias=(k % 3 != 0), seed=11)


@pytest.mark.parametrize("tokens,features,k", [
    (300, 2100, 320),            # persistent kernel, tiles hang over both edges, rows of 2100 floats (vector loads)
    (1500, 2000, 1000),          # persistent kernel, several tiles per CTA
    (700, 1001, 136),            # rows that are no multiple of four floats: element-wise loads and stores
    (2048, 2048, 2048),          # CTA pairs
    (2500, 530, 8192),           # CTA pairs, ragged, rows that tiled copies cannot write (530 floats): stores from registers
    (2500, 1100, 320),           # CTA pairs adding through tiled copies: the last pair half empty, the last box 12 columns wide
    (2300, 2052, 192),           # the same with a bias and one column box of 4
])
def test_product_added_into_its_output(tokens, features, k):
    """The accumulate form: out += x @ w.T (+ bias), every tile read and written once by its epilogue."""
    from thintensor_b200.kernels import api

    assert api.gemm_tcgen05_accumulates(tokens, features, k)
    x, w = randn(tokens, k, seed=21), randn(features, k, seed=22)
    bias = torch.randn(features, device=DEV) if k % 3 == 0 else None
    before = torch.randn(tokens, features, device=DEV) * 3.0
    out = before.clone().unsqueeze(0)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    api.gemm_tcgen05(x, w, bias, out, status, accumulate=True)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    plain = torch.empty(1, tokens, features, dtype=torch.float32, device=DEV)
    api.gemm_tcgen05(x, w, bias, plain, status)
    # the same accumulators plus the old value, in float32: bit for bit the sum of the two
    assert torch.equal(out[0], before + plain[0])
    want = before.double() + x.double() @ w.double().T + (bias.double() if bias is not None else 0)
    torch.testing.assert_close(out[0].double(), want, rtol=1e-4, atol=1e-4 * k ** 0.5)
    assert not api.gemm_tcgen05_accumulates(64, features, k) and not api.gemm_tcgen05_accumulates(512, 2048, 2048)   # few tokens; sliced k
    with pytest.raises(api.KernelError):
        api.gemm_tcgen05(x[:64], w, None, out[:, :64], status, accumulate=True)


@pytest.mark.parametrize("accumulate", [False, True])
def test_tiled_copies_of_the_output_stop_at_its_edges(accumulate):
    """The CTA pairs' plain form writes its tiles with tiled copies whose boxes hang over the last rows and columns:
    the output is a window of a larger matrix, and nothing around the window may change."""
    tokens, features, k = 2100, 1100, 136
    x, w = randn(tokens, k, seed=31), randn(features, k, seed=32)
    whole = torch.full((tokens + 40, features + 36), 7.0, dtype=torch.float32, device=DEV)    # rows of 1,136 floats: a multiple of four
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    from ctypes import c_int, c_longlong, c_void_p
    from thintensor_b200.kernels import build
    fn = build.load("gemm_tcgen05").tt_gemm_tcgen05
    fn.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                   c_void_p, c_longlong]
    fn.restype = c_int
    assert fn(x.data_ptr(), k, w.data_ptr(), k, None, whole.data_ptr(), whole.stride(0), 0, tokens, features, k, 1, 2 if accumulate else 0,
              status.data_ptr(), torch.cuda.current_stream().cuda_stream, None, 0) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = x.double() @ w.double().T + (7.0 if accumulate else 0.0)
    torch.testing.assert_close(whole[:tokens, :features].double(), want, rtol=1e-4, atol=1e-4 * k ** 0.5)
    assert bool((whole[tokens:] == 7.0).all()) and bool((whole[:, features:] == 7.0).all())


@pytest.mark.parametrize("tokens,features,k,accumulate", [
    (2560, 2048, 2048, False),   # 80 tiles for 74 pairs (two rounds, the second nearly empty): every pair a run of 34 or 35 of the 2,560 k-blocks
    (2560, 2048, 8192, True),    # the same with long k, added into the output
    (2560, 2050, 1024, False),   # rows of 2,050 floats: no tiled copies, so k is not dealt out and the shares are left alone
    (2500, 2052, 1024, True),    # 10 x 9 = 90 tiles of 16 k-blocks: runs of 19 or 20 k-blocks over two or three tiles; ragged edges and a bias
    (2100, 1100, 3072, False),   # 9 x 5 = 45 tiles: runs of 29 of a tile's 48 k-blocks, tiles shared by two or three pairs
    (2048, 2048, 2048, False),   # 64 tiles fill most of one round: whole tiles, the shares are left alone
])
def test_k_dealt_out_among_the_cta_pairs(tokens, features, k, accumulate):
    """With scratch memory for shares the CTA pairs' plain form deals the tiles' k-blocks out evenly where whole tiles
    would leave pairs idle: the same product, the flags zero again afterwards, and the same bits from call to call
    (the shares are added in a fixed order)."""
    from thintensor_b200.kernels import api

    x, w = randn(tokens, k, seed=41), randn(features, k, seed=42)
    bias = torch.randn(features, device=DEV) if features % 3 == 0 else None
    shares = torch.zeros(api.gemm_tcgen05_shares_words(), dtype=torch.int32, device=DEV)
    flags = shares[-(shares.numel() // (32 * 256 + 1)):]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    before = torch.randn(tokens, features, device=DEV) if accumulate else None
    results = []
    for _ in range(3):
        out = before.clone().unsqueeze(0) if accumulate else torch.full((1, tokens, features), float("nan"), dtype=torch.float32, device=DEV)
        api.gemm_tcgen05(x, w, bias, out, status, accumulate=accumulate, shares=shares)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert int(flags.abs().sum().item()) == 0, "a flag was left set"
        results.append(out)
    assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2])
    want = x.double() @ w.double().T + (bias.double() if bias is not None else 0) + (before.double() if accumulate else 0)
    assert torch.isfinite(results[0]).all()
    torch.testing.assert_close(results[0][0].double(), want, rtol=1e-4, atol=1e-4 * k ** 0.5)
    if features % 4 == 0 and tokens != 2048:
        assert int(shares[:-flags.numel()].abs().sum().item()) != 0, "k was not dealt out"
    else:
        assert int(shares.abs().sum().item()) == 0


def test_split_policy_and_refusals():
    from thintensor_b200.kernels import api

    assert api.gemm_tcgen05_splits(8, 2048, 2048) == 8          # 16 tiles, 32 k-blocks: four blocks per slice
    assert api.gemm_tcgen05_splits(8, 2048, 8192) == 16
    assert api.gemm_tcgen05_splits(8, 128256, 2048) == 1
    assert api.gemm_tcgen05_splits(2048, 3072, 2048) == 1
    assert api.gemm_tcgen05_splits(300, 2048, 8192) == 6        # 3 x 8 tiles of 128 x 256: the persistent kernel, 144 work items
    assert api.gemm_tcgen05_splits(256, 2048, 8192) == 4        # 2 x 16 tiles of 128 x 128 (the 16 of 256 are too few): 128 work items
    assert api.gemm_tcgen05_splits(512, 2048, 2048) == 4        # 32 tiles of 128 x 256, 32 k-blocks
    assert api.gemm_tcgen05_splits(1024, 3072, 2048) == 1       # 96 tiles: one round of the SMs already
    assert api.gemm_tcgen05_splits(4096, 256, 8192) == 1        # CTA pairs do not slice
    assert api.gemm_tcgen05_splits(300, 200, 4096) > 1          # too few tiles for it
    x, w = randn(4, 70, seed=1), randn(32, 70, seed=2)             # k = 70 is no multiple of 8
    assert not api.gemm_tcgen05_usable(x, w)
    with pytest.raises(api.KernelError):
        api.gemm_tcgen05(x, w, None, torch.empty(1, 4, 32, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("tokens,inter,k", [(129, 128, 64), (300, 200, 72), (2048, 1024, 512), (257, 8192, 2048), (5000, 1100, 200), (2048, 8192, 2048),
                                            # rows that tiled copies can write, edges inside a box of 64 features x 32 tokens: CTA pairs, one CTA
                                            (5000, 1096, 200), (400, 1064, 136),
                                            # few tokens: features on the 128-row side, gate rows paired with up rows in one tile
                                            (1, 64, 64), (8, 8192, 2048), (3, 100, 72), (16, 1000, 520), (17, 328, 200), (40, 72, 2048),
                                            (64, 14336, 4096), (65, 130, 136), (128, 1100, 512)])
def test_fused_swiglu(tokens, inter, k):
    from thintensor_b200.kernels import api

    x = randn(tokens, k, seed=5)
    w = randn(2 * inter, k, seed=6, scale=0.1)
    act = torch.full((tokens, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    api.gemm_tcgen05_swiglu(x, w, act, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    y = x.double() @ w.double().T
    g, u = y[:, :inter], y[:, inter:]
    want = g / (1 + torch.exp(-g)) * u
    torch.testing.assert_close(act.double(), want, rtol=2e-2, atol=2e-2)


def test_linear_uses_it_and_matches_exact_kernel():
    """The projection helper takes the tensor-core kernel for bfloat16 and agrees with
    the exact FMA kernel on the same operands."""
    from thintensor_b200.engine.context import StepContext, Workspace
    from thintensor_b200.kernels import api
    from thintensor_b200.parts.linear import Linear

    ws = Workspace(torch.device(DEV))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    empty = torch.zeros(1, dtype=torch.int32, device=DEV)
    ctx = StepContext(n_tokens=40, sequences=1, decode=False, max_new=40, max_total=40, tokens=empty, cu=empty, len_before=empty,
                      slots=empty, tables=[], act_dtype=torch.bfloat16, workspace=ws, status=status)
    x, w = randn(40, 2048, seed=8), randn(512, 2048, seed=9, scale=0.05)
    before = api.launch_count()
    got = Linear(w)(ctx, x, "t").sum(0)
    exact = torch.empty(1, 40, 512, device=DEV)
    api.gemm_simt(x, w, None, exact)
    torch.testing.assert_close(got, exact[0], rtol=1e-4, atol=1e-3)
    assert api.launch_count() - before == 2


@pytest.mark.parametrize("heads,kv_heads,head_dim,k,news,before", [
    (32, 8, 64, 2048, [2048], [0]),                       # CTA pairs, the 1B shape
    (8, 2, 64, 512, [700, 1, 1400], [0, 130, 64]),        # persistent kernel below the pairs' range is not taken (few tiles) ...
    (24, 8, 128, 1024, [1000, 1200], [5, 0]),             # ... but 2,200 tokens are: head size 128, two sequences, one with a cached prefix
    (4, 2, 64, 256, [2300], [77]),                        # a tile that holds q heads, k heads and v heads side by side
    (32, 8, 128, 4096, [1900], [0]),                      # the persistent kernel with at least as many tiles as SMs (8B shape)
    (32, 8, 64, 2048, [1100], [3]),                       # the persistent kernel with fewer tiles than SMs but more than half (108)
    (32, 8, 64, 2048, [700], [0]),                        # 72 tiles of 256 features are too few, 144 of 128 are not: the narrow tiles
    (8, 2, 128, 512, [900], [10]),                        # narrow tiles at head size 128: one head per tile
    (32, 8, 64, 2048, [300], [0]),                        # 3 x 24 tiles of 128: fewer than half the SMs, the separate kernels serve it
])
def test_qkv_product_rotates_and_appends_in_its_epilogue(heads, kv_heads, head_dim, k, news, before):
    """The qkv form of the prompt kernels against the separate path (product to float32, then the rotary/append
    kernel) and against plain float64 arithmetic: rotated q, rotated k in the cache at every token's position,
    v transposed inside its block; sequences packed back to back, some behind a cached prefix, blocks scattered."""
    import math

    from thintensor_b200.kernels import api

    tokens = sum(news)
    q_cols, kv_cols = heads * head_dim, kv_heads * head_dim
    x = randn(tokens, k, seed=31, scale=0.5)
    w = randn(q_cols + 2 * kv_cols, k, seed=32, scale=0.05)
    bias = torch.randn(q_cols + 2 * kv_cols, device=DEV) * 0.3 if head_dim == 128 else None
    if not api.gemm_tcgen05_qkv_rope_takes(x, w, head_dim, head_dim):
        assert tokens < 2048 and 2 * (-(-tokens // 128) * -(-(q_cols + 2 * kv_cols) // 128)) <= api.sm_count()
        pytest.skip("few tiles below the pairs' range: the separate kernels serve this shape")
    inv_freq = (10000.0 ** (-torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim)).to(DEV)
    totals = [b + n for b, n in zip(before, news)]
    blocks_per = [-(-t // 64) for t in totals]
    g = torch.Generator().manual_seed(33)
    order = torch.randperm(sum(blocks_per) + 2, generator=g).tolist()
    table = torch.full((len(news), max(blocks_per)), -1, dtype=torch.int32)
    at = 0
    for b, count in enumerate(blocks_per):
        for j in range(count):
            table[b, j] = order[at]
            at += 1
    table = table.to(DEV)
    pool_blocks = sum(blocks_per) + 2
    cu = torch.tensor([0] + torch.tensor(news).cumsum(0).tolist(), dtype=torch.int32, device=DEV)
    len_before = torch.tensor(before, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scaling = 0.75

    def pools():
        return (torch.zeros(pool_blocks, kv_heads, 64, head_dim, dtype=torch.bfloat16, device=DEV),
                torch.zeros(pool_blocks, kv_heads, head_dim, 64, dtype=torch.bfloat16, device=DEV))

    # the separate kernels
    product = torch.empty(1, tokens, q_cols + 2 * kv_cols, dtype=torch.float32, device=DEV)
    api.gemm_tcgen05(x, w, bias, product, status)
    q_want = torch.empty(tokens, q_cols, dtype=torch.bfloat16, device=DEV)
    k_want, v_want = pools()
    api.rope_append(product, inv_freq, head_dim, scaling, q_want, k_want, v_want, table, cu, len_before, len(news), tokens, heads, kv_heads, head_dim, status)
    # the fused form
    cos_sin = torch.empty(tokens, head_dim // 2, 2, dtype=torch.float32, device=DEV)
    where = torch.empty(tokens, 2, dtype=torch.int32, device=DEV)
    api.rope_table(inv_freq, head_dim, cu, len_before, len(news), tokens, cos_sin, where)
    q_got = torch.full((tokens, q_cols), float("nan"), dtype=torch.bfloat16, device=DEV)
    k_got, v_got = pools()
    api.gemm_tcgen05_qkv_rope(x, w, bias, q_got, k_got, v_got, cos_sin, where, table, heads, kv_heads, head_dim, scaling, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    positions = torch.cat([torch.arange(b, b + n) for b, n in zip(before, news)])
    assert torch.equal(where[:, 0].cpu(), positions.to(torch.int32))
    tolerance = dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(q_got.float(), q_want.float(), **tolerance)
    torch.testing.assert_close(k_got.float(), k_want.float(), **tolerance)
    torch.testing.assert_close(v_got.float(), v_want.float(), **tolerance)
    # and the formula itself at a few tokens, float64
    full = x.double().cpu() @ w.double().cpu().T + (bias.double().cpu() if bias is not None else 0)
    for t in (0, tokens // 2, tokens - 1):
        pos = int(positions[t])
        angle = inv_freq.double().cpu() * pos
        cos, sin = angle.cos() * scaling, angle.sin() * scaling
        head = full[t, :head_dim]
        a, b = head[: head_dim // 2], head[head_dim // 2:]
        want = torch.cat([a * cos - b * sin, b * cos + a * sin])
        torch.testing.assert_close(q_got[t, :head_dim].double().cpu(), want, rtol=3e-2, atol=3e-2)
        sequence = next(i for i in range(len(news)) if t < int(cu[i + 1]))
        block = int(table[sequence, pos // 64])
        vrow = full[t, q_cols + kv_cols: q_cols + kv_cols + head_dim]
        torch.testing.assert_close(v_got[block, 0, :, pos % 64].double().cpu(), vrow, rtol=3e-2, atol=3e-2)
