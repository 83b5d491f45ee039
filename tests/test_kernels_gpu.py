"""Each CUDA kernel alone against a plain float64 PyTorch statement of the same
operation, at sizes other than the engine tests' (odd widths, head sizes from 16 to 256,
groups of 1 to 8 heads, vocabularies that are no power of two), in float32 and bfloat16."""
from __future__ import annotations

import math

import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu

DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def randn(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# ------------------------------------------------------------------------------ embedding
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_gather(dtype):
    from thintensor_b200.kernels import api

    table = randn(311, 72, dtype=dtype, seed=1)
    tokens = torch.tensor([0, 310, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, dtype=torch.float32, device=DEV)
    st = status()
    api.embed_gather(table, tokens, out, 1.5, st)
    torch.testing.assert_close(out, table[tokens.long()].float() * 1.5, rtol=0, atol=0)
    assert int(st.item()) == 0
    bad = torch.tensor([3, 311], dtype=torch.int32, device=DEV)
    api.embed_gather(table, bad, out[:2], 1.0, st)
    assert int(st.item()) & api.STATUS_BAD_TOKEN


# ----------------------------------------------------------------------------------- norm
@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("hidden,splits,rows", [(72, 0, 7), (1000, 1, 7), (1002, 5, 7), (2048, 3, 7), (2048, 16, 7), (12000, 2, 7), (20000, 1, 7),
                                                # many rows: the launch with several pieces of a row per thread
                                                (2048, 1, 1100), (4096, 2, 1030), (1000, 1, 1500), (8192, 1, 1024)])
def test_add_rmsnorm(out_dtype, hidden, splits, rows):
    from thintensor_b200.kernels import api

    residual = randn(rows, hidden, seed=2)
    delta = randn(max(splits, 1), rows, hidden, seed=3) if splits else None
    weight = 1.0 + 0.1 * randn(hidden, seed=4)
    eps = 3e-6
    out = torch.empty(rows, hidden, dtype=out_dtype, device=DEV)
    x = residual.double() + (delta.double().sum(0) if splits else 0)
    want = plain_llama.rms_norm(x, weight.double(), eps)
    before = residual.clone()
    api.add_rmsnorm(residual, delta, weight, eps, out)
    torch.testing.assert_close(out.double(), want, **tol(out_dtype))
    # float32 summation of splits + 1 numbers of order one
    torch.testing.assert_close(residual.double(), x, rtol=1e-6, atol=5e-7 * (splits + 1))
    # gather form: chosen rows, residual left alone
    pick = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    residual2 = before.clone()
    out2 = torch.empty(3, hidden, dtype=out_dtype, device=DEV)
    api.add_rmsnorm(residual2, delta, weight, eps, out2, rows=pick)
    torch.testing.assert_close(out2.double(), want[pick.long()], **tol(out_dtype))
    assert torch.equal(residual2, before)


# ------------------------------------------------------------------------ cache helpers
def make_cache(sequences_len, kv_heads, head_dim, dtype, seed, extra_blocks=3):
    """A block pool holding random keys/values for sequences of the given lengths, with
    the blocks of each sequence scattered over the pool in a shuffled order."""
    blocks_per = [-(-n // 64) for n in sequences_len]
    total = sum(blocks_per) + extra_blocks
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(total, generator=g).tolist()
    width = max(blocks_per)
    table = torch.full((len(sequences_len), width), -1, dtype=torch.int32)
    k_pool = torch.zeros(total, kv_heads, 64, head_dim)
    v_pool = torch.zeros(total, kv_heads, head_dim, 64)          # values lie transposed inside a block
    keys, values = [], []
    at = 0
    for b, n in enumerate(sequences_len):
        k = torch.randn(n, kv_heads, head_dim, generator=g).to(dtype).float()
        v = torch.randn(n, kv_heads, head_dim, generator=g).to(dtype).float()
        keys.append(k)
        values.append(v)
        for j in range(blocks_per[b]):
            block = order[at]
            at += 1
            table[b, j] = block
            chunk = slice(j * 64, min(n, (j + 1) * 64))
            k_pool[block, :, : chunk.stop - chunk.start] = k[chunk].transpose(0, 1)
            v_pool[block, :, :, : chunk.stop - chunk.start] = v[chunk].permute(1, 2, 0)
    return k_pool.to(dtype).to(DEV), v_pool.to(dtype).to(DEV), table.to(DEV), keys, values


def attention_reference(q, keys, values, new_lens, heads, kv_heads, scale, window):
    """q: [tokens, heads, d] packed; sequence b's last new_lens[b] cached positions are
    the queries' positions.  float64, one (token, head) at a time."""
    group = heads // kv_heads
    out = torch.zeros(q.shape, dtype=torch.float64)
    t = 0
    for b, new in enumerate(new_lens):
        k, v = keys[b].double(), values[b].double()
        total = k.shape[0]
        for i in range(new):
            pos = total - new + i
            first = max(0, pos - window + 1) if window else 0
            for h in range(heads):
                kh = h // group
                s = (k[first: pos + 1, kh] @ q[t, h].double()) * scale
                p = torch.softmax(s, dim=0)
                out[t, h] = p @ v[first: pos + 1, kh]
            t += 1
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim", [(4, 4, 16), (6, 2, 48), (8, 1, 64), (5, 5, 80), (8, 2, 128), (3, 1, 256)])
def test_attention_prompts_with_cached_prefix(dtype, heads, kv_heads, head_dim):
    """Packed prompts of unequal length, some continuing a cached prefix."""
    from thintensor_b200.kernels import api

    totals, news = [70, 5, 130, 64], [70, 2, 9, 1]
    k_pool, v_pool, table, keys, values = make_cache(totals, kv_heads, head_dim, dtype, seed=10)
    tokens = sum(news)
    q = randn(tokens, heads, head_dim, dtype=dtype, seed=11)
    cu = torch.tensor([0] + list(torch.tensor(news).cumsum(0)), dtype=torch.int32, device=DEV)
    before = torch.tensor([t - n for t, n in zip(totals, news)], dtype=torch.int32, device=DEV)
    out = torch.empty(tokens, heads * head_dim, dtype=dtype, device=DEV)
    st = status()
    scale = head_dim ** -0.5
    api.attention(q.view(tokens, -1), k_pool, v_pool, table, cu, before, len(totals), tokens, heads, kv_heads, head_dim, scale, 0, 1,
                  out, None, None, st)
    want = attention_reference(q.float().cpu(), keys, values, news, heads, kv_heads, scale, 0)
    torch.testing.assert_close(out.double().cpu().view(tokens, heads, head_dim), want, **tol(dtype))
    assert int(st.item()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("splits", [1, 2, 5, 16])
@pytest.mark.parametrize("window", [0, 100])
def test_attention_decode_splits_and_window(dtype, splits, window):
    """One query per sequence over caches of very different lengths, keys cut into
    slices, with and without a window.  One far key of the longest sequence is made to
    dominate its scores, so a slice that is skipped or a window edge that is off by one
    changes the output outright."""
    from thintensor_b200.kernels import api

    heads, kv_heads, head_dim = 8, 2, 64
    totals = [700, 1, 65, 300]
    k_pool, v_pool, table, keys, values = make_cache(totals, kv_heads, head_dim, dtype, seed=20)
    q = randn(len(totals), heads, head_dim, dtype=dtype, seed=21)
    # the dominating key: position 3 without a window, the window's oldest position with one
    far = 3 if not window else totals[0] - window
    q0 = q[0, 0].float()
    spike = (q0 * 3.0).to(dtype)     # score about 3 |q|^2 / sqrt(d) = 24, the others are of order one
    block, offset = int(table[0, far // 64]), far % 64
    k_pool[block, 0, offset] = spike
    keys[0][far, 0] = spike.float().cpu()
    cu = torch.arange(len(totals) + 1, dtype=torch.int32, device=DEV)
    before = torch.tensor([t - 1 for t in totals], dtype=torch.int32, device=DEV)
    out = torch.empty(len(totals), heads * head_dim, dtype=dtype, device=DEV)
    rows = len(totals) * heads
    part_acc = torch.empty(rows * splits * head_dim, dtype=torch.float32, device=DEV)
    part_ml = torch.empty(rows * splits * 2, dtype=torch.float32, device=DEV)
    st = status()
    scale = head_dim ** -0.5
    api.attention(q.view(len(totals), -1), k_pool, v_pool, table, cu, before, len(totals), len(totals), heads, kv_heads, head_dim,
                  scale, window, splits, out, part_acc, part_ml, st)
    want = attention_reference(q.float().cpu(), keys, values, [1] * len(totals), heads, kv_heads, scale, window)
    torch.testing.assert_close(out.double().cpu().view(len(totals), heads, head_dim), want, **tol(dtype))
    # the spike really dominates head 0 of sequence 0
    assert torch.allclose(want[0, 0], values[0][far, 0].double(), atol=0.35)
    assert int(st.item()) == 0


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(8, 2, 64), (4, 4, 32), (6, 2, 96), (16, 1, 128), (5, 1, 64), (32, 8, 64), (12, 2, 128)])
def test_attention_mma_prompts_with_cached_prefix(heads, kv_heads, head_dim):
    """The tensor-core kernel on packed prompts of unequal length (tiles that end inside a
    sequence, groups that do not divide 16, a cached prefix)."""
    from thintensor_b200.kernels import api

    dtype = torch.bfloat16
    totals, news = [70, 5, 200, 64, 130], [70, 2, 9, 1, 130]
    k_pool, v_pool, table, keys, values = make_cache(totals, kv_heads, head_dim, dtype, seed=12)
    tokens = sum(news)
    q = randn(tokens, heads, head_dim, dtype=dtype, seed=13)
    cu = torch.tensor([0] + list(torch.tensor(news).cumsum(0)), dtype=torch.int32, device=DEV)
    before = torch.tensor([t - n for t, n in zip(totals, news)], dtype=torch.int32, device=DEV)
    out = torch.full((tokens, heads * head_dim), float("nan"), dtype=dtype, device=DEV)
    st = status()
    scale = head_dim ** -0.5
    api.attention_mma(q.view(tokens, -1), k_pool, v_pool, table, cu, before, len(totals), tokens, heads, kv_heads, head_dim, scale, 0, 1,
                      out, None, None, st)
    want = attention_reference(q.float().cpu(), keys, values, news, heads, kv_heads, scale, 0)
    torch.testing.assert_close(out.double().cpu().view(tokens, heads, head_dim), want, **tol(dtype))
    assert int(st.item()) == 0


@pytest.mark.parametrize("window", [0, 90])
@pytest.mark.parametrize("heads,kv_heads,head_dim", [(8, 2, 64), (32, 8, 64), (4, 4, 64), (24, 8, 128), (32, 8, 128), (5, 1, 64), (16, 1, 128)])
def test_attention_tcgen05_prompts(heads, kv_heads, head_dim, window):
    """The tcgen05 prompt kernel: packed prompts of unequal length with cached prefixes, tiles
    that end inside a sequence, groups that do not divide 128, many blocks per tile (both S
    accumulators and all stages in turn), a window, and a far key that dominates one row."""
    from thintensor_b200.kernels import api

    dtype = torch.bfloat16
    totals, news = [700, 5, 200, 64, 130, 333], [700, 2, 9, 1, 130, 300]
    k_pool, v_pool, table, keys, values = make_cache(totals, kv_heads, head_dim, dtype, seed=14)
    tokens = sum(news)
    q = randn(tokens, heads, head_dim, dtype=dtype, seed=15)
    # the last token of the first sequence, head 0: one far key dominates (inside the window when there is one)
    far = 5 if not window else totals[0] - window
    q_last = q[news[0] - 1, 0].float()
    spike = (q_last * (24.0 * head_dim ** 0.5 / float(q_last.norm()) ** 2)).to(dtype)
    block, offset = int(table[0, far // 64]), far % 64
    k_pool[block, 0, offset] = spike
    keys[0][far, 0] = spike.float().cpu()
    cu = torch.tensor([0] + list(torch.tensor(news).cumsum(0)), dtype=torch.int32, device=DEV)
    before = torch.tensor([t - n for t, n in zip(totals, news)], dtype=torch.int32, device=DEV)
    out = torch.full((tokens, heads * head_dim), float("nan"), dtype=dtype, device=DEV)
    st = status()
    scale = head_dim ** -0.5
    api.attention_tcgen05(q.view(tokens, -1), k_pool, v_pool, table, cu, before, len(totals), tokens, heads, kv_heads, head_dim, scale,
                          window, out, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    want = attention_reference(q.float().cpu(), keys, values, news, heads, kv_heads, scale, window)
    got = out.double().cpu().view(tokens, heads, head_dim)
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, want, **tol(dtype))
    assert torch.allclose(want[news[0] - 1, 0], values[0][far, 0].double(), atol=0.35)


@pytest.mark.parametrize("shared_tile", [False, True])
@pytest.mark.parametrize("splits", [1, 2, 5, 16])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("heads,kv_heads,head_dim", [(8, 2, 64), (3, 1, 128), (5, 1, 96), (4, 4, 32), (16, 1, 64), (24, 2, 128), (9, 1, 32)])
def test_attention_mma_decode_splits_and_window(splits, window, heads, kv_heads, head_dim, shared_tile):
    """The tensor-core kernels with one token per sequence, through the decode kernel (keys may
    be sliced) and through the prompt kernel: the same far-key construction as for the exact kernel."""
    from thintensor_b200.kernels import api

    if not shared_tile and splits > 1:
        pytest.skip("the prompt kernel does not slice keys")

    dtype = torch.bfloat16
    totals = [700, 1, 65, 300]
    k_pool, v_pool, table, keys, values = make_cache(totals, kv_heads, head_dim, dtype, seed=20)
    q = randn(len(totals), heads, head_dim, dtype=dtype, seed=21)
    far = 3 if not window else totals[0] - window
    spike = (q[0, 0].float() * (24.0 * head_dim ** 0.5 / float(q[0, 0].float().norm()) ** 2)).to(dtype)
    block, offset = int(table[0, far // 64]), far % 64
    k_pool[block, 0, offset] = spike
    keys[0][far, 0] = spike.float().cpu()
    cu = torch.arange(len(totals) + 1, dtype=torch.int32, device=DEV)
    before = torch.tensor([t - 1 for t in totals], dtype=torch.int32, device=DEV)
    out = torch.full((len(totals), heads * head_dim), float("nan"), dtype=dtype, device=DEV)
    rows = len(totals) * heads
    part_acc = torch.full((rows * splits * head_dim,), float("nan"), dtype=torch.float32, device=DEV)
    part_ml = torch.full((rows * splits * 2,), float("nan"), dtype=torch.float32, device=DEV)
    st = status()
    scale = head_dim ** -0.5
    api.attention_mma(q.view(len(totals), -1), k_pool, v_pool, table, cu, before, len(totals), len(totals), heads, kv_heads, head_dim,
                      scale, window, splits, out, part_acc, part_ml, st, one_token_each=shared_tile)
    want = attention_reference(q.float().cpu(), keys, values, [1] * len(totals), heads, kv_heads, scale, window)
    torch.testing.assert_close(out.double().cpu().view(len(totals), heads, head_dim), want, **tol(dtype))
    assert torch.allclose(want[0, 0], values[0][far, 0].double(), atol=0.35)
    assert int(st.item()) == 0
    if shared_tile and splits > 8:
        # more slices than a cluster holds: with tickets the last CTA of a (sequence, kv head) combines them itself
        # (one launch instead of two), twice in a row because the tickets have to be back at zero for the next call
        tickets = torch.zeros(len(totals) * kv_heads, dtype=torch.int32, device=DEV)
        for _ in range(2):
            again = torch.full_like(out, float("nan"))
            launches = api.launch_count()
            api.attention_mma(q.view(len(totals), -1), k_pool, v_pool, table, cu, before, len(totals), len(totals), heads, kv_heads, head_dim,
                              scale, window, splits, again, part_acc, part_ml, st, one_token_each=True, tickets=tickets)
            assert api.launch_count() - launches == 1
            torch.testing.assert_close(again.double().cpu().view(len(totals), heads, head_dim), want, **tol(dtype))
            assert int(tickets.abs().sum().item()) == 0 and int(st.item()) == 0


@pytest.mark.parametrize("splits", [1, 2, 3])
def test_attention_mma_decode_many_sequences(splits):
    """More CTAs than SMs: head size 64 then runs the variants with fewer warps and two CTAs per SM
    (200 and 600 CTAs) or three (400 CTAs)."""
    from thintensor_b200.kernels import api

    dtype, heads, kv_heads, head_dim = torch.bfloat16, 8, 4, 64
    g = torch.Generator().manual_seed(50)
    totals = [int(v) for v in torch.randint(1, 400, (50,), generator=g)]
    totals[7], totals[8], totals[9] = 64, 65, 128
    n = len(totals)
    k_pool, v_pool, table, keys, values = make_cache(totals, kv_heads, head_dim, dtype, seed=51)
    q = randn(n, heads, head_dim, dtype=dtype, seed=52)
    cu = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    before = torch.tensor([t - 1 for t in totals], dtype=torch.int32, device=DEV)
    out = torch.full((n, heads * head_dim), float("nan"), dtype=dtype, device=DEV)
    part_acc = torch.full((n * heads * splits * head_dim,), float("nan"), dtype=torch.float32, device=DEV)
    part_ml = torch.full((n * heads * splits * 2,), float("nan"), dtype=torch.float32, device=DEV)
    st = status()
    scale = head_dim ** -0.5
    assert n * kv_heads * splits > api.sm_count()
    api.attention_mma(q.view(n, -1), k_pool, v_pool, table, cu, before, n, n, heads, kv_heads, head_dim, scale, 0, splits, out,
                      part_acc, part_ml, st, one_token_each=True)
    want = attention_reference(q.float().cpu(), keys, values, [1] * n, heads, kv_heads, scale, 0)
    torch.testing.assert_close(out.double().cpu().view(n, heads, head_dim), want, **tol(dtype))
    assert int(st.item()) == 0


@pytest.mark.parametrize("window", [0, 200])
@pytest.mark.parametrize("splits", [1, 2, 4])
@pytest.mark.parametrize("sequences,heads,kv_heads,head_dim", [(120, 8, 4, 64), (80, 6, 2, 128), (150, 20, 2, 96), (40, 4, 4, 32)])
def test_attention_mma_decode_in_several_rounds(sequences, heads, kv_heads, head_dim, splits, window):
    """More (sequence, kv head, slice) CTAs than fit at once, at every head size: the grid runs in several rounds (at head
    size 64 with the smaller CTAs, two to an SM).  Lengths from one token to 1,500 (so that slices have no block for some
    warps, one block, or several rounds of the ring), sequences that end on a block's last and first slot, and in one
    sequence a far key made to dominate."""
    from thintensor_b200.kernels import api

    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(60 + head_dim)
    totals = [int(v) for v in torch.randint(1, 1500, (sequences,), generator=g)]
    totals[0], totals[1], totals[2], totals[3], totals[-1] = 1400, 1, 64, 65, 1281
    n = len(totals)
    assert n * kv_heads * splits > (3 if head_dim == 64 else 1) * api.sm_count()
    k_pool, v_pool, table, keys, values = make_cache(totals, kv_heads, head_dim, dtype, seed=61)
    q = randn(n, heads, head_dim, dtype=dtype, seed=62)
    far = 5 if not window else totals[0] - window
    spike = (q[0, 0].float() * (24.0 * head_dim ** 0.5 / float(q[0, 0].float().norm()) ** 2)).to(dtype)
    block, offset = int(table[0, far // 64]), far % 64
    k_pool[block, 0, offset] = spike
    keys[0][far, 0] = spike.float().cpu()
    cu = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    before = torch.tensor([t - 1 for t in totals], dtype=torch.int32, device=DEV)
    part_acc = torch.full((n * heads * splits * head_dim,), float("nan"), dtype=torch.float32, device=DEV)
    part_ml = torch.full((n * heads * splits * 2,), float("nan"), dtype=torch.float32, device=DEV)
    st = status()
    scale = head_dim ** -0.5
    want = attention_reference(q.float().cpu(), keys, values, [1] * n, heads, kv_heads, scale, window)
    for _ in range(2):
        out = torch.full((n, heads * head_dim), float("nan"), dtype=dtype, device=DEV)
        api.attention_mma(q.view(n, -1), k_pool, v_pool, table, cu, before, n, n, heads, kv_heads, head_dim, scale, window, splits, out,
                          part_acc, part_ml, st, one_token_each=True)
        torch.testing.assert_close(out.double().cpu().view(n, heads, head_dim), want, **tol(dtype))
        assert int(st.item()) == 0
    assert torch.allclose(want[0, 0], values[0][far, 0].double(), atol=0.35)


@pytest.mark.parametrize("write_cache", [True, False])
@pytest.mark.parametrize("splits", [1, 3, 16])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("heads,kv_heads,head_dim", [(8, 2, 64), (3, 1, 64), (32, 8, 64), (10, 5, 64), (16, 1, 64)])
def test_attention_decode_with_rotation_and_cache_write(splits, window, heads, kv_heads, head_dim, write_cache):
    """Decoding straight from the slices of the qkv product: the kernel rotates q and k, writes
    k and v at each sequence's position (first slot of a block, last slot, the middle) and
    attends.  The cache holds garbage at those positions beforehand, and the new key of one
    sequence is made to dominate, so a key that is written late or not at all shows."""
    from thintensor_b200.kernels import api

    dtype = torch.bfloat16
    totals = [700, 1, 65, 300, 128]
    n = len(totals)
    k_pool, v_pool, table, keys, values = make_cache(totals, kv_heads, head_dim, dtype, seed=40)
    cols = (heads + (2 * kv_heads if write_cache else 0)) * head_dim
    slices = 3
    qkv = randn(slices, n, cols, seed=41, scale=3 ** -0.5)
    inv_freq = plain_llama.rope_inv_freq(head_dim, 10000.0, None).to(DEV)
    x = qkv.double().sum(0).cpu()
    positions = torch.tensor([t - 1 for t in totals])
    cos, sin = plain_llama.rope_cos_sin(inv_freq.cpu(), positions, torch.float64)
    scaling = 1.25
    q = plain_llama.apply_rope(x[:, : heads * head_dim].view(n, heads, head_dim), cos, sin) * scaling
    if write_cache:
        group = heads // kv_heads
        # sequence 3: the new key is the direction of head 0's query, long enough to take all the weight
        q3 = x[3, :head_dim]
        boost = (q3 * (30.0 * head_dim ** 0.5 / float(q3.norm()) ** 2 / scaling ** 2)).float().to(DEV)
        qkv[:, 3, heads * head_dim: heads * head_dim + head_dim] = boost / slices
        x = qkv.double().sum(0).cpu()
        k_new = plain_llama.apply_rope(x[:, heads * head_dim: (heads + kv_heads) * head_dim].view(n, kv_heads, head_dim), cos, sin) * scaling
        v_new = x[:, (heads + kv_heads) * head_dim:].view(n, kv_heads, head_dim)
        table_cpu = table.cpu()
        for b, total in enumerate(totals):
            keys[b][total - 1] = k_new[b].to(dtype).float()
            values[b][total - 1] = v_new[b].to(dtype).float()
            block, off = int(table_cpu[b, (total - 1) // 64]), (total - 1) % 64
            k_pool[block, :, off] = 77.0
            v_pool[block, :, :, off] = -55.0
    before = torch.tensor([t - 1 for t in totals], dtype=torch.int32, device=DEV)
    out = torch.full((n, heads * head_dim), float("nan"), dtype=dtype, device=DEV)
    rows = n * heads
    part_acc = torch.full((rows * splits * head_dim,), float("nan"), dtype=torch.float32, device=DEV)
    part_ml = torch.full((rows * splits * 2,), float("nan"), dtype=torch.float32, device=DEV)
    st = status()
    scale = head_dim ** -0.5
    tickets = torch.zeros(n * kv_heads, dtype=torch.int32, device=DEV) if splits > 8 and heads % 2 == 0 else None     # both ways of combining many slices
    api.attention_decode_rope(qkv, inv_freq, head_dim, scaling, write_cache, k_pool, v_pool, table, before, n, heads, kv_heads, head_dim,
                              scale, window, splits, out, part_acc, part_ml, st, tickets=tickets)
    assert int(st.item()) == 0 and (tickets is None or int(tickets.abs().sum().item()) == 0)
    want = attention_reference(q.to(dtype).float(), keys, values, [1] * n, heads, kv_heads, scale, window)
    torch.testing.assert_close(out.double().cpu().view(n, heads, head_dim), want, **tol(dtype))
    if write_cache:
        assert torch.allclose(want[3, 0], values[3][totals[3] - 1, 0].double(), atol=0.35)
        for b, total in enumerate(totals):
            block, off = int(table_cpu[b, (total - 1) // 64]), (total - 1) % 64
            torch.testing.assert_close(k_pool[block, :, off].float().cpu(), keys[b][total - 1], rtol=0, atol=2 ** -7 * float(keys[b][total - 1].abs().max()))
            torch.testing.assert_close(v_pool[block, :, :, off].float().cpu(), values[b][total - 1], rtol=0, atol=2 ** -7 * float(values[b][total - 1].abs().max()))


def test_attention_refuses_bad_sizes():
    from thintensor_b200.kernels import api

    with pytest.raises(api.KernelError):
        api.check_head_dim(24)
    with pytest.raises(api.KernelError):
        api.check_head_dim(272)
    assert not api.attention_mma_supports(torch.bfloat16, 4, 2, 48) and not api.attention_mma_supports(torch.float32, 4, 2, 64)
    assert not api.attention_mma_supports(torch.bfloat16, 34, 2, 64) and api.attention_mma_supports(torch.bfloat16, 32, 8, 64)


# ----------------------------------------------------------------------------------- rope
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary_dim", [(4, 2, 16, 16), (3, 1, 32, 32), (6, 3, 48, 24), (2, 2, 128, 128), (2, 1, 16, 12), (5, 5, 80, 40)])
def test_rope_append(dtype, heads, kv_heads, head_dim, rotary_dim):
    from thintensor_b200.kernels import api

    news, befores = [5, 1, 70], [0, 130, 60]
    totals = [a + b for a, b in zip(news, befores)]
    k_pool, v_pool, table, _, _ = make_cache(totals, kv_heads, head_dim, dtype, seed=30)
    tokens = sum(news)
    cols = (heads + 2 * kv_heads) * head_dim
    splits = 2
    qkv = randn(splits, tokens, cols, seed=31)
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
    inv_freq = plain_llama.rope_inv_freq(rotary_dim, 500000.0, scaling).to(DEV)
    q_out = torch.empty(tokens, heads * head_dim, dtype=dtype, device=DEV)
    cu = torch.tensor([0] + list(torch.tensor(news).cumsum(0)), dtype=torch.int32, device=DEV)
    before = torch.tensor(befores, dtype=torch.int32, device=DEV)
    st = status()
    api.rope_append(qkv, inv_freq, rotary_dim, 1.0, q_out, k_pool, v_pool, table, cu, before, len(news), tokens, heads, kv_heads,
                    head_dim, st)
    assert int(st.item()) == 0
    x = qkv.double().sum(0).cpu()
    q = x[:, : heads * head_dim].view(tokens, heads, head_dim)
    k = x[:, heads * head_dim: (heads + kv_heads) * head_dim].view(tokens, kv_heads, head_dim)
    v = x[:, (heads + kv_heads) * head_dim:].view(tokens, kv_heads, head_dim)
    positions = torch.cat([torch.arange(b, b + n) for n, b in zip(news, befores)])
    cos, sin = plain_llama.rope_cos_sin(inv_freq.cpu(), positions, torch.float64)

    def rotate(t):
        out = t.clone()
        out[..., :rotary_dim] = plain_llama.apply_rope(t[..., :rotary_dim], cos, sin)
        return out

    torch.testing.assert_close(q_out.double().cpu().view(tokens, heads, head_dim), rotate(q), **tol(dtype))
    t = 0
    table_cpu = table.cpu()
    for b, (n, start) in enumerate(zip(news, befores)):
        for i in range(n):
            pos = start + i
            block, off = int(table_cpu[b, pos // 64]), pos % 64
            torch.testing.assert_close(k_pool[block, :, off].double().cpu(), rotate(k)[t], **tol(dtype))
            torch.testing.assert_close(v_pool[block, :, :, off].double().cpu(), v[t], **tol(dtype))
            t += 1


# --------------------------------------------------------------------------------- swiglu
@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    from thintensor_b200.kernels import api

    tokens, inter, splits = 5, 200, 3
    gate_up = randn(splits, tokens, 2 * inter, seed=40, scale=2.0)
    act = torch.empty(tokens, inter, dtype=dtype, device=DEV)
    api.swiglu(gate_up, act)
    x = gate_up.double().sum(0)
    g, u = x[:, :inter], x[:, inter:]
    torch.testing.assert_close(act.double(), g / (1 + torch.exp(-g)) * u, **tol(dtype))


# ----------------------------------------------------------------------------------- gemm
@pytest.mark.parametrize("x_dtype,w_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("m,n,k,splits", [(1, 311, 72, 1), (8, 100, 1000, 1), (70, 130, 200, 1), (33, 65, 500, 4), (200, 17, 64, 1)])
def test_gemm_simt(x_dtype, w_dtype, m, n, k, splits):
    from thintensor_b200.kernels import api

    x = randn(m, k, dtype=x_dtype, seed=50)
    w = randn(n, k, dtype=w_dtype, seed=51)
    bias = randn(n, seed=52)
    out = torch.empty(splits, m, n, dtype=torch.float32, device=DEV)
    api.gemm_simt(x, w, bias, out)
    want = x.double() @ w.double().T + bias.double()
    torch.testing.assert_close(out.double().sum(0), want, rtol=1e-5, atol=1e-4)


# ------------------------------------------------------------------------------- sampling
@pytest.mark.parametrize("vocab", [311, 1000, 8192, 128256])
def test_argmax_lowest_id_on_ties(vocab):
    from thintensor_b200.kernels import api

    logits = randn(4, vocab, seed=60)
    top = float(logits.max()) + 1.0
    logits[0, vocab - 1] = top
    logits[1, 5] = top
    logits[1, vocab // 2] = top        # a tie: the lower id wins
    logits[2, 0] = top
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    api.argmax_rows(logits, out)
    assert out.tolist()[:3] == [vocab - 1, 5, 0]
    assert out.tolist()[3] == int(torch.argmax(logits[3]))


@pytest.mark.parametrize("vocab", [311, 5000])
@pytest.mark.parametrize("params", [(0.8, 0, 1.0), (1.5, 7, 1.0), (0.6, 0, 0.5), (1.0, 50, 0.8)])
def test_sampling_follows_plain(vocab, params):
    """The tokens equal the plain sampler's for the same (seed, request, step), and over
    many draws the empirical distribution is the plain implementation's."""
    from thintensor_b200.kernels import api

    temperature, top_k, top_p = params
    rows = 64
    logits = randn(rows, vocab, seed=70, scale=3.0)
    request = torch.arange(rows, dtype=torch.int32, device=DEV) % 5
    step = torch.arange(rows, dtype=torch.int32, device=DEV) // 5
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    seed = 4
    api.sample_rows(logits, temperature, top_k, top_p, seed, request, step, out)
    cpu = logits.cpu()
    want = [plain_llama.select_token(cpu[i], temperature, top_k, top_p, seed, int(request[i]), int(step[i])) for i in range(rows)]
    assert out.tolist() == want
    # distribution: one row, many draws
    draws = 4000
    one = logits[:1].expand(draws, vocab).contiguous()
    request = torch.zeros(draws, dtype=torch.int32, device=DEV)
    step = torch.arange(draws, dtype=torch.int32, device=DEV)
    out = torch.empty(draws, dtype=torch.int32, device=DEV)
    api.sample_rows(one, temperature, top_k, top_p, 99, request, step, out)
    p = plain_llama.sampling_probabilities(cpu[0], temperature, top_k, top_p)
    counts = torch.bincount(out.long().cpu(), minlength=vocab).double() / draws
    assert float(counts[p == 0].sum()) == 0.0, "a token outside the kept set was drawn"
    assert float(0.5 * (counts - p).abs().sum()) < 0.12 + 0.5 * math.sqrt(float((p > 0).sum()) / draws)


# ------------------------------------------------------------------------ step bookkeeping
@pytest.mark.parametrize("sequences", [1, 7, 300])
def test_advance_lengths_and_step_counters(sequences):
    """After a step every sequence's length grows by the tokens it brought; the step counters,
    where the caller keeps some, go up by one; without counters only the lengths change."""
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(sequences)
    new = torch.randint(1, 9, (sequences,), generator=g)
    cu = torch.cat([torch.zeros(1, dtype=torch.int64), new.cumsum(0)]).to(torch.int32).to(DEV)
    before = torch.randint(0, 5000, (sequences,), generator=g).to(torch.int32)
    lengths, counters = before.to(DEV), torch.arange(sequences, dtype=torch.int32, device=DEV)
    api.advance_lengths(lengths, cu, sequences, counters)
    assert torch.equal(lengths.cpu(), before + new.to(torch.int32))
    assert torch.equal(counters.cpu(), torch.arange(sequences, dtype=torch.int32) + 1)
    api.advance_lengths(lengths, cu, sequences)
    assert torch.equal(lengths.cpu(), before + 2 * new.to(torch.int32))
    assert torch.equal(counters.cpu(), torch.arange(sequences, dtype=torch.int32) + 1)


def test_attention_mma_decode_beyond_the_cached_table_row():
    """A sequence of more blocks than the decode kernel keeps of a table row in shared memory (1,024): the entries beyond
    come from global memory; a far key among 70,000 must still be found, with and without slices."""
    from thintensor_b200.kernels import api

    dtype, heads, kv_heads, head_dim = torch.bfloat16, 4, 1, 64
    totals = [70000, 130]
    k_pool, v_pool, table, keys, values = make_cache(totals, kv_heads, head_dim, dtype, seed=70)
    n = len(totals)
    q = randn(n, heads, head_dim, dtype=dtype, seed=71)
    far = 69000                                                  # block 1,078
    spike = (q[0, 0].float() * (40.0 * head_dim ** 0.5 / float(q[0, 0].float().norm()) ** 2)).to(dtype)
    k_pool[int(table[0, far // 64]), 0, far % 64] = spike
    keys[0][far, 0] = spike.float().cpu()
    cu = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    before = torch.tensor([t - 1 for t in totals], dtype=torch.int32, device=DEV)
    scale = head_dim ** -0.5
    want = attention_reference(q.float().cpu(), keys, values, [1] * n, heads, kv_heads, scale, 0)
    assert torch.allclose(want[0, 0], values[0][far, 0].double(), atol=0.35)
    for splits in (1, 6, 40):
        out = torch.full((n, heads * head_dim), float("nan"), dtype=dtype, device=DEV)
        part_acc = torch.full((n * heads * splits * head_dim,), float("nan"), dtype=torch.float32, device=DEV)
        part_ml = torch.full((n * heads * splits * 2,), float("nan"), dtype=torch.float32, device=DEV)
        st = status()
        api.attention_mma(q.view(n, -1), k_pool, v_pool, table, cu, before, n, n, heads, kv_heads, head_dim, scale, 0, splits, out,
                          part_acc, part_ml, st, one_token_each=True)
        torch.testing.assert_close(out.double().cpu().view(n, heads, head_dim), want, **tol(dtype))
        assert int(st.item()) == 0
