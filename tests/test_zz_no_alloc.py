"""The entry point that allocates nothing: ``tt_attention_decode_static``.

Some users of the C interface cannot allocate device memory when a step runs: they gave
all of it to their own weight and cache arenas at start-up, or they may not pay for the
device-wide synchronisation an allocation can cause.  For them the library offers the
split-key attention with its scratch in a fixed 16 MiB array inside the library image.
This test calls it through its exported C symbol, exactly as such a user would, twice in
a row (the second call finds the first call's leftovers in the shared scratch), and
checks each result against the ordinary entry point, which gets its scratch from the
caller.  It also checks that a call too large for the array is refused with a message,
and that the second call leaves the amount of free device memory unchanged.

The file's name keeps it last in collection order, so a run that stops at the first
failure has already run every other test.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
STATIC_BYTES = 16 * 1024 * 1024
TOO_LARGE = -1


def static_library():
    from thintensor_b200.kernels import build

    lib = build.load("attention_static_scratch")
    fn = lib.tt_attention_decode_static
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                   c_float, c_int, c_int, c_void_p, c_void_p, c_void_p]
    fn.restype = c_int
    lib.tt_attention_static_last_error.restype = ctypes.c_char_p
    lib.tt_attention_static_bytes_needed.restype = ctypes.c_ulonglong
    lib.tt_attention_static_bytes_needed.argtypes = [c_int, c_int, c_int, c_int]
    return lib


def problem(dtype, lengths, news, heads, kv_heads, head_dim, seed):
    """Random queries (``news[b]`` packed tokens for sequence b, its last positions) and a block
    cache whose blocks lie scattered over the pool."""
    g = torch.Generator().manual_seed(seed)
    blocks_per = [-(-n // 64) for n in lengths]
    total = sum(blocks_per) + 2
    order = torch.randperm(total, generator=g).tolist()
    table = torch.full((len(lengths), max(blocks_per)), -1, dtype=torch.int32)
    at = 0
    for b, count in enumerate(blocks_per):
        for j in range(count):
            table[b, j] = order[at]
            at += 1
    k_pool = torch.randn(total, kv_heads, 64, head_dim, generator=g).to(dtype).to(DEV)
    v_pool = torch.randn(total, kv_heads, head_dim, 64, generator=g).to(dtype).to(DEV)
    q = torch.randn(sum(news), heads * head_dim, generator=g).to(dtype).to(DEV)
    cu = torch.tensor([0] + torch.tensor(news).cumsum(0).tolist(), dtype=torch.int32, device=DEV)
    before = torch.tensor([n - new for n, new in zip(lengths, news)], dtype=torch.int32, device=DEV)
    return q, k_pool, v_pool, table.to(DEV), cu, before


def plain_attention(q, k_pool, v_pool, table, lengths, news, heads, kv_heads, head_dim, scale, window):
    """float64, one (token, head) at a time, keys and values gathered through the block table."""
    q, k_pool, v_pool, table = q.double().cpu(), k_pool.double().cpu(), v_pool.double().cpu(), table.cpu()
    out = torch.zeros(q.shape[0], heads, head_dim, dtype=torch.float64)
    t = 0
    for b, (total, new) in enumerate(zip(lengths, news)):
        blocks = table[b, : -(-total // 64)].long()
        keys = k_pool[blocks].permute(1, 0, 2, 3).reshape(kv_heads, -1, head_dim)[:, :total]        # [kv, total, d]
        values = v_pool[blocks].permute(1, 0, 3, 2).reshape(kv_heads, -1, head_dim)[:, :total]
        for i in range(new):
            pos = total - new + i
            first = max(0, pos - window + 1) if window else 0
            for h in range(heads):
                kh = h // (heads // kv_heads)
                scores = (keys[kh, first : pos + 1] @ q[t].view(heads, head_dim)[h]) * scale
                out[t, h] = torch.softmax(scores, dim=0) @ values[kh, first : pos + 1]
            t += 1
    return out.view(q.shape[0], heads * head_dim)


def run_both(lib, dtype, lengths, heads, kv_heads, head_dim, splits, seed, news=None, window=0):
    from thintensor_b200.kernels import api

    news = news or [1] * len(lengths)
    q, k_pool, v_pool, table, cu, before = problem(dtype, lengths, news, heads, kv_heads, head_dim, seed)
    n, tokens = len(lengths), sum(news)
    scale = head_dim ** -0.5
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    want = torch.empty(tokens, heads * head_dim, dtype=dtype, device=DEV)
    part_acc = torch.empty(tokens * heads * splits * head_dim, dtype=torch.float32, device=DEV)
    part_ml = torch.empty(tokens * heads * splits * 2, dtype=torch.float32, device=DEV)
    api.attention(q, k_pool, v_pool, table, cu, before, n, tokens, heads, kv_heads, head_dim, scale, window, splits, want, part_acc, part_ml, status)
    got = torch.full_like(want, float("nan"))
    stream = torch.cuda.current_stream().cuda_stream
    code = lib.tt_attention_decode_static(
        q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), api.dtype_code(dtype), table.data_ptr(), table.shape[1], k_pool.shape[0],
        cu.data_ptr(), before.data_ptr(), n, tokens, heads, kv_heads, head_dim, scale, window, splits, got.data_ptr(), status.data_ptr(), stream)
    assert code == 0, lib.tt_attention_static_last_error().decode()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    exact = plain_attention(q, k_pool, v_pool, table, lengths, news, heads, kv_heads, head_dim, scale, window)
    return got, want, exact


def check(got, want, exact, dtype):
    """Against the ordinary entry point (the same arithmetic, so nearly the same bits) and against
    the float64 formula (so that a fault both entry points share would show)."""
    tolerance = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got.float(), want.float(), **tolerance)
    torch.testing.assert_close(got.double().cpu(), exact, **tolerance)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_matches_ordinary_entry_point(dtype):
    lib = static_library()
    # first call: long caches, many slices
    check(*run_both(lib, dtype, [900, 64, 333, 1], heads=8, kv_heads=2, head_dim=64, splits=8, seed=1), dtype)
    # second call right after it: other sizes, fewer slices; the scratch still holds the first call's partials
    free_before = torch.cuda.mem_get_info()[0]
    check(*run_both(lib, dtype, [130, 700], heads=6, kv_heads=3, head_dim=48, splits=3, seed=2), dtype)
    torch.cuda.synchronize()
    # (run_both's own torch tensors come from torch's cached pool; the driver's view of free memory must not move)
    assert torch.cuda.mem_get_info()[0] >= free_before - 4 * 1024 * 1024


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_packed_tokens_and_window(dtype):
    """More tokens than sequences (the last tokens of each sequence, packed) and a window of keys."""
    lib = static_library()
    check(*run_both(lib, dtype, [200, 70, 500], heads=4, kv_heads=2, head_dim=32, splits=4, seed=3, news=[5, 1, 9]), dtype)
    check(*run_both(lib, dtype, [300, 129], heads=6, kv_heads=2, head_dim=64, splits=3, seed=4, news=[2, 3], window=100), dtype)


def test_static_scratch_refuses_what_does_not_fit():
    lib = static_library()
    heads, head_dim, splits = 32, 128, 64
    n = 64
    assert lib.tt_attention_static_bytes_needed(n, heads, head_dim, splits) > STATIC_BYTES
    # sizes whose product leaves 64 bits must not come back small, and sizes that are not positive fit nothing
    for sizes in ((2**31 - 1, 2**31 - 1, 256, 65535), (2**31 - 1, 2**20, 16, 4096), (1 << 20, 1 << 20, 256, 1 << 15),
                  (-1, 8, 64, 2), (8, 0, 64, 2), (8, 8, -64, 2), (8, 8, 64, 0)):
        assert lib.tt_attention_static_bytes_needed(*sizes) > STATIC_BYTES, sizes
    dummy = torch.zeros(16, device=DEV)
    code = lib.tt_attention_decode_static(
        dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 0, dummy.data_ptr(), 1, 1, dummy.data_ptr(), dummy.data_ptr(), n, n,
        heads, 8, head_dim, 1.0, 0, splits, dummy.data_ptr(), dummy.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert code == TOO_LARGE
    message = lib.tt_attention_static_last_error().decode()
    assert "bytes of scratch" in message and str(STATIC_BYTES) in message
    # a count that would wrap 64 bits is refused as too large as well
    code = lib.tt_attention_decode_static(
        dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 0, dummy.data_ptr(), 1, 1, dummy.data_ptr(), dummy.data_ptr(), 1, 2**31 - 1,
        2**30, 1, 256, 1.0, 0, 65535, dummy.data_ptr(), dummy.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert code == TOO_LARGE
    # a bad head size is refused too, without touching the device
    code = lib.tt_attention_decode_static(
        dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 0, dummy.data_ptr(), 1, 1, dummy.data_ptr(), dummy.data_ptr(), 1, 1,
        4, 2, 24, 1.0, 0, 2, dummy.data_ptr(), dummy.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert code == -2
