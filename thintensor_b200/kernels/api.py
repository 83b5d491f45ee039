"""Python signatures of the CUDA kernels.

Each function checks what the kernel cannot check itself (device, dtype, contiguity,
sizes it refuses), passes raw pointers and the current CUDA stream through ctypes, and
raises on a launch error.  Nothing here computes anything and nothing falls back to
another implementation: tensors that are not on a CUDA device are an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from . import build

F32, BF16 = 0, 1
BLOCK_TOKENS = 64          # tokens of one cache block (TT_BLOCK_TOKENS in csrc/common.cuh)
MAX_HEAD_DIM = 256

STATUS_BAD_TOKEN = 1
STATUS_BAD_BLOCK = 2
STATUS_WAIT_EXPIRED = 4
STATUS_BAD_SHAPE = 8


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t: torch.Tensor | None) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("thintensor_b200 kernels run on CUDA tensors only; got a tensor on " + str(t.device))
    return c_void_p(t.data_ptr())


def _stream() -> c_void_p:
    # the raw handle of torch's current stream on the current device (torch.cuda.current_stream()
    # builds a Stream object around the same number, at ten times the cost)
    return c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


_launches = 0


def launch_count() -> int:
    """How many of this library's kernels have been launched (or captured into a graph)
    by this process so far."""
    return _launches


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch")
    _launches += kernels


def _need(t: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_functions: dict[str, object] = {}


class ClassTimer:
    """Device time per class of kernel, for looking at where a step's time goes: while one is
    active (``with api.timed_classes() as timer``) every call of an entry point of this library is
    bracketed by two CUDA events on the current stream, and ``timer.summary()`` adds the spans up
    by entry point and label (parts label their matrix products: ``attention.qkv``, ``ffn.down``
    ...).  The events keep a kernel from starting under the tail of the one before it, so the
    spans are those of kernels run one after another, like a profiler's: compare shares, and take
    a step's duration from an untimed run.  Not for use while a CUDA graph is being captured.
    The reference's counterpart brackets layers the same way (LayerProfileEvents,
    thinruntime/gpu_runtime.py:4770-4797, summed at :7464-7543)."""

    def __init__(self):
        self.spans: list[tuple[str, torch.cuda.Event, torch.cuda.Event]] = []

    def wrap(self, name: str, fn):
        def timed(*args):
            global _label
            key = name if _label is None else f"{name}[{_label}]"
            _label = None
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            code = fn(*args)
            stop.record()
            self.spans.append((key, start, stop))
            return code

        return timed

    def summary(self) -> dict[str, dict]:
        """class -> {"calls": n, "ms": total}; synchronises."""
        torch.cuda.synchronize()
        out: dict[str, dict] = {}
        for key, start, stop in self.spans:
            entry = out.setdefault(key, {"calls": 0, "ms": 0.0})
            entry["calls"] += 1
            entry["ms"] += start.elapsed_time(stop)
        return dict(sorted(out.items(), key=lambda item: -item[1]["ms"]))


_timer: ClassTimer | None = None
_label: str | None = None


def set_label(label: str) -> None:
    """Name the next kernel call for an active :class:`ClassTimer` (no effect otherwise)."""
    global _label
    if _timer is not None:
        _label = label


class timed_classes:
    """Context manager that switches a :class:`ClassTimer` on for the calls inside it."""

    def __enter__(self) -> ClassTimer:
        global _timer
        if _timer is not None:
            raise KernelError("a class timer is already active")
        _timer = ClassTimer()
        return _timer

    def __exit__(self, *exc) -> None:
        global _timer, _label
        _timer, _label = None, None


def _fn(lib: str, name: str, argtypes: list):
    """The C entry point ``name`` of library ``lib`` (built and loaded at first use), with its prototype set."""
    fn = _functions.get(name)
    if fn is None:
        fn = getattr(build.load(lib), name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _functions[name] = fn
    if _timer is not None:
        return _timer.wrap(name, fn)
    return fn


# ------------------------------------------------------------------------- elementwise
def embed_gather(table: torch.Tensor, tokens: torch.Tensor, residual: torch.Tensor, scale: float, status: torch.Tensor) -> None:
    """residual[t] = table[tokens[t]] * scale, float32 out."""
    _need(tokens, torch.int32, "tokens")
    _need(residual, torch.float32, "residual")
    if not table.is_contiguous():
        raise KernelError("embedding table must be contiguous")
    n, hidden = tokens.numel(), table.shape[1]
    fn = _fn("elementwise", "tt_embed_gather", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(fn(_ptr(table), dtype_code(table.dtype), _ptr(tokens), _ptr(residual), n, hidden, table.shape[0], scale, _ptr(status), _stream()), "embed_gather")


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: torch.Tensor | None = None, weight_offset: float = 0.0) -> None:
    """residual += sum(delta over its first axis); out = rmsnorm(residual) * weight.
    With ``rows`` (int32), out[i] comes from residual row rows[i] and residual is left
    as it was."""
    _need(residual, torch.float32, "residual")
    _need(weight, torch.float32, "norm weight")
    if not out.is_contiguous():
        raise KernelError("norm output must be contiguous")
    hidden = residual.shape[-1]
    splits, stride = 0, 0
    if delta is not None:
        _need(delta, torch.float32, "delta")
        splits = delta.shape[0]
        stride = delta.stride(0)
    n_rows = rows.numel() if rows is not None else residual.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows")
    fn = _fn("elementwise", "tt_add_rmsnorm", [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_float, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(residual), _ptr(delta), splits, stride, _ptr(weight), weight_offset, eps, _ptr(out), dtype_code(out.dtype), _ptr(rows), n_rows, hidden, _stream()), "add_rmsnorm")


def rope_append(qkv: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, attention_scaling: float, q_out: torch.Tensor,
                k_pool: torch.Tensor | None, v_pool: torch.Tensor | None, table: torch.Tensor | None, cu: torch.Tensor,
                len_before: torch.Tensor, sequences: int, n_tokens: int, heads: int, kv_heads: int, head_dim: int,
                status: torch.Tensor) -> None:
    """Rotate q and k of float32 partial sums ``qkv`` [splits, tokens, cols], write q in
    the activation dtype and append k and v to the block pools.  Without pools the
    projection holds queries only."""
    _need(qkv, torch.float32, "qkv")
    _need(inv_freq, torch.float32, "inv_freq")
    write = k_pool is not None
    cols = heads * head_dim + (2 * kv_heads * head_dim if write else 0)
    if qkv.shape[-1] != cols:
        raise KernelError(f"qkv has {qkv.shape[-1]} columns, expected {cols}")
    if write and (k_pool.dtype != q_out.dtype or v_pool.dtype != q_out.dtype):
        raise KernelError("cache pools and activations must share a dtype")
    fn = _fn("elementwise", "tt_rope_append", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int,
                                               c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(qkv), qkv.shape[0], qkv.stride(0), _ptr(inv_freq), rotary_dim, attention_scaling, _ptr(q_out), _ptr(k_pool), _ptr(v_pool),
              dtype_code(q_out.dtype), _ptr(table), table.shape[1] if table is not None else 0,
              k_pool.shape[0] if write else 0, _ptr(cu), _ptr(len_before), sequences, n_tokens, heads, kv_heads, head_dim,
              1 if write else 0, _ptr(status), _stream()), "rope_append")


def rope_table(inv_freq: torch.Tensor, rotary_dim: int, cu: torch.Tensor, len_before: torch.Tensor, sequences: int, n_tokens: int,
               cos_sin: torch.Tensor, where: torch.Tensor) -> None:
    """What the rotations of all layers of a step share: ``where[t] = (position, sequence)`` of packed token t
    (int32 [tokens, 2]) and ``cos_sin[t, i] = (cos, sin)(inv_freq[i] * position)`` (float32 [tokens, rotary_dim / 2, 2])."""
    _need(inv_freq, torch.float32, "inv_freq")
    _need(cos_sin, torch.float32, "cos/sin table")
    _need(where, torch.int32, "token positions")
    half = rotary_dim // 2
    if tuple(cos_sin.shape) != (n_tokens, half, 2) or tuple(where.shape) != (n_tokens, 2) or inv_freq.numel() < half:
        raise KernelError(f"rope_table: cos_sin must be [{n_tokens}, {half}, 2] and where [{n_tokens}, 2]")
    fn = _fn("elementwise", "tt_rope_table", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(inv_freq), half, _ptr(cu), _ptr(len_before), sequences, n_tokens, _ptr(cos_sin), _ptr(where), _stream()), "rope_table")


def swiglu(gate_up: torch.Tensor, act: torch.Tensor) -> None:
    """act = silu(gate) * up from float32 partial sums [splits, tokens, 2 * inter]."""
    _need(gate_up, torch.float32, "gate_up")
    inter = gate_up.shape[-1] // 2
    fn = _fn("elementwise", "tt_swiglu", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(gate_up), gate_up.shape[0], gate_up.stride(0), _ptr(act), dtype_code(act.dtype), gate_up.shape[1], inter, _stream()), "swiglu")


def copy_int32(dst: torch.Tensor, src: torch.Tensor, extra: torch.Tensor | None = None) -> None:
    """dst[:n] = src for small int32 vectors; either side may be pinned host memory.  With ``extra``
    (one int32 on the device, the status word say) ``dst`` has n + 1 entries and dst[n] = extra[0]."""
    for t, name in ((dst, "dst"), (src, "src")):
        if t.dtype != torch.int32 or not t.is_contiguous() or not (t.is_cuda or t.is_pinned()):
            raise KernelError(f"copy_int32: {name} must be contiguous int32 on the device or in pinned host memory")
    if dst.numel() != src.numel() + (1 if extra is not None else 0):
        raise KernelError("copy_int32: sizes differ")
    if extra is not None and (extra.dtype != torch.int32 or extra.numel() != 1 or not extra.is_cuda):
        raise KernelError("copy_int32: the extra word must be one int32 on the device")
    fn = _fn("elementwise", "tt_copy_int32", [c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    _check(fn(c_void_p(dst.data_ptr()), c_void_p(src.data_ptr()), src.numel(), _ptr(extra), _stream()), "copy_int32")


def advance_lengths(lengths: torch.Tensor, cu: torch.Tensor, sequences: int, counters: torch.Tensor | None = None) -> None:
    """lengths[b] += cu[b + 1] - cu[b] after a step; ``counters`` (int32, one per sequence), if given, go up by one."""
    if counters is not None:
        _need(counters, torch.int32, "step counters")
    fn = _fn("elementwise", "tt_advance_lengths", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(lengths), _ptr(cu), _ptr(counters), sequences, _stream()), "advance_lengths")


# --------------------------------------------------------------------------- attention
def check_head_dim(head_dim: int) -> None:
    if head_dim <= 0 or head_dim % 16 or head_dim > MAX_HEAD_DIM:
        raise KernelError(f"attention kernels take head sizes that are multiples of 16 up to {MAX_HEAD_DIM}, not {head_dim}")


def attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor, cu: torch.Tensor,
              len_before: torch.Tensor, sequences: int, n_tokens: int, heads: int, kv_heads: int, head_dim: int,
              scale: float, window: int, splits: int, out: torch.Tensor, part_acc: torch.Tensor | None,
              part_ml: torch.Tensor | None, status: torch.Tensor) -> None:
    """Exact causal attention of ``n_tokens`` packed query tokens over the block cache."""
    check_head_dim(head_dim)
    if heads % kv_heads:
        raise KernelError(f"{heads} query heads are not a multiple of {kv_heads} key/value heads")
    if not (q.dtype == k_pool.dtype == v_pool.dtype == out.dtype):
        raise KernelError("queries, cache and output must share a dtype")
    fn = _fn("attention", "tt_attention", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                                           c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(q), _ptr(k_pool), _ptr(v_pool), dtype_code(q.dtype), _ptr(table), table.shape[1], k_pool.shape[0], _ptr(cu),
              _ptr(len_before), sequences, n_tokens, heads, kv_heads, head_dim, scale, window, splits, _ptr(out),
              _ptr(part_acc), _ptr(part_ml), _ptr(status), _stream()), "attention", 2 if splits > 1 else 1)


def _attention_launches(splits: int, decode: bool, tickets: bool = False) -> int:
    """Kernels one call launches: the decode kernel combines up to 8 slices itself (a thread-block
    cluster) and, given tickets, any number; otherwise more slices need the merge kernel."""
    return 1 if splits == 1 or (decode and (splits <= 8 or tickets)) else 2


def _check_tickets(tickets: torch.Tensor | None, sequences: int, kv_heads: int) -> None:
    if tickets is not None:
        _need(tickets, torch.int32, "tickets")
        if tickets.numel() < sequences * kv_heads:
            raise KernelError(f"decode attention needs {sequences * kv_heads} tickets, got {tickets.numel()}")


def attention_mma_supports(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether the tensor-core attention kernel takes these sizes (bfloat16, head size 32,
    64, 96 or 128, at most 16 query heads per key/value head)."""
    return dtype == torch.bfloat16 and head_dim in (32, 64, 96, 128) and heads % kv_heads == 0 and heads // kv_heads <= 16


def attention_mma(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor, cu: torch.Tensor,
                  len_before: torch.Tensor, sequences: int, n_tokens: int, heads: int, kv_heads: int, head_dim: int,
                  scale: float, window: int, splits: int, out: torch.Tensor, part_acc: torch.Tensor | None,
                  part_ml: torch.Tensor | None, status: torch.Tensor, one_token_each: bool = False,
                  tickets: torch.Tensor | None = None) -> None:
    """Causal attention of packed bfloat16 query tokens over the block cache on tensor cores.
    ``one_token_each`` (decoding): the warps of a CTA share a sequence's tile and split its keys.
    ``tickets`` (decoding; int32, one per sequence and key/value head, zero before the call and after it): with
    more slices than a cluster combines, the CTA that finishes last combines them and no second kernel runs."""
    if not attention_mma_supports(q.dtype, heads, kv_heads, head_dim):
        raise KernelError(f"the tensor-core attention kernel does not take {q.dtype}, {heads}/{kv_heads} heads of size {head_dim}")
    if not (k_pool.dtype == v_pool.dtype == out.dtype == torch.bfloat16):
        raise KernelError("queries, cache and output must all be bfloat16")
    if one_token_each and n_tokens != sequences:
        raise KernelError("one_token_each needs exactly one token per sequence")
    tickets = tickets if one_token_each else None
    _check_tickets(tickets, sequences, kv_heads)
    fn = _fn("attention_mma", "tt_attention_mma", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                                                   c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(table), table.shape[1], k_pool.shape[0], _ptr(cu), _ptr(len_before), sequences,
              n_tokens, heads, kv_heads, head_dim, scale, window, splits, sequences if one_token_each else 0, _ptr(out), _ptr(part_acc),
              _ptr(part_ml), _ptr(tickets), _ptr(status),
              _stream()), "attention_mma", _attention_launches(splits, one_token_each, tickets is not None))


def attention_mma_failure_drill(wait_limit_ns: int, undelivered_bytes: int) -> None:
    """For tests of the failure path, never for serving.  ``wait_limit_ns``: the limit of the bounded waits in the
    tensor-core decode attention (0 restores the default of two seconds).  ``undelivered_bytes``: from now on the first
    stage of every warp expects that many bytes more than its copies bring (0 restores normal operation), so its barrier
    never completes; the kernel must then raise ``STATUS_WAIT_EXPIRED`` and return."""
    lib = build.load("attention_mma")
    lib.tt_attention_mma_failure_drill.argtypes = [c_ulonglong, c_int]
    lib.tt_attention_mma_failure_drill.restype = c_int
    code = lib.tt_attention_mma_failure_drill(int(wait_limit_ns), int(undelivered_bytes))
    if code != 0:
        raise KernelError(f"the decode attention's failure drill could not be set: CUDA error {code}")


def attention_decode_rope_supports(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int, rotary_dim: int) -> bool:
    """Whether decoding may rotate q and k and write the cache inside the attention kernel
    (bfloat16, head size 64 rotated whole, at most 16 query heads per key/value head)."""
    return attention_mma_supports(dtype, heads, kv_heads, head_dim) and head_dim == 64 and rotary_dim == head_dim


def attention_decode_rope(qkv: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, attention_scaling: float, write_cache: bool,
                          k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor, len_before: torch.Tensor,
                          sequences: int, heads: int, kv_heads: int, head_dim: int, scale: float, window: int, splits: int,
                          out: torch.Tensor, part_acc: torch.Tensor | None, part_ml: torch.Tensor | None,
                          status: torch.Tensor, tickets: torch.Tensor | None = None) -> None:
    """One decode step of attention straight from the float32 partial sums ``qkv``
    [slices, sequences, cols] of the qkv product: q and k are rotated, k and v are written to
    the cache (``write_cache``; else ``qkv`` holds queries only), then every sequence's token
    attends over its cache: one launch where rope_append and attention_mma would be two."""
    _need(qkv, torch.float32, "qkv")
    _need(inv_freq, torch.float32, "inv_freq")
    if not attention_decode_rope_supports(out.dtype, heads, kv_heads, head_dim, rotary_dim):
        raise KernelError(f"the fused decode attention does not take {out.dtype}, {heads}/{kv_heads} heads of size {head_dim}, rotary part {rotary_dim}")
    if not (k_pool.dtype == v_pool.dtype == torch.bfloat16):
        raise KernelError("cache and output must be bfloat16")
    cols = heads * head_dim + (2 * kv_heads * head_dim if write_cache else 0)
    if qkv.shape[-1] != cols or qkv.shape[1] != sequences:
        raise KernelError(f"qkv is {tuple(qkv.shape)}, expected [slices, {sequences}, {cols}]")
    _check_tickets(tickets, sequences, kv_heads)
    fn = _fn("attention_mma", "tt_attention_decode_rope", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p,
                                                           c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                                           c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(qkv), qkv.shape[0], qkv.stride(0), _ptr(inv_freq), rotary_dim, attention_scaling, 1 if write_cache else 0, _ptr(k_pool),
              _ptr(v_pool), _ptr(table), table.shape[1], k_pool.shape[0], _ptr(len_before), sequences, heads, kv_heads, head_dim, scale,
              window, splits, _ptr(out), _ptr(part_acc), _ptr(part_ml), _ptr(tickets), _ptr(status), _stream()), "attention_decode_rope",
           _attention_launches(splits, True, tickets is not None))


def attention_tcgen05_supports(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether the tcgen05 prompt attention takes these sizes (bfloat16, head size 64 or 128,
    at most 16 query heads per key/value head)."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and heads % kv_heads == 0 and heads // kv_heads <= 16


def attention_tcgen05(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor, cu: torch.Tensor,
                      len_before: torch.Tensor, sequences: int, n_tokens: int, heads: int, kv_heads: int, head_dim: int,
                      scale: float, window: int, out: torch.Tensor, status: torch.Tensor) -> None:
    """Causal attention of packed bfloat16 prompts over the block cache with both products on
    the tcgen05 tensor cores."""
    if not attention_tcgen05_supports(q.dtype, heads, kv_heads, head_dim):
        raise KernelError(f"the tcgen05 attention kernel does not take {q.dtype}, {heads}/{kv_heads} heads of size {head_dim}")
    if not (k_pool.dtype == v_pool.dtype == out.dtype == torch.bfloat16) or not q.is_contiguous():
        raise KernelError("queries, cache and output must all be contiguous bfloat16")
    fn = _fn("attention_tcgen05", "tt_attention_tcgen05", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                                                           c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(table), table.shape[1], k_pool.shape[0], _ptr(cu), _ptr(len_before), sequences,
              n_tokens, heads, kv_heads, head_dim, scale, window, _ptr(out), _ptr(status), _stream()), "attention_tcgen05")


# -------------------------------------------------------------------------------- gemm
def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor) -> None:
    """out[s] = x @ w[:, k-slice s].T in float32 FMA; ``out`` is float32
    [splits, m, n]; bias (float32 [n]) goes into slice 0."""
    _need(out, torch.float32, "gemm output")
    if x.stride(-1) != 1 or w.stride(-1) != 1:
        raise KernelError("gemm operands must be contiguous along k")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[1:] != (m, n):
        raise KernelError(f"gemm shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    fn = _fn("gemm_simt", "tt_gemm_simt", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_longlong,
                                           c_longlong, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), dtype_code(x.dtype), x.stride(0), _ptr(w), dtype_code(w.dtype), w.stride(0), _ptr(bias), _ptr(out), out.stride(1),
              out.stride(0), m, n, k, out.shape[0], _stream()), "gemm_simt")


# ---------------------------------------------------------------------------- sampling
_argmax_scratch: dict[torch.device, tuple[torch.Tensor, torch.Tensor]] = {}


def argmax_rows(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[i] = argmax of logits[i], lowest id on ties.  Large vocabularies are reduced in
    two stages through a small scratch buffer kept per device."""
    _need(logits, torch.float32, "logits")
    _need(out, torch.int32, "token output")
    rows = logits.shape[0]
    scratch = _argmax_scratch.get(logits.device)
    if scratch is None or scratch[0].numel() < rows * 32:
        count = max(rows, 256) * 32
        scratch = (torch.empty(count, dtype=torch.float32, device=logits.device), torch.empty(count, dtype=torch.int32, device=logits.device))
        _argmax_scratch[logits.device] = scratch
    fn = _fn("sampling", "tt_argmax_rows", [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    two_stage = logits.shape[1] >= 8192
    _check(fn(_ptr(logits), logits.stride(0), rows, logits.shape[1], _ptr(out), _ptr(scratch[0]), _ptr(scratch[1]), _stream()),
           "argmax_rows", 2 if two_stage else 1)


def sample_rows(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int, request: torch.Tensor,
                step: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits, torch.float32, "logits")
    _need(request, torch.int32, "request ids")
    _need(step, torch.int32, "step ids")
    _need(out, torch.int32, "token output")
    fn = _fn("sampling", "tt_sample_rows", [c_void_p, c_longlong, c_int, c_int, c_float, c_int, c_float, c_ulonglong, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], temperature, top_k, top_p, seed & ((1 << 64) - 1),
              _ptr(request), _ptr(step), _ptr(out), _stream()), "sample_rows")


# ----------------------------------------------------------------- tensor-core kernels
_sm_counts: dict[int, int] = {}


def sm_count(device: torch.device | int | None = None) -> int:
    """Streaming multiprocessors of a CUDA device (the current one by default), asked of the device
    once: it sizes the k-slices of few-token products and the key slices of decode attention, which
    the launchers in C++ size from the same attribute."""
    index = torch.cuda.current_device() if device is None else (device if isinstance(device, int) else (device.index if device.index is not None else torch.cuda.current_device()))
    count = _sm_counts.get(index)
    if count is None:
        count = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return count


SKINNY_TOKENS = 128         # up to this many tokens the weights go on the 128-row side of the tile


def gemm_tcgen05_usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    """TMA needs 16-byte aligned bases and row strides, i.e. k and both leading
    dimensions must be multiples of 8 bfloat16 numbers."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and x.stride(1) == 1 and w.stride(1) == 1)


PERSISTENT_TILES = 8        # from this many 128 x 256 output tiles on, prompts run the persistent kernel
PAIR_TOKENS = 2048          # from this many tokens on, CTA pairs run them, which do not slice k
PERSISTENT_SLICE_BLOCKS = 8  # a k-slice of the persistent kernel has at least this many 64-wide k-blocks


def gemm_tcgen05_splits(tokens: int, features: int, k: int, sms: int | None = None) -> int:
    """Into how many slices k is cut so that few output tiles still fill the GPU.  Few tokens:
    about two CTAs per SM, at least four 64-wide k-blocks per slice, at most 16 slices.
    Prompts (more than 128 tokens) with at least 8 tiles of 128 x 256 run the persistent kernel,
    one CTA per SM: as many slices as keep its work items within one round of the SMs (a
    512-token prompt has 32 tiles in the 1B shape's output projection), none of them empty.
    ``sms``: the device's multiprocessors (asked of the current device when not given)."""
    sms = sm_count() if sms is None else sms
    k_blocks = -(-k // 64)
    if tokens > SKINNY_TOKENS and -(-tokens // 128) * -(-features // 256) >= PERSISTENT_TILES:
        if tokens >= PAIR_TOKENS:
            return 1
        tiles = -(-tokens // 128) * -(-features // 256)
        if tiles * 8 <= sms:                  # tiles of 128 features where those of 256 fill at most an eighth of the SMs (the launcher does the same)
            tiles = -(-tokens // 128) * -(-features // 128)
        splits = max(1, min(sms // tiles, k_blocks // PERSISTENT_SLICE_BLOCKS, 16))
        while splits > 1 and (splits - 1) * -(-k_blocks // splits) >= k_blocks:
            splits -= 1
        return splits
    tiles = -(-features // 128) * (1 if tokens <= SKINNY_TOKENS else -(-tokens // 128))
    return max(1, min(2 * sms // tiles, k_blocks // 4, 16))


def gemm_tcgen05_accumulates(tokens: int, features: int, k: int, sms: int | None = None) -> bool:
    """Whether the product of these sizes can be added into its output by the kernel itself: prompts
    on the persistent or CTA-pair kernel whose k is not cut into slices, so that every output tile
    has one writer."""
    return (tokens > SKINNY_TOKENS and -(-tokens // 128) * -(-features // 256) >= PERSISTENT_TILES
            and gemm_tcgen05_splits(tokens, features, k, sms) == 1)


def gemm_tcgen05_accumulate_pays(tokens: int, features: int, k: int, sms: int | None = None) -> bool:
    """Whether adding into the output inside the kernel is also the faster way.  Where the output's rows are a multiple
    of 16 bytes the tiles are added by tiled copies from shared memory, which read nothing back, and the norm after the
    product then reads the stream alone: taken wherever it can be (measured on a B200 with the 1B shape's output and down
    projections, whole prefill: 2,048 tokens 3.98 -> 3.91 ms, 4,096 tokens 8.62 -> 8.51).  Other widths add from
    registers after reading the old values, which pays only where every CTA (or CTA pair) has at least two tiles, so
    that a tile's epilogue runs under the next tile's products."""
    sms = sm_count() if sms is None else sms
    if not gemm_tcgen05_accumulates(tokens, features, k, sms):
        return False
    if features % 4 == 0:
        return True
    if tokens >= PAIR_TOKENS:
        return -(-tokens // 256) * -(-features // 256) >= 2 * (sms // 2)
    return -(-tokens // 128) * -(-features // 256) >= 2 * sms


_shares_words: dict[int, int] = {}


def gemm_tcgen05_shares_words() -> int:
    """int32 words of scratch memory with which the CTA pairs of a prompt's plain product may deal the tiles' k-blocks out
    evenly among themselves (``shares`` of :func:`gemm_tcgen05`): a share of a tile per epilogue warp, and a flag word
    each at the end, which must be zero before a call and is zero again after it."""
    device = torch.cuda.current_device()
    words = _shares_words.get(device)
    if words is None:
        lib = build.load("gemm_tcgen05")
        lib.tt_gemm_tcgen05_shares_bytes.argtypes = []
        lib.tt_gemm_tcgen05_shares_bytes.restype = c_longlong
        words = _shares_words[device] = int(lib.tt_gemm_tcgen05_shares_bytes()) // 4
    return words


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor, status: torch.Tensor,
                 operands_checked: bool = False, accumulate: bool = False, shares: torch.Tensor | None = None) -> None:
    """out[s] = x @ w[:, k-slice s].T on the tensor cores; bfloat16 operands, float32
    ``out`` [splits, tokens, features]; bias (float32) goes into slice 0.  ``operands_checked``: the
    caller has already called :func:`gemm_tcgen05_usable` on these operands.  ``accumulate``: the
    product is added to ``out`` [1, tokens, features] (only where :func:`gemm_tcgen05_accumulates`).
    ``shares``: zeroed int32 scratch memory of :func:`gemm_tcgen05_shares_words` words; with it, prompts on
    CTA pairs whose tiles would leave pairs idle share the tiles' k among the pairs."""
    _need(out, torch.float32, "gemm output")
    tokens, k = x.shape
    features = w.shape[0]
    if accumulate and (out.shape[0] != 1 or not gemm_tcgen05_accumulates(tokens, features, k)):
        raise KernelError(f"tcgen05 gemm cannot add a product of {tokens} x {features} x {k} into its output")
    if not (operands_checked or gemm_tcgen05_usable(x, w)) or w.shape[1] != k or tuple(out.shape[1:]) != (tokens, features):
        raise KernelError(f"tcgen05 gemm cannot take x {tuple(x.shape)} / w {tuple(w.shape)} / out {tuple(out.shape)} (k and strides must be multiples of 8)")
    if out.shape[0] > -(-k // 64):
        raise KernelError(f"{out.shape[0]} k-slices for k = {k}: a slice needs at least one block of 64")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    if shares is not None and (shares.dtype != torch.int32 or not shares.is_contiguous()):
        raise KernelError("the shares of a tcgen05 gemm must be contiguous int32")
    fn = _fn("gemm_tcgen05", "tt_gemm_tcgen05", [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_longlong,
                                                 c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_longlong])
    _check(fn(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out), out.stride(1), out.stride(0), tokens, features, k,
              out.shape[0], 2 if accumulate else 0, _ptr(status), _stream(), _ptr(shares), 0 if shares is None else shares.numel() * 4),
           "gemm_tcgen05")


def gemm_tcgen05_qkv_rope_takes(x: torch.Tensor, w: torch.Tensor, head_dim: int, rotary_dim: int) -> bool:
    """Whether the qkv product of these operands can rotate, narrow and append to the cache in its own epilogue:
    a prompt on the persistent or CTA-pair kernel without k-slices, head size 64 or 128 rotated whole."""
    if rotary_dim != head_dim or head_dim not in (64, 128) or not gemm_tcgen05_usable(x, w):
        return False
    lib = build.load("gemm_tcgen05")
    lib.tt_gemm_tcgen05_qkv_rope_takes.argtypes = [c_int, c_int, c_int, c_int]
    lib.tt_gemm_tcgen05_qkv_rope_takes.restype = c_int
    return bool(lib.tt_gemm_tcgen05_qkv_rope_takes(x.shape[0], w.shape[0], x.shape[1], head_dim))


def gemm_tcgen05_qkv_rope(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, q_out: torch.Tensor, k_pool: torch.Tensor,
                          v_pool: torch.Tensor, cos_sin: torch.Tensor, where: torch.Tensor, table: torch.Tensor, heads: int,
                          kv_heads: int, head_dim: int, attention_scaling: float, status: torch.Tensor) -> None:
    """The qkv projection of a prompt with the rotation, the narrowing to bfloat16 and the cache append done by the
    product's epilogue: q (rotated) to ``q_out`` [tokens, heads * head_dim], k (rotated) and v into the block pools at
    each token's position.  ``cos_sin`` and ``where`` are the step's :func:`rope_table`.  Only where
    :func:`gemm_tcgen05_qkv_rope_takes`."""
    tokens, k = x.shape
    q_cols, kv_cols = heads * head_dim, kv_heads * head_dim
    if w.shape != (q_cols + 2 * kv_cols, k) or tuple(q_out.shape) != (tokens, q_cols):
        raise KernelError(f"qkv product: w {tuple(w.shape)} / q_out {tuple(q_out.shape)} do not fit {heads}/{kv_heads} heads of {head_dim}")
    for t, name in ((q_out, "q_out"), (k_pool, "key pool"), (v_pool, "value pool")):
        _need(t, torch.bfloat16, name)
    if bias is not None:
        _need(bias, torch.float32, "bias")
    _need(cos_sin, torch.float32, "cos/sin table")
    _need(where, torch.int32, "token positions")
    if tuple(cos_sin.shape) != (tokens, head_dim // 2, 2) or tuple(where.shape) != (tokens, 2):
        raise KernelError("qkv product: the rope table does not fit the step")
    fn = _fn("gemm_tcgen05", "tt_gemm_tcgen05_qkv_rope", [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                          c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                                          c_void_p, c_void_p])
    code = fn(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias), tokens, k, _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _ptr(cos_sin),
              _ptr(where), _ptr(table), table.shape[1], k_pool.shape[0], heads, kv_heads, head_dim, attention_scaling, _ptr(status), _stream())
    if code < 0:
        raise KernelError("qkv product with rotation: " + ("a tensor map could not be made" if code == -1 else "the shape is not taken"))
    _check(code, "gemm_tcgen05_qkv_rope")


def gemm_tcgen05_failure_drill(wait_limit_ns: int, undelivered_bytes: int) -> None:
    """For tests of the failure path, never for serving.  ``wait_limit_ns``: the limit of every
    bounded wait in the tensor-core product kernels (0 restores the default of two seconds).
    ``undelivered_bytes``: from now on the first stage of the few-token and small-prompt kernel
    expects that many bytes more than its copies bring (0 restores normal operation), so its
    barrier never completes; the kernel must then raise ``STATUS_WAIT_EXPIRED``, free what it
    holds and return."""
    lib = build.load("gemm_tcgen05")
    lib.tt_gemm_tcgen05_set_wait_limit_ns.argtypes = [c_ulonglong]
    lib.tt_gemm_tcgen05_set_wait_limit_ns.restype = c_int
    lib.tt_gemm_tcgen05_expect_undelivered_bytes.argtypes = [c_int]
    lib.tt_gemm_tcgen05_expect_undelivered_bytes.restype = None
    code = lib.tt_gemm_tcgen05_set_wait_limit_ns(int(wait_limit_ns))
    if code != 0:
        raise KernelError(f"setting the wait limit failed: CUDA error {code}")
    lib.tt_gemm_tcgen05_expect_undelivered_bytes(int(undelivered_bytes))


def gemm_tcgen05_swiglu(x: torch.Tensor, w: torch.Tensor, act: torch.Tensor, status: torch.Tensor) -> None:
    """act = silu(x @ gate.T) * (x @ up.T) in bfloat16, where ``w`` [2 * inter, k] holds
    the gate rows followed by the up rows; the activation never exists in float32 in
    global memory."""
    _need(act, torch.bfloat16, "activation output")
    tokens, k = x.shape
    inter = w.shape[0] // 2
    if not gemm_tcgen05_usable(x, w) or w.shape[1] != k or tuple(act.shape) != (tokens, inter):
        raise KernelError(f"tcgen05 swiglu gemm cannot take x {tuple(x.shape)} / w {tuple(w.shape)} / act {tuple(act.shape)}")
    fn = _fn("gemm_tcgen05", "tt_gemm_tcgen05", [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_longlong,
                                                 c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_longlong])
    _check(fn(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(None), _ptr(act), act.stride(0), 0, tokens, inter, k, 1, 1,
              _ptr(status), _stream(), _ptr(None), 0), "gemm_tcgen05_swiglu")
