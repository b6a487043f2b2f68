"""Python face of the CUDA kernels: argument checks, then a ``ctypes`` call on the current stream.

Every function here launches hand-written kernels from this folder (matrix products
with many rows go to cuBLAS through ``torch.matmul``, as the reference's prefill does
with ``cublasGemmEx``/``cublasSgemm``, src/gpu_cuda.cu:11788-11879).  Nothing falls
back to the CPU: tensors that are not on a CUDA device are refused.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

from . import build

PAGE = 64  # tokens per cache page; must equal BN_PAGE in common.cuh

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}") from None


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _stream() -> c_void_p:
    """The current stream of the current device as a raw handle (asked of torch's C layer directly:
    ``torch.cuda.current_stream()`` builds a Python object per call, several microseconds of a launch)."""
    try:
        return c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))
    except AttributeError:  # a torch without these entry points
        return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None) -> None:
    # the usual case in one test (a launch asks this of ten tensors); what fails it is named below
    if (t.__class__ is torch.Tensor and t.is_cuda and t.is_contiguous() and (dtype is None or t.dtype is dtype)
            and (dims is None or t.dim() == dims)):
        return
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, got {tuple(t.shape)}")


def _check(status: int, what: str) -> None:
    if status == 0:
        return
    if status == 1:
        raise KernelError(f"{what}: sizes or pointers refused by the kernel launcher")
    raise KernelError(f"{what}: CUDA launch failed with error {status - 2}")


LAUNCHES = 0  # kernels of this library launched through this module (bench.py reads and resets it)
PROFILE = None  # a dict while kernel classes are being timed (engine/diagnostics.py): entry point -> [(event, event)]


def _timed(key: str, call):
    """Run ``call`` between two CUDA events kept under ``key`` (only while PROFILE is a dict)."""
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    out = call()
    b.record()
    PROFILE.setdefault(key, []).append((a, b))
    return out


_entry_points = {}  # (family, name) -> the library's entry point, its result type set


def _fn(family: str, name: str):
    global LAUNCHES
    LAUNCHES += 1
    f = _entry_points.get((family, name))
    if f is None:
        f = getattr(build.library(family), name)
        f.restype = c_int
        _entry_points[(family, name)] = f
    if PROFILE is not None:
        return lambda *args: _timed(f"{family}.{name}", lambda: f(*args))
    return f


# Arguments that never change, made once: building a ctypes object costs a fifth of a microsecond, and
# a launch has twenty of them.  (Python ints go to C as int without a wrapper; pointers need c_void_p,
# an int would be cut to 32 bits; floats need c_float.)
_NULL = c_void_p(None)
_F0 = c_float(0.0)


# ---- embedding ----------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, bad_token: torch.Tensor,
                 scale: float = 1.0) -> torch.Tensor:
    """out[t] = float32(table[tokens[t]]) * scale; sets bad_token[0] = 1 on an id outside the table."""
    _need(table, "table", dims=2)
    _need(tokens, "tokens", torch.int32, 1)
    _need(out, "out", torch.float32, 2)
    _need(bad_token, "bad_token", torch.int32)
    n, width = tokens.shape[0], table.shape[1]
    if out.shape[0] < n or out.shape[1] != width:
        raise KernelError(f"out {tuple(out.shape)} does not hold {n} rows of width {width}")
    _check(_fn("embed", "bn_embed_gather")(_ptr(table), _code(table), _ptr(tokens), _ptr(out), int(n),
                                           int(width), int(table.shape[0]), c_float(scale),
                                           _ptr(bad_token), _stream()), "embed_gather")
    return out


# ---- norm ---------------------------------------------------------------------------------
def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, write_x: bool = True) -> torch.Tensor:
    """x += delta (if given), out = rmsnorm(x) * weight.  With ``rows`` only those rows are read
    and ``out`` holds them densely; x is then left as it is."""
    _need(x, "x", torch.float32, 2)
    _need(weight, "weight", dims=1)
    _need(out, "out", dims=2)
    width = x.shape[1]
    if weight.shape[0] != width or out.shape[1] != width:
        raise KernelError(f"widths differ: x {width}, weight {weight.shape[0]}, out {out.shape[1]}")
    n_parts, part_stride = 1, 0
    if delta is not None:
        _need(delta, "delta")
        if delta.dim() == 3:  # partial sums of a product that split its inner dimension
            n_parts, part_stride = delta.shape[0], delta.shape[1] * delta.shape[2]
        if tuple(delta.shape[-2:]) != tuple(x.shape) or delta.dim() not in (2, 3):
            raise KernelError(f"delta {tuple(delta.shape)} does not match x {tuple(x.shape)}")
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n_rows, write_x = rows.shape[0], False
    else:
        n_rows = x.shape[0]
    if out.shape[0] < n_rows:
        raise KernelError(f"out has {out.shape[0]} rows, {n_rows} are written")
    _check(_fn("norm", "bn_add_rmsnorm")(_ptr(x), _ptr(delta), int(_code(delta) if delta is not None else 0),
                                         int(n_parts), ctypes.c_longlong(part_stride), _ptr(weight), int(_code(weight)), _ptr(out), int(_code(out)),
                                         _ptr(rows), int(n_rows), int(width), c_float(eps),
                                         int(1 if write_x else 0), _stream()), "add_rmsnorm")
    return out


# ---- activation ---------------------------------------------------------------------------
def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Stack gate and up rows as alternating blocks of 8 rows: [g0..g7, u0..u7, g8..g15, u8..u15, ...]."""
    I, K = gate.shape
    if I % 8:
        raise KernelError(f"feed-forward width {I} must be a multiple of 8")
    return torch.stack([gate.reshape(I // 8, 8, K), up.reshape(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()


def silu_mul(h: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, i] = silu(gate_i) * up_i for rows of h that alternate 8 gate and 8 up values
    (the layout ``interleave_gate_up`` gives the product's output)."""
    _need(h, "h", dims=2)
    _need(out, "out", h.dtype, 2)
    inter = h.shape[1] // 2
    if h.shape[1] != 2 * inter or out.shape != (h.shape[0], inter):
        raise KernelError(f"silu_mul: h {tuple(h.shape)} and out {tuple(out.shape)} do not fit")
    _check(_fn("act", "bn_silu_mul")(_ptr(h), _ptr(out), int(_code(h)), int(h.shape[0]), int(inter),
                                     _stream()), "silu_mul")
    return out


def scale_softcap(x: torch.Tensor, scale: float, softcap: float) -> torch.Tensor:
    """In place on float32 x: x * scale, then softcap * tanh(x / softcap) when softcap is not 0."""
    _need(x, "x", torch.float32)
    _check(_fn("act", "bn_scale_softcap")(_ptr(x), ctypes.c_longlong(x.numel()), c_float(scale), c_float(softcap),
                                          _stream()), "scale_softcap")
    return x


# ---- rotary + cache append ----------------------------------------------------------------
def rope_append(x: torch.Tensor, n_rot_heads: int, head_dim: int, rotary_dims: int, theta_scale: float,
                tok_pos: torch.Tensor, *, k_off: int = 0, v_off: int = 0, n_kv_heads: int = 0,
                tok_seq: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
                page_table: Optional[torch.Tensor] = None, k_cache: Optional[torch.Tensor] = None,
                v_cache: Optional[torch.Tensor] = None) -> None:
    """Rotate the first ``n_rot_heads`` heads of every row of x in place; when a cache is given,
    write the key heads at ``k_off`` and the value heads at ``v_off`` of each row into it."""
    _need(x, "x", dims=2)
    _need(tok_pos, "tok_pos", torch.int32, 1)
    n = tok_pos.shape[0]
    if x.shape[0] < n or n_rot_heads * head_dim > x.shape[1]:
        raise KernelError("rope_append: x is too small for the heads and tokens given")
    pt_stride = 0
    if k_cache is not None:
        for t, nm in ((tok_seq, "tok_seq"), (slots, "slots")):
            _need(t, nm, torch.int32, 1)
        _need(page_table, "page_table", torch.int32, 2)
        _need(k_cache, "k_cache", x.dtype, 4)
        _need(v_cache, "v_cache", x.dtype, 4)
        if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
            raise KernelError(f"rope_append: cache {tuple(k_cache.shape)} is not [pages, {n_kv_heads}, {PAGE}, {head_dim}]")
        if max(k_off, v_off) + n_kv_heads * head_dim > x.shape[1]:
            raise KernelError("rope_append: key/value offsets run past the row")
        pt_stride = page_table.shape[1]
    _check(_fn("rope", "bn_rope_append")(_ptr(x), int(_code(x)), int(n), int(x.shape[1]), int(n_rot_heads),
                                         int(head_dim), int(rotary_dims), c_float(theta_scale), _ptr(tok_pos),
                                         int(k_off), int(v_off), int(n_kv_heads), _ptr(tok_seq), _ptr(slots),
                                         _ptr(page_table), int(pt_stride), _ptr(k_cache), _ptr(v_cache),
                                         _stream()), "rope_append")


# ---- attention ----------------------------------------------------------------------------
def attention_general(q: torch.Tensor, q_stride: int, out: torch.Tensor, n_tokens: int, n_heads: int,
                      n_kv_heads: int, head_dim: int, scale: float, window: int, tok_seq: torch.Tensor,
                      tok_pos: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                      k_cache: torch.Tensor, v_cache: torch.Tensor) -> torch.Tensor:
    """Causal attention of every new token over its sequence's pages; q may be a view into a wider row."""
    if not q.is_cuda or q.stride(-1) != 1:
        raise KernelError("attention: q must be a CUDA tensor with unit inner stride")
    _need(out, "out", q.dtype, 2)
    for t, nm in ((tok_seq, "tok_seq"), (tok_pos, "tok_pos"), (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    _need(k_cache, "k_cache", q.dtype, 4)
    _need(v_cache, "v_cache", q.dtype, 4)
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention: cache {tuple(k_cache.shape)} is not [pages, {n_kv_heads}, {PAGE}, {head_dim}]")
    if head_dim % 16 or head_dim > 256:
        raise KernelError(f"attention: head_dim={head_dim} must be a multiple of 16 up to 256")
    if n_heads % n_kv_heads:
        raise KernelError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} key/value heads")
    if out.shape[0] < n_tokens or out.shape[1] != n_heads * head_dim:
        raise KernelError("attention: out does not fit")
    _check(_fn("attention", "bn_attention_general")(
        _ptr(q), int(q_stride), _ptr(out), int(out.shape[1]), int(_code(q)), int(n_tokens), int(n_heads),
        int(n_kv_heads), int(head_dim), c_float(scale), int(window), _ptr(tok_seq), _ptr(tok_pos),
        _ptr(slots), _ptr(page_table), int(page_table.shape[1]), _ptr(k_cache), _ptr(v_cache), _stream()),
        "attention_general")
    return out


def attention_prefill(q: torch.Tensor, q_stride: int, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                      scale: float, window: int, tile_seq: torch.Tensor, tile_row0: torch.Tensor,
                      seq_start: torch.Tensor, seq_pos0: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                      k_cache: torch.Tensor, v_cache: torch.Tensor) -> torch.Tensor:
    """bfloat16 causal attention of runs of new tokens on the tensor cores; block i handles up to 64
    new tokens of sequence tile_seq[i] from its row tile_row0[i] on."""
    if not q.is_cuda or q.stride(-1) != 1 or q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill: q must be a bfloat16 CUDA tensor with unit inner stride")
    _need(out, "out", torch.bfloat16, 2)
    for t, nm in ((tile_seq, "tile_seq"), (tile_row0, "tile_row0"), (seq_start, "seq_start"), (seq_pos0, "seq_pos0"),
                  (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention_prefill: cache {tuple(k_cache.shape)} is not [pages, {n_kv_heads}, {PAGE}, {head_dim}]")
    if head_dim % 16 or head_dim > 256 or n_heads % n_kv_heads:
        raise KernelError(f"attention_prefill: head_dim={head_dim}, heads {n_heads}/{n_kv_heads} not supported")
    if out.shape[1] != n_heads * head_dim or q_stride % 8:
        raise KernelError("attention_prefill: out or q_stride does not fit")
    _check(_fn("attention_prefill", "bn_attention_prefill")(
        _ptr(q), int(q_stride), _ptr(out), int(out.shape[1]), int(tile_seq.shape[0]), int(n_heads),
        int(n_kv_heads), int(head_dim), c_float(scale), int(window), _ptr(tile_seq), _ptr(tile_row0),
        _ptr(seq_start), _ptr(seq_pos0), _ptr(slots), _ptr(page_table), int(page_table.shape[1]), _ptr(k_cache),
        _ptr(v_cache), _stream()), "attention_prefill")
    return out


USE_TCGEN05_ATTENTION = True  # prefill attention with head sizes up to 128 runs on tcgen05 (attention_prefill_tc.cu)


def attention_prefill_tc(q: torch.Tensor, q_stride: int, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                         scale: float, window: int, tile_seq: torch.Tensor, tile_row0: torch.Tensor,
                         seq_start: torch.Tensor, seq_pos0: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                         k_cache: torch.Tensor, v_cache: torch.Tensor) -> torch.Tensor:
    """bfloat16 causal attention of runs of new tokens on tcgen05 tensor cores with TMA-fed operands;
    block i handles up to 128 new tokens of sequence tile_seq[i] from its row tile_row0[i] on.
    Head sizes up to 128."""
    if not q.is_cuda or q.dim() != 2 or q.stride(-1) != 1 or q.stride(0) != q_stride or q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_tc: q must be a bfloat16 CUDA matrix with unit inner stride")
    _need(out, "out", torch.bfloat16, 2)
    for t, nm in ((tile_seq, "tile_seq"), (tile_row0, "tile_row0"), (seq_start, "seq_start"), (seq_pos0, "seq_pos0"),
                  (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention_prefill_tc: cache {tuple(k_cache.shape)} is not [pages, {n_kv_heads}, {PAGE}, {head_dim}]")
    if head_dim % 16 or head_dim > 128 or n_heads % n_kv_heads:
        raise KernelError(f"attention_prefill_tc: head_dim={head_dim}, heads {n_heads}/{n_kv_heads} not supported")
    if out.shape[1] != n_heads * head_dim or q_stride % 8 or n_heads * head_dim > q_stride or out.shape[0] < q.shape[0]:
        raise KernelError("attention_prefill_tc: out or q_stride does not fit")
    _check(_fn("attention_prefill_tc", "bn_attention_prefill_tc")(
        _ptr(q), int(q_stride), int(q.shape[0]), _ptr(out), int(out.shape[1]), int(tile_seq.shape[0]),
        int(n_heads), int(n_kv_heads), int(head_dim), c_float(scale), int(window), _ptr(tile_seq), _ptr(tile_row0),
        _ptr(seq_start), _ptr(seq_pos0), _ptr(slots), _ptr(page_table), int(page_table.shape[1]), _ptr(k_cache),
        _ptr(v_cache), int(k_cache.shape[0]), _ptr(tc_status(q.device)), _stream()), "attention_prefill_tc")
    return out


DECODE_CHUNK = 128  # positions per block of the decode attention; must equal DEC_CHUNK in attention_decode.cu


def attention_decode(q: torch.Tensor, q_stride: int, out: torch.Tensor, n_seqs: int, n_heads: int, n_kv_heads: int,
                     head_dim: int, scale: float, window: int, tok_pos: torch.Tensor, slots: torch.Tensor,
                     page_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, max_len: int) -> torch.Tensor:
    """bfloat16 attention of one new token per sequence (row b of q is sequence b), split over the
    keys.  ``max_len`` bounds every sequence's length after this step; it sizes the scratch."""
    if not q.is_cuda or q.stride(-1) != 1 or q.dtype != torch.bfloat16:
        raise KernelError("attention_decode: q must be a bfloat16 CUDA tensor with unit inner stride")
    _need(out, "out", torch.bfloat16, 2)
    for t, nm in ((tok_pos, "tok_pos"), (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention_decode: cache {tuple(k_cache.shape)} is not [pages, {n_kv_heads}, {PAGE}, {head_dim}]")
    if head_dim % 16 or head_dim > 256 or n_heads % n_kv_heads:
        raise KernelError(f"attention_decode: head_dim={head_dim}, heads {n_heads}/{n_kv_heads} not supported")
    if out.shape[0] < n_seqs or out.shape[1] != n_heads * head_dim or tok_pos.shape[0] < n_seqs:
        raise KernelError("attention_decode: out or tok_pos does not fit")
    n_splits = max(1, (max_len + DECODE_CHUNK - 1) // DECODE_CHUNK)
    part_o = torch.empty((n_seqs * n_heads * n_splits * head_dim,), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((n_seqs * n_heads * n_splits * 2,), dtype=torch.float32, device=q.device)
    _check(_fn("attention_decode", "bn_attention_decode")(
        _ptr(q), int(q_stride), _ptr(out), int(out.shape[1]), int(n_seqs), int(n_heads), int(n_kv_heads),
        int(head_dim), c_float(scale), int(window), _ptr(tok_pos), _ptr(slots), _ptr(page_table),
        int(page_table.shape[1]), _ptr(k_cache), _ptr(v_cache), _ptr(part_o), _ptr(part_ml), int(n_splits),
        _stream()), "attention_decode")
    return out


_FORCE_SPLITS = 0  # tests and experiments: a fixed number of blocks per sequence in attention_decode_fused
# (more than eight take the path that merges through global memory and a ticket)


def decode_splits(pages: int, blocks_per_split: int) -> int:
    """How many blocks share one sequence's pages in ``attention_decode_fused``.

    A block walks its pages one after another, about 0.75 us each; blocks that share a sequence
    merge their results inside a thread-block cluster, which costs about as much as five pages.
    So a split pays only when it shortens the walk by more than that: few sequences, or long
    ones.  Up to eight blocks per sequence are one cluster; more (up to 32) merge through global
    memory block by block, which costs as much as 0.7 pages more for every block and pays from
    some 16,000 positions on for one or two sequences.  No more than 256 blocks in all: clusters
    are placed within one GPC, and beyond that number a second wave of blocks starts.
    ``pages`` is the bound the step was recorded for; sequences are taken to fill three quarters
    of it, and the kernel shares a sequence's pages evenly among its blocks whatever the bound.
    Measured at 8 key/value heads of 128 (us, 520 positions, 1 against the chosen number of
    splits): 1 sequence 10.3 / 5.5, 4: 10.6 / 7.6, 8: 11.4 / 10.2, 12: 12.2 / 11.2 (three
    splits 18.6), 16: 12.6 / 12.2 (four 20.1), 24: 13.6 (two 15.7); at 2,000 positions 8
    sequences 31.7 / 15.6, 16: 34.9 / 26.0; one sequence of 64,000 positions: 8 splits 111, 32
    splits 59."""
    cap = max(1, min(pages, 256 // max(1, blocks_per_split)))
    filled = 0.75 * pages
    best, best_cost = 1, filled
    for s in (2, 3, 4, 5, 6, 7, 8, 12, 16, 24, 32):
        if s > cap:
            break
        cost = float(-(-int(filled) // s)) + (5.0 if s <= 8 else 5.0 + 0.7 * s)
        if cost < best_cost:
            best, best_cost = s, cost
    return best


DECODE_ITEM_BLOCKS = 450  # a work list may come to so many blocks (three per SM run at once)
_FORCE_ITEM_GROUP = 0  # tests: a work list in groups of this many whatever the batch


def decode_items(seq_pages, blocks_per_seq: int, group: Optional[int] = None, capacity: Optional[int] = None):
    """For a batch of unequal lengths: which block of ``attention_decode_fused`` works on what.

    ``seq_pages[b]`` is the number of cache pages sequence b's new token sees.  Returns
    ``(group, items)`` or None when the plain grid (every sequence alike) serves as well: few
    blocks (the plain grid then splits every sequence), lengths that differ little, or so many
    sequences that more blocks would only queue.  ``items`` lists, in the order in which blocks
    start, ``sequence | split << 16 | splits << 24`` or -1 (nothing); its length is a multiple of
    ``group``, and each run of ``group`` entries (one thread-block cluster) is either the
    ``group`` splits of one long sequence or sequences that are not split.  A sequence is long
    when it has more than 1/group of the longest one's pages; long sequences come first, so that
    the launch does not end on them.  ``group`` is the largest of 2, 3, 4 that keeps the blocks
    within ``DECODE_ITEM_BLOCKS``.  Measured (us per launch, plain grid against work list): 8
    sequences of 513 to 2,560 positions at 40 heads of 128: 49 / 34; 32 sequences of 129 to 2,176
    at 8 key/value heads of 128: 36 / 31; 64 such sequences at 8 heads of 64: 37 / 40 (not used).
    With ``group`` given (a recorded step keeps the shape of its grid) only the list is made,
    padded to ``capacity`` entries."""
    n = len(seq_pages)
    if n == 0 or n > 65535:
        return None
    total, longest = sum(seq_pages), max(seq_pages)

    def long_ones(s: int):
        limit = -(-longest // s)
        return [b for b in range(n) if seq_pages[b] > limit]

    def fits(s: int) -> bool:
        k = len(long_ones(s))
        return (s * k + n - k) * blocks_per_seq <= DECODE_ITEM_BLOCKS

    uneven = longest >= 12 and longest * n >= 1.5 * total
    if group is None and _FORCE_ITEM_GROUP:
        group = _FORCE_ITEM_GROUP
        chosen = long_ones(group) if group > 1 else []
    elif group is None:
        sizes = [s for s in (2, 3, 4) if fits(s)]
        if n * blocks_per_seq <= 128 or not uneven or not sizes:
            return None
        group = max(sizes)
        chosen = long_ones(group)
    else:
        # the grid's shape is given; if the batch has meanwhile become even, or splitting its long
        # sequences would now take too many blocks, nothing is split and the list only orders
        chosen = long_ones(group) if group > 1 and (_FORCE_ITEM_GROUP or (uneven and fits(group))) else []
    is_long = set(chosen)
    items = []
    for b in sorted(chosen, key=lambda b: -seq_pages[b]):
        items.extend(b | (z << 16) | (group << 24) for z in range(group))
    items.extend(b | (1 << 24) for b in sorted((b for b in range(n) if b not in is_long), key=lambda b: -seq_pages[b]))
    size = capacity if capacity is not None else -(-len(items) // group) * group
    if len(items) > size or size % group:
        raise KernelError(f"decode_items: {len(items)} entries do not fit a capacity of {size} in groups of {group}")
    items.extend([-1] * (size - len(items)))
    return group, items


def attention_decode_fused(qkv: torch.Tensor, k_off: int, v_off: int, out: torch.Tensor, n_seqs: int, n_heads: int,
                           n_kv_heads: int, head_dim: int, scale: float, window: int, rotary_dims: int,
                           theta_scale: float, tok_pos: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                           k_cache: torch.Tensor, v_cache: torch.Tensor, max_len: int,
                           items: Optional[torch.Tensor] = None, item_group: int = 0) -> torch.Tensor:
    """The decode step's attention in one launch on tensor cores (attention_decode_tc.cu): rotary
    encoding of the raw queries and of the new key (``rotary_dims`` = 0: none), the new key and value
    written into the cache at ``tok_pos``, attention split over the keys, and the combination of
    the splits.  ``qkv`` holds one raw
    q|k|v row per sequence with the key heads at element ``k_off`` and the value heads at ``v_off``.
    ``items`` / ``item_group``: the work list of ``decode_items`` on the device, for batches of
    unequal lengths."""
    _need(qkv, "qkv", torch.bfloat16, 2)
    _need(out, "out", torch.bfloat16, 2)
    for t, nm in ((tok_pos, "tok_pos"), (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention_decode_fused: cache {tuple(k_cache.shape)} is not [pages, {n_kv_heads}, {PAGE}, {head_dim}]")
    if head_dim % 16 or head_dim > 256 or n_heads % n_kv_heads or rotary_dims % 2 or rotary_dims > head_dim:
        raise KernelError(f"attention_decode_fused: head_dim={head_dim}, heads {n_heads}/{n_kv_heads}, "
                          f"rotary_dims={rotary_dims} not supported")
    if max(k_off, v_off) + n_kv_heads * head_dim > qkv.shape[1] or n_heads * head_dim > qkv.shape[1]:
        raise KernelError("attention_decode_fused: offsets run past the row")
    if out.shape[0] < n_seqs or out.shape[1] != n_heads * head_dim or tok_pos.shape[0] < n_seqs or qkv.shape[0] < n_seqs:
        raise KernelError("attention_decode_fused: out, qkv or tok_pos does not fit")
    if items is not None:
        _need(items, "items", torch.int32, 1)
        if not 1 <= item_group <= 8 or items.shape[0] % item_group or items.shape[0] == 0:
            raise KernelError(f"attention_decode_fused: {items.shape[0]} items in groups of {item_group}")
        part_o = torch.empty((n_seqs * n_heads * item_group * head_dim,), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((n_seqs * n_heads * item_group * 2,), dtype=torch.float32, device=qkv.device)
        _scr, counters = _split_scratch(qkv.device)
        _check(_fn("attention_decode_tc", "bn_attention_decode_tc_items")(
            _ptr(qkv), int(qkv.shape[1]), int(k_off), int(v_off), _ptr(out), int(out.shape[1]), int(n_seqs),
            int(n_heads), int(n_kv_heads), int(head_dim), c_float(scale), int(window), int(rotary_dims),
            c_float(theta_scale), _ptr(tok_pos), _ptr(slots), _ptr(page_table), int(page_table.shape[1]), _ptr(k_cache),
            _ptr(v_cache), int(k_cache.shape[0]), _ptr(tc_status(qkv.device)), _ptr(part_o), _ptr(part_ml), _ptr(counters),
            int(counters.numel()), _ptr(items), int(items.shape[0]), int(item_group), _stream()), "attention_decode_fused")
        return out
    pages = max(1, (max_len + PAGE - 1) // PAGE)
    blocks_per_split = n_seqs * n_kv_heads * ((n_heads // n_kv_heads + 15) // 16)
    want_splits = decode_splits(pages, blocks_per_split)
    if _FORCE_SPLITS:
        want_splits = max(1, min(pages, _FORCE_SPLITS))
    pages_per_block = (pages + want_splits - 1) // want_splits
    n_splits = (pages + pages_per_block - 1) // pages_per_block
    part_o = torch.empty((n_seqs * n_heads * n_splits * head_dim,), dtype=torch.float32, device=qkv.device)
    part_ml = torch.empty((n_seqs * n_heads * n_splits * 2,), dtype=torch.float32, device=qkv.device)
    _scr, counters = _split_scratch(qkv.device)
    _check(_fn("attention_decode_tc", "bn_attention_decode_tc")(
        _ptr(qkv), int(qkv.shape[1]), int(k_off), int(v_off), _ptr(out), int(out.shape[1]), int(n_seqs),
        int(n_heads), int(n_kv_heads), int(head_dim), c_float(scale), int(window), int(rotary_dims),
        c_float(theta_scale), _ptr(tok_pos), _ptr(slots), _ptr(page_table), int(page_table.shape[1]), _ptr(k_cache),
        _ptr(v_cache), int(k_cache.shape[0]), _ptr(tc_status(qkv.device)), _ptr(part_o), _ptr(part_ml), int(n_splits),
        int(pages_per_block), _ptr(counters),
        int(counters.numel()), _stream()), "attention_decode_fused")
    return out


# ---- matrix products ----------------------------------------------------------------------
SKINNY_MAX_ROWS = 16  # float32: warp-per-column kernel up to this many rows
MMA_MAX_ROWS = 64  # bfloat16: the streaming kernels (linear_tc.cu, linear_mma.cu) up to this many rows; the library
# product is faster beyond (5.5 against 5.8 ms for a decode step of 96 sequences at 32 layers of width 4096)
TC_MAX_ROWS = MMA_MAX_ROWS
USE_TCGEN05 = True  # small-batch bfloat16 products run on tcgen05 (linear_tc.cu); False: mma.sync (linear_mma.cu)
_n_sms = {}


def n_sms(device) -> int:
    """Streaming multiprocessors of ``device`` (asked once)."""
    key = torch.device(device).index or 0
    if key not in _n_sms:
        _n_sms[key] = int(torch.cuda.get_device_properties(key).multi_processor_count)
    return _n_sms[key]



_SCRATCH_FLOATS = 8 * 1024 * 1024  # 32 MB of split-K partial tiles, shared by all products of a device
_N_COUNTERS = 8192
_scratch = {}


def _split_scratch(device):
    """Scratch and ticket counters of the split-K reduction, one set per device, made on first use."""
    key = torch.device(device).index or 0
    got = _scratch.get(key)
    if got is None:
        got = _scratch[key] = (torch.empty(_SCRATCH_FLOATS, dtype=torch.float32, device=device),
                               torch.zeros(_N_COUNTERS, dtype=torch.int32, device=device))
    return got


def _mma_splits(M: int, N: int, K: int, sms: int) -> int:
    """How many ways the inner dimension is split so that about four blocks per SM stream weights."""
    blocks = (N + 63) // 64
    want = 4 * sms
    if blocks >= want or blocks > _N_COUNTERS:
        return 1
    mp = 8 if M <= 8 else 16 if M <= 16 else 32 if M <= 32 else 64
    fit = _SCRATCH_FLOATS // (blocks * 64 * mp)
    splits = max(1, min((want + blocks - 1) // blocks, K // 256, fit))
    chunks = (K + 127) // 128  # the kernel works in chunks of 128 along K and leaves no split empty
    per = (chunks + splits - 1) // splits
    return (chunks + per - 1) // per


_tc_status = {}


def tc_status(device) -> torch.Tensor:
    """One int per device that a TMA-fed kernel (the tcgen05 product, the tensor-core decode
    attention) sets when a wait inside it gave up (0 = fine)."""
    key = torch.device(device).index or 0
    got = _tc_status.get(key)
    if got is None:
        got = _tc_status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return got


_tc_status_ptr = {}


def _tc_status_arg(device: torch.device) -> c_void_p:
    """The status word of ``device`` as a launch argument (made once per device)."""
    got = _tc_status_ptr.get(device.index)
    if got is None:
        got = _tc_status_ptr[device.index] = _ptr(tc_status(device))
    return got


def check_tc_status(device) -> None:
    """Raise if a TMA-fed kernel on ``device`` reported a wait that gave up (synchronises)."""
    code = int(tc_status(device).item())
    if code:
        tc_status(device).zero_()
        _split_scratch(device)[1].zero_()  # tickets of the launch that gave up may be left over
        what = {1: "linear_tc: a stage never filled (TMA load)", 2: "linear_tc: a stage was never released (MMA commit)",
                3: "linear_tc: the accumulator never completed",
                4: "attention_decode_tc: a cache page never arrived (TMA load)",
                5: "attention_prefill_tc: a wait inside the kernel gave up",
                6: "linear_tc: a slice of partial sums from another block of the cluster never arrived",
                7: "gemm_tc: a wait inside the kernel gave up"}.get(code, f"code {code}")
        raise KernelError(f"{what}; the result of that launch is not valid")


class RowScaled:
    """Rows of activations that still lack their RMS scale: the value of row m is
    ``x[m] / sqrt(sum_p ss[p, m] / width + eps)``.  A product whose epilogue added to the residual
    (``linear(..., sink=...)``) leaves the next norm's output in this form: x = residual * gain in
    bfloat16 and, per block of the product, the sum of squares of its slice of every residual row.
    The product that consumes the rows scales its result rows instead (W (s x) = s (W x))."""

    def __init__(self, x: torch.Tensor, ss: torch.Tensor, width: int, eps: float):
        self.x, self.ss, self.width, self.eps = x, ss, int(width), float(eps)

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype

    @property
    def device(self):
        return self.x.device

    def dense(self) -> torch.Tensor:
        """The rows with their scale applied (for a consumer that cannot apply it itself)."""
        scale = torch.rsqrt(self.ss.sum(0)[: self.x.shape[0]] / self.width + self.eps)
        return (self.x.float() * scale[:, None]).to(self.x.dtype)


class NormSink:
    """Where a product's result goes when the RMSNorm after it is fused into its epilogue: the
    float32 residual it is added to, and that norm's weight and eps."""

    def __init__(self, residual: torch.Tensor, weight: torch.Tensor, eps: float):
        self.residual, self.weight, self.eps = residual, weight, float(eps)


USE_FUSED_NORM = True  # products of few rows add to the residual and prepare the next norm in their epilogue
# (tests and comparisons set it to False)


def linear_tc(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None, swiglu: bool = False,
              cluster: int = 0, sink: Optional[NormSink] = None, _checked: bool = False):
    """x[M, K] . w[N, K]^T for M <= 64 in bfloat16 on tcgen05 tensor cores with TMA-fed operands.
    ``cluster`` blocks (1 to 8) share the inner dimension of each 128-row tile of w and add their
    parts up through distributed shared memory (0: chosen from the number of tiles).  ``x`` may be
    ``RowScaled``.  With ``sink`` the product is added to ``sink.residual`` in place and the result
    is the ``RowScaled`` output of the norm that follows.  (``_checked``: ``linear`` has looked at w
    and at the sizes already.)"""
    scaled = x if isinstance(x, RowScaled) else None
    if scaled is not None:
        x = scaled.x
    _need(x, "x", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if not _checked:
        _need(w, "w", torch.bfloat16, 2)
        if w.shape[1] != K or M > TC_MAX_ROWS or K % 8 or (swiglu and N % 16) or not 0 <= cluster <= 8:
            raise KernelError(f"linear_tc: x {tuple(x.shape)}, w {tuple(w.shape)}, cluster {cluster} not supported")
    fn = _fn("linear_tc", "bn_linear_tc_ex")
    dev = x.device
    if scaled is not None:
        ss_rows = scaled.ss
        _need(ss_rows, "ss", torch.float32, 2)
        if ss_rows.shape[1] < M or scaled.width != K:
            raise KernelError(f"linear_tc: row sums {tuple(ss_rows.shape)} of width {scaled.width} do not fit x {tuple(x.shape)}")
        row = (c_void_p(ss_rows.data_ptr()), ss_rows.shape[0], ss_rows.shape[1], c_float(1.0 / scaled.width), c_float(scaled.eps))
    else:
        row = (_NULL, 0, 0, _F0, _F0)
    if sink is not None:
        res = sink.residual
        _need(res, "residual", torch.float32, 2)
        _need(sink.weight, "norm weight", dims=1)
        if swiglu or tuple(res.shape) != (M, N) or sink.weight.shape[0] != N or sink.weight.dtype not in _DT:
            raise KernelError(f"linear_tc: residual {tuple(res.shape)} / norm weight {tuple(sink.weight.shape)} do not fit "
                              f"a product [{M}, {N}]")
        if cluster == 0:
            cluster = _auto_cluster(N, K)
        tiles = (N + 127) // 128
        xg = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        ss = torch.empty((tiles * cluster, M), dtype=torch.float32, device=dev)
        _check(fn(c_void_p(x.data_ptr()), c_void_p(w.data_ptr()), c_void_p(res.data_ptr()), 0, M, N, K, N, 3,
                  cluster, *row, c_void_p(sink.weight.data_ptr()), _DT[sink.weight.dtype], c_void_p(xg.data_ptr()),
                  c_void_p(ss.data_ptr()), M, _tc_status_arg(dev), _stream()), "linear_tc")
        return RowScaled(xg, ss, N, sink.eps)
    out_dtype = out_dtype or x.dtype
    cols = N // 2 if swiglu else N
    out = torch.empty((M, cols), dtype=out_dtype, device=dev)
    _check(fn(c_void_p(x.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), _DT[out_dtype], M, N, K, cols,
              2 if swiglu else 0, cluster, *row, _NULL, 0, _NULL, _NULL, 0, _tc_status_arg(dev), _stream()), "linear_tc")
    return out


_auto_clusters = {}  # (N, K) -> how many blocks share a tile's inner dimension (a property of the sizes and the device)


def _auto_cluster(N: int, K: int) -> int:
    got = _auto_clusters.get((N, K))
    if got is None:
        f = getattr(build.library("linear_tc"), "bn_linear_tc_auto_cluster")
        f.restype = c_int
        got = _auto_clusters[(N, K)] = int(f(int(N), int(K)))
    return got


# Many-row bfloat16 products on this library's tcgen05 kernel (gemm_tc.cu) instead of the library product
# followed by separate kernels.  "fused": where the kernel's epilogue replaces a pass over the activations
# and that saves more than its main loop loses against the library's (measured on a B200 at widths 4096
# and 14336: the SwiGLU epilogue from 1,024 rows on, 0.88 to 0.98 of the library product + activation
# kernel; the residual + norm epilogue from 2,048 rows on for inner sizes up to 8192, 0.85 to 0.95 of the
# library product + norm kernel; plain products are 1.09 to 1.16 of the library's and stay there).
# True: every product that fits.  False: none.
USE_OWN_GEMM = "fused"
GEMM_MIN_ROWS = 65            # True: from so many rows on
OWN_GEMM_SWIGLU_MIN_ROWS = 1024
OWN_GEMM_SINK_MIN_ROWS = 2048
OWN_GEMM_SINK_MAX_K = 8192


def own_gemm_sink_rows(rows: int) -> bool:
    """Whether a product of so many rows may take the residual + norm epilogue of ``gemm_tc``."""
    if USE_OWN_GEMM is True:
        return rows >= GEMM_MIN_ROWS
    return USE_OWN_GEMM == "fused" and rows >= OWN_GEMM_SINK_MIN_ROWS


def gemm_tc(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None, swiglu: bool = False,
            sink: Optional[NormSink] = None):
    """x[M, K] . w[N, K]^T for many rows in bfloat16 on tcgen05 tensor cores (gemm_tc.cu).  ``x`` may be
    ``RowScaled``; ``swiglu`` and ``sink`` as for ``linear`` (the activation, or the residual add with
    the next norm's gain and sums of squares, happen in the product's epilogue)."""
    scaled = x if isinstance(x, RowScaled) else None
    if scaled is not None:
        x = scaled.x
    _need(x, "x", torch.bfloat16, 2)
    _need(w, "w", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or K % 8 or N % 8 or (swiglu and N % 16) or (swiglu and sink is not None):
        raise KernelError(f"gemm_tc: x {tuple(x.shape)}, w {tuple(w.shape)} not supported")
    fn = _fn("gemm_tc", "bn_gemm_tc")
    if scaled is not None:
        _need(scaled.ss, "ss", torch.float32, 2)
        if scaled.ss.shape[1] < M or scaled.width != K:
            raise KernelError(f"gemm_tc: row sums {tuple(scaled.ss.shape)} of width {scaled.width} do not fit x {tuple(x.shape)}")
        row = (_ptr(scaled.ss), int(scaled.ss.shape[0]), int(scaled.ss.shape[1]), c_float(1.0 / scaled.width),
               c_float(scaled.eps))
    else:
        row = (c_void_p(None), int(0), int(0), c_float(0.0), c_float(0.0))
    status = _ptr(tc_status(x.device))
    if sink is not None:
        res = sink.residual
        _need(res, "residual", torch.float32, 2)
        _need(sink.weight, "norm weight", dims=1)
        if scaled is not None or tuple(res.shape) != (M, N) or sink.weight.shape[0] != N or sink.weight.dtype not in _DT:
            raise KernelError(f"gemm_tc: residual {tuple(res.shape)} / norm weight {tuple(sink.weight.shape)} do not fit "
                              f"a product [{M}, {N}]")
        xg = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        parts = getattr(build.library("gemm_tc"), "bn_gemm_tc_parts")
        parts.restype = c_int
        ss = torch.empty((parts(int(N)), M), dtype=torch.float32, device=x.device)
        _check(fn(_ptr(x), _ptr(w), int(M), int(N), int(K), c_void_p(None), int(0), int(0), int(3), *row,
                  _ptr(res), _ptr(sink.weight), int(_DT[sink.weight.dtype]), _ptr(xg), _ptr(ss), int(M), status,
                  _stream()), "gemm_tc")
        return RowScaled(xg, ss, N, sink.eps)
    out_dtype = out_dtype or x.dtype
    cols = N // 2 if swiglu else N
    out = torch.empty((M, cols), dtype=out_dtype, device=x.device)
    _check(fn(_ptr(x), _ptr(w), int(M), int(N), int(K), _ptr(out), int(_DT[out_dtype]), int(cols),
              int(2 if swiglu else 0), *row, c_void_p(None), c_void_p(None), int(0), c_void_p(None), c_void_p(None),
              int(0), status, _stream()), "gemm_tc")
    return out


def gemm_pairs(on: Optional[bool] = None) -> bool:
    """Whether ``gemm_tc`` runs pairs of blocks as one (tcgen05 cta_group::2, the default) or every block
    alone; with an argument, sets it.  Returns the setting before the call."""
    f = getattr(build.library("gemm_tc"), "bn_gemm_tc_pairs")
    f.restype = c_int
    return bool(f(int(-1 if on is None else int(bool(on)))))


def _own_gemm_fits(x, w: torch.Tensor, swiglu: bool, out_dtype, kind: str) -> bool:
    """``kind``: "plain", "swiglu", "sink", or "scaled" (rows that lack their scale: the library product
    would need them made dense first)."""
    M, K = x.shape
    N = w.shape[0]
    if not (USE_OWN_GEMM and w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and M >= GEMM_MIN_ROWS
            and K % 8 == 0 and N % (16 if swiglu else 8) == 0 and (N // 2 if swiglu else N) % 8 == 0
            and out_dtype in (None, torch.bfloat16, torch.float32)):
        return False
    if USE_OWN_GEMM is True or kind == "scaled":
        return True
    if kind == "swiglu":
        return M >= OWN_GEMM_SWIGLU_MIN_ROWS
    if kind == "sink":
        return M >= OWN_GEMM_SINK_MIN_ROWS and K <= OWN_GEMM_SINK_MAX_K
    return False


def linear(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None, swiglu: bool = False,
           partial_sums: bool = False, sink: Optional[NormSink] = None):
    """x[M, K] . w[N, K]^T.  A weight kept in float32 makes the product float32 whatever x is.

    ``x`` may be ``RowScaled`` (the output of a norm that a product's epilogue prepared).  With
    ``sink`` the product is added to ``sink.residual`` and the result is the output of the norm
    that follows it: ``RowScaled`` when the product of few rows does it in its epilogue,
    else a tensor from the norm kernel.

    ``swiglu``: w holds gate and up rows in alternating blocks of 8 and the result is
    silu(gate) * up, ``[M, N / 2]``.  ``partial_sums``: return the float32 partial sums
    ``[parts, M, N]`` of a product that split its inner dimension instead of their sum
    (``add_rmsnorm`` can add them up); by default the product sums them itself.
    """
    _need(w, "w", dims=2)
    if x.shape[1] != w.shape[1] or len(x.shape) != 2:
        raise KernelError(f"linear: x {tuple(x.shape)} and w {tuple(w.shape)} do not share the inner size")
    M, K = x.shape
    N = w.shape[0]
    few = w.dtype == torch.bfloat16 and K % 8 == 0 and (not swiglu or N % 16 == 0)
    small = few and M <= MMA_MAX_ROWS
    streams = few and M <= TC_MAX_ROWS and not partial_sums and USE_TCGEN05
    fast = streams and x.dtype == torch.bfloat16
    if sink is not None:
        if fast and USE_FUSED_NORM and not swiglu and tuple(sink.residual.shape) == (M, N):
            return linear_tc(x, w, sink=sink, _checked=True)
        if (not swiglu and not isinstance(x, RowScaled) and tuple(sink.residual.shape) == (M, N)
                and _own_gemm_fits(x, w, False, None, "sink") and not partial_sums):
            return gemm_tc(x, w, sink=sink)
        delta = linear(x, w, out_dtype=out_dtype, swiglu=swiglu)
        normed = torch.empty((M, sink.residual.shape[1]), dtype=delta.dtype, device=delta.device)
        return add_rmsnorm(sink.residual, delta, sink.weight, sink.eps, normed)
    if isinstance(x, RowScaled):
        if fast:
            return linear_tc(x, w, out_dtype=out_dtype or x.dtype, swiglu=swiglu, _checked=True)
        if _own_gemm_fits(x.x, w, swiglu, out_dtype, "scaled") and not partial_sums:
            return gemm_tc(x, w, out_dtype=out_dtype or x.dtype, swiglu=swiglu)
        x = x.dense()
    _need(x, "x", dims=2)
    out_dtype = out_dtype or x.dtype
    if x.dtype != w.dtype:
        x = x.to(w.dtype)
    if streams:
        return linear_tc(x, w, out_dtype=out_dtype, swiglu=swiglu, _checked=True)
    if _own_gemm_fits(x, w, swiglu, out_dtype, "swiglu" if swiglu else "plain") and not partial_sums:
        return gemm_tc(x, w, out_dtype=out_dtype, swiglu=swiglu)
    if small:
        fn = _fn("linear_mma", "bn_linear_mma")
        splits = _mma_splits(M, N, K, n_sms(x.device))
        scratch, counters = _split_scratch(x.device)
        tail = (_ptr(scratch), ctypes.c_longlong(scratch.numel()), _ptr(counters), int(counters.numel()), _stream())
        if swiglu:
            out = torch.empty((M, N // 2), dtype=out_dtype, device=x.device)
            _check(fn(_ptr(x), _ptr(w), _ptr(out), int(_DT[out_dtype]), int(M), int(N), int(K), int(N // 2),
                      int(2), int(splits), *tail), "linear_mma")
            return out
        if partial_sums and splits > 1:
            out = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
            _check(fn(_ptr(x), _ptr(w), _ptr(out), int(0), int(M), int(N), int(K), int(N), int(1),
                      int(splits), *tail), "linear_mma")
            return out
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        _check(fn(_ptr(x), _ptr(w), _ptr(out), int(_DT[out_dtype]), int(M), int(N), int(K), int(N), int(0),
                  int(splits), *tail), "linear_mma")
        return out
    if M <= SKINNY_MAX_ROWS and K % 8 == 0:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        # a matrix with few rows shares its inner dimension out over several blocks (a property of the matrix alone)
        n_splits = getattr(build.library("linear"), "bn_linear_skinny_splits")
        n_splits.restype = c_int
        splits = n_splits(int(N), int(K))
        partial = torch.empty((splits, M, N), dtype=torch.float32, device=x.device) if splits > 1 else None
        _check(_fn("linear", "bn_linear_skinny")(_ptr(x), _ptr(w), int(_code(w)), _ptr(out), int(_DT[out_dtype]),
                                                 int(M), int(N), int(K), int(N),
                                                 _ptr(partial) if partial is not None else c_void_p(None), _stream()),
               "linear_skinny")
        if splits > 1:
            global LAUNCHES
            LAUNCHES += 1  # the kernel that adds the splits
    else:
        # Many rows: the library product, float32 accumulation, no reduced-precision float32 mode.
        if w.dtype == torch.float32:
            if torch.backends.cuda.matmul.allow_tf32:
                raise KernelError("float32 products need torch.backends.cuda.matmul.allow_tf32 = False")
            product = lambda: torch.matmul(x, w.t())
        elif out_dtype == torch.float32:
            product = lambda: torch.mm(x, w.t(), out_dtype=torch.float32)
        else:
            product = lambda: torch.matmul(x, w.t())
        out = product() if PROFILE is None else _timed("library.matmul", product)
        out = out if out.dtype == out_dtype else out.to(out_dtype)
    if swiglu:
        act = torch.empty((M, N // 2), dtype=out.dtype, device=x.device)
        return silu_mul(out, act)
    return out


# ---- sampling -----------------------------------------------------------------------------
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(logits, "logits", torch.float32, 2)
    out = out if out is not None else torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, 1)
    n = logits.shape[0]
    _scr, counters = _split_scratch(logits.device)
    if n > counters.numel():
        raise KernelError(f"argmax: at most {counters.numel()} rows at a time")
    part_v = torch.empty(n * 64, dtype=torch.float32, device=logits.device)
    part_i = torch.empty(n * 64, dtype=torch.int32, device=logits.device)
    _check(_fn("sampling", "bn_argmax")(_ptr(logits), int(logits.shape[1]), int(n), int(logits.shape[1]),
                                        _ptr(out), _ptr(part_v), _ptr(part_i), _ptr(counters), _stream()), "argmax")
    return out


def sample_temperature(logits: torch.Tensor, temperature: float, rng_state: torch.Tensor,
                       out: Optional[torch.Tensor] = None, index: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One draw per row from softmax(logits / temperature).  ``rng_state`` holds xorshift64* states
    (int64 bit patterns); row r uses and advances state ``index[r]`` (or r without an index)."""
    _need(logits, "logits", torch.float32, 2)
    _need(rng_state, "rng_state", torch.int64, 1)
    if index is not None:
        _need(index, "index", torch.int32, 1)
    elif rng_state.shape[0] < logits.shape[0]:
        raise KernelError("sample_temperature: one generator state per row is needed")
    out = out if out is not None else torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, 1)
    _check(_fn("sampling", "bn_sample_temperature")(_ptr(logits), int(logits.shape[1]), int(logits.shape[0]),
                                                    int(logits.shape[1]), c_float(temperature), _ptr(rng_state),
                                                    _ptr(index), _ptr(out), _stream()), "sample_temperature")
    return out


def sample_topp(logits: torch.Tensor, temperature: float, topp: float, rng_state: torch.Tensor,
                out: Optional[torch.Tensor] = None, index: Optional[torch.Tensor] = None,
                probs: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Nucleus sampling: one draw per row from the smallest set of most probable tokens whose
    mass exceeds ``topp``.  ``probs`` is scratch of the shape of ``logits``."""
    _need(logits, "logits", torch.float32, 2)
    _need(rng_state, "rng_state", torch.int64, 1)
    if index is not None:
        _need(index, "index", torch.int32, 1)
    if probs is None:
        probs = torch.empty_like(logits)
    _need(probs, "probs", torch.float32, 2)
    if probs.shape[0] < logits.shape[0] or probs.shape[1] != logits.shape[1]:
        raise KernelError("sample_topp: probs scratch does not fit")
    out = out if out is not None else torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, 1)
    _check(_fn("sampling", "bn_sample_topp")(_ptr(logits), int(logits.shape[1]), int(logits.shape[0]),
                                             int(logits.shape[1]), c_float(temperature), c_float(topp),
                                             _ptr(rng_state), _ptr(index), _ptr(probs), _ptr(out), _stream()),
           "sample_topp")
    return out


def repeat_penalty(logits: torch.Tensor, recent: torch.Tensor, recent_len: torch.Tensor, penalty: float,
                   index: Optional[torch.Tensor] = None) -> None:
    """In place: for each distinct id among the first recent_len[s] entries of recent[s] (s = index[r]
    or r), logit > 0 ? logit / penalty : logit * penalty."""
    _need(logits, "logits", torch.float32, 2)
    _need(recent, "recent", torch.int32, 2)
    _need(recent_len, "recent_len", torch.int32, 1)
    if index is not None:
        _need(index, "index", torch.int32, 1)
    _check(_fn("sampling", "bn_repeat_penalty")(_ptr(logits), int(logits.shape[1]), int(logits.shape[0]),
                                                int(logits.shape[1]), _ptr(recent), int(recent.shape[1]),
                                                _ptr(recent_len), _ptr(index), c_float(penalty), _stream()),
           "repeat_penalty")


def sampler_accept(recent: torch.Tensor, recent_len: torch.Tensor, recent_pos: torch.Tensor, tokens: torch.Tensor,
                   index: Optional[torch.Tensor] = None) -> None:
    """Push tokens[r] into the ring of recent tokens of state row index[r] (or r)."""
    _need(recent, "recent", torch.int32, 2)
    _need(recent_len, "recent_len", torch.int32, 1)
    _need(recent_pos, "recent_pos", torch.int32, 1)
    _need(tokens, "tokens", torch.int32, 1)
    if index is not None:
        _need(index, "index", torch.int32, 1)
    _check(_fn("sampling", "bn_sampler_accept")(_ptr(recent), int(recent.shape[1]), _ptr(recent_len),
                                                _ptr(recent_pos), _ptr(index), _ptr(tokens), int(tokens.shape[0]),
                                                _stream()), "sampler_accept")
