"""Thin Python entry to the kernels: torch tensors in, pointers out.

Each function checks what the C side cannot (device, contiguity, dtype), passes
pointers, sizes and the current CUDA stream to ``libferrox_b200.so`` and raises
:class:`KernelError` on a non-zero status.  Nothing here computes: there is no
torch fallback, and a CPU tensor is an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_long, c_ulonglong, c_void_p
from typing import Optional

import torch

from . import lib as _libmod

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

_ERRORS = {
    -1: "combination of element types not built",
    -2: "a size outside what the kernel handles",
    -3: "pointer or stride not aligned as the kernel requires",
    -4: "a bounded wait inside a kernel ran out",
    -5: "the request needs more scratch than the library's fixed array holds",
}


class KernelError(RuntimeError):
    pass


_P, _I, _L, _F = c_void_p, c_int, c_long, c_float
_SIGNATURES = {
    "fx_set_pdl": [_I],
    "fx_gemm": [_P, _I, _L, _P, _P, _I, _L, _P, _I, _P, _I, _L, _I, _I, _I, _I, _P, _I, _L, _P],
    "fx_embed": [_P, _I, _P, _P, _I, _I, _I, _P, _P],
    "fx_rmsnorm": [_P, _P, _P, _I, _F, _P, _I, _I, _I, _P],
    "fx_silu_mul": [_P, _L, _P, _L, _I, _P, _I, _I, _P],
    "fx_rope_kv_write": [_P, _I, _L, _P, _P, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "fx_rope_table": [_P, _P, _I, _I, _P, _P],
    "fx_gemm_tc": [_P, _L, _P, _L, _L, _I, _P, _I, _P, _I, _L, _I, _I, _I, _I, _I, _I, _P, _I, _P, _P],
    "fx_gemm_tc_swap": [_P, _L, _P, _L, _L, _I, _P, _I, _P, _I, _L, _I, _I, _I, _I, _I, _I, _P, _I, _I, _I, _I, _P, _P, _P],
    "fx_gemm_tc2": [_P, _L, _P, _L, _I, _P, _I, _P, _I, _L, _I, _I, _I, _I, _I, _I, _P, _P],
    "fx_gather_rows": [_P, _L, _P, _P, _L, _I, _I, _I, _P],
    "fx_route_small": [_P, _L, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _P],
    "fx_route": [_P, _L, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _I, _P],
    "fx_route_fused": [_P, _L, _P, _L, _I, _I, _I, _I, _I, _I, _P, _L, _P, _P, _P, _P, _P, _P, _I, _P, _L, _P],
    "fx_moe_combine": [_P, _P, _I, _P, _P, _I, _P, _P, _L, _I, _I, _P],
    "fx_moe_combine_norm": [_P, _P, _I, _P, _P, _I, _P, _P, _L, _I, _I, _P, _I, _F, _P, _P],
    "fx_residual_add": [_P, _P, _I, _L, _P],
    "fx_paged_attention": [_P, _L, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _F, _P],
    "fx_prefill_attention": [_P, _L, _P, _P, _P, _I, _I, _P, _I, _P, _P, _L, _I, _I, _I, _I, _F, _P],
    "fx_prefill_attention_tc": [_P, _L, _I, _P, _P, _I, _P, _I, _I, _P, _I, _P, _P, _L, _I, _I, _I, _I, _F, _P, _P, _P,
                                _P, _I, _P],
    "fx_router_topk": [_P, _L, _I, _I, _I, _I, _P, _P, _P],
    "fx_moe_align": [_P, _I, _I, _I, _P, _P, _P, _P, _P, _I, _P],
    "fx_gemm_slab_ok": [_I, _I, _I],
    "fx_gemm_slab": [_P, _L, _P, _L, _P, _I, _P, _I, _L, _I, _I, _I, _I, _P, _P],
    "fx_gemm_skinny": [_P, _L, _P, _P, _L, _L, _P, _I, _P, _I, _L, _I, _I, _I, _I, _I, _I, _P, _P, _I, _I, _I, _P],
    "fx_decode_attention": [_P, _L, _P, _P, _I, _I, _P, _I, _I, _P, _P, _P, _P, _L, _P, _P, _I, _I, _I, _I, _I, _F, _I,
                            _I, _P, _P, _I, _I, _I, _P, _P],
    "fx_argmax": [_P, _L, _I, _I, _P, _P],
    "fx_repetition_penalty": [_P, _L, _I, _I, _P, _P, _P, _P],
    "fx_sample": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P],
    "fx_sample_or": [_P, _L, _P, _L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P],
    "fx_random_normal": [_P, _I, _L, c_ulonglong, c_double, c_double, _P],
}

_fn = {}

# kernels launched by one call of an entry point (fx_moe_align: count, scan, place)
_KERNELS = {"fx_moe_align": 3, "fx_route": 2, "fx_decode_attention": 2}   # (a split-K product adds a second kernel; not counted)
_launches = 0


def launch_count() -> int:
    """Kernels of this library launched so far by this process."""
    return _launches


def count_launches(n: int) -> None:
    """Account for kernels launched outside :func:`call` (a CUDA graph's replay)."""
    global _launches
    _launches += n


def _get(name: str):
    f = _fn.get(name)
    if f is None:
        lib = _libmod.load()
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[name]
        f.restype = c_int
        _fn[name] = f
    return f


def register_signature(name: str, argtypes) -> None:
    """Lets further source files of the library declare their entry points."""
    _SIGNATURES[name] = list(argtypes)


def call(name: str, *args) -> None:
    global _launches
    _launches += _KERNELS.get(name, 1)
    if _trace is not None:
        return _call_traced(name, args)
    rc = _get(name)(*args)
    if rc != 0:
        if rc > 0:
            raise KernelError(f"{name}: CUDA error {rc} at launch ({torch.cuda.get_device_name()})")
        raise KernelError(f"{name}: refused: {_ERRORS.get(rc, rc)}")


# ---- tracing: device time per class of kernel, behind a switch -------------------------------------------
# The reference prints phase rates only (crates/ferrox-cli/src/run.rs:680-695); with the switch on, every entry
# point's launches are bracketed by CUDA events on their own stream and summed by (scope, entry point), where the
# scope is what the parts announce with :class:`trace_scope` (mixer, feed-forward, norm, head ...).  Launches then
# run without programmatic dependent launch, so that a kernel's time is its own; the engine leaves CUDA graphs off.
_trace = None          # None: off; else {key: [n_calls, [(start event, end event), ...]]}
_trace_scope = []


def trace_enabled() -> bool:
    return _trace is not None


def trace_start() -> None:
    global _trace
    _trace = {}
    _get("fx_set_pdl")(0)


def trace_stop() -> dict:
    """Ends tracing; returns {"scope:entry point": (launches, milliseconds on the device)}."""
    global _trace
    t, _trace = _trace or {}, None
    _get("fx_set_pdl")(1)
    torch.cuda.synchronize()
    return {k: (n, sum(a.elapsed_time(b) for a, b in evs)) for k, (n, evs) in t.items()}


class trace_scope:
    """Names the part whose kernels follow (no cost while tracing is off)."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if _trace is not None:
            _trace_scope.append(self.name)
        return self

    def __exit__(self, *exc):
        if _trace is not None and _trace_scope:
            _trace_scope.pop()
        return False


def _call_traced(name: str, args) -> None:
    stream = torch.cuda.ExternalStream(args[-1]) if args and isinstance(args[-1], int) and args[-1] else torch.cuda.current_stream()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    rc = _get(name)(*args)
    b.record(stream)
    if rc != 0:
        raise KernelError(f"{name}: status {rc}")
    key = f"{_trace_scope[-1] if _trace_scope else '-'}:{name}"
    rec = _trace.setdefault(key, [0, []])
    rec[0] += _KERNELS.get(name, 1)
    rec[1].append((a, b))


_scoped_stream = None
_sm_count = 0


def sm_count() -> int:
    """Streaming multiprocessors of the current device, asked once; launch shapes and the choices between kernels are
    functions of it.  Without a device (the choices are also tested on the CPU): the B200's 148."""
    global _sm_count
    if _sm_count == 0:
        if not torch.cuda.is_available():
            return 148
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def stream_ptr() -> int:
    """The stream kernels go to when none is named: the one a step has announced, else torch's current stream."""
    if _scoped_stream is not None:
        return _scoped_stream
    return torch.cuda.current_stream().cuda_stream


class stream_scope:
    """While a step runs, its stream is known: asking torch for the current stream costs more than a launch."""

    def __init__(self, ptr: int):
        self.ptr = ptr

    def __enter__(self):
        global _scoped_stream
        self.prev, _scoped_stream = _scoped_stream, self.ptr
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self.prev
        return False


def code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not handled by the kernels") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernels take CUDA tensors only (there is no CPU path)")
    return t.data_ptr()


def _rows(t: torch.Tensor) -> int:
    """Row stride of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"expected a 2-D tensor with contiguous rows, found shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


# ---------------------------------------------------------------------------
def gemm(a, w, out, *, bias=None, accumulate=False, a_rows=None, group_offsets=None, stream=None):
    """out[M,N] (+)= a[M,K] . w[N,K]^T (+ bias).  With ``group_offsets`` ([G+1],
    int32) ``w`` is [G,N,K] and rows off[g]..off[g+1] use matrix g; ``a_rows``
    gathers rows of ``a``."""
    M, N = out.shape
    if group_offsets is not None:
        G, Nw, K = w.shape
        wstride = w.stride(0)
        ldw = w.stride(1)
        if w.stride(2) != 1:
            raise KernelError("grouped weights must have contiguous rows")
    else:
        G, wstride = 1, 0
        Nw, K = w.shape
        ldw = _rows(w)
    if Nw != N or a.shape[1] != K or (a_rows is None and a.shape[0] != M):
        raise KernelError(f"gemm shapes do not agree: a {tuple(a.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    call(
        "fx_gemm", _ptr(a), code(a), _rows(a), _ptr(a_rows), _ptr(w), code(w), ldw,
        _ptr(bias), code(bias) if bias is not None else 0, _ptr(out), code(out), _rows(out), int(accumulate),
        M, N, K, _ptr(group_offsets), G, wstride, stream if stream is not None else stream_ptr(),
    )
    return out


def embed(table, ids, out, status=None, stream=None):
    T = ids.numel()
    call("fx_embed", _ptr(table), code(table), _ptr(ids), _ptr(out), T, table.shape[1], table.shape[0], _ptr(status),
         stream if stream is not None else stream_ptr())
    return out


def rmsnorm(x, weight, eps, out, rows=None, stream=None):
    if x.dtype != torch.float32:
        raise KernelError("rmsnorm reads the 32-bit residual stream")
    n = out.shape[0]
    call("fx_rmsnorm", _ptr(x), _ptr(rows), _ptr(weight), code(weight), float(eps), _ptr(out), code(out), n, x.shape[1],
         stream if stream is not None else stream_ptr())
    return out


def silu_mul(gu, out, stream=None):
    rows, n = out.shape
    if gu.shape[1] != 2 * n:
        raise KernelError("silu_mul expects [gate | up] rows of twice the output width")
    call("fx_silu_mul", _ptr(gu), _rows(gu), _ptr(out), _rows(out), code(gu), None, rows, n,
         stream if stream is not None else stream_ptr())
    return out


def rope_table(positions, inv_freq, out, stream=None):
    """out[t, i] = (cos, sin)(positions[t] * inv_freq[i]); out is float32 [T, half, 2]."""
    call("fx_rope_table", _ptr(positions), _ptr(inv_freq), positions.numel(), inv_freq.numel(), _ptr(out),
         stream if stream is not None else stream_ptr())
    return out


def route_small(logits, top_k, renorm, ids, weights, offsets, src_token, inv_perm, active=None, n_experts=None,
                stream=None):
    """router_topk and moe_align of a small step (at most 1024 tokens) in one launch."""
    T, E = logits.shape[0], (n_experts or logits.shape[1])
    call("fx_route_small", _ptr(logits), _rows(logits), T, E, top_k, int(renorm), _ptr(ids), _ptr(weights), _ptr(offsets),
         _ptr(src_token), _ptr(inv_perm), _ptr(active), active.numel() if active is not None else 0,
         stream if stream is not None else stream_ptr())


ROUTE_FUSED_MAX_TOKENS = 8     # the kernel keeps a sum per token in registers
ROUTE_FUSED_MAX_ROWS = 1024


def route_fused_ok(x, w_route, n_experts: int, top_k: int = 1) -> bool:
    """Whether :func:`route_fused` takes these operands."""
    T, H = x.shape
    R = w_route.shape[0]
    smem = 8 * H * 2 + (8 * R + 8 * n_experts) * 4 + (2 * n_experts + 1 + 16 * top_k) * 4
    return (T <= ROUTE_FUSED_MAX_TOKENS and top_k <= 64 and x.dtype == torch.bfloat16 and w_route.dtype == torch.bfloat16
            and w_route.dim() == 2 and R <= ROUTE_FUSED_MAX_ROWS and smem <= 200 * 1024 and H % 8 == 0
            and w_route.shape[1] == H and x.stride(0) % 8 == 0 and w_route.stride(0) % 8 == 0 and x.stride(1) == 1
            and w_route.stride(1) == 1 and x.data_ptr() % 16 == 0 and w_route.data_ptr() % 16 == 0)


def route_fused(x, w_route, logits, top_k, renorm, ids, weights, offsets, src_token, inv_perm, active=None, n_experts=None,
                xp_out=None, stream=None):
    """What stands between the norm and the experts in a step of a few tokens, in one launch of one thread-block
    cluster (see :func:`route_fused_ok`): the router's product logits = x . w_route^T (32-bit sums; ``w_route`` may carry
    rows beyond the experts', whose logits later kernels read), :func:`route_small` on the first ``n_experts`` columns
    and, with ``xp_out`` [tokens * top_k, hidden], the rows of ``x`` copied into expert order."""
    T, H = x.shape
    R = w_route.shape[0]
    E = n_experts or R
    call("fx_route_fused", _ptr(x), _rows(x), _ptr(w_route), _rows(w_route), T, R, E, H, top_k, int(renorm), _ptr(logits),
         _rows(logits), _ptr(ids), _ptr(weights), _ptr(offsets), _ptr(src_token), _ptr(inv_perm), _ptr(active),
         active.numel() if active is not None else 0, _ptr(xp_out), _rows(xp_out) if xp_out is not None else 0,
         stream if stream is not None else stream_ptr())


ROUTE_SMALL_MAX_TOKENS = 48    # measured with 60 experts: the one-block kernel 4 to 8 us up to here, the two kernels 8 us
ROUTE_SMALL_MAX_EXPERTS = 256  # its shared memory: 32 warps x experts x 4 bytes


def route(logits, top_k, renorm, ids, weights, scratch, offsets, src_token, inv_perm, active=None, n_experts=None,
          stream=None):
    """router_topk and moe_align of a step of any size: the top-k kernel counts each expert's rows as it chooses,
    the placing kernel sums the counts itself.  ``scratch``: 2 * n_experts int32."""
    T, E = logits.shape[0], (n_experts or logits.shape[1])
    call("fx_route", _ptr(logits), _rows(logits), T, E, top_k, int(renorm), _ptr(ids), _ptr(weights), _ptr(scratch),
         _ptr(offsets), _ptr(src_token), _ptr(inv_perm), _ptr(active), active.numel() if active is not None else 0,
         stream if stream is not None else stream_ptr())


PAIR_HALVES, PAIR_ADJACENT = 0, 1


def rope_kv_write(qkv, positions, token_seq, seq_slot, inv_freq, rotary_dim, k_pages, v_pages, block_table, page_size,
                  n_heads, n_kv_heads, head_dim, write_cache=True, status=None, stream=None, cos_sin=None,
                  pairing=PAIR_HALVES):
    """Rotates the q and k heads of the fused [q|k|v] rows in place at each token's position and stores k and v in
    their cache pages.  ``inv_freq`` ([rotary_dim/2] float32, or None for no rotation) gives each pair's frequency,
    ``pairing`` which elements form pair i: PAIR_HALVES (i, i + rotary_dim/2) or PAIR_ADJACENT (2i, 2i+1);
    ``cos_sin`` ([T, rotary_dim/2, 2], optional) holds this step's cos and sin, made by :func:`rope_table`."""
    T = qkv.shape[0]
    call("fx_rope_kv_write", _ptr(qkv), code(qkv), _rows(qkv), _ptr(positions), _ptr(token_seq), _ptr(seq_slot),
         _ptr(inv_freq), _ptr(cos_sin), rotary_dim, int(pairing), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1], page_size,
         T, n_heads, n_kv_heads, head_dim, int(write_cache), _ptr(status), stream if stream is not None else stream_ptr())


def paged_attention(q, k_pages, v_pages, block_table, page_size, positions, token_seq, seq_slot, out, n_heads,
                    n_kv_heads, head_dim, window, scale, stream=None):
    """``q`` is a [T, >= n_heads*head_dim] view whose rows start with the query heads."""
    T = q.shape[0]
    call("fx_paged_attention", _ptr(q), _rows(q), _ptr(k_pages), _ptr(v_pages), code(q), _ptr(block_table),
         block_table.shape[1], page_size, _ptr(positions), _ptr(token_seq), _ptr(seq_slot), _ptr(out), _rows(out), T,
         n_heads, n_kv_heads, head_dim, int(window or 0), float(scale), stream if stream is not None else stream_ptr())
    return out


PREFILL_TILE = 64


def prefill_attention(q, k_pages, v_pages, block_table, page_size, tiles, seq_slot, out, n_heads, n_kv_heads, head_dim,
                      window, scale, stream=None):
    """Flash attention of prompt portions (bfloat16).  ``tiles``: int32 [n, 4] rows of
    (first flat token, rows <= 64, entry index, absolute position of the first row)."""
    if q.dtype != torch.bfloat16:
        raise KernelError("prefill_attention is a bfloat16 kernel")
    call("fx_prefill_attention", _ptr(q), _rows(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
         block_table.shape[1], page_size, _ptr(tiles), tiles.shape[0], _ptr(seq_slot), _ptr(out), _rows(out), n_heads,
         n_kv_heads, head_dim, int(window or 0), float(scale), stream if stream is not None else stream_ptr())
    return out


WIDE_PREFILL_TILE = 256


def prefill_ok(q, out, k_pages, head_dim) -> bool:
    """Whether the mma.sync prompt attention kernel takes these operands (bfloat16, head sizes in steps of 16)."""
    return (q.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16 and 0 < head_dim <= 256 and head_dim % 16 == 0
            and q.stride(0) % 8 == 0 and out.stride(0) % 2 == 0 and q.data_ptr() % 16 == 0 and k_pages.data_ptr() % 16 == 0)


def prefill_tc_ok(q, out, k_pages, page_size, head_dim) -> bool:
    """Whether the tcgen05 prompt attention kernel takes these operands."""
    return (q.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16 and head_dim in (64, 128)
            and page_size >= 64 and page_size % 64 == 0 and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


PREFILL_KEY_BLOCK = 128          # positions per key block of the tcgen05 prompt attention kernel
PREFILL_MAX_RUNS = 32            # runs of key blocks a tile may be cut into (a lane of the merging warp each)
# The planner's cost model, in units of the time a block of 128 keys takes a tile (measured on a B200, 16 heads of
# 128: 2.7 us): what an item costs beside its key blocks (set-up, the first block's latency, its output), and the
# second kernel that adds the runs of cut tiles up.
PREFILL_ITEM_OVERHEAD, PREFILL_MERGE_COST = 5, 3
PREFILL_RUN_CHOICES = (0, 16, 12, 8, 6, 4)   # key blocks a run (0: tiles stay whole)


def _prefill_items(tiles, run: int):
    items, merges, parts = [], [], 0
    for tok0, rows, b, pos0, first, end in tiles:
        n_blk = end - first
        runs = min(PREFILL_MAX_RUNS, -(-n_blk // run)) if run > 0 else 1
        if runs <= 1:
            items.append((tok0, rows, b, pos0, first, end, -1, 0))
            continue
        per = -(-n_blk // runs)
        first_part = parts
        for kb in range(first, end, per):
            items.append((tok0, rows, b, pos0, kb, min(end, kb + per), parts, 0))
            parts += 1
        merges.append((tok0, rows, first_part, parts - first_part))
    items.sort(key=lambda it: it[4] - it[5])      # most key blocks first (stable: ties stay in order)
    return items, merges, parts


def _prefill_makespan(items, parts: int, n_heads: int, sms: int) -> float:
    """How long the items take on ``sms`` SMs that take them heaviest first, each head its own copy of every item:
    no less than the heaviest item, than an even share of all work, and than the two items that must share an SM once
    there are more items than SMs; plus the adding up of the parts."""
    costs = [it[5] - it[4] + PREFILL_ITEM_OVERHEAD for it in items]           # descending already
    n = len(costs) * n_heads
    est = max(costs[0], sum(costs) * n_heads / sms)
    if n > sms:
        est = max(est, costs[(sms - 1) // n_heads] + costs[sms // n_heads])
    return est + (PREFILL_MERGE_COST if parts else 0)


def prefill_tc_plan(entries, window, n_heads: int, sms: int = 0, run_blocks: int = -1):
    """The work items of the tcgen05 prompt attention kernel for a step.  ``entries``: (tokens, first position) of
    each entry, in the order of the flattened batch.  A tile is up to 256 queries of one entry; it sees the key blocks
    (of 128 positions) from its first query's first visible key to its last query's own.  Tiles with many key blocks
    may be cut into runs whose partial results a second kernel adds up: a portion behind a long cached prefix is one
    tile with all the keys, and without the cut it would keep as many SMs busy as there are heads.  A cut item costs
    (PREFILL_ITEM_OVERHEAD), so the run length is the one of PREFILL_RUN_CHOICES whose items finish first by
    :func:`_prefill_makespan`, and whole tiles stay unless a cut is 15 % faster by that estimate.  Returns (items int32 [n, 8], merges int32 [m, 4], parts) as
    ``fx_prefill_attention_tc`` takes them: heavy items first; a tile's runs have consecutive parts in the order of
    their keys.  ``run_blocks`` >= 0: this many key blocks a run instead of the choice (0: no cut; tests)."""
    import numpy as np

    sms = sms or sm_count()
    W = int(window or 0)
    tiles, flat = [], 0
    for b, (n, start) in enumerate(entries):
        for i in range(0, n, WIDE_PREFILL_TILE):
            rows, pos0 = min(WIDE_PREFILL_TILE, n - i), start + i
            first = (max(0, pos0 - W + 1) if W > 0 else 0) // PREFILL_KEY_BLOCK
            end = (pos0 + rows - 1) // PREFILL_KEY_BLOCK + 1
            tiles.append((flat + i, rows, b, pos0, first, end))
        flat += n
    best = first = None
    whole = 0.0
    for run in (PREFILL_RUN_CHOICES if run_blocks < 0 else (run_blocks,)):
        items, merges, parts = _prefill_items(tiles, run)
        if run > 0 and not parts and best is not None:
            continue                                  # nothing was cut: the same items as the whole tiles
        est = _prefill_makespan(items, parts, n_heads, sms)
        # (whole tiles stay unless a cut promises a clear gain: the model is good to a tenth or so)
        if best is None or est < (0.85 * whole if best[1] is first else best[0] - 1e-9):
            best = (est, items, merges, parts)
            if first is None:
                first, whole = items, est
    _, items, merges, parts = best
    return (np.asarray(items, dtype=np.int32).reshape(-1, 8), np.asarray(merges, dtype=np.int32).reshape(-1, 4), parts)


def prefill_attention_tc(q, k_pages, v_pages, block_table, page_size, items, seq_slot, out, n_heads, n_kv_heads,
                         head_dim, window, scale, status=None, stream=None, merges=None, part_o=None, part_ml=None):
    """Flash attention of prompt portions on the tcgen05 tensor cores (bfloat16, head_dim 64 or 128, pages of a
    multiple of 64 positions).  ``items``, ``merges``: device copies of what :func:`prefill_tc_plan` returns;
    ``part_o`` float32 [parts, n_heads, 256, head_dim] and ``part_ml`` float32 [parts, n_heads, 256, 2]: scratch for the
    tiles that were cut into runs of key blocks (a second kernel adds the runs up)."""
    global _launches
    n_merges = merges.shape[0] if merges is not None else 0
    if n_merges:
        _launches += 1
    call("fx_prefill_attention_tc", _ptr(q), _rows(q), q.shape[0], _ptr(k_pages), _ptr(v_pages), k_pages.shape[0],
         _ptr(block_table), block_table.shape[1], page_size, _ptr(items), items.shape[0], _ptr(seq_slot), _ptr(out),
         _rows(out), n_heads, n_kv_heads, head_dim, int(window or 0), float(scale), _ptr(status),
         _ptr(part_o) if n_merges else None, _ptr(part_ml) if n_merges else None, _ptr(merges) if n_merges else None,
         n_merges, stream if stream is not None else stream_ptr())
    return out


def router_topk(logits, top_k, renorm, ids, weights, n_experts=None, stream=None):
    """``n_experts``: the first columns of ``logits`` that are router logits (default: all)."""
    T, E = logits.shape[0], (n_experts or logits.shape[1])
    call("fx_router_topk", _ptr(logits), _rows(logits), T, E, top_k, int(renorm), _ptr(ids), _ptr(weights),
         stream if stream is not None else stream_ptr())


def moe_align(ids, n_experts, scratch, offsets, src_token, inv_perm, active=None, stream=None):
    """``active`` (optional, int32 [n_slots]) receives the experts that got rows, then -1."""
    T, K = ids.shape
    call("fx_moe_align", _ptr(ids), T, K, n_experts, _ptr(scratch), _ptr(offsets), _ptr(src_token), _ptr(inv_perm),
         _ptr(active), active.numel() if active is not None else 0, stream if stream is not None else stream_ptr())


SKINNY_MAX_TOKENS = 64


def skinny_ok(x, w) -> bool:
    """Whether the decode-sized product kernel takes these operands."""
    K = x.shape[1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 32 == 0 and x.stride(0) % 8 == 0
            and w.stride(-2) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(x, w, out, *, bias=None, accumulate=False, gated=False, x_rows=None, group_offsets=None,
                active_groups=None, tokens_hint=0, transposed_out=False, stream=None):
    """out[rows, N] (+)= x . w^T for few rows: streams ``w`` once.  ``gated``: ``w`` is
    [gate rows ; up rows] (2N rows) and out = silu(gate) * up.  Grouped: ``w`` is
    [G, rows, K], ``group_offsets``/``active_groups`` come from :func:`moe_align`."""
    rows, N = (out.shape[1], out.shape[0]) if transposed_out else out.shape   # transposed: out is [N, rows]
    K = x.shape[1]
    if group_offsets is not None:
        wrows, wstride, ldw = w.shape[1], w.stride(0), w.stride(1)
        n_slots = active_groups.numel()
    else:
        wrows, wstride, ldw = w.shape[0], 0, w.stride(0)
        n_slots = 1
    if wrows != (2 * N if gated else N) or w.shape[-1] != K:
        raise KernelError(f"gemm_skinny shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    call("fx_gemm_skinny", _ptr(x), _rows(x), _ptr(x_rows), _ptr(w), ldw, wstride, _ptr(bias),
         code(bias) if bias is not None else 0, _ptr(out), code(out), _rows(out), int(accumulate), rows, N, K,
         int(gated), N if gated else 0, _ptr(group_offsets), _ptr(active_groups), n_slots, int(tokens_hint),
         int(transposed_out), stream if stream is not None else stream_ptr())
    return out


SLAB_MAX_TOKENS = 32      # the kernel walks its tokens 8 at a time over a matrix it holds in shared memory
# up to here it is the faster one (measured on a B200, 8 layers' decode step: 16 tokens 1,728 against 1,742 us, 24 tokens
# 2,271 against 2,221, 32 tokens 2,449 against 2,353; 1 to 8 tokens 1 to 2 % faster)
SLAB_BETTER_MAX_TOKENS = 16


def slab_ok(x, w) -> bool:
    """Whether :func:`gemm_slab` takes the product: bfloat16, few tokens, a plain matrix that fits the shared
    memory of all SMs together (a slab of rows a block), K a multiple of 128, rows 16-byte aligned."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.dim() != 2 or x.shape[0] > SLAB_MAX_TOKENS:
        return False
    if x.stride(0) % 8 or w.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16 or x.stride(1) != 1 or w.stride(1) != 1:
        return False
    return bool(_get("fx_gemm_slab_ok")(w.shape[0], w.shape[1], x.shape[0]))


def gemm_slab(x, w, out, *, bias=None, accumulate=False, status=None, stream=None):
    """out[T, N] (+)= x . w^T (+ bias) by the kernel that asks for its whole slab of ``w`` before it waits for the
    kernel before it on the stream (gemm_slab.cu): for a matrix that kernel did not write."""
    T, K = x.shape
    N = w.shape[0]
    if out.shape != (T, N) or w.shape[1] != K:
        raise KernelError(f"gemm_slab shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    call("fx_gemm_slab", _ptr(x), _rows(x), _ptr(w), w.stride(0), _ptr(bias), code(bias) if bias is not None else 0,
         _ptr(out), code(out), _rows(out), int(accumulate), T, N, K, _ptr(status),
         stream if stream is not None else stream_ptr())
    return out


DECODE_BLOCK_OVERHEAD = 128       # start and end of a block, in keys' worth of a block's time
DECODE_MERGE_COST = 256           # the merge of the key ranges, in the same unit
DECODE_BLOCKS_TO_SATURATE = 160   # blocks streaming at the same time that draw the machine's whole bandwidth
DECODE_MAX_SPLITS = 16
DECODE_RUN_LATENCY = 0.15         # share of a run's length that a block's own chain of tiles adds


def decode_tma_blocks_per_sm(dtype, head_dim: int, page_size: int) -> int:
    """Blocks an SM holds of the decode attention kernel that streams pages by TMA (attention_decode_tma.cu);
    0 where it does not apply (then the cp.async kernel runs, three blocks an SM).  Mirrors the kernel's ring:
    stages of 2 x head_dim x 64 x 2 bytes, as many as fit 96 KB (at least 3, at most 8)."""
    if dtype != torch.bfloat16 or head_dim <= 0 or head_dim % 64 or head_dim > 256 or page_size < 64 or page_size % 64:
        return 0
    stage = 2 * (head_dim // 64) * 8192
    stages = max(3, min(8, (96 * 1024) // stage))
    smem = 1024 + max(stages * stage, 4 * 16 * (head_dim + 8) * 4) + 16 * (head_dim * 2 + 16)
    return min(2, (227 * 1024) // (smem + 1024))


def decode_split_plan(n_tokens: int, n_kv_blocks: int, max_positions: int, blocks_per_sm: int = 3,
                      single_is_final: bool = False, run_latency: float = 0.0):
    """(split_len, n_splits) for :func:`decode_attention`.  split_len 0: every token's visible keys are cut
    into n_splits runs of equal length, so that all blocks have work whatever the context length is.
    n_splits is a function of the step's size and the context limit only (a CUDA graph keeps its grid).  The cost
    of n runs, in the time one block takes for a key: the keys stream at the rate of the whole machine
    (DECODE_BLOCKS_TO_SATURATE blocks' worth) or, with few or unevenly many blocks, at the rate of the blocks of a
    wave one after the other; every wave pays a block's start and end and a share of a run's length (a block's own
    chain of tiles, which nothing hides at its start and its end); more than one run pays the merge
    (``single_is_final``: a kernel that writes a single run's result itself, so only n > 1 pays it).
    ``run_latency``: the share of a run's length counted once more per wave; the kernel that streams pages by TMA is
    planned with DECODE_RUN_LATENCY.  Measured with it on a B200 with 16 kv heads of 128, context 2,048 of 4,096, 8
    layers' step in microseconds: 3 requests 864 with 4 runs and 848 with 6; 4 requests 956 with 3 and 936 with 4;
    5 requests 1,081 with 2 and 1,046 with 3; 6 requests 1,167 with 2 and 1,133 with 3; 8 requests 1,258 with 2 and
    1,357 with 3 (384 blocks where 296 fit); 9 requests 1,482 with 1, 1,376 with 2, 1,464 with 3."""
    blocks = max(1, n_tokens * n_kv_blocks)
    slots = sm_count() * blocks_per_sm
    best, best_cost = 1, None
    for n in range(1, min(DECODE_MAX_SPLITS, max(1, -(-max_positions // 64))) + 1):
        waves = -(-blocks * n // slots)
        stream = max(blocks * max_positions / DECODE_BLOCKS_TO_SATURATE, waves * max_positions / n)
        cost = (stream + waves * (DECODE_BLOCK_OVERHEAD + run_latency * max_positions / n)
                + (DECODE_MERGE_COST if n > 1 or not single_is_final else 0))
        if best_cost is None or cost < best_cost * 0.98:   # more runs only for a clear gain
            best, best_cost = n, cost
    return 0, best


def decode_store_ok(qkv, k_pages, head_dim: int, page_size: int) -> bool:
    """Whether :func:`decode_attention` can rotate and store the step's own keys and values itself (``store_new``):
    where the kernel that streams pages by TMA runs."""
    return (decode_tma_blocks_per_sm(qkv.dtype, head_dim, page_size) > 0 and k_pages.dtype == torch.bfloat16
            and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0 and k_pages.data_ptr() % 16 == 0)


def decode_attention(q, k_pages, v_pages, block_table, page_size, positions, token_seq, seq_slot, out, n_heads,
                     n_kv_heads, head_dim, window, scale, split_len, n_splits, part_acc, part_ml, status=None,
                     counters=None, stream=None, fresh_positions=0, store_new=False, write_pages=True, cos_sin=None):
    """``counters``: zeroed int32 scratch that the call leaves zeroed, at least tokens x ceil(group / 16) x kv heads;
    with it the kernel that streams pages by TMA merges the key ranges itself (one kernel instead of two).
    ``fresh_positions``: 0 assumes nothing about the kernel launched just before on the stream.  N > 0 promises that
    that kernel wrote, of all this call reads, only the queries and the keys and values of at most the last N
    positions of each request; older keys are then fetched while it still runs (a false promise reads stale keys).
    ``store_new`` (one token a request; see :func:`decode_store_ok`): ``q`` is the fused [q | k | v] rows as the
    projection left them and the kernel does the rotary kernel's work itself: queries and each token's own key
    rotated (split-half pairs over the whole head, ``cos_sin`` from :func:`rope_table`; None: no rotation), key and
    value put where the attention reads them and, if ``write_pages``, into the pages."""
    global _launches
    T = q.shape[0]
    per_sm = decode_tma_blocks_per_sm(q.dtype, head_dim, page_size)
    blocks = T * n_kv_heads * -(-(n_heads // n_kv_heads) // 16)
    # Merging in the kernel pays while all blocks run at the same time: the count and the fence lengthen the end of
    # every block, which costs nothing only where no other block waits for its place.
    if counters is not None and not (per_sm > 0 and 1 < n_splits <= 32 and counters.numel() >= blocks
                                     and blocks * n_splits <= sm_count() * per_sm):
        counters = None
    if per_sm > 0 and (counters is not None or n_splits == 1):
        _launches -= 1      # no merge kernel
    call("fx_decode_attention", _ptr(q), _rows(q), _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], code(q),
         _ptr(block_table), block_table.shape[1], page_size, _ptr(positions), _ptr(token_seq), _ptr(seq_slot),
         _ptr(out), _rows(out), _ptr(part_acc), _ptr(part_ml), T, n_heads, n_kv_heads, head_dim, int(window or 0),
         float(scale), split_len, n_splits, _ptr(status), _ptr(counters), int(fresh_positions), int(store_new),
         int(write_pages), _ptr(cos_sin), stream if stream is not None else stream_ptr())
    return out


TC_MAX_GROUPS = 1024        # experts the grouped tcgen05 kernel keeps its tile table for (gemm_tc.cu)
TC_SWAP_MAX_GROUPS = 512    # and the swapped-role kernel (gemm_tc_swap.cu)


def tc_ok(x, w) -> bool:
    """Whether the tcgen05 kernel takes these operands (bfloat16, 16-byte aligned rows)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and w.stride(-2) % 8 == 0 and (w.dim() == 2 or w.stride(0) % 8 == 0) and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and x.stride(1) == 1 and w.stride(-1) == 1)


def gemm_tc(x, w, out, *, bias=None, accumulate=False, gated=False, group_offsets=None, status=None, stream=None):
    """out[M, N] (+)= x . w^T on the tcgen05 tensor cores.  ``gated``: ``w`` is [gate rows ; up rows] and
    out = silu(gate) * up.  Grouped: ``w`` is [G, rows, K] and the rows of ``x``/``out`` are sorted by group."""
    M, N = out.shape
    K = x.shape[1]
    if group_offsets is not None:
        G, wrows, ldw, wstride = w.shape[0], w.shape[1], w.stride(1), w.stride(0)
    else:
        G, wrows, ldw, wstride = 0, w.shape[0], w.stride(0), 0
    if wrows != (2 * N if gated else N) or w.shape[-1] != K or x.shape[0] != M:
        raise KernelError(f"gemm_tc shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    call("fx_gemm_tc", _ptr(x), _rows(x), _ptr(w), ldw, wstride, wrows, _ptr(bias), code(bias) if bias is not None else 0,
         _ptr(out), code(out), _rows(out), int(accumulate), M, N, K, int(gated), N if gated else 0,
         _ptr(group_offsets), G, _ptr(status), stream if stream is not None else stream_ptr())
    return out


def gemm_tc_swap(x, w, out, *, bias=None, accumulate=False, gated=False, group_offsets=None, tokens_per_tile=0,
                 weights_first=None, k_splits=1, status=None, stream=None):
    """The same product as :func:`gemm_tc` with the roles swapped: 128 features of ``w`` fill the lanes of a tile,
    the tokens its columns (multiples of 16 up to ``tokens_per_tile``: 32, 64 or 128; 0 = chosen from the sizes).
    For few tokens per weight matrix: decode batches beyond the weight-streaming kernel's, experts of a prompt.
    ``weights_first``: the kernel may fetch its first weights before the kernel launched just before it has finished;
    true by default for dense products, and for grouped ones only if the caller says that ``group_offsets`` is older
    than that kernel.  ``k_splits`` > 1 (plain dense products): K is cut into runs taken by separate CTAs and a second
    kernel adds the partial sums in run order, for matrices of too few rows to fill the machine with tiles."""
    M, N = out.shape
    K = x.shape[1]
    if group_offsets is not None:
        G, wrows, ldw, wstride = w.shape[0], w.shape[1], w.stride(1), w.stride(0)
    else:
        G, wrows, ldw, wstride = 0, w.shape[0], w.stride(0), 0
    if wrows != (2 * N if gated else N) or w.shape[-1] != K or x.shape[0] != M:
        raise KernelError(f"gemm_tc_swap shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    call("fx_gemm_tc_swap", _ptr(x), _rows(x), _ptr(w), ldw, wstride, wrows, _ptr(bias), code(bias) if bias is not None else 0,
         _ptr(out), code(out), _rows(out), int(accumulate), M, N, K, int(gated), N if gated else 0,
         _ptr(group_offsets), G, int(tokens_per_tile),
         int(group_offsets is None if weights_first is None else weights_first), int(k_splits),
         _ptr(torch.empty(k_splits, M, N, dtype=torch.float32, device=out.device)) if k_splits > 1 else None,
         _ptr(status), stream if stream is not None else stream_ptr())
    return out


def gemm_tc2(x, w, out, *, bias=None, accumulate=False, gated=False, status=None, stream=None):
    """The dense product of :func:`gemm_tc` on pairs of SMs (tcgen05 cta_group::2: 256 x 256 tiles shared by the two
    CTAs of a cluster, each fetching half of the tile's operands).  For prompt-sized dense products."""
    M, N = out.shape
    K = x.shape[1]
    if w.dim() != 2 or w.shape[0] != (2 * N if gated else N) or w.shape[1] != K or x.shape[0] != M:
        raise KernelError(f"gemm_tc2 shapes do not agree: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    call("fx_gemm_tc2", _ptr(x), _rows(x), _ptr(w), w.stride(0), w.shape[0], _ptr(bias), code(bias) if bias is not None else 0,
         _ptr(out), code(out), _rows(out), int(accumulate), M, N, K, int(gated), N if gated else 0, _ptr(status),
         stream if stream is not None else stream_ptr())
    return out


def gather_rows(x, rows, out, stream=None):
    call("fx_gather_rows", _ptr(x), _rows(x), _ptr(rows), _ptr(out), _rows(out), code(x), out.shape[0], x.shape[1],
         stream if stream is not None else stream_ptr())
    return out


def swap_better(T: int, N: int, K: int) -> bool:
    """Few tokens against a weight matrix: whether the tcgen05 kernel with the roles swapped (features in the
    lanes, tokens in the columns, weights by TMA) beats the weight-streaming mma.sync kernel.  Measured on a
    B200: beyond 32 tokens for matrices of a few thousand rows, from 8 tokens on for very large ones (the
    vocabulary head); matrices of few rows give the swapped kernel too few tiles."""
    return (T > 32 and N >= 4096) or (T >= 8 and N * K >= (1 << 27))


def pairs_better(M: int, N: int, gated: bool = False) -> bool:
    """Prompt-sized dense products: whether the kernel on pairs of SMs (256 x 256 tiles) beats the one with a CTA per
    128 x 256 tile.  Measured on a B200: from two rounds of tiles for the 74 pairs on (3 to 13 % faster, more with more
    rows); with fewer tiles than SMs the pairs leave SMs idle."""
    tiles = -(-M // 256) * -(-N // (128 if gated else 256))
    return M >= 1024 and tiles >= sm_count()


def swap_k_splits(T: int, N: int, K: int) -> int:
    """Runs of K for the swapped-role kernel on a plain dense product of few tokens, or 0 where the weight-streaming
    kernel is as good.  A matrix of N rows gives N / 128 tiles; with fewer than the machine has SMs, K is cut so that
    some 150 to 300 CTAs stream it.  Measured on a B200 (decode batches of 32 and 64): ahead from 33 tokens on, and from
    17 tokens for matrices of 8M elements and more."""
    if T > 32 or (T > 16 and N * K >= (1 << 23)):
        tiles = -(-N // 128) * -(-T // (32 if T <= 32 else 64))
        return max(1, min(8, K // 256, round(192 / tiles)))
    return 0


def linear(x, w, out, *, bias=None, accumulate=False, status=None, stream=None, after_short_kernel=False):
    """out (+)= x . w^T (+ bias): picks the kernel by size and element type.  ``after_short_kernel``: the kernel before
    this one on the stream is short and leaves the memory system idle; a few tokens then go to the kernel that asks
    for the whole matrix before it waits for that kernel (:func:`gemm_slab`), where the matrix fits."""
    T = x.shape[0]
    if after_short_kernel and T <= SLAB_BETTER_MAX_TOKENS and slab_ok(x, w) and out.dtype in _CODES:
        return gemm_slab(x, w, out, bias=bias, accumulate=accumulate, status=status, stream=stream)
    if (T > SKINNY_MAX_TOKENS and w.shape[0] <= SKINNY_MAX_TOKENS and bias is None and skinny_ok(w, x)):
        # many tokens, a narrow output (router logits): the weight-streaming kernel with the roles swapped,
        # x streamed once as the "matrix", w as the few "tokens", stored transposed
        return gemm_skinny(w, x, out, accumulate=accumulate, transposed_out=True, stream=stream)
    if T <= SKINNY_MAX_TOKENS and w.dim() == 2 and tc_ok(x, w):
        N, K = w.shape
        if T >= 8 and N * K >= (1 << 27):   # the vocabulary head: tiles enough without cutting K
            return gemm_tc_swap(x, w, out, bias=bias, accumulate=accumulate, status=status, stream=stream)
        ks = swap_k_splits(T, N, K)
        if ks:
            return gemm_tc_swap(x, w, out, bias=bias, accumulate=accumulate, k_splits=ks, status=status, stream=stream)
    if T <= SKINNY_MAX_TOKENS and skinny_ok(x, w):
        return gemm_skinny(x, w, out, bias=bias, accumulate=accumulate, stream=stream)
    if T > SKINNY_MAX_TOKENS and tc_ok(x, w):
        if w.dim() == 2 and pairs_better(T, w.shape[0]):
            return gemm_tc2(x, w, out, bias=bias, accumulate=accumulate, status=status, stream=stream)
        return gemm_tc(x, w, out, bias=bias, accumulate=accumulate, status=status, stream=stream)
    return gemm(x, w, out, bias=bias, accumulate=accumulate, stream=stream)


def gated_linear(x, w_gu, out, *, status=None, stream=None):
    """out = silu(x . gate^T) * (x . up^T) with ``w_gu`` = [gate rows ; up rows]: picks the kernel as
    :func:`linear` does; the gate|up intermediate reaches memory only on the CUDA-core path."""
    T, I = out.shape
    if T <= SKINNY_MAX_TOKENS and tc_ok(x, w_gu) and swap_better(T, 2 * I, x.shape[1]):
        return gemm_tc_swap(x, w_gu, out, gated=True, status=status, stream=stream)
    if T <= SKINNY_MAX_TOKENS and skinny_ok(x, w_gu):
        return gemm_skinny(x, w_gu, out, gated=True, stream=stream)
    if T > SKINNY_MAX_TOKENS and tc_ok(x, w_gu):
        if w_gu.dim() == 2 and pairs_better(T, I, gated=True):
            return gemm_tc2(x, w_gu, out, gated=True, status=status, stream=stream)
        return gemm_tc(x, w_gu, out, gated=True, status=status, stream=stream)
    gu = torch.empty(T, 2 * I, dtype=out.dtype, device=out.device)
    gemm(x, w_gu, gu, stream=stream)
    return silu_mul(gu, out, stream=stream)


def combine_norm_ok(h, y) -> bool:
    """Whether :func:`moe_combine` can also write the normed rows (a thread keeps its part of a row in registers)."""
    vw = 4 if y.dtype == torch.float32 else 8
    H = h.shape[1]
    return y.dtype in _CODES and H % vw == 0 and H // vw <= 4 * 256


def moe_combine(h, y, inv_perm, topk_w, shared=None, shared_gate_logit=None, stream=None, norm=None):
    """h[t] += sum_k topk_w[t, k] * y[inv_perm[t, k]] (+ sigmoid(gate logit) * shared[t]).  ``norm`` = (weight, eps,
    out): also out[t] = rmsnorm(h[t]) * weight on the new rows, in the same kernel (see :func:`combine_norm_ok`)."""
    T, H = h.shape
    if norm is not None:
        w, eps, out = norm
        call("fx_moe_combine_norm", _ptr(h), _ptr(y), code(y), _ptr(inv_perm), _ptr(topk_w), topk_w.shape[1],
             _ptr(shared), _ptr(shared_gate_logit), shared_gate_logit.stride(0) if shared_gate_logit is not None else 0,
             T, H, _ptr(w), code(w), float(eps), _ptr(out), stream if stream is not None else stream_ptr())
        return out
    call("fx_moe_combine", _ptr(h), _ptr(y), code(y), _ptr(inv_perm), _ptr(topk_w), topk_w.shape[1], _ptr(shared),
         _ptr(shared_gate_logit), shared_gate_logit.stride(0) if shared_gate_logit is not None else 0, T, H, stream if stream is not None else stream_ptr())


def residual_add(h, y, stream=None):
    call("fx_residual_add", _ptr(h), _ptr(y), code(y), h.numel(), stream if stream is not None else stream_ptr())


def argmax(logits, out, stream=None):
    n, V = logits.shape
    call("fx_argmax", _ptr(logits), _rows(logits), n, V, _ptr(out), stream if stream is not None else stream_ptr())
    return out


def repetition_penalty(work, history, hist_offsets, penalty, stream=None):
    n, V = work.shape
    call("fx_repetition_penalty", _ptr(work), _rows(work), n, V, _ptr(history), _ptr(hist_offsets), _ptr(penalty),
         stream if stream is not None else stream_ptr())


def sample_or(scores, work, temperature, top_k, top_p, draw, use_sample, instead, out, stream=None):
    """Row r of ``out``: a sample of ``scores[r]`` as :func:`sample` draws it if ``use_sample[r]``, else ``instead[r]``
    (also when every candidate was filtered away).  ``scores`` stay untouched; ``work`` is scratch of the same shape."""
    n, V = scores.shape
    call("fx_sample_or", _ptr(scores), _rows(scores), _ptr(work), _rows(work), n, V, _ptr(temperature), _ptr(top_k),
         _ptr(top_p), _ptr(draw), _ptr(use_sample), _ptr(instead), _ptr(out),
         stream if stream is not None else stream_ptr())
    return out


def random_normal(out, key: int, mean: float, std: float, stream=None):
    """out[i] = mean + std * z_i, z the standard normal stream of the 64-bit ``key`` (the rule of
    ``weights.random_init``, which states it for the CPU bit for bit).  ``out``: contiguous float32 or bfloat16."""
    if not out.is_contiguous():
        raise KernelError("random_normal fills contiguous tensors")
    call("fx_random_normal", _ptr(out), code(out), out.numel(), key & ((1 << 64) - 1), float(mean), float(std),
         stream if stream is not None else stream_ptr())
    return out


def sample(work, temperature, top_k, top_p, draw, out, stream=None):
    n, V = work.shape
    call("fx_sample", _ptr(work), _rows(work), n, V, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(draw), _ptr(out),
         stream if stream is not None else stream_ptr())
    return out
