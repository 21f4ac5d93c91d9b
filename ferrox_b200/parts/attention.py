"""Grouped-query attention over paged keys and values.

    q = Wq x + bq, k = Wk x + bk, v = Wv x + bv     (one fused product, [q|k|v] rows)
    q, k rotated at the token's absolute position; k, v written to the cache pages
    head h attends with kv head h / (n_heads / n_kv_heads), scale 1/sqrt(head_dim),
    over positions max(0, p-W+1)..p of its own request
    h += Wo . concat(heads)

Reference: crates/ferrox-models/src/decoder.rs:2075-2157 (one token), :3230-3549 (a
batch), attention in crates/ferrox-core/src/attention.rs:402-524.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from ..cache.specs import CacheSpec, KvCacheSpec
from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Mixer, build_part, register_part
from .specs import NoPositionSpec


RANGE_COUNTERS = 16384            # (token, block of heads) pairs of a decode step whose key ranges one kernel merges
DECODE_ATTENTION_MAX_NEW = 8  # entries that bring at most this many tokens use the split-key kernel
# A decode step of up to this many requests leaves the rotary kernel's work to the attention kernel (measured on a
# B200, 16 heads of 128: 2 us a layer gained at 1 request, 4 at 8, 1.5 lost at 64, where every one of a thousand
# blocks pays for what one short kernel did).
ROTARY_IN_DECODE_KERNEL_MAX_TOKENS = 32


def _common_dtype(tensors):
    return torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype


def query_tiles(batch, rows: int) -> torch.Tensor:
    """The work list of a prompt-attention kernel that takes ``rows`` queries of one request at a time: int32
    [n_tiles, 4] rows of (first flat token, rows in the tile, entry index, absolute position of the first row).
    Made once a step for each tile size and shared by the layers (``batch.shared``)."""
    key = ("attention query tiles", rows)
    t = batch.shared.get(key)
    if t is None:
        out, flat = [], 0
        for b, e in enumerate(batch.entries):
            n = len(e.tokens)
            for i in range(0, n, rows):
                out.append((flat + i, min(rows, n - i), b, e.start + i))
            flat += n
        t = torch.from_numpy(np.asarray(out, dtype=np.int32).reshape(-1, 4)).to(batch.token_ids.device)
        batch.shared[key] = t
    return t


def prefill_tc_plan(batch, window, n_heads: int):
    """This step's work items for the tcgen05 prompt attention kernel (``ops.prefill_tc_plan``) on the device: made
    once a step for each window and shared by the layers that have it."""
    key = ("attention tcgen05 items", window, n_heads)
    plan = batch.shared.get(key)
    if plan is None:
        items, merges, parts = ops.prefill_tc_plan([(len(e.tokens), e.start) for e in batch.entries], window, n_heads)
        both = torch.from_numpy(np.concatenate([items.reshape(-1), merges.reshape(-1)])).to(batch.token_ids.device)
        plan = (both[:items.size].view(-1, 8), both[items.size:].view(-1, 4) if merges.size else None, parts)
        batch.shared[key] = plan
    return plan


class GqaAttention(Mixer):
    @property
    def graph_safe(self):
        # this mixer only enqueues kernels; whether its position part does is that part's word
        return self.position.graph_safe

    def __init__(self, spec):
        super().__init__(spec)
        s = spec
        if s.head_dim % 2 or s.head_dim > 256:
            raise ValueError(f"head_dim={s.head_dim}: must be even and at most 256")
        if s.window is not None and s.window < 1:
            raise ValueError(f"window={s.window}: a window holds at least the query's own position")
        if s.n_heads % s.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        # the position encoding is a part of its own: it rotates q and k and stores k and v (no encoding: it only stores)
        self.position = build_part(s.position if s.position is not None else NoPositionSpec())
        self.q_size = s.n_heads * s.head_dim
        self.kv_size = s.n_kv_heads * s.head_dim
        self.scale = s.softmax_scale if s.softmax_scale is not None else 1.0 / math.sqrt(s.head_dim)

    def cache_spec(self):
        return CacheSpec(paged=KvCacheSpec(self.spec.n_kv_heads, self.spec.head_dim, self.spec.window))

    def tensor_decls(self):
        s, p = self.spec, self.spec.prefix
        d = [
            TensorDecl(p + "q_proj.weight", (self.q_size, s.hidden)),
            TensorDecl(p + "k_proj.weight", (self.kv_size, s.hidden)),
            TensorDecl(p + "v_proj.weight", (self.kv_size, s.hidden)),
            TensorDecl(p + "o_proj.weight", (s.hidden, self.q_size)),
        ]
        if s.qkv_bias:
            d += [
                TensorDecl(p + "q_proj.bias", (self.q_size,)),
                TensorDecl(p + "k_proj.bias", (self.kv_size,)),
                TensorDecl(p + "v_proj.bias", (self.kv_size,)),
            ]
        return d

    def load(self, src, rt):
        super().load(src, rt)
        p = self.spec.prefix
        ws = [src.get(p + f"{n}_proj.weight") for n in "qkv"]
        dt = _common_dtype(ws)
        self.w_qkv = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
        self.b_qkv = None
        if self.spec.qkv_bias:
            bs = [src.get(p + f"{n}_proj.bias") for n in "qkv"]
            bdt = _common_dtype(bs)
            self.b_qkv = torch.cat([b.to(bdt) for b in bs]).contiguous()
        self.w_o = src.get(p + "o_proj.weight")
        self.position.load(src, rt)
        # zeroed scratch of the decode attention kernel that merges its own key ranges (it leaves it zeroed)
        self._range_counters = (torch.zeros(RANGE_COUNTERS, dtype=torch.int32, device=rt.device)
                                if rt.device.type == "cuda" else None)

    def reset_after_fault(self):
        # blocks that gave up never counted themselves: the counters of the merge must start at zero again
        if self._range_counters is not None:
            self._range_counters.zero_()
        self.position.reset_after_fault()

    def forward_add(self, x, h, batch, cache):
        s = self.spec
        T = x.shape[0]
        qkv = self.rt.empty(T, self.q_size + 2 * self.kv_size)
        # (what runs before a block's first product is a norm or the combination before it: short kernels)
        ops.linear(x, self.w_qkv, qkv, bias=self.b_qkv, status=batch.status, stream=batch.stream, after_short_kernel=True)
        # A decode step of one token a request: where the attention kernel can, it rotates the queries and rotates and
        # stores the keys and values itself (one launch less on every layer's path); else the position part does.
        in_kernel = None
        if (batch.max_new == 1 and T <= ROTARY_IN_DECODE_KERNEL_MAX_TOKENS
                and ops.decode_store_ok(qkv, cache.k, s.head_dim, cache.page_size)):
            in_kernel = self.position.in_decode_kernel(batch, s.head_dim)
        if in_kernel is None:
            self.position.rotate_and_store(qkv, batch, cache, s.n_heads, s.n_kv_heads, s.head_dim)
        attn = self.rt.empty(T, self.q_size)
        if batch.max_new <= DECODE_ATTENTION_MAX_NEW:
            # few query tokens: split each request's keys over many blocks
            group = s.n_heads // s.n_kv_heads
            per_sm = ops.decode_tma_blocks_per_sm(qkv.dtype, s.head_dim, cache.page_size)
            # blocks per token: the tensor-core kernels take 16 query heads of a kv head at a time, the CUDA-core one 8
            kv_blocks = s.n_kv_heads * -(-group // (16 if qkv.dtype == torch.bfloat16 else 8))
            split_len, n_splits = ops.decode_split_plan(
                T, kv_blocks, cache.block_table.shape[1] * cache.page_size, per_sm or 3, single_is_final=per_sm > 0,
                run_latency=ops.DECODE_RUN_LATENCY if per_sm else 0.0)
            part_acc = self.rt.empty(T, s.n_heads, n_splits, s.head_dim, dtype=torch.float32)
            part_ml = self.rt.empty(T, s.n_heads, n_splits, 2, dtype=torch.float32)
            ops.decode_attention(
                qkv, cache.k, cache.v, cache.block_table, cache.page_size, batch.positions, batch.token_seq,
                batch.seq_slot, attn, s.n_heads, s.n_kv_heads, s.head_dim, s.window, self.scale, split_len, n_splits,
                part_acc, part_ml, status=batch.status, counters=self._range_counters, stream=batch.stream,
                # the kernel just before (the position part's, or the projection) wrote these rows' q and at most the
                # k, v of the step's own positions, max_new of a request
                fresh_positions=batch.max_new,
                store_new=in_kernel is not None, write_pages=cache.writes, cos_sin=in_kernel[0] if in_kernel else None,
            )
        elif ops.prefill_tc_ok(qkv, attn, cache.k, cache.page_size, s.head_dim):
            # prompt portions: tiles of 256 queries (long ones cut into runs of key blocks), tcgen05
            items, merges, parts = prefill_tc_plan(batch, s.window, s.n_heads)
            part_o = part_ml = None
            if parts:
                part_o = self.rt.empty(parts, s.n_heads, ops.WIDE_PREFILL_TILE, s.head_dim, dtype=torch.float32)
                part_ml = self.rt.empty(parts, s.n_heads, ops.WIDE_PREFILL_TILE, 2, dtype=torch.float32)
            ops.prefill_attention_tc(
                qkv, cache.k, cache.v, cache.block_table, cache.page_size, items, batch.seq_slot, attn,
                s.n_heads, s.n_kv_heads, s.head_dim, s.window, self.scale, status=batch.status, stream=batch.stream,
                merges=merges, part_o=part_o, part_ml=part_ml,
            )
        elif ops.prefill_ok(qkv, attn, cache.k, s.head_dim):
            # prompt portions, other head and page sizes: tiles of 64 queries, mma.sync
            ops.prefill_attention(
                qkv, cache.k, cache.v, cache.block_table, cache.page_size, query_tiles(batch, ops.PREFILL_TILE),
                batch.seq_slot, attn,
                s.n_heads, s.n_kv_heads, s.head_dim, s.window, self.scale, stream=batch.stream,
            )
        else:
            # 32-bit, and head sizes that are no multiple of 16: a warp per (token, head)
            ops.paged_attention(
                qkv, cache.k, cache.v, cache.block_table, cache.page_size, batch.positions, batch.token_seq,
                batch.seq_slot, attn, s.n_heads, s.n_kv_heads, s.head_dim, s.window, self.scale, stream=batch.stream,
            )
        # (the attention's last blocks only add up key ranges: the memory system is idle under them)
        ops.linear(attn, self.w_o, h, accumulate=True, status=batch.status, stream=batch.stream, after_short_kernel=True)


register_part("gqa_attention", GqaAttention, replace=True)
