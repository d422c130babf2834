"""Causal grouped-query attention over the paged cache
(crates/glassbox-core/src/model.rs:260-325).

h -> qkv = h Wqkv^T (q, k, v stacked by rows) -> position encoding of q and k at each row's own
position, k and v stored at the row's cache slot (all rows of the step before any attention)
-> per (row, head) softmax(q k^T * scale) v over the row's visible keys of its own request
-> residual += att Wo^T. No bias anywhere. With ``writes_cache`` False the keys and values of
this run are not stored and attention reads what the named cache layer already holds.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.binding import ParamSpec
from .base import Mixer, PagedKvSpec, Position, build_part, register_part
from .linear import _resolve, linear, weights_ahead


class GqaAttention(Mixer):
    accepts_deferred_input = True
    launches_through_kernels_only = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"num_heads {s.num_heads} is not a multiple of num_kv_heads {s.num_kv_heads}")
        if s.head_dim % 2 or s.head_dim > 256:
            raise ValueError(f"head_dim {s.head_dim} must be even and at most 256")
        if s.window is not None and s.window <= 0:
            raise ValueError(f"window {s.window} must be positive")
        self.hidden_size = hidden_size
        self.nh, self.nkv, self.hd = s.num_heads, s.num_kv_heads, s.head_dim
        self.qd, self.kvd = self.nh * self.hd, self.nkv * self.hd
        self.position = build_part("position", s.position)

    def sub_parts(self):
        return {"position": self.position}

    def param_specs(self):
        d = self.hidden_size
        return {"wqkv": ParamSpec((self.qd + 2 * self.kvd, d), pieces=(self.qd, self.kvd, self.kvd)),
                "wo": ParamSpec((d, self.qd))}

    def cache_spec(self):
        return PagedKvSpec(self.nkv, self.hd, self.spec.window)

    def forward(self, ctx, h, residual, cache, writes_cache: bool) -> None:
        n = h.shape[0]
        qkv = ctx.scratch("qkv", (n, self.qd + 2 * self.kvd))
        table = self.position.fused_table(qkv.device)
        x, norm, _, scale = _resolve(h, self.params["wqkv"])
        plain_rotary = (table is not None and self.position.rotary_dim == self.hd) or \
            (table is None and type(self.position).apply_qk is Position.apply_qk)
        if (plain_rotary and (norm is not None or x.dtype == torch.bfloat16)
                and kernels.gemm_stream_qkv_supported(x, self.params["wqkv"], self.hd, qkv)):
            # few rows: one kernel normalises, projects, rotates and writes the cache
            kernels.gemm_stream_qkv(x, self.params["wqkv"], qkv, table, ctx.positions, cache.slots, cache.k, cache.v,
                                    self.nh, self.nkv, self.hd, cache.page_size, writes_cache, ctx.status, norm=norm,
                                    prefetch=weights_ahead(ctx, self.params["wqkv"]))
        elif (plain_rotary and norm is None and n > kernels.STREAM_MAX_ROWS
              and kernels.gemm_tc_qkv_supported(x, self.params["wqkv"], self.hd, qkv, cache.k)):
            # many rows: the tile kernel projects; its epilogue rotates from the float32 sums and writes the cache
            # (and completes the norm, if the product before this layer prepared it)
            kernels.gemm_tc_qkv(x, self.params["wqkv"], qkv, table, ctx.positions, cache.slots, cache.k, cache.v,
                                self.nh, self.nkv, self.hd, cache.page_size, writes_cache, ctx.status, row_scale=scale)
        else:
            linear(ctx, h, self.params["wqkv"], qkv)
            if table is None:
                self.position.apply_qk(ctx, qkv, self.nh, self.nkv, self.hd)
            kernels.rope_kv_write(qkv, table, ctx.positions, cache.slots, cache.k, cache.v, self.nh, self.nkv, self.hd,
                                  self.position.rotary_dim, cache.page_size, writes_cache, ctx.status)
        att = ctx.scratch("att", (n, self.qd))
        self.attend(ctx, qkv[:, :self.qd], att, cache)
        linear(ctx, att, self.params["wo"], residual, accumulate=True)


    #: Prefetch a layer's share of the cache into L2 only when it is small; above it the hook launches an empty kernel.
    #: The hook runs on a second stream beside the feed-forward of the layer before: the step's graph then has a fork
    #: after that layer's mixer and a join in front of this one. Measured on a B200 (decode, context 4096, ms per step
    #: with the prefetch / with an empty kernel in its place / with no second stream at all): 135M shapes batch 1
    #: (3 MB a layer) 0.628 / 0.632 / 0.684, batch 8 (25 MB) 0.735 / 0.713 / 0.779; with the empty kernel against
    #: nothing: 360M batch 8 1.165 / 1.213, 1.7B batch 1 1.358 / 1.436, batch 8 2.854 / 2.905. Most of the gain
    #: belongs to the fork and join themselves, not to the bytes moved (why a chain of kernels under programmatic
    #: dependent launch runs faster with them has not been found out; it is kept because it is measured, at every size).
    PREFETCH_MAX_BYTES = 8 << 20

    def prefetch(self, ctx, cache) -> None:
        if not ctx.decode_only or cache is None:
            return
        n = ctx.n
        step_bytes = 2 * n * min(ctx.max_context, self.spec.window or ctx.max_context) * self.kvd * cache.k.element_size()
        if step_bytes > self.PREFETCH_MAX_BYTES:
            kernels.stream_marker()
            return
        kernels.kv_prefetch(cache.k, cache.v, cache.block_tables, ctx.row_seq, ctx.positions, self.nkv, self.hd,
                            cache.page_size, self.spec.window, blocks_per_row=max(1, 148 // max(n, 1)))

    def attend(self, ctx, q, att, cache) -> None:
        """att[row, head, :] = softmax over the row's visible keys; the kernel is picked by the shape
        of the batch: rows that are single decoded tokens share the keys of a request between
        several blocks (on the tensor cores in bfloat16 where the head size is one the kernel is built
        for, else with float32 FMA); prompt portions take a flash kernel in bfloat16 at head sizes one
        is built for; anything else takes the one-warp-per-(row, head) kernel. A mixed batch that starts
        with many single-token requests (the scheduler puts them first) is split: those rows go to the
        decode kernel, the portions to the flash kernel, which would otherwise spend a 128-row tile per
        head on each of them."""
        n = q.shape[0]
        if ctx.decode_only:
            if self._attend_decode(ctx, q, att, cache, n):
                return
        else:
            k = ctx.leading_single if ctx.leading_single * self.nh > SPLIT_MIXED_ABOVE else 0
            if k and self._has_flash(q, att, cache) and self._attend_decode(ctx, q[:k], att[:k], cache, k):
                self._attend_flash(ctx, q, att, cache, k)
                return
            if self._attend_flash(ctx, q, att, cache, 0):
                return
        kernels.attention_rows(q, att, cache.k, cache.v, cache.block_tables, ctx.row_seq, ctx.positions, self.nh,
                               self.nkv, self.hd, cache.page_size, self.spec.scale, self.spec.window, ctx.status)

    def _attend_decode(self, ctx, q, att, cache, n: int) -> bool:
        """Rows 0 .. n-1, one per request (request i is row i); False if no decode kernel takes the shape."""
        if kernels.attention_decode_mma_supported(q.dtype, self.nh, self.nkv, self.hd, cache.page_size):
            splits, block_keys, warps = kernels.decode_mma_plan(n, self.nkv, self.hd, ctx.max_context)
            part_acc = ctx.scratch("decode_part_acc", (n, self.nh * warps * splits * self.hd), torch.float32, grow=True)
            part_ml = ctx.scratch("decode_part_ml", (n, self.nh * warps * splits * 2), torch.float32, grow=True)
            counters = ctx.zeros_once("decode_counters", ctx.max_rows * self.nh, torch.int32)
            kernels.attention_decode_mma(q, att, cache.k, cache.v, cache.block_tables, ctx.row_seq[:n], ctx.positions[:n],
                                         self.nh, self.nkv, self.hd, cache.page_size, self.spec.scale,
                                         self.spec.window, splits, part_acc, part_ml, counters, ctx.status, block_keys, warps)
            return True
        if self.hd % 16 == 0 and self.hd >= 16:
            splits = kernels.decode_splits(n, self.nh, self.nkv, ctx.max_context)
            part_acc = part_ml = counters = None
            if splits > 1:
                part_acc = ctx.scratch("decode_part_acc", (n, self.nh * splits * self.hd), torch.float32, grow=True)
                part_ml = ctx.scratch("decode_part_ml", (n, self.nh * splits * 2), torch.float32, grow=True)
                counters = ctx.zeros_once("decode_counters", ctx.max_rows * self.nh, torch.int32)
            kernels.attention_decode(q, att, cache.k, cache.v, cache.block_tables, ctx.row_seq[:n], ctx.positions[:n],
                                     self.nh, self.nkv, self.hd, cache.page_size, self.spec.scale, self.spec.window,
                                     splits, part_acc, part_ml, counters, ctx.status)
            return True
        return False

    def _has_flash(self, q, att, cache) -> bool:
        return (kernels.attention_prefill_tc_supported(q, att, self.nh, self.nkv, self.hd, cache.page_size)
                or kernels.attention_prefill_supported(q.dtype, self.nh, self.nkv, self.hd, cache.page_size))

    def _attend_flash(self, ctx, q, att, cache, first_seq: int) -> bool:
        """The requests from ``first_seq`` on (runs of consecutive rows); False if no flash kernel takes the shape."""
        tables = cache.block_tables[first_seq:]
        first_row, start_pos = ctx.seq_first_row[first_seq:], ctx.seq_start_pos[first_seq:]
        if kernels.attention_prefill_tc_supported(q, att, self.nh, self.nkv, self.hd, cache.page_size):
            kernels.attention_prefill_tc(q, att, cache.k, cache.v, tables, first_row, start_pos, ctx.max_rows_per_seq,
                                         self.nh, self.nkv, self.hd, cache.page_size, self.spec.scale, self.spec.window,
                                         ctx.status)
            return True
        if kernels.attention_prefill_supported(q.dtype, self.nh, self.nkv, self.hd, cache.page_size):
            kernels.attention_prefill(q, att, cache.k, cache.v, tables, first_row, start_pos, ctx.max_rows_per_seq,
                                      self.nh, self.nkv, self.hd, cache.page_size, self.spec.scale, self.spec.window,
                                      ctx.status)
            return True
        return False


#: a mixed batch is split between the decode and the flash kernel when its leading single-token requests would
#: otherwise add more 128-row tiles (one per request and head) than the GPU has SMs
SPLIT_MIXED_ABOVE = 148

register_part("mixer", "gqa_attention", GqaAttention, replace=True)
