"""Causal grouped-query attention as a mixer.

x -> [Q | K | V] = x . Wqkv^T -> per-head RMSNorm on Q and K (optional) ->
position encoding on Q and K -> keys and values into the cache -> softmax(q.k *
scale) v over the keys the query may see (all earlier ones, or the last
``window``) -> . Wo^T, added into the residual stream.

berniehans/titan: engine/engine-core/src/forward_cpu.rs:300-366 and 440-507;
driver steps forward_driver.rs:1010-1133 (prompt) and 2168-2259 (one token).
Q, K and V are three launches there; here their weights are concatenated at
bind time into one [Q + 2 KV, H] matrix.  Which tensors those are is the spec's
business (``MixerSpec.names``): by default q_proj / k_proj / v_proj / o_proj
``.weight`` under the prefix; a checkpoint that stores one fused tensor names
it under the role "qkv".

A step of single tokens writes K and V into the cache inside the norm/rotary
kernel and attends over the cache.  A step with longer runs of tokens keeps the
step's own K and V beside the cache, attends over both, and appends afterwards,
which is what makes a ring of ``window`` rows safe.

With ``cache_from`` the mixer owns no keys: it projects queries only and reads
the named layer's cache.
"""
from __future__ import annotations

import ctypes
import math
from typing import List, Optional

import torch

from .. import kernels as K
from ..cache.groups import CacheNeed, KVGroup
from ..weights.loader import WeightSpec
from . import linear
from .base import MIXERS, POSITIONS, Mixer
from .norm import DeferredNorm, rows_of


def decode_split(lay, kv_heads: int, options, fast: bool):
    """(fewest keys per split, most splits) of decode attention; the kernels cut every sequence by its own
    length from these two numbers (``tb_split_keys``).  Neither depends on what the sequences hold or on the
    longest context the engine allows, so a sequence's borders are the same in any cache and beside any
    neighbours, and a captured step and an eager one cut the keys at the same places.

    The any-size kernel takes splits of ``attn_chunk`` keys, as many as the longest sequence needs (an eager
    step) or as the context limit needs (a captured one, whose grid is fixed; the spare ones leave at once):
    the borders are multiples of ``attn_chunk`` either way.  The tensor-core kernel takes the number of splits
    that fills the machine once at this batch size: two of its CTAs fit an SM, and (sequences x kv heads x splits)
    stays within 7/8 of those 2 x SMs places, because the splits of a (sequence, kv head) are a thread-block cluster,
    which is placed as a whole inside one part of the chip: with every place counted, some clusters wait for a
    second round (measured after 2,048-token prompts: 5 sequences 3.28 -> 3.03 ms per step with 6 splits instead
    of 7, 6 sequences 3.36 -> 3.09, 9 sequences 3.54 -> 3.29, 12 sequences 3.80 -> 3.50).  At most 16 splits merge
    inside a cluster (no scratch, no merge kernel), and clusters of more than 8 CTAs only while they fill half of
    the machine (16 / 9 / 8 / 4 / 2 / 1 splits at batch 1 / 2 / 4 / 8 / 16 / 32 with 8 kv heads)."""
    if not fast:
        chunk = int(options.get("attn_chunk", 256))
        cover = int(options.get("max_context", 0)) if options.get("fixed_splits") else 0
        return chunk, max(1, -(-(cover or lay.max_kv_len) // chunk))
    sms = int(options.get("sm_count", 148))
    pairs = lay.B * kv_heads
    splits = max(1, min(16, (2 * sms * 7 // 8) // pairs))
    if splits > 8:
        splits = max(8, min(splits, sms // pairs))
    forced = int(options.get("attn_splits", 0))
    return int(options.get("attn_min_chunk", 128)), forced or splits


class AttentionMixer(Mixer):
    folds_norm = True           # a decode step's Q|K|V product takes the norm before it in

    def __init__(self, spec):
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ValueError(f"{s.num_heads} query heads are not a multiple of {s.num_kv_heads} kv heads")
        if s.head_dim % 16 or not 16 <= s.head_dim <= 256:
            raise ValueError(f"head_dim {s.head_dim} is not supported: multiples of 16 from 16 to 256")
        if s.window is not None and s.window <= 0:
            raise ValueError("an attention window must be positive")
        if s.cache_from is not None and s.window is not None:
            raise ValueError("a mixer that reads another layer's cache cannot have a window")
        self.spec = s
        self.Q, self.KV = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        self.shared = s.cache_from is not None
        self.position = POSITIONS.build(s.position)
        self.scale = s.softmax_scale if s.softmax_scale is not None else 1.0 / math.sqrt(s.head_dim)
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None
        self._views = {}

    # -- declaration ------------------------------------------------------ #
    def cache_need(self) -> Optional[CacheNeed]:
        if self.shared:
            return None
        return CacheNeed("kv", self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def _names(self):
        """Tensor names (relative to the prefix) by role; "qkv" only if the spec names a fused tensor."""
        s = self.spec
        names = {role: s.name(role, role + "_proj.weight") for role in ("q", "k", "v", "o")}
        names["qkv"] = s.name("qkv")
        if names["qkv"] is not None and self.shared:
            raise ValueError("a mixer that reads another layer's cache has queries only: it cannot name a fused q|k|v tensor")
        return names

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        s, p, n = self.spec, prefix + self.spec.prefix, self._names()
        specs = [WeightSpec(p + n["o"], (s.hidden_size, self.Q))]
        if n["qkv"] is not None:
            specs.append(WeightSpec(p + n["qkv"], (self.Q + 2 * self.KV, s.hidden_size)))
        else:
            specs.append(WeightSpec(p + n["q"], (self.Q, s.hidden_size)))
            if not self.shared:
                specs += [WeightSpec(p + n["k"], (self.KV, s.hidden_size)),
                          WeightSpec(p + n["v"], (self.KV, s.hidden_size))]
        if s.qk_norm is not None:
            for which in ("q",) if self.shared else ("q", "k"):
                specs.append(WeightSpec(p + s.qk_norm.weight.format(which), (s.head_dim,), "vector", ("one_plus_normal", 0.1)))
        return specs

    def bind(self, get) -> None:
        s, p, n = self.spec, self.spec.prefix, self._names()
        if n["qkv"] is not None:
            self.w_qkv = get(p + n["qkv"])
        else:
            parts = [get(p + n["q"])]
            if not self.shared:
                parts += [get(p + n["k"]), get(p + n["v"])]
            self.w_qkv = torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else parts[0]
        self.w_o = get(p + n["o"])
        if s.qk_norm is not None:
            self.q_norm = get(p + s.qk_norm.weight.format("q"))
            self.k_norm = None if self.shared else get(p + s.qk_norm.weight.format("k"))

    # -- one step --------------------------------------------------------- #
    def _view(self, cache) -> K.KvView:
        group, index = cache
        key = (id(group), index)
        if key not in self._views:
            if not isinstance(group, KVGroup):
                raise TypeError(f"attention reads keys and values from a 'kv' cache group, not from {type(group).__name__}")
            self._views[key] = K.KvView(group.layer_storage(index).data_ptr(), group.table.data_ptr(), group.table_width,
                                        group.ring_rows, group.page_size, group.num_pages, group.need.num_kv_heads,
                                        group.need.head_dim)
        return self._views[key]

    def _qk_args(self, qkv, width, q_buf, q_stride, view, lay, rope, T, hd, append: bool, zero_in: bool) -> K.QkArgs:
        s = self.spec
        qa = K.QkArgs()
        qa.inp, qa.in_stride = (None if qkv is None else qkv.data_ptr()), width
        qa.q_out, qa.q_stride = q_buf.data_ptr(), q_stride
        qa.k_out, qa.k_stride = None, 0
        qa.q_w = None if self.q_norm is None else self.q_norm.data_ptr()
        qa.k_w = None if self.k_norm is None else self.k_norm.data_ptr()
        qa.rope = rope                              # the position encoding's block, passed on as it is
        qa.eps = s.qk_norm.eps if s.qk_norm is not None else 0.0
        qa.nh, qa.nkv, qa.hd = s.num_heads, (0 if self.shared else s.num_kv_heads), hd
        qa.pos_of, qa.seq_of, qa.slot_of_seq = lay.pos_of.data_ptr(), lay.seq_of.data_ptr(), lay.slot_of_seq.data_ptr()
        qa.cache, qa.append, qa.T = view, int(append), T
        qa.zero_in = int(zero_in)
        qa.kv_len = lay.kv_len.data_ptr()
        return qa

    def forward(self, h, ctx, cache, out: torch.Tensor) -> None:
        s, lay = self.spec, ctx.layout
        T, Q, KV, hd = lay.T, self.Q, self.KV, s.head_dim
        width = Q if self.shared else Q + 2 * KV
        view = self._view(cache)
        decode = lay.all_single
        rope = self.position.kernel_args(ctx.device)
        # A decode step in bfloat16 sums Q | K | V in float32 (K slices of the product add into a zeroed
        # buffer), and the norm/rotary kernel rounds once, into the query buffer and the cache.
        wide_sum = decode and not self.shared and h.dtype == torch.bfloat16 and ctx.options.get("gemm", "fast") != "plain"
        row_sums = None
        if wide_sum:
            key = f"acc_qkv_{T}x{width}"            # zeroed once; the norm/rotary kernel leaves it zeroed again (Engine.reset_accumulators after a failed step)
            qkv = ctx.scratch.get(key)
            if qkv is None:
                qkv = ctx.scratch[key] = torch.zeros((T, width), dtype=torch.float32, device=ctx.device)
            # The norm before the projection, if it was handed over unevaluated, goes into the product: the kernel
            # adds the products of the unscaled rows into the sums and leaves the rows' sums of squares, one part per
            # K slice, at a place of this step's own; the head norm/rotary kernel adds the parts and scales the rows first.
            if isinstance(h, DeferredNorm) and T <= 32:
                row_sums = ctx.row_sums()
                if row_sums is not None and K.gemm_tc_normed_accepts(h.x, h.weight, self.w_qkv, qkv, linear.EPI_ADD, row_sums):
                    K.gemm_tc_normed(h.x, h.weight, h.eps, self.w_qkv, qkv, linear.EPI_ADD, ctx.stream, sumsq=row_sums,
                                     ordered=bool(ctx.options.get("reproducible", False)))
                else:
                    row_sums = None
            if row_sums is None:
                linear.matmul(rows_of(h), self.w_qkv, qkv, linear.EPI_ADD, ctx)
            q_buf, q_stride = ctx.empty((T, Q)), Q
        else:
            qkv = ctx.empty((T, width))
            linear.matmul(rows_of(h), self.w_qkv, qkv, linear.EPI_STORE, ctx)
            q_buf, q_stride = qkv, width
        # K and V go into the cache in this kernel when nothing of this step still has to read the rows
        # they replace: always for single tokens and for caches that keep everything; in a ring only if
        # every sequence starts at position 0 (attention then reads the step's own rows alone).
        append_now = not self.shared and (decode or view.ring_rows == 0 or lay.all_fresh)
        qa = self._qk_args(qkv, width, q_buf, q_stride, view, lay, rope, T, hd, append=append_now, zero_in=wide_sum)
        if not (self.shared or wide_sum):
            qa.k_out, qa.k_stride = qkv.data_ptr() + Q * qkv.element_size(), width
        if row_sums is not None:
            qa.row_sumsq = row_sums.data_ptr()
            qa.row_parts = K.gemm_tc_normed_slices(self.w_qkv, linear.EPI_ADD, T, bool(ctx.options.get("reproducible", False)))
            qa.row_width, qa.row_eps = s.hidden_size, h.eps
        # A decode step whose Q | K | V are float32 sums may leave head norm, rotation and append to the attention
        # kernel itself (one kernel less between the projection and the attention); decided below, where the
        # attention's arguments are known.  Everything else runs the kernel now.
        folds_head_norm = wide_sum and ctx.options.get("fold_head_norm", True)
        if not folds_head_norm:
            K.qk_norm_rope(qa, qkv.dtype, q_buf.dtype, ctx.stream)

        attn = ctx.empty((T, Q))
        aa = K.AttnArgs()
        aa.q, aa.q_stride = q_buf.data_ptr(), q_stride
        aa.out, aa.out_stride = attn.data_ptr(), Q
        aa.cache, aa.batch = view, lay.c_struct()
        aa.nh, aa.nkv, aa.hd = s.num_heads, view.kv_heads, hd
        aa.window, aa.scale = s.window or 0, self.scale
        if decode:
            fast = ctx.options.get("attention", "fast") != "plain" and q_buf.dtype == torch.bfloat16 and hd in (64, 128)
            chunk, splits = decode_split(lay, view.kv_heads, ctx.options, fast)
            need = lay.B * s.num_heads * splits * (hd + 2)
            scratch = ctx.scratch.get("attn_partials")
            if scratch is None or scratch.numel() < need:
                scratch = ctx.scratch["attn_partials"] = torch.empty(need, dtype=torch.float32, device=ctx.device)
            aa.kv_new, aa.kv_stride = None, 0
            aa.chunk, aa.n_splits, aa.scratch = chunk, splits, scratch.data_ptr()
            if ctx.options.get("early_pages", True):       # lengths the kernel may read before its predecessors end
                if lay.lengths_by_copy:
                    aa.early_len, aa.early_mode = lay.kv_len.data_ptr(), 1
                elif lay.committed_len is not None:
                    aa.early_len, aa.early_mode = lay.committed_len.data_ptr(), 2
            if folds_head_norm:
                aa.fused_qk = ctypes.pointer(qa)
                if not (fast and K.attn_decode_mma_accepts(aa, q_buf.dtype)):      # the kernel cannot take it in: as a kernel of its own, then
                    aa.fused_qk = None
                    K.qk_norm_rope(qa, qkv.dtype, q_buf.dtype, ctx.stream)
            if fast and K.attn_decode_mma_accepts(aa, q_buf.dtype):
                K.attn_decode_mma(aa, ctx.stream)
            else:
                K.attn_decode(aa, q_buf.dtype, ctx.stream)
        else:
            if self.shared:
                aa.kv_new, aa.kv_stride = None, 0
            else:
                aa.kv_new, aa.kv_stride = qkv.data_ptr() + Q * qkv.element_size(), width
            mode = ctx.options.get("attention", "fast")   # "fast" | "mma" | "plain"
            # The tensor-core kernels read keys and values from the step's own rows when every sequence starts at
            # position 0, and else from the cache's pages, if the step's keys lie there already (a cache that keeps
            # everything; a reader of another layer's cache finds them there in any case).
            if lay.all_fresh and not self.shared:
                source = K.KV_FROM_STEP
            elif view.ring_rows == 0 and (self.shared or append_now):
                source = K.KV_FROM_CACHE
            else:
                source = K.KV_NOWHERE
            if mode == "fast" and source and K.attn_prefill_tc_accepts(aa, q_buf.dtype, source):
                K.attn_prefill_tc(aa, source, ctx.stream)
            elif mode in ("fast", "mma") and source and K.attn_prefill_mma_accepts(aa, q_buf.dtype, source):
                K.attn_prefill_mma(aa, source, ctx.stream)
            else:
                K.attn_prefill(aa, q_buf.dtype, ctx.stream)
            if not self.shared and not append_now:
                K.kv_append(qkv[:, Q:], view, lay.c_struct(), ctx.stream)
        linear.matmul(attn, self.w_o, out, linear.EPI_ADD, ctx)


MIXERS.register("attention", AttentionMixer)
