"""Causal grouped-query attention as a mixer.

x -> [Q | K | V] = x . Wqkv^T -> per-head RMSNorm on Q and K (optional) ->
position encoding on Q and K -> keys and values into the cache -> softmax(q.k *
scale) v over the keys the query may see (all earlier ones, or the last
``window``) -> . Wo^T, added into the residual stream.

berniehans/titan: engine/engine-core/src/forward_cpu.rs:300-366 and 440-507;
driver steps forward_driver.rs:1010-1133 (prompt) and 2168-2259 (one token).
Q, K and V are three launches there; here their weights are concatenated at
bind time into one [Q + 2 KV, H] matrix.

A step of single tokens writes K and V into the cache inside the norm/rotary
kernel and attends over the cache.  A step with longer runs of tokens keeps the
step's own K and V beside the cache, attends over both, and appends afterwards,
which is what makes a ring of ``window`` rows safe.

With ``cache_from`` the mixer owns no keys: it projects queries only and reads
the named layer's cache.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import kernels as K
from ..cache.groups import CacheNeed, KVGroup
from ..weights.loader import WeightSpec
from . import linear
from .base import MIXERS, POSITIONS, Mixer


def decode_split(lay, kv_heads: int, options, fast: bool):
    """(keys per split, number of splits) of decode attention.  Both depend on the batch size and on the
    context limit only, so a sequence's result is the same whatever the other sequences hold, and a
    captured step (whose grid is fixed) and an eager one cut the keys at the same places."""
    bound = int(options.get("max_context", 0)) or lay.max_kv_len
    if not fast:
        chunk = int(options.get("attn_chunk", 256))
    else:
        # Two CTAs of the tensor-core kernel fit an SM.  Measured over batch sizes 1 to 8 at 8,192 keys: one
        # round of CTAs on about 0.6 of those places is fastest (a second round costs a whole chunk, more
        # splits a longer merge), chunks under 512 keys never pay, and at most 16 splits: up to 16 merge
        # inside a thread-block cluster (no scratch, no merge kernel), which at batch 1 beats more, smaller
        # chunks through scratch.
        places = 2 * int(options.get("sm_count", 148))
        pairs = lay.B * kv_heads
        want = min(16, max(1, (3 * places // 5 + pairs // 2) // pairs))
        chunk = max(512, -(-(-(-bound // want)) // 64) * 64)
    # an eager step launches the splits its longest sequence needs; a captured one, whose grid cannot
    # change, launches what the context limit needs (the extra CTAs leave at once)
    cover = bound if options.get("fixed_splits") else lay.max_kv_len
    return chunk, max(1, -(-cover // chunk))


class AttentionMixer(Mixer):
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

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        s, p = self.spec, prefix + self.spec.prefix
        specs = [WeightSpec(p + "q_proj.weight", (self.Q, s.hidden_size)),
                 WeightSpec(p + "o_proj.weight", (s.hidden_size, self.Q))]
        if not self.shared:
            specs += [WeightSpec(p + "k_proj.weight", (self.KV, s.hidden_size)),
                      WeightSpec(p + "v_proj.weight", (self.KV, s.hidden_size))]
        if s.qk_norm is not None:
            for which in ("q",) if self.shared else ("q", "k"):
                specs.append(WeightSpec(p + s.qk_norm.weight.format(which), (s.head_dim,), "vector", ("one_plus_normal", 0.1)))
        return specs

    def bind(self, get) -> None:
        s, p = self.spec, self.spec.prefix
        parts = [get(p + "q_proj.weight")]
        if not self.shared:
            parts += [get(p + "k_proj.weight"), get(p + "v_proj.weight")]
        self.w_qkv = torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else parts[0]
        self.w_o = get(p + "o_proj.weight")
        if s.qk_norm is not None:
            self.q_norm = get(p + s.qk_norm.weight.format("q"))
            self.k_norm = None if self.shared else get(p + s.qk_norm.weight.format("k"))

    # -- one step --------------------------------------------------------- #
    def _view(self, cache) -> K.KvView:
        group, index = cache
        key = (id(group), index)
        if key not in self._views:
            assert isinstance(group, KVGroup)
            self._views[key] = K.KvView(group.layer_storage(index).data_ptr(), group.table.data_ptr(), group.table_width,
                                        group.ring_rows, group.page_size, group.num_pages, group.need.num_kv_heads,
                                        group.need.head_dim)
        return self._views[key]

    def _qk_args(self, qkv, width, q_buf, q_stride, view, lay, inv_freq, T, hd, append: bool, zero_in: bool) -> K.QkArgs:
        s = self.spec
        qa = K.QkArgs()
        qa.inp, qa.in_stride = (None if qkv is None else qkv.data_ptr()), width
        qa.q_out, qa.q_stride = q_buf.data_ptr(), q_stride
        qa.k_out, qa.k_stride = None, 0
        qa.q_w = None if self.q_norm is None else self.q_norm.data_ptr()
        qa.k_w = None if self.k_norm is None else self.k_norm.data_ptr()
        qa.inv_freq = None if inv_freq is None else inv_freq.data_ptr()
        qa.eps = s.qk_norm.eps if s.qk_norm is not None else 0.0
        qa.rot, qa.nh, qa.nkv, qa.hd = self.position.rotary_dim, s.num_heads, (0 if self.shared else s.num_kv_heads), hd
        qa.pos_of, qa.seq_of, qa.slot_of_seq = lay.pos_of.data_ptr(), lay.seq_of.data_ptr(), lay.slot_of_seq.data_ptr()
        qa.cache, qa.append, qa.T = view, int(append), T
        qa.zero_in = int(zero_in)
        qa.kv_len = lay.kv_len.data_ptr()
        return qa

    def forward(self, h: torch.Tensor, ctx, cache, out: torch.Tensor) -> None:
        s, lay = self.spec, ctx.layout
        T, Q, KV, hd = lay.T, self.Q, self.KV, s.head_dim
        width = Q if self.shared else Q + 2 * KV
        view = self._view(cache)
        decode = lay.all_single
        tables = self.position.tables(ctx.device)
        inv_freq = tables.get("inv_freq")
        # A decode step in bfloat16 sums Q | K | V in float32 (K slices of the product add into a zeroed
        # buffer), and the norm/rotary kernel rounds once, into the query buffer and the cache.
        wide_sum = decode and not self.shared and h.dtype == torch.bfloat16 and ctx.options.get("gemm", "fast") != "plain"
        # ... or, on request (option qkv="fused") and where the kernel takes the shapes (heads of 128, at most
        # 16 tokens), the projection itself sums its K slices inside a thread-block cluster and does norm,
        # rotation and append.
        fused = None
        if wide_sum and ctx.options.get("qkv", "split") == "fused":
            q_buf = ctx.empty((T, Q))
            fused = self._qk_args(None, 0, q_buf, Q, view, lay, inv_freq, T, hd, append=True, zero_in=False)
            if not K.gemm_qkv_accepts(h, self.w_qkv, fused, q_buf.dtype):
                fused = None
        if fused is not None:
            K.gemm_qkv(h, self.w_qkv, fused, ctx.stream)
            q_stride = Q
        elif wide_sum:
            key = f"qkv_sum_{T}x{width}"            # zeroed once; the norm/rotary kernel leaves it zeroed again
            qkv = ctx.scratch.get(key)
            if qkv is None:
                qkv = ctx.scratch[key] = torch.zeros((T, width), dtype=torch.float32, device=ctx.device)
            linear.matmul(h, self.w_qkv, qkv, linear.EPI_ADD, ctx)
            q_buf, q_stride = ctx.empty((T, Q)), Q
        else:
            qkv = ctx.empty((T, width))
            linear.matmul(h, self.w_qkv, qkv, linear.EPI_STORE, ctx)
            q_buf, q_stride = qkv, width
        if fused is None:
            # K and V go into the cache in this kernel when nothing of this step still has to read the rows
            # they replace: always for single tokens and for caches that keep everything; in a ring only if
            # every sequence starts at position 0 (attention then reads the step's own rows alone).
            append_now = not self.shared and (decode or view.ring_rows == 0 or lay.all_fresh)
            qa = self._qk_args(qkv, width, q_buf, q_stride, view, lay, inv_freq, T, hd, append=append_now, zero_in=wide_sum)
            if not (self.shared or wide_sum):
                qa.k_out, qa.k_stride = qkv.data_ptr() + Q * qkv.element_size(), width
            K.qk_norm_rope(qa, qkv.dtype, q_buf.dtype, ctx.stream)
        else:
            append_now = True

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
            if fast and K.attn_decode_mma_accepts(aa, q_buf.dtype):
                K.attn_decode_mma(aa, ctx.stream)
            else:
                K.attn_decode(aa, q_buf.dtype, ctx.stream)
        else:
            if self.shared:
                aa.kv_new, aa.kv_stride = None, 0
            else:
                aa.kv_new, aa.kv_stride = qkv.data_ptr() + Q * qkv.element_size(), width
            mode = "plain" if self.shared else ctx.options.get("attention", "fast")   # "fast" | "mma" | "plain"
            if mode == "fast" and K.attn_prefill_tc_accepts(aa, q_buf.dtype, lay.all_fresh):
                K.attn_prefill_tc(aa, lay.all_fresh, ctx.stream)
            elif mode in ("fast", "mma") and K.attn_prefill_mma_accepts(aa, q_buf.dtype, lay.all_fresh):
                K.attn_prefill_mma(aa, lay.all_fresh, ctx.stream)
            else:
                K.attn_prefill(aa, q_buf.dtype, ctx.stream)
            if not self.shared and not append_now:
                K.kv_append(qkv[:, Q:], view, lay.c_struct(), ctx.stream)
        linear.matmul(attn, self.w_o, out, linear.EPI_ADD, ctx)


MIXERS.register("attention", AttentionMixer)
