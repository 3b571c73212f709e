"""Python face of the hand-written CUDA library: argument structs and checked calls.

Every function here launches kernels of ``titan_b200/csrc`` on the given CUDA
stream and raises ``KernelError`` with the launcher's message when it refuses
its arguments.  Nothing here computes on the host and nothing falls back to a
library: if the extension cannot be built or loaded, the first call raises.
"""
from __future__ import annotations

import ctypes
import sys
from ctypes import POINTER, Structure, byref, c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .csrc import build as _build

EPI_STORE, EPI_F32, EPI_ADD, EPI_SWIGLU = 0, 1, 2, 3
F32, BF16 = 0, 1

launch_count = 0          # launcher calls since import (a launcher starts one or two kernels)
_launch_log = None        # while a log is open: launcher name -> calls (berniehans/titan keeps such a record per launch, engine-cuda/src/dispatch_telemetry.rs:13-143)


def launch_log_start() -> None:
    """Begin counting launcher calls by name (what a step launched, and how often)."""
    global _launch_log
    _launch_log = {}


def launch_log_stop() -> dict:
    """End the count; {launcher name: calls}, in the order of first use."""
    global _launch_log
    log, _launch_log = _launch_log or {}, None
    return log


class KernelError(RuntimeError):
    pass


def timeline_attach(buffer: Optional[torch.Tensor]) -> bool:
    """Names the buffer (int64, 1 + 8 * records) in which the decode kernels' timeline probe keeps its records, or
    takes it away (None).  False if the tensor-core library was built without the probe (csrc/timeline.cuh: it is
    compiled in with TITAN_B200_NVCC_FLAGS=-DTB_TIMELINE and costs nothing otherwise)."""
    lib_ = tlib()
    ptr = None if buffer is None else buffer.data_ptr()
    on = [int(f(c_void_p(ptr))) for f in (lib_.tb_gemm_tc_timeline, lib_.tb_attn_mma_timeline)]
    return all(v == 1 for v in on)


class KvView(Structure):
    _fields_ = [("storage", c_void_p), ("table", c_void_p), ("table_width", c_int), ("ring_rows", c_int),
                ("page_size", c_int), ("num_pages", c_int), ("kv_heads", c_int), ("head_dim", c_int)]


class Batch(Structure):
    _fields_ = [("tokens", c_void_p), ("seq_of", c_void_p), ("pos_of", c_void_p), ("slot_of_seq", c_void_p),
                ("q_start", c_void_p), ("start_pos", c_void_p), ("kv_len", c_void_p),
                ("T", c_int), ("B", c_int), ("max_new", c_int), ("max_kv_len", c_int)]


class RotaryArgs(Structure):
    """What a position encoding hands to the kernels; a mixer passes it on without looking inside.
    angle_k(position) = (position + offset) * inv_freq[k]; cosines and sines are scaled by ``magnitude``."""
    _fields_ = [("inv_freq", c_void_p), ("rot", c_int), ("offset", c_float), ("magnitude", c_float)]


class QkArgs(Structure):
    _fields_ = [("inp", c_void_p), ("in_stride", c_int), ("q_out", c_void_p), ("q_stride", c_int),
                ("k_out", c_void_p), ("k_stride", c_int), ("q_w", c_void_p), ("k_w", c_void_p),
                ("rope", RotaryArgs), ("eps", c_float), ("nh", c_int), ("nkv", c_int),
                ("hd", c_int), ("pos_of", c_void_p), ("seq_of", c_void_p), ("slot_of_seq", c_void_p),
                ("cache", KvView), ("append", c_int), ("T", c_int), ("zero_in", c_int), ("kv_len", c_void_p),
                ("row_sumsq", c_void_p), ("row_parts", c_int), ("row_width", c_int), ("row_eps", c_float)]


class AttnArgs(Structure):
    _fields_ = [("q", c_void_p), ("q_stride", c_int), ("kv_new", c_void_p), ("kv_stride", c_int),
                ("out", c_void_p), ("out_stride", c_int), ("cache", KvView), ("batch", Batch),
                ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("window", c_int), ("scale", c_float),
                ("chunk", c_int), ("n_splits", c_int), ("scratch", c_void_p),
                ("early_len", c_void_p), ("early_mode", c_int), ("fused_qk", POINTER(QkArgs))]


class SampleArgs(Structure):
    _fields_ = [("logits", c_void_p), ("ld", c_int), ("V", c_int), ("B", c_int), ("slot_of_row", c_void_p),
                ("temperature", c_void_p), ("top_k", c_void_p), ("top_p", c_void_p), ("penalty", c_void_p),
                ("seed", c_void_p), ("sequence_id", c_void_p), ("sample_step", c_void_p),
                ("last_token", c_void_p), ("seen", c_void_p), ("seen_words", c_int), ("out", c_void_p),
                ("part_best", c_void_p), ("part_idx", c_void_p), ("parts", c_int)]


_lib = None


def lib():
    """The loaded extension (built on first use)."""
    global _lib
    if _lib is None:
        l = _build.load()
        l.tb_last_error.restype = ctypes.c_char_p
        l.tb_uniform24.restype = ctypes.c_uint
        l.tb_uniform24.argtypes = [c_longlong, c_longlong, c_longlong]
        l.tb_embed.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        l.tb_fill_random.argtypes = [c_void_p, c_int, c_longlong, ctypes.c_ulonglong, c_float, c_float, c_void_p]
        l.tb_scale_f32.argtypes = [c_void_p, c_longlong, c_float, c_void_p]
        l.tb_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p]
        l.tb_gemm_simt.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
        l.tb_qk_norm_rope.argtypes = [POINTER(QkArgs), c_int, c_int, c_void_p]
        l.tb_kv_append.argtypes = [c_void_p, c_int, c_int, POINTER(KvView), POINTER(Batch), c_void_p]
        l.tb_attn_prefill.argtypes = [POINTER(AttnArgs), c_int, c_void_p]
        l.tb_attn_decode.argtypes = [POINTER(AttnArgs), c_int, c_void_p]
        l.tb_sample.argtypes = [POINTER(SampleArgs), c_void_p]
        l.tb_decode_prepare.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        l.tb_commit_lengths.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        l.tb_mark_seen.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
        _lib = l
    return _lib


_tlib = None


def tlib():
    """The library of tensor-core kernels (tcgen05 / TMA / mma.sync), built and loaded when first asked for."""
    global _tlib
    if _tlib is None:
        lib()
        l = _build.load("tensor")
        l.tb_gemm_tc.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
        l.tb_gemm_tc_normed.argtypes = [c_void_p, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
        l.tb_gemm_tc_normed_check.argtypes = [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        l.tb_gemm_tc_check.argtypes = [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]
        l.tb_attn_decode_mma.argtypes = [POINTER(AttnArgs), c_void_p]
        l.tb_attn_decode_mma_check.argtypes = [POINTER(AttnArgs), c_int]
        l.tb_attn_prefill_mma.argtypes = [POINTER(AttnArgs), c_int, c_void_p]
        l.tb_attn_prefill_mma_check.argtypes = [POINTER(AttnArgs), c_int, c_int]
        l.tb_attn_prefill_tc.argtypes = [POINTER(AttnArgs), c_int, c_void_p]
        l.tb_attn_prefill_tc_check.argtypes = [POINTER(AttnArgs), c_int, c_int]
        _tlib = l
    return _tlib


def _check(rc: int) -> None:
    global launch_count
    launch_count += 1
    if _launch_log is not None:
        name = sys._getframe(1).f_code.co_name
        _launch_log[name] = _launch_log.get(name, 0) + 1
    if rc:
        raise KernelError(lib().tb_last_error().decode())


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"the kernels take float32 and bfloat16, not {dt}")


def current_stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on CUDA tensors only; there is no CPU path")


# --------------------------------------------------------------------------- #
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, stream: int) -> None:
    _need_cuda(table, tokens, out)
    _check(lib().tb_embed(table.data_ptr(), dtype_code(table.dtype), tokens.data_ptr(), out.data_ptr(),
                          tokens.numel(), table.shape[1], table.shape[0], stream))


def fill_random(out: torch.Tensor, key: int, std: float, mean: float) -> None:
    """out[i] = normal(key, i) * std + mean (float32 or bfloat16), or 15-bit integers (int32): the counter-based
    generator of titan_b200.weights.random_init, on the device."""
    _need_cuda(out)
    if not out.is_contiguous():
        raise KernelError("fill_random: a contiguous tensor is wanted")
    code = -1 if out.dtype == torch.int32 else dtype_code(out.dtype)
    _check(lib().tb_fill_random(out.data_ptr(), code, out.numel(), key & ((1 << 64) - 1), std, mean, current_stream()))


def scale_f32(x: torch.Tensor, factor: float, stream: int) -> None:
    """x *= factor in place (float32, contiguous)."""
    _need_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale_f32: a contiguous float32 tensor is wanted")
    _check(lib().tb_scale_f32(x.data_ptr(), x.numel(), factor, stream))


def rmsnorm(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, eps: float, stream: int,
            rows: Optional[torch.Tensor] = None) -> None:
    _need_cuda(x, w, y, rows)
    n = y.shape[0]
    _check(lib().tb_rmsnorm(x.data_ptr(), w.data_ptr(), y.data_ptr(), dtype_code(y.dtype), _ptr(rows), n,
                            x.shape[-1], eps, stream))


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int, stream: int) -> None:
    """out (epilogue ``epi``) = x[M,K] . w[N,K]^T; x and out may be row-strided views."""
    _need_cuda(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or not w.is_contiguous() or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm: shapes do not fit: x {tuple(x.shape)} w {tuple(w.shape)}")
    _check(lib().tb_gemm_simt(x.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(w.dtype), M, N, K,
                              x.stride(0), out.stride(0), epi, stream))


def gemm_tc_accepts(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int) -> bool:
    """Whether the tensor-core kernel's alignment rules hold for this product."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous():
        return False
    if x.stride(1) != 1 or out.stride(1) != 1 or x.shape[1] != w.shape[1]:
        return False
    return tlib().tb_gemm_tc_check(x.shape[0], w.shape[0], x.shape[1], x.stride(0), out.stride(0), epi,
                                  x.data_ptr(), w.data_ptr(), out.data_ptr()) == 0


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int, stream: int, splits: int = 0, ordered: bool = False) -> None:
    """out (epilogue ``epi``) = x[M,K] . w[N,K]^T on the tcgen05 tensor cores (bfloat16 operands).  ``ordered``: partial
    sums along K add up in a fixed order (the K slices of a decode product inside a thread-block cluster, no prompt tile
    cut along K), so that the same inputs give the same bits on every run; the default lets float32 reductions meet at
    L2 in the order they arrive, which is faster and differs from run to run in the last bits."""
    _need_cuda(x, w, out)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc: operands must be bfloat16")
    want = torch.bfloat16 if epi in (EPI_STORE, EPI_SWIGLU) else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm_tc: this epilogue writes {want}, the output is {out.dtype}")
    M, K_ = x.shape
    N = w.shape[0]
    if w.shape[1] != K_ or not w.is_contiguous() or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm_tc: shapes do not fit: x {tuple(x.shape)} w {tuple(w.shape)}")
    _check(tlib().tb_gemm_tc(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K_, x.stride(0), out.stride(0), epi,
                            -1 if ordered and not splits else splits, stream))


def gemm_tc_normed_accepts(x: torch.Tensor, norm_w: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int,
                           sumsq: Optional[torch.Tensor]) -> bool:
    """Can the product run with the RMS norm of its input folded in (tb_gemm_tc_normed)?"""
    if x.dtype != torch.float32 or norm_w.dtype != torch.float32 or w.dtype != torch.bfloat16 or not w.is_contiguous():
        return False
    if x.stride(1) != 1 or out.stride(1) != 1 or x.shape[1] != w.shape[1] or norm_w.numel() != x.shape[1]:
        return False
    return tlib().tb_gemm_tc_normed_check(x.shape[0], w.shape[0], x.shape[1], x.stride(0), out.stride(0), epi, x.data_ptr(),
                                         norm_w.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(sumsq)) == 0


def gemm_tc_normed(x: torch.Tensor, norm_w: torch.Tensor, eps: float, w: torch.Tensor, out: torch.Tensor, epi: int, stream: int,
                   sumsq: Optional[torch.Tensor] = None, ordered: bool = False) -> None:
    """out (epilogue ``epi``) = rmsnorm(x; norm_w, eps) . w^T for the rows of a decode step, the norm folded into the
    product: x is the float32 residual stream.  EPI_SWIGLU: complete.  EPI_ADD: ``out`` (float32) receives the products
    of the rows times the norm's weight WITHOUT the rows' scales, and ``sumsq`` [slices, 32] (float32; ``gemm_tc_normed_slices``
    rows of it are written) the rows' sums of squares per K slice; the consumer multiplies row m by
    1/sqrt(sum_z sumsq[z, m] / K + eps).  ``ordered``: as for ``gemm_tc``."""
    _need_cuda(x, norm_w, w, out, sumsq)
    want = torch.bfloat16 if epi == EPI_SWIGLU else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm_tc_normed: this epilogue writes {want}, the output is {out.dtype}")
    _check(tlib().tb_gemm_tc_normed(x.data_ptr(), x.stride(0), norm_w.data_ptr(), eps, w.data_ptr(), out.data_ptr(), x.shape[0],
                                   w.shape[0], x.shape[1], out.stride(0), epi, _ptr(sumsq), int(bool(ordered)), stream))


def gemm_tc_normed_slices(w: torch.Tensor, epi: int, rows: int = 1, ordered: bool = False) -> int:
    """K slices that gemm_tc_normed cuts this product into (one row of partial sums of squares each) for a step of
    ``rows`` rows; ``ordered``: as it cuts when the slices add up in a fixed order (a cluster per tile: fewer fit)."""
    return int(tlib().tb_gemm_tc_normed_slices(w.shape[0], w.shape[1], epi, int(rows), int(bool(ordered))))


def gemm_tc_error() -> int:
    """Error word of the tensor-core kernels (0: none); synchronises the device and clears the word."""
    return int(tlib().tb_gemm_tc_error())


def qk_norm_rope(args: QkArgs, in_dtype: torch.dtype, out_dtype: torch.dtype, stream: int) -> None:
    _check(lib().tb_qk_norm_rope(byref(args), dtype_code(in_dtype), dtype_code(out_dtype), stream))


def kv_append(kv: torch.Tensor, cache: KvView, batch: Batch, stream: int) -> None:
    _check(lib().tb_kv_append(kv.data_ptr(), kv.stride(0), dtype_code(kv.dtype), byref(cache), byref(batch), stream))


def attn_prefill(args: AttnArgs, dtype: torch.dtype, stream: int) -> None:
    _check(lib().tb_attn_prefill(byref(args), dtype_code(dtype), stream))


def attn_decode(args: AttnArgs, dtype: torch.dtype, stream: int) -> None:
    _check(lib().tb_attn_decode(byref(args), dtype_code(dtype), stream))


def attn_decode_mma_accepts(args: AttnArgs, dtype: torch.dtype) -> bool:
    return dtype == torch.bfloat16 and tlib().tb_attn_decode_mma_check(byref(args), BF16) == 0


def attn_decode_mma(args: AttnArgs, stream: int) -> None:
    """Decode attention on tensor cores (bfloat16, head_dim 64 or 128), then the merge of the splits."""
    _check(tlib().tb_attn_decode_mma(byref(args), stream))


def set_attn_decode_cluster(on: bool) -> None:
    """Decode attention with up to 16 splits: merge them inside a thread-block cluster (on by default) or through
    scratch memory and the merge kernel."""
    tlib().tb_attn_decode_set_cluster(int(bool(on)))


def set_attn_decode_late_trigger(on: bool) -> None:
    """Decode attention lets the kernel after it start once its own pages have been requested and read (on by
    default), or at once: the next kernel's first weight requests then queue in front of the pages."""
    tlib().tb_attn_decode_set_late_trigger(int(bool(on)))


# Where the tensor-core prompt kernels take keys and values from: nowhere they can (0), the step's own rows (every
# sequence starts at position 0), or the cache's pages (the step's keys are appended already; no ring).
KV_NOWHERE, KV_FROM_STEP, KV_FROM_CACHE = 0, 1, 2


def attn_prefill_mma_accepts(args: AttnArgs, dtype: torch.dtype, source: int) -> bool:
    return dtype == torch.bfloat16 and tlib().tb_attn_prefill_mma_check(byref(args), BF16, int(source)) == 0


def attn_prefill_mma(args: AttnArgs, source: int, stream: int) -> None:
    """Causal attention of prompts and continuation chunks on tensor cores (bfloat16, head_dim 64 or 128)."""
    _check(tlib().tb_attn_prefill_mma(byref(args), int(source), stream))


def attn_prefill_tc_accepts(args: AttnArgs, dtype: torch.dtype, source: int) -> bool:
    return dtype == torch.bfloat16 and tlib().tb_attn_prefill_tc_check(byref(args), BF16, int(source)) == 0


def attn_prefill_tc(args: AttnArgs, source: int, stream: int) -> None:
    """Causal attention of prompts and continuation chunks on the tcgen05 tensor cores (bfloat16, head_dim 128)."""
    _check(tlib().tb_attn_prefill_tc(byref(args), int(source), stream))


def attn_tc_error() -> int:
    return int(tlib().tb_attn_tc_error())


def attn_mma_error() -> int:
    return int(tlib().tb_attn_mma_error())


def sample(args: SampleArgs, stream: int) -> None:
    _check(lib().tb_sample(byref(args), stream))


def set_sample_team(ctas: int) -> None:
    """CTAs (a thread-block cluster) that share a row that is not greedy: 0 = by the size of the vocabulary
    (8 from 65,536 tokens, 4 from 16,384, else 1), or 1, 2, 4, 8."""
    lib().tb_sample_set_team(int(ctas))


def mark_seen(tokens, seq_of, slot_of_seq, seen: torch.Tensor, T: int, stream: int) -> None:
    _check(lib().tb_mark_seen(tokens.data_ptr(), seq_of.data_ptr(), slot_of_seq.data_ptr(), seen.data_ptr(),
                              seen.shape[1], T, stream))


def decode_prepare(slot_of_seq, seq_len, last_token, feed_last: bool, tokens, pos_of, start_pos, kv_len, stream: int) -> None:
    _check(lib().tb_decode_prepare(slot_of_seq.data_ptr(), seq_len.data_ptr(), last_token.data_ptr(), int(feed_last),
                                   tokens.data_ptr(), pos_of.data_ptr(), start_pos.data_ptr(), kv_len.data_ptr(),
                                   slot_of_seq.numel(), stream))


def commit_lengths(slot_of_seq, kv_len, seq_len, stream: int) -> None:
    _check(lib().tb_commit_lengths(slot_of_seq.data_ptr(), kv_len.data_ptr(), seq_len.data_ptr(), slot_of_seq.numel(), stream))


def wait_errors() -> dict:
    """The error words of the kernels whose waits are bounded (a wait that gave up leaves a code there and the
    step's result is invalid).  Reads and clears them; synchronises the device.  Empty if all is well, and
    if the tensor-core library was never loaded."""
    if _tlib is None:
        return {}
    found = {"gemm_tc": gemm_tc_error(), "attn_prefill_tc": attn_tc_error(), "attn_mma": attn_mma_error()}
    return {k: v for k, v in found.items() if v}


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for every kernel launched afterwards (on by default)."""
    lib().tb_set_pdl(int(bool(on)))


def set_gemm_tail_split(on: bool) -> None:
    """Prompt products with the ADD epilogue: cut the tiles of a last, partly filled round along K (on by default) or keep them whole."""
    tlib().tb_gemm_tc_set_tail_split(int(bool(on)))


def set_gemm_pair(on: bool) -> None:
    """Prompt products on pairs of CTAs that share one MMA (on by default) or on single CTAs."""
    tlib().tb_gemm_tc_set_pair(int(bool(on)))


def set_gemm_swap_below(m: int) -> None:
    """Products with fewer rows than this run in swap mode (weights on the 128-row side): 128 by default, at most 129."""
    tlib().tb_gemm_tc_set_swap_below(int(m))


def set_gemm_plain_tile(which: int) -> None:
    """Prompt products: 0 lets the launcher choose the tile shape (default), 1 forces CTA pairs with 256 x 256 tiles
    (from 256 x 256 outputs on), 2 single CTAs with 128 x 256 tiles, 3 single CTAs with 128 x 128 tiles."""
    tlib().tb_gemm_tc_set_plain_tile(int(which))


def gemm_pair_clusters(epi: int) -> int:
    """CTA pairs the device holds at once for the pair kernel of this epilogue (0: it cannot run)."""
    return int(tlib().tb_gemm_tc_pair_clusters(int(epi)))


def uniform24(seed: int, sequence: int, step: int) -> int:
    return int(lib().tb_uniform24(seed, sequence, step))
