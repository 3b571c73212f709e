"""Each CUDA kernel alone against a plain float32/float64 reference, at sizes other than the engine's
test models: head sizes in steps of 16, odd head counts and groups, widths and vocabularies that are
no power of two."""
import math

import pytest
import torch

from helpers import rel_l2
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KTOL = {"float32": 2e-6, "bfloat16": 6e-3}      # one kernel: float32 summation order / one bfloat16 rounding


@pytest.fixture(scope="module")
def K():
    from titan_b200 import kernels
    kernels.lib()
    return kernels


def dev(t):
    return t.cuda()


def stream():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(K, dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(777, 203, generator=g).to(DT[dtype])
    toks = torch.tensor([0, 776, 5, 5, 301], dtype=torch.int32)
    out = torch.empty(5, 203, device="cuda")
    K.embed(dev(table), dev(toks), out, stream())
    assert torch.equal(out.cpu(), P.embed_lookup(table, toks))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [48, 1000, 4100])
def test_rmsnorm(K, dtype, H):
    g = torch.Generator().manual_seed(H)
    x, w = torch.randn(9, H, generator=g) * 3, 1 + 0.1 * torch.randn(H, generator=g)
    y = torch.empty(9, H, dtype=DT[dtype], device="cuda")
    K.rmsnorm(dev(x), dev(w), y, 1e-3, stream())
    assert rel_l2(y.float().cpu(), P.rms_norm(x, w, 1e-3)) < KTOL[dtype]
    rows = torch.tensor([7, 0, 7], dtype=torch.int32)
    y2 = torch.empty(3, H, dtype=DT[dtype], device="cuda")
    K.rmsnorm(dev(x), dev(w), y2, 1e-3, stream(), dev(rows))
    assert torch.equal(y2, y[[7, 0, 7]])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,Kd", [(1, 130, 72), (37, 250, 200), (130, 66, 1032)])
def test_gemm_plain_all_epilogues(K, dtype, M, N, Kd):
    g = torch.Generator().manual_seed(M * N)
    x = (torch.randn(M, Kd, generator=g)).to(DT[dtype])
    w = (torch.randn(N, Kd, generator=g) * 0.1).to(DT[dtype])
    want = P.linear(x.float(), w.float())
    out = torch.empty(M, N, dtype=DT[dtype], device="cuda")
    K.gemm_simt(dev(x), dev(w), out, K.EPI_STORE, stream())
    assert rel_l2(out.float().cpu(), want) < KTOL[dtype]
    f = torch.empty(M, N, device="cuda")
    K.gemm_simt(dev(x), dev(w), f, K.EPI_F32, stream())
    assert rel_l2(f.cpu(), want) < 2e-6
    res = torch.randn(M, N, generator=g)
    acc = dev(res.clone())
    K.gemm_simt(dev(x), dev(w), acc, K.EPI_ADD, stream())
    assert rel_l2(acc.cpu(), res + want) < 2e-6
    act = torch.empty(M, N // 2, dtype=DT[dtype], device="cuda")
    K.gemm_simt(dev(x), dev(w), act, K.EPI_SWIGLU, stream())
    assert rel_l2(act.float().cpu(), P.swiglu(want[:, 0::2], want[:, 1::2])) < KTOL[dtype]
    # a strided view as input and output
    big = torch.zeros(M, Kd + 16, dtype=DT[dtype], device="cuda")
    big[:, 8:8 + Kd] = dev(x)
    wide = torch.zeros(M, N + 8, dtype=DT[dtype], device="cuda")
    K.gemm_simt(big[:, 8:8 + Kd], dev(w), wide[:, :N], K.EPI_STORE, stream())
    assert torch.equal(wide[:, :N], out) and float(wide[:, N:].abs().sum()) == 0


def test_gemm_refuses_what_it_cannot_run(K):
    x, w = torch.zeros(2, 8, device="cuda"), torch.zeros(5, 8, device="cuda")
    with pytest.raises(K.KernelError, match="even"):
        K.gemm_simt(x, w, torch.zeros(2, 2, device="cuda"), K.EPI_SWIGLU, stream())
    with pytest.raises(K.KernelError):
        K.gemm_simt(x, torch.zeros(5, 9, device="cuda"), torch.zeros(2, 5, device="cuda"), K.EPI_STORE, stream())
    with pytest.raises(K.KernelError, match="CUDA"):
        K.gemm_simt(x.cpu(), w, torch.zeros(2, 5, device="cuda"), K.EPI_STORE, stream())


class Paged:
    """A paged cache for tests: pages handed out in a scrambled order, other slots filled with noise."""

    def __init__(self, K, slots, lengths, nkv, hd, dtype, ring_rows=0, page=64, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.page, self.ring_rows, self.nkv, self.hd = page, ring_rows, nkv, hd
        width = max(-(-max(lengths) // page), 1) if not ring_rows else ring_rows // page
        per = [min(-(-n // page), width) for n in lengths]
        self.num_pages = sum(per) + 3
        order = torch.randperm(self.num_pages, generator=g).tolist()
        table = torch.full((max(slots) + 1, width), 0, dtype=torch.int32)
        for s, n in zip(slots, per):
            for j in range(n):
                table[s, j] = order.pop()
        self.table = table.cuda()
        self.storage = (torch.randn(2, self.num_pages, nkv, page, hd, generator=g) * 50).to(dtype).cuda()   # noise: a stale read shows
        self.view = K.KvView(self.storage.data_ptr(), self.table.data_ptr(), width, ring_rows, page, self.num_pages, nkv, hd)

    def put(self, slot, pos, k, v):
        """k, v: [nkv, hd] at position pos."""
        row = pos % self.ring_rows if self.ring_rows else pos
        page = int(self.table[slot, row // self.page])
        self.storage[0, page, :, row % self.page] = k.to(self.storage.dtype).cuda()
        self.storage[1, page, :, row % self.page] = v.to(self.storage.dtype).cuda()

    def get(self, slot, pos):
        row = pos % self.ring_rows if self.ring_rows else pos
        page = int(self.table[slot, row // self.page])
        return self.storage[0, page, :, row % self.page].float().cpu(), self.storage[1, page, :, row % self.page].float().cpu()


def layout_for(slots, starts, news):
    from titan_b200.engine.batch import StepEntry, StepLayout
    return StepLayout([StepEntry(s, [0] * n, []) for s, n in zip(slots, news)], starts, "cuda")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,rot", [(3, 1, 48, 48), (6, 2, 16, 8), (4, 4, 112, 112)])
def test_qk_norm_rope_in_place_and_append(K, dtype, nh, nkv, hd, rot):
    g = torch.Generator().manual_seed(hd)
    slots, starts, news = [4, 1], [70, 0], [3, 5]
    lay = layout_for(slots, starts, news)
    T, Q, KV = 8, nh * hd, nkv * hd
    qkv = torch.randn(T, Q + 2 * KV, generator=g).to(DT[dtype])
    qw, kw = 1 + 0.1 * torch.randn(hd, generator=g), 1 + 0.1 * torch.randn(hd, generator=g)
    k = torch.arange(rot // 2, dtype=torch.float64)
    inv = (torch.tensor(1e4, dtype=torch.float64) ** (-2 * k / rot)).float()
    pos = torch.tensor([70, 71, 72, 0, 1, 2, 3, 4])

    def ref(x, w):
        y = P.rms_norm(x.float(), w, 1e-5)
        r = P.rope_neox(y[..., :rot], pos, 1e4)
        return torch.cat([r, y[..., rot:]], -1)
    want_q = ref(qkv[:, :Q].view(T, nh, hd), qw)
    want_k = ref(qkv[:, Q:Q + KV].view(T, nkv, hd), kw)
    cache = Paged(K, slots, [73, 5], nkv, hd, DT[dtype])
    for append in (0, 1):
        buf = dev(qkv.clone())
        a = K.QkArgs()
        esz = buf.element_size()
        a.inp, a.in_stride, a.q_out, a.q_stride = buf.data_ptr(), Q + 2 * KV, buf.data_ptr(), Q + 2 * KV
        a.k_out, a.k_stride = buf.data_ptr() + Q * esz, Q + 2 * KV
        keep = (dev(qw), dev(kw), dev(inv))
        a.q_w, a.k_w = keep[0].data_ptr(), keep[1].data_ptr()
        a.rope = K.RotaryArgs(keep[2].data_ptr(), rot, 0.0, 1.0)
        a.eps, a.nh, a.nkv, a.hd = 1e-5, nh, nkv, hd
        a.pos_of, a.seq_of, a.slot_of_seq = lay.pos_of.data_ptr(), lay.seq_of.data_ptr(), lay.slot_of_seq.data_ptr()
        a.cache, a.append, a.T = cache.view, append, T
        K.qk_norm_rope(a, DT[dtype], DT[dtype], stream())
        got = buf.float().cpu()
        assert rel_l2(got[:, :Q], want_q.reshape(T, Q)) < KTOL[dtype]
        assert rel_l2(got[:, Q:Q + KV], want_k.reshape(T, KV)) < KTOL[dtype]
        assert torch.equal(got[:, Q + KV:], qkv[:, Q + KV:].float())          # V is left alone
    for t, (s, p) in enumerate(zip([4, 4, 4, 1, 1, 1, 1, 1], pos.tolist())):
        ck, cv = cache.get(s, p)
        assert torch.equal(ck, got[t, Q:Q + KV].view(nkv, hd)) and torch.equal(cv, got[t, Q + KV:].view(nkv, hd))
    with pytest.raises(K.KernelError, match="rotary_dim"):
        a.rope.rot = hd + 2
        K.qk_norm_rope(a, DT[dtype], DT[dtype], stream())


def test_attention_prefill_tensor_cores_long_prompt_many_times(K):
    """A long prompt (125 key tiles for the last query block, 32 heads) run repeatedly: the roles of the tcgen05 kernel
    hand tiles to each other through barriers whose phases must never get two apart, which only shows
    after many tiles and not on every run.  Checked against the mma.sync kernel and the error words."""
    nh, nkv, hd, T = 32, 8, 128, 8000
    g = torch.Generator().manual_seed(3)
    lay = layout_for([0], [0], [T])
    Q, KV = nh * hd, nkv * hd
    buf = torch.randn(T, Q + 2 * KV, generator=g).to(torch.bfloat16).cuda()
    outs = {}
    for which, reps in (("mma", 1), ("tc", 40)):
        for _ in range(reps):
            out = torch.full((T, Q), float("nan"), dtype=torch.bfloat16, device="cuda")
            a = K.AttnArgs()
            a.q, a.q_stride, a.out, a.out_stride = buf.data_ptr(), Q + 2 * KV, out.data_ptr(), Q
            a.kv_new, a.kv_stride = buf.data_ptr() + Q * 2, Q + 2 * KV
            a.batch = lay.c_struct()
            a.nh, a.nkv, a.hd, a.window, a.scale = nh, nkv, hd, 0, 1 / math.sqrt(hd)
            if which == "tc":
                K.attn_prefill_tc(a, True, stream())
                assert K.attn_tc_error() == 0
                if _ % 10 == 0:
                    assert rel_l2(out.float().cpu(), outs["mma"]) < 8e-3
            else:
                K.attn_prefill_mma(a, True, stream())
                assert K.attn_mma_error() == 0
                outs["mma"] = out.float().cpu()
    assert not torch.isnan(outs["mma"]).any()


@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 128), (3, 1, 48)])
def test_qk_norm_rope_scales_rows_whose_norm_was_folded_into_the_projection(K, nh, nkv, hd):
    """Float32 sums of unscaled rows in, with the rows' sums of squares: the kernel scales every row (Q, K and V
    heads) by 1/sqrt(sum / width + eps) first, and the result equals that of scaled rows."""
    g = torch.Generator().manual_seed(nh + hd)
    T, Q, KV, width, eps = 5, nh * hd, nkv * hd, 777, 1e-6
    slots, lens = [1, 3, 0, 2, 4], [9, 70, 1, 64, 200]
    lay = layout_for(slots, [n - 1 for n in lens], [1] * T)
    rows = torch.randn(T, Q + 2 * KV, generator=g)
    parts = torch.zeros(16, 32)
    parts[:3, :T] = torch.rand(3, T, generator=g) * 2000 + 10            # three K slices' partial sums
    parts[3:] = float("nan")                                              # parts beyond the count are not read
    sums = parts[:3, :T].sum(0)
    scale = 1.0 / torch.sqrt(sums / width + eps)
    qw, kw = 1 + 0.1 * torch.randn(hd, generator=g), 1 + 0.1 * torch.randn(hd, generator=g)
    k_ = torch.arange(hd // 2, dtype=torch.float64)
    inv = (torch.tensor(1e4, dtype=torch.float64) ** (-2 * k_ / hd)).float().cuda()
    keep = (qw.cuda(), kw.cuda(), parts.cuda())
    outs = []
    for folded in (True, False):
        cache = Paged(K, slots, lens, nkv, hd, torch.bfloat16)
        buf = (rows if folded else rows * scale[:, None]).cuda()
        q_out = torch.empty(T, Q, dtype=torch.bfloat16, device="cuda")
        a = K.QkArgs()
        a.inp, a.in_stride, a.q_out, a.q_stride, a.k_out, a.k_stride = buf.data_ptr(), Q + 2 * KV, q_out.data_ptr(), Q, None, 0
        a.q_w, a.k_w, a.rope = keep[0].data_ptr(), keep[1].data_ptr(), K.RotaryArgs(inv.data_ptr(), hd, 0.0, 1.0)
        a.eps, a.nh, a.nkv, a.hd = 1e-5, nh, nkv, hd
        a.pos_of, a.seq_of, a.slot_of_seq, a.kv_len = lay.pos_of.data_ptr(), lay.seq_of.data_ptr(), lay.slot_of_seq.data_ptr(), lay.kv_len.data_ptr()
        a.cache, a.append, a.T, a.zero_in = cache.view, 1, T, 1
        if folded:
            a.row_sumsq, a.row_parts, a.row_width, a.row_eps = keep[2].data_ptr(), 3, width, eps
        K.qk_norm_rope(a, torch.float32, torch.bfloat16, stream())
        assert float(buf.abs().sum()) == 0                                          # the sums are left cleared
        kv = [torch.cat(cache.get(s, n - 1)) for s, n in zip(slots, lens)]
        outs.append((q_out.float().cpu(), torch.stack(kv)))
    assert rel_l2(outs[0][0], outs[1][0]) < 4e-3 and rel_l2(outs[0][1], outs[1][1]) < 4e-3
    v_want = (rows[:, Q + KV:] * scale[:, None]).view(T, nkv, hd)
    assert rel_l2(outs[0][1][:, nkv:], v_want) < 4e-3                               # V rows: scaled, else untouched


def reference_attention(q, keys, vals, qpos, window, scale):
    """q [nh, hd] at position qpos; keys/vals [len, nkv, hd]; float64."""
    nh, nkv = q.shape[0], keys.shape[1]
    lo = max(0, qpos - window + 1) if window else 0
    out = torch.zeros_like(q, dtype=torch.float64)
    for h in range(nh):
        kh = h // (nh // nkv)
        s = (keys[lo:qpos + 1, kh].double() @ q[h].double()) * scale
        out[h] = torch.softmax(s, 0) @ vals[lo:qpos + 1, kh].double()
    return out.float()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,window,ring", [(6, 2, 32, 0, 0), (5, 1, 48, 20, 64), (4, 4, 16, 70, 128), (8, 2, 128, 0, 0)])
def test_attention_prefill_over_cache_and_new_keys(K, dtype, nh, nkv, hd, window, ring):
    """Three sequences in one step: a fresh prompt, a continuation on a filled cache and a single
    token.  One far key of each sequence is made to stand out, so a kernel that skips or misplaces
    it is far off, not slightly off."""
    g = torch.Generator().manual_seed(nh * hd)
    slots, starts, news = [2, 0, 5], [0, 150, 33], [90, 40, 1]
    lay = layout_for(slots, starts, news)
    T, Q, KV = sum(news), nh * hd, nkv * hd
    scale = 1 / math.sqrt(hd)
    full_k = [torch.randn(s + n, nkv, hd, generator=g) for s, n in zip(starts, news)]
    full_v = [torch.randn(s + n, nkv, hd, generator=g) for s, n in zip(starts, news)]
    q = torch.randn(T, nh, hd, generator=g)
    for i in range(3):
        far = 3 if not window else max(0, starts[i] + news[i] - window)       # the window's first key
        full_k[i][far] *= 6.0
    q, full_k, full_v = (q.to(DT[dtype]), [k.to(DT[dtype]) for k in full_k], [v.to(DT[dtype]) for v in full_v])
    cache = Paged(K, slots, [s + n for s, n in zip(starts, news)], nkv, hd, DT[dtype], ring_rows=ring)
    for i, s in enumerate(slots):
        lo = max(0, starts[i] - ring) if ring else 0
        for p in range(lo, starts[i]):
            cache.put(s, p, full_k[i][p], full_v[i][p])
    qkv = torch.zeros(T, Q + 2 * KV, dtype=DT[dtype])
    qkv[:, :Q] = q.reshape(T, Q)
    at = 0
    for i in range(3):
        qkv[at:at + news[i], Q:Q + KV] = full_k[i][starts[i]:].reshape(news[i], KV)
        qkv[at:at + news[i], Q + KV:] = full_v[i][starts[i]:].reshape(news[i], KV)
        at += news[i]
    buf = dev(qkv)
    out = torch.empty(T, Q, dtype=DT[dtype], device="cuda")
    a = K.AttnArgs()
    a.q, a.q_stride, a.out, a.out_stride = buf.data_ptr(), Q + 2 * KV, out.data_ptr(), Q
    a.kv_new, a.kv_stride = buf.data_ptr() + Q * buf.element_size(), Q + 2 * KV
    a.cache, a.batch = cache.view, lay.c_struct()
    a.nh, a.nkv, a.hd, a.window, a.scale = nh, nkv, hd, window, scale
    K.attn_prefill(a, DT[dtype], stream())
    want = torch.zeros(T, nh, hd)
    at = 0
    for i in range(3):
        for j in range(news[i]):
            want[at + j] = reference_attention(q[at + j].float(), full_k[i].float(), full_v[i].float(), starts[i] + j, window, scale)
        at += news[i]
    assert rel_l2(out.float().cpu(), want.reshape(T, Q)) < KTOL[dtype]
    # then append, and decode one more token per sequence from the cache alone
    K.kv_append(buf[:, Q:], cache.view, lay.c_struct(), stream())
    lens = [s + n for s, n in zip(starts, news)]
    for i, s in enumerate(slots):
        lo = max(0, lens[i] - ring) if ring else 0
        for p in (lo, lens[i] - 1):
            ck, cv = cache.get(s, p)
            assert torch.equal(ck, full_k[i][p].float()) and torch.equal(cv, full_v[i][p].float())
    dlay = layout_for(slots, [n - 1 for n in lens], [1, 1, 1])
    q1 = torch.randn(3, nh, hd, generator=g).to(DT[dtype])
    qb = dev(q1.reshape(3, Q))
    o1 = torch.empty(3, Q, dtype=DT[dtype], device="cuda")
    for chunk in (256, 64, 32):
        splits = -(-max(lens) // chunk)
        scratch = torch.full((3 * nh * splits * (hd + 2),), float("nan"), device="cuda")
        d = K.AttnArgs()
        d.q, d.q_stride, d.out, d.out_stride = qb.data_ptr(), Q, o1.data_ptr(), Q
        d.cache, d.batch = cache.view, dlay.c_struct()
        d.nh, d.nkv, d.hd, d.window, d.scale = nh, nkv, hd, window, scale
        d.chunk, d.n_splits, d.scratch = chunk, splits, scratch.data_ptr()
        K.attn_decode(d, DT[dtype], stream())
        want1 = torch.stack([reference_attention(q1[i].float(), full_k[i].float(), full_v[i].float(), lens[i] - 1, window, scale) for i in range(3)])
        assert rel_l2(o1.float().cpu(), want1.reshape(3, Q)) < KTOL[dtype], chunk
    # fewer splits than the chunk covers: every sequence is cut into that many equal parts of its own length
    for splits in (1, 3):
        d.chunk, d.n_splits = 32, splits
        o1.fill_(float("nan"))
        K.attn_decode(d, DT[dtype], stream())
        assert rel_l2(o1.float().cpu(), want1.reshape(3, Q)) < KTOL[dtype], splits


@pytest.mark.parametrize("nh,nkv,hd,window", [(8, 2, 128, 0), (4, 4, 64, 0), (6, 1, 128, 100), (16, 8, 64, 300)])
def test_attention_of_continuation_chunks_on_tensor_cores(K, nh, nkv, hd, window):
    """The tensor-core prompt kernels with keys and values taken from the cache's pages: one step holds a fresh
    prompt, a chunk of 200 tokens onto 450 cached ones (query blocks and key tiles that straddle the border), a
    chunk that starts inside a page, and a single token on a long sequence.  A far key of every sequence
    stands out.  Against float64, and the two kernels against each other."""
    g = torch.Generator().manual_seed(nh + hd + window)
    slots, starts, news = [2, 0, 5, 3], [0, 450, 37, 700], [130, 200, 64, 1]
    lay = layout_for(slots, starts, news)
    T, Q, KV = sum(news), nh * hd, nkv * hd
    scale = 1 / math.sqrt(hd)
    full_k = [torch.randn(s + n, nkv, hd, generator=g) for s, n in zip(starts, news)]
    full_v = [torch.randn(s + n, nkv, hd, generator=g) for s, n in zip(starts, news)]
    q = torch.randn(T, nh, hd, generator=g).to(torch.bfloat16)
    for i in range(4):
        far = 3 if not window else max(0, starts[i] + news[i] - window)
        full_k[i][far] *= 5.0
    full_k, full_v = [k.to(torch.bfloat16) for k in full_k], [v.to(torch.bfloat16) for v in full_v]
    cache = Paged(K, slots, [s + n for s, n in zip(starts, news)], nkv, hd, torch.bfloat16)
    for i, s in enumerate(slots):
        for p in range(starts[i] + news[i]):                       # the step's own keys are in the cache already
            cache.put(s, p, full_k[i][p], full_v[i][p])
    qb = q.reshape(T, Q).cuda()
    want = torch.zeros(T, nh, hd)
    at = 0
    for i in range(4):
        for j in range(news[i]):
            want[at + j] = reference_attention(q[at + j].float(), full_k[i].float(), full_v[i].float(), starts[i] + j, window, scale)
        at += news[i]
    outs = {}
    for name in ("tc", "mma"):
        if name == "tc" and hd != 128:
            continue
        out = torch.full((T, Q), float("nan"), dtype=torch.bfloat16, device="cuda")
        a = K.AttnArgs()
        a.q, a.q_stride, a.out, a.out_stride = qb.data_ptr(), Q, out.data_ptr(), Q
        a.kv_new, a.kv_stride = None, 0
        a.cache, a.batch = cache.view, lay.c_struct()
        a.nh, a.nkv, a.hd, a.window, a.scale = nh, nkv, hd, window, scale
        accepts, run = (K.attn_prefill_tc_accepts, K.attn_prefill_tc) if name == "tc" else (K.attn_prefill_mma_accepts, K.attn_prefill_mma)
        assert accepts(a, torch.bfloat16, K.KV_FROM_CACHE)
        assert not accepts(a, torch.bfloat16, K.KV_FROM_STEP) and not accepts(a, torch.bfloat16, K.KV_NOWHERE)
        run(a, K.KV_FROM_CACHE, stream())
        assert K.wait_errors() == {}
        outs[name] = out.float().cpu()
        assert rel_l2(outs[name], want.reshape(T, Q)) < 8e-3, name
        rows = ((outs[name] - want.reshape(T, Q)).norm(dim=1) / want.reshape(T, Q).norm(dim=1))
        assert float(rows.max()) < 3e-2, (name, int(rows.argmax()))
    if len(outs) == 2:
        assert rel_l2(outs["tc"], outs["mma"]) < 8e-3
    ring = Paged(K, slots, [s + n for s, n in zip(starts, news)], nkv, hd, torch.bfloat16, ring_rows=128)
    a.cache = ring.view
    assert not K.attn_prefill_mma_accepts(a, torch.bfloat16, K.KV_FROM_CACHE)       # a ring has lost the early keys


def test_attention_refuses_bad_heads(K):
    a = K.AttnArgs()
    a.nh, a.nkv, a.hd = 5, 2, 32
    with pytest.raises(K.KernelError, match="multiple"):
        K.attn_prefill(a, torch.float32, stream())
    a.nh, a.nkv, a.hd = 4, 2, 272
    with pytest.raises(K.KernelError, match="head_dim"):
        K.attn_prefill(a, torch.float32, stream())


# ------------------------------------------------------------------ sampling
class SamplerBench:
    def __init__(self, K, V, B, seed=0, parts=None):
        from titan_b200.cache import SlotState
        from titan_b200.sampling import DeviceSampler
        self.K, self.V, self.B = K, V, B
        self.state = SlotState(B + 3, "cuda")
        self.sampler = DeviceSampler(self.state, B + 3, V, "cuda", parts=parts)
        self.slots = list(range(2, 2 + B))
        self.slot_t = torch.tensor(self.slots, dtype=torch.int32, device="cuda")

    def run(self, logits, params, seq_ids, context=None, steps=1):
        from titan_b200.engine.batch import StepEntry, StepLayout
        self.sampler.configure(self.slots, params, seq_ids)
        if context is not None:
            lay = StepLayout([StepEntry(s, c, []) for s, c in zip(self.slots, context)], [0] * self.B, "cuda")
            self.sampler.observe(lay, stream())
        outs = []
        for _ in range(steps):
            outs.append(self.sampler.sample(logits.cuda(), self.slot_t, stream()).cpu().tolist())
        return outs


def test_uniform_numbers_match_the_plain_hash(K):
    for seed, seq, step in [(0, 0, 0), (42, 3, 17), ((1 << 63) - 1, 12345, 99999), (7, 1 << 40, 5)]:
        assert K.uniform24(seed, seq, step) / float(1 << 24) == P.uniform_draw(seed, seq, step)


@pytest.mark.parametrize("V", [509, 5003, 151936])
def test_argmax_whole_vocabulary_lowest_index_on_ties(K, V):
    from titan_b200.sampling import SamplerParams
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(4, V, generator=g)
    logits[0, V - 1] = 9.0                      # the last entry: a vocabulary tail must not be skipped
    logits[1, 77] = logits[1, 400] = 8.0        # a tie
    logits[2, :] = -1.0                         # all equal
    logits[3, 5] = float("nan")
    b = SamplerBench(K, V, 4, parts=None if V > 1000 else 3)
    got = b.run(logits, [SamplerParams.greedy()] * 4, [0, 1, 2, 3])[0]
    assert got[:3] == [V - 1, 77, 0] and got[3] == int(torch.argmax(torch.nan_to_num(logits[3], nan=-1e30)))


@pytest.fixture(params=[0, 1, 2, 8], ids=lambda t: f"team{t}")
def team(request, K):
    """CTAs per row in the sampling kernel: by the vocabulary's size (0), one, or a cluster of 2 or 8."""
    K.set_sample_team(request.param)
    yield request.param
    K.set_sample_team(0)


@pytest.mark.parametrize("parts", [0, 7])       # the row's maximum by one block, and by seven blocks of uneven slices
def test_sampling_matches_the_plain_sampler(K, parts, team):
    from titan_b200.sampling import SamplerParams
    V, B = 1000, 6
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(B, V, generator=g) * 3
    logits[4, 10] = logits[4, 20] = logits[4, 30] = logits[4].max() + 1     # ties at the top_k border
    params = [SamplerParams(1.0, 1.0, 0, 1.0, 3), SamplerParams(0.7, 1.0, 5, 1.0, 3), SamplerParams(1.3, 0.6, 0, 1.0, 4),
              SamplerParams(0.9, 0.8, 50, 1.5, 5), SamplerParams(1.0, 1.0, 2, 1.0, 6), SamplerParams(0.0, 1.0, 0, 2.0, 7)]
    context = [random_ctx.tolist() for random_ctx in torch.randint(0, V, (B, 40), generator=g)]
    context[5] = [int(torch.argmax(logits[5]))] * 3          # the greedy row's winner is penalised away
    b = SamplerBench(K, V, B, parts=parts)
    steps = 40
    got = b.run(logits, params, [10, 11, 12, 13, 14, 15], context, steps=steps)
    seen = [set(c) for c in context]
    agree = total = 0
    for step in range(steps):
        for r in range(B):
            p = params[r]
            u = P.uniform_draw(p.seed_value(), 10 + r, step)
            want = P.sample(logits[r], seen[r], p.temperature, p.top_k, p.top_p, p.repetition_penalty, u)
            total += 1
            agree += int(want == got[step][r])
            if p.top_k:
                allowed = torch.topk(penalised(logits[r], seen[r], p.repetition_penalty), p.top_k + 2).indices.tolist()
                assert got[step][r] in allowed
            seen[r].add(got[step][r])
    # the device sums exact fixed-point masses, the plain sampler float64 ones: a draw that falls
    # within 2^-24 of a border may differ, nothing else
    assert agree >= total - 2, (agree, total)
    assert all(got[s][4] in (10, 20) for s in range(steps))   # top_k = 2 of three tied: the two lowest indices


_PLAIN_DRAWS = {}


@pytest.mark.parametrize("V", [40000, 151936])
def test_sampling_large_vocabulary_matches_the_plain_sampler(K, V, team):
    """Vocabularies of several selection bins and several levels of the ordered search: top_k on the gathered
    list (up to 1,024 kept) and over the whole row (more), top_p alone, ties at both borders that lie far apart."""
    from titan_b200.sampling import SamplerParams
    B = 7 if V < 100000 else 3
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(B, V, generator=g) * 2.5
    logits[1] = torch.round(logits[1] * 2) / 2                       # thousands of ties everywhere: top_p cuts inside a tie
    logits[2, 5] = logits[2, V // 2] = logits[2, V - 1] = logits[2].max() + 1   # top_k = 2 of three tied, far apart
    params = [SamplerParams(0.8, 0.95, 40, 1.0, 3), SamplerParams(1.0, 0.7, 0, 1.0, 4), SamplerParams(1.0, 1.0, 2, 1.0, 5),
              SamplerParams(1.1, 1.0, 2000, 1.0, 6), SamplerParams(0.9, 0.5, 1024, 1.2, 7), SamplerParams(1.0, 1.0, 0, 1.0, 8),
              SamplerParams(0.7, 0.9, 1500, 1.0, 9)][:B]
    context = [torch.randint(0, V, (30,), generator=g).tolist() for _ in range(B)]
    b = SamplerBench(K, V, B)
    steps = 4 if V < 100000 else 2
    got = b.run(logits, params, list(range(20, 20 + B)), context, steps=steps)
    seen = [set(c) for c in context]
    agree = total = 0
    for step in range(steps):
        for r in range(B):
            p = params[r]
            key = (V, r, step, tuple(sorted(seen[r])) if p.repetition_penalty > 1 else None)
            if key not in _PLAIN_DRAWS:          # the plain sampler is slow at these sizes and does not depend on the team
                _PLAIN_DRAWS[key] = P.sample(logits[r], seen[r], p.temperature, p.top_k, p.top_p, p.repetition_penalty,
                                             P.uniform_draw(p.seed_value(), 20 + r, step))
            want = _PLAIN_DRAWS[key]
            total += 1
            agree += int(want == got[step][r])
            seen[r].add(got[step][r])
    assert agree >= total - 1, (agree, total, got)
    assert all(got[s][2] in (5, V // 2) for s in range(steps))


@pytest.mark.parametrize("case", range(12))
def test_sampling_on_a_grid_of_tied_logits(K, case):
    """Logits rounded to a coarse grid: both borders fall inside groups of equal values, zeros come with both signs
    (one value: -0.0 == 0.0), and a top_k border that cuts a group must not cut the group at the top_p border."""
    import random
    from titan_b200.sampling import SamplerParams
    r = random.Random(case)
    V, B = r.choice([227, 803, 1446, 2819]), 4
    g = torch.Generator().manual_seed(case)
    logits = torch.round(torch.randn(B, V, generator=g) * r.choice([2.0, 6.0]) * 2) / 2
    assert bool(((logits == 0) & torch.signbit(logits)).any()) and bool(((logits == 0) & ~torch.signbit(logits)).any())
    params = [SamplerParams(r.choice([0.8, 1.0, 1.7]), r.choice([1.0, 0.9, 0.5, 0.01]), r.choice([V // 2, V // 3, 40, 0, 2000]),
                            r.choice([1.0, 1.3]), r.randint(0, 99)) for _ in range(B)]
    K.set_sample_team(r.choice([1, 2, 4]))
    try:
        context = [torch.randint(0, V, (10,), generator=g).tolist() for _ in range(B)]
        got = SamplerBench(K, V, B, parts=r.choice([0, 3])).run(logits, params, list(range(B)), context, steps=3)
    finally:
        K.set_sample_team(0)
    seen = [set(c) for c in context]
    for step in range(3):
        for row in range(B):
            p = params[row]
            want = P.sample(logits[row], seen[row], p.temperature, p.top_k, p.top_p, p.repetition_penalty,
                            P.uniform_draw(p.seed_value(), row, step))
            assert want == got[step][row], (case, row, step, p)
            seen[row].add(want)


def test_sampling_borders_built_by_hand(K, team):
    """Row 0: the top_k border cuts a group of zeros whose low indices hold -0.0 and whose high indices hold +0.0
    (one value; the low indices are kept).  Row 1: top_k cuts a group of ties at index 20, and the top_p border
    needs ALL of a higher group that has a member beyond index 20."""
    from titan_b200.sampling import SamplerParams
    V = 64
    logits = torch.full((2, V), -5.0)
    logits[0, 0:10] = -0.0
    logits[0, 10:20] = 0.0
    logits[0, 20:25] = 1.0
    logits[1, 50] = 3.0
    logits[1, 5] = logits[1, 60] = 2.0
    logits[1, 10] = logits[1, 20] = logits[1, 30] = logits[1, 40] = 1.0
    params = [SamplerParams(1.0, 1.0, 15, 1.0, 1), SamplerParams(1.0, 0.8, 5, 1.0, 2)]
    steps = 60
    got = SamplerBench(K, V, 2).run(logits, params, [0, 1], None, steps=steps)
    for step in range(steps):
        for row, p in enumerate(params):
            want = P.sample(logits[row], set(), p.temperature, p.top_k, p.top_p, 1.0, P.uniform_draw(p.seed_value(), row, step))
            assert want == got[step][row], (row, step)
    assert {g[0] for g in got} <= set(range(0, 10)) | set(range(20, 25)) and {g[0] for g in got} & set(range(0, 10))
    assert {g[1] for g in got} == {50, 5, 60}


def penalised(row, seen, pen):
    x = row.clone()
    for t in seen:
        x[t] = x[t] / pen if x[t] > 0 else x[t] * pen
    return x


def test_sampling_follows_the_distribution(K):
    from titan_b200.sampling import SamplerParams
    V = 37
    logits = torch.linspace(-2, 2, V)[None, :].repeat(1, 1)
    b = SamplerBench(K, V, 1)
    got = [o[0] for o in b.run(logits, [SamplerParams(1.0, 1.0, 0, 1.0, 123)], [0], steps=6000)]
    freq = torch.bincount(torch.tensor(got), minlength=V).float() / 6000
    assert float((freq - torch.softmax(logits[0], 0)).abs().max()) < 0.02


@pytest.mark.parametrize("nh,nkv,hd,window,ring", [(32, 8, 128, 0, 0), (6, 2, 64, 0, 0), (24, 2, 128, 0, 0), (4, 4, 64, 100, 128), (8, 1, 128, 200, 256)])
def test_attention_decode_on_tensor_cores(K, nh, nkv, hd, window, ring):
    """The mma kernel against float64 and against the plain kernel: long and short sequences in one
    batch, lengths that end inside a page, a far key that stands out, chunks of several sizes."""
    g = torch.Generator().manual_seed(nh + hd)
    lens = [1, 63, 64, 65, 700, 1500]
    slots = [3, 0, 5, 1, 2, 4]
    B, Q = len(lens), nh * hd
    scale = 1 / math.sqrt(hd)
    ks = [torch.randn(n, nkv, hd, generator=g).to(torch.bfloat16) for n in lens]
    vs = [torch.randn(n, nkv, hd, generator=g).to(torch.bfloat16) for n in lens]
    q = torch.randn(B, nh, hd, generator=g).to(torch.bfloat16)
    for i, n in enumerate(lens):
        far = max(0, n - window) if window else min(3, n - 1)
        ks[i][far] = (ks[i][far].float() * 5).to(torch.bfloat16)
    cache = Paged(K, slots, lens, nkv, hd, torch.bfloat16, ring_rows=ring)
    for i, s in enumerate(slots):
        for p in range(max(0, lens[i] - ring) if ring else 0, lens[i]):
            cache.put(s, p, ks[i][p], vs[i][p])
    lay = layout_for(slots, [n - 1 for n in lens], [1] * B)
    qb = q.reshape(B, Q).cuda()
    want = torch.stack([reference_attention(q[i].float(), ks[i].float(), vs[i].float(), lens[i] - 1, window, scale) for i in range(B)]).reshape(B, Q)
    # splits of ``chunk`` keys: 24 (through scratch), 12 (a cluster beyond the portable 8), 6, 2; then fewer splits
    # than the chunk covers, which cut every sequence into equal parts of its own length (4, 16 and 1 parts)
    for chunk, splits in ((64, 24), (128, 12), (256, 6), (1024, 2), (128, 4), (64, 16), (128, 1)):
        outs = []
        for mode in ("mma", "mma through scratch", "plain"):     # up to 16 splits merge inside a cluster unless told otherwise
            fast = mode != "plain"
            out = torch.full((B, Q), float("nan"), dtype=torch.bfloat16, device="cuda")
            scratch = torch.full((B * nh * splits * (hd + 2),), float("nan"), device="cuda")
            d = K.AttnArgs()
            d.q, d.q_stride, d.out, d.out_stride = qb.data_ptr(), Q, out.data_ptr(), Q
            d.cache, d.batch = cache.view, lay.c_struct()
            d.nh, d.nkv, d.hd, d.window, d.scale = nh, nkv, hd, window, scale
            d.chunk, d.n_splits, d.scratch = chunk, splits, scratch.data_ptr()
            if fast:
                assert K.attn_decode_mma_accepts(d, torch.bfloat16)
                K.set_attn_decode_cluster(mode == "mma")
                try:
                    K.attn_decode_mma(d, stream())
                    assert K.attn_mma_error() == 0
                finally:
                    K.set_attn_decode_cluster(True)
            else:
                K.attn_decode(d, torch.bfloat16, stream())
            outs.append(out.float().cpu())
        assert rel_l2(outs[0], want) < 8e-3, chunk        # P is rounded to bfloat16 before P.V
        assert rel_l2(outs[1], want) < 8e-3, chunk
        assert rel_l2(outs[0], outs[2]) < 8e-3, chunk
        assert rel_l2(outs[0], outs[1]) < 1e-5, chunk     # the two merges add the same parts in the same order
        # lengths named as final before the step: the same numbers by sequence (1), or committed lengths by slot (2);
        # pages of older positions are then requested before the dependency wait, and nothing else changes
        committed = torch.zeros(max(slots) + 1, dtype=torch.int32)
        for sl, n in zip(slots, lens):
            committed[sl] = n - 1
        committed = committed.cuda()
        for early, mode in ((lay.kv_len, 1), (committed, 2)):
            out = torch.full((B, Q), float("nan"), dtype=torch.bfloat16, device="cuda")
            d.out, d.early_len, d.early_mode = out.data_ptr(), early.data_ptr(), mode
            K.attn_decode_mma(d, stream())
            assert K.attn_mma_error() == 0
            assert torch.equal(out.float().cpu(), outs[0]), (chunk, mode)
        committed -= 1                                    # an early length that is not the step's is reported
        K.attn_decode_mma(d, stream())
        assert K.attn_mma_error() == 7
        d.early_len, d.early_mode = None, 0
    d.chunk = 100
    assert not K.attn_decode_mma_accepts(d, torch.bfloat16)
    d.chunk, d.hd = 64, 96
    assert not K.attn_decode_mma_accepts(d, torch.bfloat16)


@pytest.mark.parametrize("nh,nkv,hd,window", [(8, 2, 128, 0), (6, 6, 64, 0), (4, 1, 128, 100), (3, 1, 64, 64), (2, 1, 128, 300)])
def test_attention_prefill_on_tensor_cores(K, nh, nkv, hd, window):
    """Fresh prompts of ragged lengths (1 token, ends inside a tile, several tiles) in one step."""
    g = torch.Generator().manual_seed(nh * hd + window)
    lens = [1, 200, 64, 333, 65, 128, 700]
    slots = list(range(len(lens)))
    lay = layout_for(slots, [0] * len(lens), lens)
    T, Q, KV = sum(lens), nh * hd, nkv * hd
    scale = 1 / math.sqrt(hd)
    qkv = torch.randn(T, Q + 2 * KV, generator=g).to(torch.bfloat16)
    at = 0
    for n in lens:                                   # a far key that stands out: the first the last query may see
        far = max(0, n - window) if window else 0
        qkv[at + far, Q:Q + KV] = (qkv[at + far, Q:Q + KV].float() * 4).to(torch.bfloat16)
        at += n
    buf = qkv.cuda()
    outs = {}
    for which in (["tc"] if hd == 128 else []) + ["mma", "plain"]:
        out = torch.full((T, Q), float("nan"), dtype=torch.bfloat16, device="cuda")
        a = K.AttnArgs()
        a.q, a.q_stride, a.out, a.out_stride = buf.data_ptr(), Q + 2 * KV, out.data_ptr(), Q
        a.kv_new, a.kv_stride = buf.data_ptr() + Q * 2, Q + 2 * KV
        a.batch = lay.c_struct()
        a.nh, a.nkv, a.hd, a.window, a.scale = nh, nkv, hd, window, scale
        if which == "tc":
            assert K.attn_prefill_tc_accepts(a, torch.bfloat16, True) and not K.attn_prefill_tc_accepts(a, torch.bfloat16, False)
            K.attn_prefill_tc(a, True, stream())
            assert K.attn_tc_error() == 0
        elif which == "mma":
            assert K.attn_prefill_mma_accepts(a, torch.bfloat16, True)
            assert not K.attn_prefill_mma_accepts(a, torch.bfloat16, False)
            K.attn_prefill_mma(a, True, stream())
            assert K.attn_mma_error() == 0
        else:
            K.attn_prefill(a, torch.bfloat16, stream())
        outs[which] = out.float().cpu()
    want = torch.zeros(T, nh, hd)
    at = 0
    for n in lens:
        k = qkv[at:at + n, Q:Q + KV].float().view(n, nkv, hd)
        v = qkv[at:at + n, Q + KV:].float().view(n, nkv, hd)
        for j in range(n):
            want[at + j] = reference_attention(qkv[at + j, :Q].float().view(nh, hd), k, v, j, window, scale)
        at += n
    for which, got in outs.items():
        assert not torch.isnan(got).any(), which
        assert rel_l2(got, want.reshape(T, Q)) < 8e-3, which
