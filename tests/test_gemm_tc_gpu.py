"""The tcgen05 matrix product against float64, at sizes that fill tiles exactly and at sizes that do
not (ragged M, N and K; vocabulary-like N; strided views), in both operand orders and all epilogues."""
import pytest
import torch

from helpers import rel_l2
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from titan_b200 import kernels
    kernels.lib()
    return kernels


def stream():
    return torch.cuda.current_stream().cuda_stream


SHAPES = [(1, 128, 64), (5, 384, 256), (16, 200, 72), (17, 1000, 520), (40, 130, 4096), (64, 509, 96), (100, 256, 128),
          (128, 256, 64), (200, 300, 1032), (333, 1000, 200), (256, 128, 512),
          (1100, 5000, 520), (2048, 6144, 256)]      # more tiles than SMs: a CTA walks over two or three tiles


@pytest.fixture(params=["auto", "pairs", "single 128x256", "single 128x128"])
def cta_mode(request, K):
    """Prompt products choose among three tile shapes; every shape is forced in turn and tested on every size."""
    K.set_gemm_plain_tile(["auto", "pairs", "single 128x256", "single 128x128"].index(request.param))
    yield request.param
    K.set_gemm_plain_tile(0)


@pytest.mark.parametrize("M,N,Kd", SHAPES + [(256, 256, 64), (300, 700, 136), (520, 264, 1032), (130, 512, 128), (255, 1000, 264)])
def test_all_epilogues(K, M, N, Kd, cta_mode):
    if cta_mode != "auto" and M < 128:
        pytest.skip("decode-sized products have one kernel")
    if cta_mode == "pairs" and (M <= 128 or N < 256):
        pytest.skip("pairs are only used from 129 rows and 256 columns on")
    g = torch.Generator().manual_seed(M + N + Kd)
    x = torch.randn(M, Kd, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, Kd, generator=g) * 0.1).to(torch.bfloat16)
    want = P.linear(x.float(), w.float())
    xd, wd = x.cuda(), w.cuda()
    n8 = -(-N // 8) * 8
    out = torch.zeros(M, n8, dtype=torch.bfloat16, device="cuda")[:, :N]
    K.gemm_tc(xd, wd, out, K.EPI_STORE, stream())
    assert K.gemm_tc_error() == 0
    assert rel_l2(out.float().cpu(), want) < 4e-3
    f = torch.zeros(M, n8, device="cuda")[:, :N]
    K.gemm_tc(xd, wd, f, K.EPI_F32, stream())
    assert rel_l2(f.cpu(), want) < 1e-5
    res = torch.randn(M, N, generator=g)
    acc = torch.zeros(M, n8, device="cuda")[:, :N]
    acc.copy_(res)
    K.gemm_tc(xd, wd, acc, K.EPI_ADD, stream())
    assert rel_l2(acc.cpu(), res + want) < 1e-5
    if M < 128 and Kd >= 512:
        acc2 = torch.zeros(M, n8, device="cuda")[:, :N]
        acc2.copy_(res)
        K.gemm_tc(xd, wd, acc2, K.EPI_ADD, stream(), splits=1)       # one slice: no atomics
        assert rel_l2(acc2.cpu(), res + want) < 1e-5
    if N % 2 == 0:
        h8 = -(-(N // 2) // 8) * 8
        act = torch.zeros(M, h8, dtype=torch.bfloat16, device="cuda")[:, :N // 2]
        K.gemm_tc(xd, wd, act, K.EPI_SWIGLU, stream())
        assert rel_l2(act.float().cpu(), P.swiglu(want[:, 0::2], want[:, 1::2])) < 6e-3
    assert K.gemm_tc_error() == 0


@pytest.mark.parametrize("M,N,Kd", [(1100, 5000, 520), (2048, 4096, 1024), (300, 20000, 64), (512, 1024, 2048)])
def test_tail_split_and_whole_tiles(K, M, N, Kd, cta_mode):
    """ADD epilogue with a last round of tiles that does not fill the SMs (or fewer tiles than SMs
    altogether): those tiles cut along K (partial sums meet through atomics), and whole tiles per CTA,
    both against float64."""
    g = torch.Generator().manual_seed(N)
    x = torch.randn(M, Kd, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, Kd, generator=g) * 0.1).to(torch.bfloat16)
    res = torch.randn(M, N, generator=g)
    want = res + P.linear(x.float(), w.float())
    try:
        for on in (True, False):
            K.set_gemm_tail_split(on)
            acc = res.cuda()
            K.gemm_tc(x.cuda(), w.cuda(), acc, K.EPI_ADD, stream())
            assert K.gemm_tc_error() == 0
            assert rel_l2(acc.cpu(), want) < 1e-5      # the same bound whichever way the sum is cut
    finally:
        K.set_gemm_tail_split(True)


def test_pairs_are_available(K):
    """On a B200 every epilogue's pair kernel fits: the default path is the cta_group::2 one."""
    for epi in (K.EPI_STORE, K.EPI_F32, K.EPI_ADD, K.EPI_SWIGLU):
        assert K.gemm_pair_clusters(epi) >= 32


def test_strided_input_rows(K):
    g = torch.Generator().manual_seed(1)
    big = torch.randn(150, 400, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(96, 200, generator=g) * 0.1).to(torch.bfloat16).cuda()
    for rows in (150, 20):
        x = big[:rows, 8:208]
        out = torch.zeros(rows, 96, device="cuda")
        K.gemm_tc(x, w, out, K.EPI_F32, stream())
        assert rel_l2(out.cpu(), P.linear(x.float().cpu(), w.float().cpu())) < 1e-5
    assert K.gemm_tc_error() == 0


def test_refuses_misaligned(K):
    x = torch.zeros(4, 12, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(8, 12, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(4, 8, device="cuda")
    assert not K.gemm_tc_accepts(x, w, out, K.EPI_F32)
    with pytest.raises(K.KernelError, match="multiples of 8"):
        K.gemm_tc(x, w, out, K.EPI_F32, stream())
    with pytest.raises(K.KernelError, match="bfloat16"):
        K.gemm_tc(x.float(), w.float(), out, K.EPI_F32, stream())


@pytest.mark.parametrize("M,N,Kd", [(1, 256, 64), (1, 6144, 4096), (3, 200, 72), (8, 1000, 520), (13, 4096, 1024), (16, 24576, 4096),
                                    (17, 384, 256), (32, 2600, 1096)])
def test_the_norm_before_a_decode_product_folded_into_it(K, M, N, Kd):
    """tb_gemm_tc_normed: rmsnorm(x) . W^T with the norm inside the product, against the plain functions.  With
    the SwiGLU epilogue the result is complete; with float32 sums (K cut into slices) the product of the unscaled
    rows comes out beside the rows' sums of squares, and the head norm / rotary kernel applies the scale.  The
    rows' sizes differ by orders of magnitude, so a scale that is lost or taken from another row shows."""
    g = torch.Generator().manual_seed(M * 31 + N + Kd)
    x = torch.randn(M, Kd, generator=g) * (10.0 ** torch.linspace(-1, 2, M))[:, None]
    nw = 1 + 0.2 * torch.randn(Kd, generator=g)
    w = (torch.randn(N - N % 2, Kd, generator=g) * 0.1).to(torch.bfloat16)
    N = w.shape[0]
    eps = 1e-5
    h = P.rms_norm(x, nw, eps)
    want = P.linear(h, w.float())
    xd, nd, wd = x.cuda(), nw.cuda(), w.cuda()
    # SwiGLU: gate and up rows interleaved, as the feed-forward part binds them
    act = torch.full((M, -(-(N // 2) // 8) * 8), float("nan"), dtype=torch.bfloat16, device="cuda")[:, :N // 2]
    assert K.gemm_tc_normed_accepts(xd, nd, wd, act, K.EPI_SWIGLU, None)
    K.gemm_tc_normed(xd, nd, eps, wd, act, K.EPI_SWIGLU, stream())
    assert K.gemm_tc_error() == 0
    assert rel_l2(act.float().cpu(), P.swiglu(want[:, 0::2], want[:, 1::2])) < 6e-3
    per_row = (act.float().cpu() - P.swiglu(want[:, 0::2], want[:, 1::2])).norm(dim=1) / P.swiglu(want[:, 0::2], want[:, 1::2]).norm(dim=1)
    assert float(per_row.max()) < 1.2e-2, per_row
    # float32 sums + sums of squares, twice in a row into the same buffers (cleared by the caller in between)
    n4 = -(-N // 4) * 4
    for _ in range(2):
        acc = torch.zeros(M, n4, device="cuda")[:, :N]
        parts = torch.full((16, 32), float("nan"), device="cuda")      # one row per K slice is written, nothing is added to
        assert K.gemm_tc_normed_accepts(xd, nd, wd, acc, K.EPI_ADD, parts)
        K.gemm_tc_normed(xd, nd, eps, wd, acc, K.EPI_ADD, stream(), sumsq=parts)
        assert K.gemm_tc_error() == 0
        n_parts = K.gemm_tc_normed_slices(wd, K.EPI_ADD)
        assert 1 <= n_parts <= 16 and not torch.isnan(parts[:n_parts, :M]).any() and torch.isnan(parts[n_parts:]).all()
        sums = parts[:n_parts, :M].sum(0)
        assert rel_l2(sums.cpu(), (x.double() ** 2).sum(1).float()) < 1e-5
        scale = 1.0 / torch.sqrt(sums.cpu() / Kd + eps)
        got = acc.cpu() * scale[:, None]
        assert rel_l2(got, want) < 6e-3
        rows = (got - want).norm(dim=1) / want.norm(dim=1)
        assert float(rows.max()) < 1.2e-2, rows
    # what it refuses
    assert not K.gemm_tc_normed_accepts(xd, nd, wd, acc, K.EPI_ADD, None)                   # sums need their place
    assert not K.gemm_tc_normed_accepts(xd, nd, wd, act, K.EPI_SWIGLU, parts)
    big = torch.zeros(33, Kd, device="cuda")
    assert not K.gemm_tc_normed_accepts(big, nd, wd, torch.zeros(33, N // 2, dtype=torch.bfloat16, device="cuda"), K.EPI_SWIGLU, None)


@pytest.mark.parametrize("M,N,Kd", [(1, 4096, 4096), (8, 4096, 12288), (13, 1000, 4104), (17, 384, 2048), (40, 2600, 1096), (64, 4096, 4096),
                                    (100, 520, 4096), (127, 4096, 2048)])
def test_k_slices_added_in_a_fixed_order_give_the_same_bits_every_time(K, M, N, Kd):
    """``ordered``: the K slices of a decode product meet inside a thread-block cluster and are added in slice order, one
    writer per element.  Six runs from the same residual must agree bit for bit (reductions at L2 do so only by luck),
    and agree with float64 as closely as the default does."""
    g = torch.Generator().manual_seed(7 * M + N)
    x = torch.randn(M, Kd, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, Kd, generator=g) * 0.1).to(torch.bfloat16).cuda()
    res = torch.randn(M, N, generator=g)
    want = res + P.linear(x.float().cpu(), w.float().cpu())
    n4 = -(-N // 4) * 4
    runs = []
    for _ in range(6):
        acc = torch.zeros(M, n4, device="cuda")[:, :N]
        acc.copy_(res)
        K.gemm_tc(x, w, acc, K.EPI_ADD, stream(), ordered=True)
        runs.append(acc.clone())
    assert K.gemm_tc_error() == 0
    assert rel_l2(runs[0].cpu(), want) < 1e-5
    for r in runs[1:]:
        assert torch.equal(r, runs[0])
    if M <= 32:                  # and with the norm folded in
        xf = torch.randn(M, Kd, generator=g).cuda()
        nw = (1 + 0.2 * torch.randn(Kd, generator=g)).cuda()
        runs = []
        for _ in range(6):
            acc = torch.zeros(M, n4, device="cuda")[:, :N]
            parts = torch.zeros(16, 32, device="cuda")
            K.gemm_tc_normed(xf, nw, 1e-6, w, acc, K.EPI_ADD, stream(), sumsq=parts, ordered=True)
            runs.append((acc.clone(), parts.clone()))
        assert K.gemm_tc_error() == 0
        n_parts = K.gemm_tc_normed_slices(w, K.EPI_ADD, M, ordered=True)
        assert 1 <= n_parts <= K.gemm_tc_normed_slices(w, K.EPI_ADD, M)
        scale = 1.0 / torch.sqrt(runs[0][1][:n_parts, :M].sum(0).cpu() / Kd + 1e-6)
        assert rel_l2(runs[0][0].cpu() * scale[:, None], P.linear(P.rms_norm(xf.cpu(), nw.cpu(), 1e-6), w.float().cpu())) < 6e-3
        for acc, parts in runs[1:]:
            assert torch.equal(acc, runs[0][0]) and torch.equal(parts, runs[0][1])


def test_the_timeline_probe_is_absent_from_the_default_build(K):
    """The decode kernels' timeline probe costs nothing unless the library is built with -DTB_TIMELINE: the default
    build says so when a buffer is offered, and runs on as before."""
    import os
    buf = torch.zeros(1 + 8 * 16, dtype=torch.int64, device="cuda")
    built_in = "TB_TIMELINE" in os.environ.get("TITAN_B200_NVCC_FLAGS", "")
    assert K.timeline_attach(buf) == built_in
    x = torch.randn(4, 256).to(torch.bfloat16).cuda()
    w = torch.randn(128, 256).to(torch.bfloat16).cuda()
    out = torch.zeros(4, 128, device="cuda")
    K.gemm_tc(x, w, out, K.EPI_F32, stream())
    torch.cuda.synchronize()
    assert K.gemm_tc_error() == 0 and rel_l2(out.cpu(), P.linear(x.float().cpu(), w.float().cpu())) < 1e-5
    assert int(buf[0]) == (1 if built_in else 0)          # one CTA's record, or nothing
    K.timeline_attach(None)
