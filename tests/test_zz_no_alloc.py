"""The entry point that allocates nothing (titan_b200/csrc/attention_noalloc.h), called through its
exported C symbol, against the ordinary entry point that takes the caller's scratch buffer.

Some host programs may not allocate device memory while they run: a process that gave the whole GPU
to its own pool at start-up, or a loop that cannot afford the device-wide synchronisation inside
cudaMalloc.  For them the split-KV decode attention exists in a form whose scratch is a fixed 8 MiB
array inside the library.  This file is collected last on purpose (its name), so that a run that
stops at the first failure has already run everything else.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
SCRATCH_FLOATS = 2 * 1024 * 1024


def build_case(K, seed, lens, nh, nkv, hd, dtype):
    """A paged cache with scrambled pages and noise in unused rows, one query per sequence."""
    g = torch.Generator().manual_seed(seed)
    page, B = 64, len(lens)
    per = [-(-n // page) for n in lens]
    num_pages = sum(per) + 2
    order = torch.randperm(num_pages, generator=g).tolist()
    table = torch.zeros((B, max(per)), dtype=torch.int32)
    storage = (torch.randn(2, num_pages, nkv, page, hd, generator=g) * 30).to(dtype)
    keys, vals = [], []
    for s in range(B):
        for j in range(per[s]):
            table[s, j] = order.pop()
        k = torch.randn(lens[s], nkv, hd, generator=g).to(dtype)
        v = torch.randn(lens[s], nkv, hd, generator=g).to(dtype)
        for p in range(lens[s]):
            storage[0, int(table[s, p // page]), :, p % page] = k[p]
            storage[1, int(table[s, p // page]), :, p % page] = v[p]
        keys.append(k)
        vals.append(v)
    q = torch.randn(B, nh * hd, generator=g).to(dtype)
    dev = dict(table=table.cuda(), storage=storage.cuda(), q=q.cuda(),
               slots=torch.arange(B, dtype=torch.int32).cuda(), kv_len=torch.tensor(lens, dtype=torch.int32).cuda())
    # what the attention must give, in float64, from the keys and values themselves (not from the paged copy)
    want = torch.zeros(B, nh, hd, dtype=torch.float64)
    for s in range(B):
        for h in range(nh):
            kh = h // (nh // nkv)
            score = (keys[s][:, kh].double() @ q[s].view(nh, hd)[h].double()) / math.sqrt(hd)
            want[s, h] = torch.softmax(score, 0) @ vals[s][:, kh].double()
    return dev, want.reshape(B, nh * hd).float()


def make_args(K, dev, lens, nh, nkv, hd, chunk, out, scratch_ptr):
    B = len(lens)
    a = K.AttnArgs()
    a.q, a.q_stride, a.out, a.out_stride = dev["q"].data_ptr(), nh * hd, out.data_ptr(), nh * hd
    a.cache = K.KvView(dev["storage"].data_ptr(), dev["table"].data_ptr(), dev["table"].shape[1], 0, 64,
                       dev["storage"].shape[1], nkv, hd)
    a.batch = K.Batch(None, None, None, dev["slots"].data_ptr(), None, None, dev["kv_len"].data_ptr(), B, B, 1, max(lens))
    a.nh, a.nkv, a.hd, a.window, a.scale = nh, nkv, hd, 0, 1 / math.sqrt(hd)
    a.chunk, a.n_splits, a.scratch = chunk, -(-max(lens) // chunk), scratch_ptr
    return a


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row(dtype):
    from titan_b200 import kernels as K
    lib = K.lib()
    entry = lib.tb_attn_decode_noalloc                      # the exported C symbol itself
    entry.argtypes = [ctypes.POINTER(K.AttnArgs), ctypes.c_int, ctypes.c_void_p]
    entry.restype = ctypes.c_int
    stream = torch.cuda.current_stream().cuda_stream
    code = K.dtype_code(dtype)
    # two calls in a row with different shapes: the second finds the first one's leftovers in the array
    for seed, lens, nh, nkv, hd, chunk in [(1, [300, 17, 129], 6, 2, 48, 64), (2, [64, 500], 4, 4, 32, 128)]:
        dev, exact = build_case(K, seed, lens, nh, nkv, hd, dtype)
        B = len(lens)
        want = torch.empty(B, nh * hd, dtype=dtype, device="cuda")
        scratch = torch.empty(B * nh * -(-max(lens) // chunk) * (hd + 2), device="cuda")
        K.attn_decode(make_args(K, dev, lens, nh, nkv, hd, chunk, want, scratch.data_ptr()), dtype, stream)
        got = torch.full((B, nh * hd), float("nan"), dtype=dtype, device="cuda")
        # The first call on a device looks up the scratch array's address (and may load the module that holds it):
        # make it, then watch the driver's own count of free device memory around a second call.  That count moves
        # with any cudaMalloc or cudaFree in the process, by torch's allocator or by the library itself.
        args = make_args(K, dev, lens, nh, nkv, hd, chunk, got, None)
        assert entry(ctypes.byref(args), code, stream) == 0, lib.tb_last_error().decode()
        torch.cuda.synchronize()
        got.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = entry(ctypes.byref(args), code, stream)
        assert rc == 0, lib.tb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        # against float64 from the keys and values themselves: the bound of the other kernel tests
        exact_err = float((got.float().cpu() - exact).norm() / exact.norm())
        assert exact_err < (2e-6 if dtype == torch.float32 else 6e-3), exact_err
        # the same kernels on another scratch: the bound of the other kernel tests (2e-6 float32, 6e-3 bfloat16)
        err = float((got.float() - want.float()).norm() / want.float().norm())
        assert err < (2e-6 if dtype == torch.float32 else 6e-3), err
        assert torch.equal(got, want)                       # and in fact the same bits


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from titan_b200 import kernels as K
    lib = K.lib()
    entry = lib.tb_attn_decode_noalloc
    entry.argtypes = [ctypes.POINTER(K.AttnArgs), ctypes.c_int, ctypes.c_void_p]
    entry.restype = ctypes.c_int
    a = K.AttnArgs()
    a.batch = K.Batch(None, None, None, None, None, None, None, 64, 64, 1, 8192)
    a.nh, a.nkv, a.hd, a.chunk, a.n_splits = 32, 8, 128, 256, 32
    assert 64 * 32 * 32 * 130 > SCRATCH_FLOATS
    assert entry(ctypes.byref(a), K.BF16, None) != 0
    msg = lib.tb_last_error().decode()
    assert "8519680" in msg and str(SCRATCH_FLOATS) in msg
