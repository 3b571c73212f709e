"""The number of splits of decode attention by batch size: it depends on the batch size and the machine alone
(never on what the sequences hold), fills the machine's places once, and leaves an eighth of them free because
the splits of a (sequence, kv head) are a thread-block cluster that is placed as a whole."""
from types import SimpleNamespace

from titan_b200.parts.attention import decode_split


def splits(B, kv_heads=8, **options):
    return decode_split(SimpleNamespace(B=B, max_kv_len=5000), kv_heads, dict(sm_count=148, **options), fast=True)


def test_splits_by_batch_size():
    got = {B: splits(B)[1] for B in (1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 12, 14, 16, 20, 32, 64, 200)}
    assert got == {1: 16, 2: 9, 3: 8, 4: 8, 5: 6, 6: 5, 7: 4, 8: 4, 9: 3, 10: 3, 12: 2, 14: 2, 16: 2, 20: 1, 32: 1, 64: 1, 200: 1}
    for B, s in got.items():
        assert B * 8 * s <= 2 * 148 * 7 // 8 or s == 1           # within 7/8 of the places
        assert splits(B)[0] == 128                               # splits of at least 128 keys


def test_splits_do_not_depend_on_lengths_and_can_be_forced():
    a = decode_split(SimpleNamespace(B=8, max_kv_len=100), 8, dict(sm_count=148), fast=True)
    b = decode_split(SimpleNamespace(B=8, max_kv_len=30000), 8, dict(sm_count=148, max_context=32768), fast=True)
    assert a == b
    assert splits(8, attn_splits=7, attn_min_chunk=512) == (512, 7)
    assert splits(3, kv_heads=1)[1] == 16 and splits(40, kv_heads=2)[1] == 3


def test_the_any_size_kernel_cuts_at_multiples_of_its_chunk():
    lay = SimpleNamespace(B=3, max_kv_len=1000)
    assert decode_split(lay, 8, dict(attn_chunk=256), fast=False) == (256, 4)
    assert decode_split(lay, 8, dict(attn_chunk=256, fixed_splits=True, max_context=8192), fast=False) == (256, 32)
