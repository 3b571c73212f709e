"""The packed layout of a step and the command line's options (no GPU)."""
import pytest
import torch

from titan_b200.cli import build_parser
from titan_b200.engine.batch import StepEntry, StepLayout


def test_layout_packs_without_padding():
    lay = StepLayout([StepEntry(4, [9, 8, 7], [0, 2]), StepEntry(1, [5], [0]), StepEntry(6, [1, 2], [])], [10, 0, 63], "cpu")
    assert (lay.T, lay.B, lay.W) == (6, 3, 3)
    assert lay.tokens.tolist() == [9, 8, 7, 5, 1, 2]
    assert lay.seq_of.tolist() == [0, 0, 0, 1, 2, 2]
    assert lay.pos_of.tolist() == [10, 11, 12, 0, 63, 64]
    assert lay.slot_of_seq.tolist() == [4, 1, 6] and lay.q_start.tolist() == [0, 3, 4, 6]
    assert lay.start_pos.tolist() == [10, 0, 63] and lay.kv_len.tolist() == [13, 1, 65]
    assert lay.want.tolist() == [0, 2, 3]                      # rows among the packed tokens
    assert (lay.max_new, lay.max_kv_len, lay.all_single, lay.all_fresh) == (3, 65, False, False)
    one = StepLayout([StepEntry(0, [3], [0]), StepEntry(2, [4], [0])], [0, 0], "cpu")
    assert one.all_single and one.all_fresh and one.h2d_bytes == one.buffer.numel() * 4
    for part in (lay.tokens, lay.seq_of, lay.pos_of, lay.slot_of_seq, lay.q_start, lay.start_pos, lay.kv_len, lay.want):
        assert part.dtype == torch.int32 and part.data_ptr() % 16 == 0


def test_command_line_keeps_the_references_options():
    ap = build_parser()
    a = ap.parse_args(["run", "-m", "dir", "--prompt-ids", "1,2,3", "--prompt-ids", "4 5"])
    assert (a.model, a.kv_capacity, a.temperature, a.top_p, a.top_k, a.repetition_penalty, a.seed, a.max_tokens) == \
        ("dir", 2048, 0.7, 0.9, 40, 1.1, None, 512)
    assert a.prompt_ids == [[1, 2, 3], [4, 5]]
    b = ap.parse_args(["chat", "folder", "-c", "4096", "-t", "0", "--top-p", "0.5", "--stop-ids", "7,8", "--dtype", "float32"])
    assert (b.model_pos, b.kv_capacity, b.temperature, b.top_p, b.stop_ids, b.dtype) == ("folder", 4096, 0.0, 0.5, [7, 8], "float32")
    for alias in ("--temp", "--temperature"):
        assert ap.parse_args(["run", alias, "1.5"]).temperature == 1.5
    assert ap.parse_args(["bench", "--random", "cfg.json"]).random == "cfg.json"
    c = ap.parse_args(["run", "-m", "dir", "--max-context", "300", "--max-batch", "2"])
    assert (c.max_context, c.max_batch) == (300, 2) and (a.max_context, a.max_batch) == (None, 64)
    with pytest.raises(SystemExit):
        ap.parse_args(["serve"])                               # servers are outside this library
