"""The random-weights mode gives the same bits on the CPU (numpy) and on the device (a CUDA kernel): a
model made with a seed on one can be made again on the other."""
import numpy as np
import pytest
import torch

from helpers import TINY_B

pytestmark = pytest.mark.gpu


def test_a_model_folder_and_a_model_made_on_the_device_hold_the_same_tensors(tmp_path):
    from titan_b200 import Engine, StepEntry
    from titan_b200.config import config_from_dict
    from titan_b200.parts import declare_weights
    from titan_b200.weights import write_model_folder
    from titan_b200.weights.random_init import make_tensor
    cfg = config_from_dict(TINY_B)
    for d in declare_weights(cfg.to_model_spec()):
        for dtype in (torch.bfloat16, torch.float32):
            host, dev = make_tensor(d, 9, dtype, "cpu"), make_tensor(d, 9, dtype, "cuda")
            assert host.dtype == dev.dtype == dtype and torch.equal(host, dev.cpu()), d.name
    folder = write_model_folder(str(tmp_path / "m"), cfg, 9)
    a = Engine.from_pretrained(folder, dtype="float32", max_tokens=256)
    b = Engine.from_random(cfg, 9, dtype="float32", max_tokens=256)
    toks = [5, 400, 17, 99, 3, 250]
    outs = []
    for e in (a, b):
        s = e.alloc_slot()
        outs.append(e.step([StepEntry(s, toks, list(range(len(toks))))]))
    assert torch.equal(outs[0], outs[1])


def test_slices_of_a_large_matrix_and_its_moments():
    """One matrix of the benchmark's sizes, made on the device; rows and scattered slices of it made again on
    the CPU from the element index alone."""
    from titan_b200.weights.loader import WeightSpec
    from titan_b200.weights.random_init import make_tensor, tensor_key, values
    spec = WeightSpec("model.layers.0.mlp.down_proj.weight", (4096, 12288), "matrix", ("normal", 0.02))
    dev32 = make_tensor(spec, 2, torch.float32, "cuda")
    dev16 = make_tensor(spec, 2, torch.bfloat16, "cuda")
    assert torch.equal(dev32.to(torch.bfloat16), dev16)
    key = tensor_key(2, spec.name)
    flat = dev32.flatten().cpu()
    rng = np.random.default_rng(0)
    for start in [0, 12288 * 2047 + 5, 4096 * 12288 - 70000] + [int(v) for v in rng.integers(0, 4096 * 12288 - 70000, 6)]:
        want = torch.from_numpy(values(key, start, 70000, 0.02, 0.0))
        assert torch.equal(flat[start:start + 70000], want), start
    assert abs(float(dev32.mean())) < 2e-5 and abs(float(dev32.std()) - 0.02) < 2e-5
    assert 0.09 < float(dev32.abs().max()) < 0.14                      # about 5.4 sigma in 50 million draws
    ints = make_tensor(WeightSpec("t", (1000,), "int_table"), 1, torch.int32, "cuda").cpu()
    assert torch.equal(ints, make_tensor(WeightSpec("t", (1000,), "int_table"), 1, torch.int32, "cpu")) and 0 <= int(ints.min()) and int(ints.max()) < 1 << 15
