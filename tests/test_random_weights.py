"""Seeded random weights are a function of (seed, tensor name, element index): the package's
host path (NumPy), its CUDA kernel and the plain one-value-at-a-time statement under
``tests/plain`` give the same bits."""
import random
import tempfile

import numpy as np
import pytest
import torch

from plain import random_plain as R
from util import config_json


def _spec(name="B"):
    from llmario_b200.config import Qwen3Config

    return Qwen3Config.from_dict(config_json(name)).to_spec()


def test_host_values_equal_the_plain_statement():
    from llmario_b200.weights import expected_tensors, random_tensors

    spec = _spec("B")
    rng = random.Random(0)
    for dtype in (torch.float32, torch.bfloat16):
        tensors = random_tensors(spec, 1, dtype, "cpu")
        assert set(tensors) == set(expected_tensors(spec))
        for name, t in tensors.items():
            flat = t.reshape(-1).float()
            picks = [0, flat.numel() - 1] + [rng.randrange(flat.numel()) for _ in range(6)]
            for i in picks:
                want = R.weight(1, name, i, t.dim() == 1, dtype == torch.bfloat16)
                assert float(flat[i]) == want, (name, i, float(flat[i]), want)


def test_values_do_not_depend_on_order_or_slabs():
    from llmario_b200.weights.random_normal import normal_f32, standard_normal, tensor_key

    key = tensor_key(3, "model.layers.0.mlp.up_proj.weight")
    assert key == R.key_of(3, "model.layers.0.mlp.up_proj.weight")
    whole = standard_normal(key, 0, 5000)
    assert (standard_normal(key, 1234, 777) == whole[1234:2011]).all()
    assert whole[4321] == R.standard_normal(key, 4321)
    assert tensor_key(3, "a") != tensor_key(4, "a") != tensor_key(3, "b")
    # the distribution: a standard normal within sampling error
    z = standard_normal(key, 0, 200000)
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1.0) < 0.01
    assert abs(((z - z.mean()) ** 4).mean() / z.var() ** 2 - 3.0) < 0.1
    assert np.isfinite(z).all()
    f = normal_f32(key, 0, 1000, 1.0, 0.01)
    assert f.dtype == np.float32 and abs(f.mean() - 1.0) < 0.002


def test_extreme_uniforms_stay_finite():
    # the smallest and the largest first uniform, every quarter turn
    assert R.ln_unit(1 << 32) == 0.0
    assert R.ln_unit(1) == -32 * 0.6931471805599453
    assert R.cos_turn(0) == 1.0 and R.cos_turn(1 << 31) == -1.0
    assert abs(R.cos_turn(1 << 30)) < 1e-15 and abs(R.cos_turn(3 << 30)) < 1e-15
    for k in (1, (1 << 30) - 1, (1 << 30) + 1, (1 << 32) - 1):
        import math
        assert abs(R.cos_turn(k) - math.cos(2 * math.pi * k / 2 ** 32)) < 1e-14


@pytest.mark.gpu
def test_device_values_equal_host_values():
    """``Model.random`` on the GPU holds what ``write_random_model`` writes on the CPU, tensor
    by tensor and bit by bit, in both precisions."""
    from llmario_b200.config import Qwen3Config
    from llmario_b200.weights import random_tensors, write_random_model
    from llmario_b200.weights.safetensors_io import SafetensorsFolder

    cfg = Qwen3Config.from_dict(config_json("B"))
    for dtype in (torch.float32, torch.bfloat16):
        dev = random_tensors(cfg.to_spec(), 1, dtype, "cuda:0")
        with tempfile.TemporaryDirectory() as d:
            write_random_model(d, cfg, 1, dtype)
            folder = SafetensorsFolder(d)
            assert sorted(folder.names()) == sorted(dev)
            for name, t in dev.items():
                assert torch.equal(folder.tensor(name), t.cpu()), (name, dtype)
        with tempfile.TemporaryDirectory() as d:      # made on the device, then written
            write_random_model(d, cfg, 1, dtype, device="cuda:0")
            folder = SafetensorsFolder(d)
            for name, t in dev.items():
                assert torch.equal(folder.tensor(name), t.cpu()), (name, dtype)


@pytest.mark.gpu
def test_a_large_matrix_on_the_device_equals_the_host_in_slabs():
    """One matrix of the benchmark model's feed-forward size (4096 x 12288): the first, a middle
    and the last slab against NumPy, single values against the plain statement."""
    from llmario_b200 import kernels
    from llmario_b200.weights.random_normal import normal_f32, tensor_key

    name = "model.layers.0.mlp.down_proj.weight"
    key = tensor_key(0, name)
    n = 4096 * 12288
    t = torch.empty(4096, 12288, dtype=torch.bfloat16, device="cuda:0")
    kernels.random_normal(t, key, 0.0, 0.02)
    flat = t.view(-1)
    for first, count in ((0, 1 << 19), (n // 2 + 12345, 1 << 19), (n - (1 << 19), 1 << 19)):
        want = torch.from_numpy(normal_f32(key, first, count, 0.0, 0.02)).to(torch.bfloat16)
        assert torch.equal(flat[first:first + count].cpu(), want), first
    host = flat.float().cpu()
    rng = random.Random(1)
    for i in [0, n - 1] + [rng.randrange(n) for _ in range(20)]:
        assert float(host[i]) == R.weight(0, name, i, False, True), i
    assert abs(float(host.std()) - 0.02) < 2e-4 and abs(float(host.mean())) < 1e-4
    # a slab made with an offset continues the sequence
    part = torch.empty(1000, dtype=torch.float32, device="cuda:0")
    kernels.random_normal(part, key, 0.0, 0.02, first=777)
    assert np.array_equal(part.cpu().numpy(), normal_f32(key, 777, 1000, 0.0, 0.02))
