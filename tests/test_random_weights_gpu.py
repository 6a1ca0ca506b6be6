"""The random-weights mode on the GPU: device memory filled by the kernel holds the same bits as
the folder written on the CPU, and a model made that way is the model the plain implementation
reads from the folder."""
import tempfile

import pytest
import torch

from helpers import BF16_TOL, F32_TOL, TINY_B, WIDE, random_prompts, rel_err
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_device_fill_equals_the_folder_bit_for_bit(dtype):
    from builderforce_inference_b200.engine.decoder import expected_tensors
    from builderforce_inference_b200.registry import describe_model
    from builderforce_inference_b200.weights.random_init import random_tensors
    exp = expected_tensors(describe_model(TINY_B))
    cpu = dict(random_tensors(exp, 21, dtype, torch.device("cpu")))
    gpu = dict(random_tensors(exp, 21, dtype, torch.device("cuda:0")))
    assert set(cpu) == set(gpu)
    for name in cpu:
        assert gpu[name].dtype == dtype and torch.equal(gpu[name].cpu(), cpu[name]), name


def test_device_fill_of_a_large_tensor_at_scattered_places():
    from plain import random_fill_plain as R
    from builderforce_inference_b200.parts.base import ParamSpec
    from builderforce_inference_b200.weights.random_init import random_tensor
    shape = (151936, 2560)                      # past 2^28 elements: 64-bit indices on the device
    t = random_tensor("model.embed_tokens.weight", ParamSpec(shape, "table"), 0, torch.bfloat16, torch.device("cuda:0"))
    flat = t.view(-1)
    n = flat.numel()
    for i in (0, 1, 2 ** 28 - 1, 2 ** 28, 2 ** 28 + 12345, n - 1):
        got = int(flat[i].view(torch.int16).item()) & 0xFFFF
        assert got == R.bf16_bits(R.value(0, "model.embed_tokens.weight", i, "table")), i
    assert abs(float(flat[:10_000_000].float().std()) - 0.02) < 2e-4


def test_conversion_kernel_rounds_to_nearest_even():
    from builderforce_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    x = torch.randn(100_003, generator=g) * 3.0
    x[:4] = torch.tensor([1.00390625, 1.01171875, -1.00390625, 0.0])      # ties: to even
    dev = x.cuda()
    assert torch.equal(ops.convert(dev, torch.bfloat16).cpu(), x.bfloat16())
    assert torch.equal(ops.convert(x.bfloat16().cuda(), torch.float32).cpu(), x.bfloat16().float())
    assert torch.equal(ops.convert(dev, torch.float32).cpu(), x)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_model_from_random_is_the_model_of_the_written_folder(dtype):
    """Two layers at the benchmark model's widths, made in device memory from (config, seed), give
    the plain implementation's logits for the folder written from the same (config, seed)."""
    from builderforce_inference_b200 import write_model_folder
    from builderforce_inference_b200.engine.engine import Engine, SequenceStep
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    prompt = random_prompts(WIDE["vocab_size"], [150], seed=3)[0]
    eng = Engine.from_random(WIDE, 17, dtype=dtype, max_tokens=1024)
    s = eng.acquire()
    got = eng.step([SequenceStep(s, prompt, list(range(len(prompt))))]).cpu()
    with tempfile.TemporaryDirectory() as folder:
        write_model_folder(WIDE, 17, folder, store)
        cfg, w = P.load_folder(folder)
        ref = P.forward_each(w, cfg, prompt)
        loaded = Engine.load(folder, dtype=dtype, max_tokens=1024)
        s2 = loaded.acquire()
        same = loaded.step([SequenceStep(s2, prompt, list(range(len(prompt))))]).cpu()
    assert torch.equal(got, same)
    assert rel_err(got, ref) < (F32_TOL if dtype == "float32" else BF16_TOL)
