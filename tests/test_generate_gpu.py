"""Generation through the Python entry point and the command line against the plain
implementation: greedy ids, stop tokens, unequal batches, seeded temperature sampling."""
import subprocess
import sys

import pytest
import torch

from helpers import CONFIGS, ROOT, model_folder, plain_model, random_prompts, store_dtype
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu


def load(name, dtype, **kw):
    from builderforce_inference_b200 import Model
    kw.setdefault("max_tokens", 4096)
    return Model.load(model_folder(name, store_dtype(dtype)), dtype=dtype, **kw)


def plain_greedy_with_margin(folder, prompt, got, stop=()):
    """Walk the plain implementation along the engine's tokens: each must be the plain argmax, or
    lie within ``margin`` of it (bfloat16 may swap near-ties; float32 gets no slack to speak of)."""
    cfg, w = plain_model(folder)
    ids = list(prompt)
    margins = []
    for tok in got:
        logits = P.forward_each(w, cfg, ids)[-1]
        margins.append(float(logits.max() - logits[tok]))
        ids.append(tok)
    return margins


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_batch_matches_plain(name, dtype):
    model = load(name, dtype)
    folder = model_folder(name, store_dtype(dtype))
    cfg, w = plain_model(folder)
    from builderforce_inference_b200 import SampleParams
    lens = [5, 11, 17] if name == "A" else [1, 7, 32, 64]
    prompts = random_prompts(CONFIGS[name]["vocab_size"], lens, seed=3)
    outs = model.generate_batch(prompts, SampleParams(max_tokens=32), ignore_eos=True)
    assert model.last_batch_decode_steps == 31 and model.last_generated_tokens == 32 * len(prompts)
    for p, got in zip(prompts, outs):
        assert len(got) == 32
        if dtype == "float32":
            assert got == P.greedy_generate(w, cfg, p, 32)
        else:
            scale = float(P.forward_each(w, cfg, p)[-1].abs().max())
            assert max(plain_greedy_with_margin(folder, p, got)) < 2e-2 * scale
    # alone, each request generates what it generated in the batch
    for p, got in zip(prompts[:2], outs[:2]):
        assert model.generate(p, SampleParams(max_tokens=32), ignore_eos=True) == got


def test_stop_tokens_budgets_and_reuse():
    from builderforce_inference_b200 import SampleParams
    name, dtype = "A", "float32"
    model = load(name, dtype, max_batch=2, max_tokens=64 * 6)
    folder = model_folder(name, store_dtype(dtype))
    cfg, w = plain_model(folder)
    prompts = random_prompts(256, [9, 3, 30, 12, 6], seed=14)
    free = [P.greedy_generate(w, cfg, p, 20) for p in prompts]
    stop = [free[0][6], free[3][0]]
    outs = model.generate_batch(prompts, SampleParams(max_tokens=20), stop_ids=stop)
    for p, got, why in zip(prompts, outs, model.last_finish_reasons):
        want = P.greedy_generate(w, cfg, p, 20, stop)
        assert got == want and why == ("stop" if len(want) < 20 else "length")
        assert not set(got) & set(stop)
    assert outs[3] == []
    assert model.engine.cache.slots.n_held == 0
    model.engine.cache.check()
    # the model's own eos id (7 in this configuration) is the default stop token
    assert model.stop_ids == (7,)
    # context end: max_tokens 0 runs until the context (128) is full
    out = model.generate(prompts[2], SampleParams(max_tokens=0), ignore_eos=True)
    assert len(out) == 128 - 30
    trace = model.generate_greedy_trace(prompts[0], 5)
    assert trace.token_ids == P.greedy_generate(w, cfg, prompts[0], 5, (7,)) and trace.last_logits.numel() == 256


@pytest.mark.parametrize("params", [dict(temperature=0.8, seed=5), dict(temperature=1.3, seed=9, min_p=0.05),
                                    dict(temperature=0.7, seed=2, top_k=12), dict(temperature=0.9, seed=4, top_p=0.8),
                                    dict(temperature=0.0, repeat_penalty=1.3, presence_penalty=0.4)])
def test_sampling_is_seeded_and_follows_the_plain_distribution(params):
    """Every sampled token must be what the plain sampler draws at the same uniform number from
    the plain logits, unless the number falls on the edge of the token's interval."""
    from builderforce_inference_b200 import SampleParams
    from builderforce_inference_b200.sampling import uniform_draw
    name, dtype = "B", "float32"
    model = load(name, dtype)
    folder = model_folder(name, store_dtype(dtype))
    cfg, w = plain_model(folder)
    prompts = random_prompts(384, [1, 7, 32, 64], seed=8)
    sp = SampleParams(max_tokens=16, **params)
    outs = model.generate_batch(prompts, sp, ignore_eos=True)
    assert outs == model.generate_batch(prompts, sp, ignore_eos=True)
    if sp.temperature > 0:
        other = SampleParams(max_tokens=16, **dict(params, seed=params["seed"] + 1))
        assert outs != model.generate_batch(prompts, other, ignore_eos=True)
        assert len({tuple(o) for o in outs}) == len(outs)
    pp = P.PlainSampleParams(**{k: v for k, v in params.items()})
    for r, (p, got) in enumerate(zip(prompts, outs)):
        ids = list(p)
        for step, tok in enumerate(got):
            logits = P.forward_each(w, cfg, ids)[-1]
            kind, val = P.target(logits.tolist(), ids, pp)
            if kind == "token":
                assert tok == val
            else:
                u = uniform_draw(sp.seed, r, step)
                total = sum(pr for _, pr in val)
                cum, ok = 0.0, False
                for i, pr in val:
                    lo, cum = cum, cum + pr
                    if i == tok:
                        ok = lo - 1e-4 * total <= u * total <= cum + 1e-4 * total
                assert ok, (r, step, tok)
            ids.append(tok)


def test_command_line_run_and_bench():
    folder = model_folder("A", torch.float32)
    cfg, w = plain_model(folder)
    prompt = [5, 9, 200, 31]
    r = subprocess.run([sys.executable, "-m", "builderforce_inference_b200", "run", folder, "5 9 200,31",
                        "--dtype", "float32", "--max-tokens", "12", "--ignore-eos"], cwd=ROOT, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [int(t) for t in r.stdout.split()] == P.greedy_generate(w, cfg, prompt, 12)
    r = subprocess.run([sys.executable, "-m", "builderforce_inference_b200", "bench", folder, "--pp", "64", "--tg",
                        "16", "--dtype", "bfloat16"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "| pp64 |" in r.stdout and "| tg16 |" in r.stdout
