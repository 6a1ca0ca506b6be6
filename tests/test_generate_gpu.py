"""Generation through the Python entry point and the command line against the plain
implementation: greedy ids, stop tokens, unequal batches, seeded temperature sampling."""
import json
import math
import os
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


NEAR_TIE = 1e-2      # of max |logit|: a plain top-2 gap below this may flip under bfloat16 rounding


def walk_plain_greedy(folder, prompt, got):
    """Walk the plain implementation along the engine's tokens.  Returns the steps at which the
    engine's token is not the plain argmax, each with the gap between the plain best logit and the
    engine's choice, as a fraction of the largest |logit| of that step."""
    cfg, w = plain_model(folder)
    ids = list(prompt)
    swaps = []
    for step, tok in enumerate(got):
        logits = P.forward_each(w, cfg, ids)[-1]
        if tok != P.argmax_first(logits.tolist()):
            swaps.append((step, float(logits.max() - logits[tok]) / float(logits.abs().max())))
        ids.append(tok)
    return swaps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_batch_matches_plain(name, dtype):
    """32 greedy tokens per request.  float32: the plain implementation's ids exactly.  bfloat16:
    the same ids (the reference asks for exact top-1 agreement, crates/bfi-runtime/tests/
    golden_greedy.rs:102-144), except at steps where the plain top-2 gap is a near-tie, and those
    are counted: from a swap on, the walk follows the engine's token, so later steps are judged on
    the engine's own prefix."""
    model = load(name, dtype)
    folder = model_folder(name, store_dtype(dtype))
    cfg, w = plain_model(folder)
    from builderforce_inference_b200 import SampleParams
    lens = [5, 11, 17] if name == "A" else [1, 7, 32, 64]
    prompts = random_prompts(CONFIGS[name]["vocab_size"], lens, seed=3)
    outs = model.generate_batch(prompts, SampleParams(max_tokens=32), ignore_eos=True)
    assert model.last_batch_decode_steps == 31 and model.last_generated_tokens == 32 * len(prompts)
    n_swaps = 0
    for p, got in zip(prompts, outs):
        assert len(got) == 32
        if dtype == "float32":
            assert got == P.greedy_generate(w, cfg, p, 32)
        else:
            swaps = walk_plain_greedy(folder, p, got)
            assert all(gap < NEAR_TIE for _, gap in swaps), swaps
            n_swaps += len(swaps)
    # near-ties that bfloat16 rounding turned, over all requests and steps of this configuration
    assert n_swaps <= MAX_BF16_SWAPS[name], n_swaps
    # alone, each request generates what it generated in the batch
    for p, got in zip(prompts[:2], outs[:2]):
        assert model.generate(p, SampleParams(max_tokens=32), ignore_eos=True) == got


MAX_BF16_SWAPS = {"A": 2, "B": 3}     # of 96 and 128 steps


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


def test_model_exposes_the_step_function_the_slots_and_its_configuration():
    from builderforce_inference_b200 import Qwen3Config, SequenceStep, registry
    model = load("B", "float32")
    cfg = model.config
    assert isinstance(cfg, Qwen3Config) and cfg.head_dim == 32 and cfg.num_key_value_heads == 3
    with pytest.raises(Exception):
        cfg.head_dim = 64                                   # read-only
    assert registry() == ["Qwen3ForCausalLM", "qwen3"]
    assert (model.n_layer(), model.n_vocab(), model.n_ctx(), model.n_embd()) == (3, 384, 256, 96)
    folder = model_folder("B", torch.float32)
    p = random_prompts(384, [9], seed=1)[0]
    slot = model.alloc_slot()
    got = model.step([SequenceStep(slot, p, [8])]).cpu()
    from helpers import plain_logits, rel_err
    assert rel_err(got, plain_logits(folder, p)[8:9]) < 1e-4
    model.free_slot(slot)
    assert model.engine.cache.slots.n_held == 0


def test_seeded_temperature_sampling_in_bfloat16():
    """Tiny B at temperature 0.8, seeded, in bfloat16.  The engine's logits differ from the plain
    ones by at most e = BF16_TOL * max|logit|, so every probability moves by a factor within
    exp(+-2e/T) and the cumulative distribution by at most d = exp(2e/T) - 1 anywhere: the sampled
    token's plain interval, widened by d, must hold the uniform number.  Most tokens must be the
    plain sampler's exact choice."""
    from builderforce_inference_b200 import SampleParams
    from builderforce_inference_b200.sampling import uniform_draw
    from helpers import BF16_TOL
    import math
    model = load("B", "bfloat16")
    cfg, w = plain_model(model_folder("B", torch.bfloat16))
    prompts = random_prompts(384, [1, 7, 32, 64], seed=8)
    sp = SampleParams(max_tokens=16, temperature=0.8, seed=5)
    outs = model.generate_batch(prompts, sp, ignore_eos=True)
    assert outs == model.generate_batch(prompts, sp, ignore_eos=True)
    exact = total_tokens = 0
    pp = P.PlainSampleParams(temperature=0.8, seed=5)
    for r, (p, got) in enumerate(zip(prompts, outs)):
        ids = list(p)
        assert len(got) == 16
        for step, tok in enumerate(got):
            logits = P.forward_each(w, cfg, ids)[-1]
            kind, val = P.target(logits.tolist(), ids, pp)
            assert kind == "weights"
            u = uniform_draw(sp.seed, r, step)
            total = sum(pr for _, pr in val)
            d = math.exp(2.0 * BF16_TOL * float(logits.abs().max()) / 0.8) - 1.0
            cum, ok = 0.0, False
            for i, pr in val:
                lo, cum = cum, cum + pr
                if i == tok:
                    ok = lo / total - d <= u <= cum / total + d
                    exact += int(P.draw(val, u) == tok)
            assert ok, (r, step, tok, d)
            total_tokens += 1
            ids.append(tok)
    assert exact >= 0.9 * total_tokens, (exact, total_tokens)


def test_command_line_run_and_bench():
    folder = model_folder("A", torch.float32)
    cfg, w = plain_model(folder)
    prompt = [5, 9, 200, 31]
    r = subprocess.run([sys.executable, "-m", "builderforce_inference_b200", "run", folder, "5 9 200,31",
                        "--dtype", "float32", "--max-new-tokens", "12", "--ignore-eos"], cwd=ROOT, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [int(t) for t in r.stdout.split()] == P.greedy_generate(w, cfg, prompt, 12)
    r = subprocess.run([sys.executable, "-m", "builderforce_inference_b200", "bench", folder, "--pp", "64", "--tg",
                        "16", "--dtype", "bfloat16"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "| pp64 |" in r.stdout and "| tg16 |" in r.stdout
    rates = [float(line.split("|")[4]) for line in r.stdout.splitlines() if "| pp64 |" in line or "| tg16 |" in line]
    assert len(rates) == 2 and all(math.isfinite(x) and x > 0 for x in rates), r.stdout
    r = subprocess.run([sys.executable, "-m", "builderforce_inference_b200", "bench", folder, "--pp", "32", "--tg",
                        "8", "--batch", "3", "--prompt-len-min", "5", "--prompt-len-max", "40", "--reps", "2", "--json",
                        "--dtype", "float32"], cwd=ROOT,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    rates = json.loads(r.stdout.strip().splitlines()[-1])
    assert set(rates) == {"pp32", "tg8"} and all(math.isfinite(x) and x > 0 for x in rates.values())


def test_command_line_prompt_file_random_weights_cache_budget_and_stop_ids(tmp_path):
    """``--prompt-ids FILE`` serves the file's prompts as one batch; ``--random-weights SEED`` makes
    the model of a config.json in device memory (the same model a written folder holds);
    ``--cache-gib`` sizes the cache; stop ids come from generation_config.json when it is there."""
    import shutil
    from builderforce_inference_b200 import write_model_folder
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(CONFIGS["A"]))
    folder = str(tmp_path / "model")
    write_model_folder(CONFIGS["A"], 31, folder, torch.float32)
    cfg, w = P.load_folder(folder)
    prompts = [[5, 9, 200, 31], [17], [3, 4, 5, 6, 7, 8, 9]]
    ids_file = tmp_path / "prompts.txt"
    ids_file.write_text("\n".join(" ".join(str(t) for t in p) for p in prompts) + "\n")
    r = subprocess.run([sys.executable, "-m", "builderforce_inference_b200", "run", str(cfg_path), "--random-weights",
                        "31", "--prompt-ids", str(ids_file), "--dtype", "float32", "--max-tokens", "10", "--ignore-eos",
                        "--cache-gib", "0.001"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [[int(t) for t in line.split()] for line in r.stdout.strip().splitlines()]
    assert lines == [P.greedy_generate(w, cfg, p, 10) for p in prompts]
    # stop ids: config.json says 7; generation_config.json names the token the first prompt's
    # free run produces at step 4, so that run now ends there
    free = P.greedy_generate(w, cfg, prompts[0], 10, ())
    stop = free[4]
    with open(os.path.join(folder, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": [stop, 300000]}, f)
    from builderforce_inference_b200 import Model, SampleParams
    model = Model.load(folder, dtype="float32", cache_bytes=1 << 20, cache_slots=4)
    assert model.stop_ids == (stop, 300000, 7)
    assert model.engine.cache_plan.max_tokens == model.engine.cache.n_pages * 64
    assert model.engine.cache_plan.kv_bytes <= 1 << 20 < model.engine.cache_plan.kv_bytes + 256 * model.engine.cache.bytes_per_token()
    assert model.generate(prompts[0], SampleParams(max_tokens=10)) == P.greedy_generate(w, cfg, prompts[0], 10, (stop, 7))
    shutil.rmtree(folder)


def test_replay_subcommand_is_trace_run(tmp_path):
    from helpers import run_trace
    folder = model_folder("A", torch.float32)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3, 4, 5], "want": [4]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [6], "want": [0]}], "end": ["a"]}]
    a = run_trace(folder, "float32", steps, 256)
    text = "".join(json.dumps(s) + "\n" for s in steps)
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, "-m", "builderforce_inference_b200", "replay", "--model", folder, "--dtype",
                        "float32", "--out", str(out), "--max-tokens", "256"], input=text, cwd=ROOT, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.split() == ["done", "0", "done", "1"], r.stderr[-2000:]
    import numpy as np
    for s in (0, 1):
        assert torch.equal(torch.from_numpy(np.fromfile(out / f"{s}.f32", dtype="<f4")), a[s].reshape(-1))
