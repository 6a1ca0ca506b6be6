"""Shared by the tests: the tiny configurations, model folders with random weights, the error
metric, and the plain reference's logits."""
import functools
import json
import os
import subprocess
import sys
import tempfile

import torch

from plain import qwen3_plain as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg(**kw):
    base = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
                attention_bias=False, rope_scaling=None)
    base.update(kw)
    return base


# Two tiny configurations that differ in every size and option, plus a windowed one.
TINY_A = _cfg(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True, max_position_embeddings=128, eos_token_id=7)
TINY_B = _cfg(num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=3, head_dim=32,
              intermediate_size=224, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
              tie_word_embeddings=False, max_position_embeddings=256, eos_token_id=[11, 12])
# odd sizes: width and vocabulary no power of two, one kv head for six q heads, head_dim 48,
# a window of 40 on two of four layers
TINY_C = _cfg(num_hidden_layers=4, hidden_size=72, num_attention_heads=6, num_key_value_heads=1, head_dim=48,
              intermediate_size=200, vocab_size=301, rope_theta=50000.0, rms_norm_eps=3e-6,
              tie_word_embeddings=False, max_position_embeddings=512, use_sliding_window=True,
              sliding_window=40, max_window_layers=2)
# as many kv heads as q heads, long context for far-key tests
TINY_D = _cfg(num_hidden_layers=2, hidden_size=80, num_attention_heads=5, num_key_value_heads=5, head_dim=16,
              intermediate_size=144, vocab_size=259, rope_theta=10000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True, max_position_embeddings=1024)

# head sizes the bfloat16 decode attention takes (64 and 128), groups of 4 and 2, a window of 70
TINY_E = _cfg(num_hidden_layers=2, hidden_size=128, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
              intermediate_size=192, vocab_size=500, rope_theta=10000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True, max_position_embeddings=512, use_sliding_window=True,
              sliding_window=70, max_window_layers=1)
TINY_F = _cfg(num_hidden_layers=2, hidden_size=96, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
              intermediate_size=160, vocab_size=333, rope_theta=1000000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=False, max_position_embeddings=1024)

# the layer sizes of the benchmark model (Qwen3-4B shape) with two layers and a small vocabulary:
# the kernels at the sizes they are tuned for
WIDE = _cfg(num_hidden_layers=2, hidden_size=2560, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
            intermediate_size=9728, vocab_size=4099, rope_theta=1000000.0, rms_norm_eps=1e-6,
            tie_word_embeddings=True, max_position_embeddings=4096)

CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F, "WIDE": WIDE}

F32_TOL = 1e-4     # max |got - ref| / max |ref|, float32 run against the plain implementation
BF16_TOL = 2e-2    # bfloat16 run against the plain implementation on the same (bfloat16) weights


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max |got - ref| / max(1e-6, max |ref|): the reference's metric
    (crates/bfi-core/src/fused_gemv.rs:83-93)."""
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    if not torch.isfinite(got).all():
        return float("inf")
    return float((got - ref).abs().max() / max(1e-6, float(ref.abs().max())))


_FOLDERS = {}


def model_folder(name: str, store: torch.dtype, seed: int = 11) -> str:
    """A temporary folder with config.json and model.safetensors for tiny config ``name``."""
    from builderforce_inference_b200.weights import write_model_folder
    key = (name, store, seed)
    if key not in _FOLDERS:
        d = tempfile.mkdtemp(prefix=f"bfi_tiny_{name}_")
        write_model_folder(CONFIGS[name], seed, d, store)
        _FOLDERS[key] = d
    return _FOLDERS[key]


@functools.lru_cache(maxsize=None)
def plain_model(folder: str):
    return P.load_folder(folder, torch.float32)


def plain_logits(folder: str, tokens) -> torch.Tensor:
    cfg, w = plain_model(folder)
    return P.forward_each(w, cfg, list(tokens))


def random_prompts(vocab: int, lengths, seed: int = 5):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def store_dtype(run_dtype: str) -> torch.dtype:
    return torch.float32 if run_dtype == "float32" else torch.bfloat16


def tol(run_dtype: str) -> float:
    return F32_TOL if run_dtype == "float32" else BF16_TOL


def run_trace(folder: str, dtype: str, steps, max_tokens: int, out_dir: str = None, env=None, cwd=None,
              trace_run=None):
    """Drive bin/trace_run with ``steps`` (a list of step dictionaries); returns {step: tensor}."""
    import numpy as np
    out_dir = out_dir or tempfile.mkdtemp(prefix="bfi_trace_")
    exe = trace_run or os.path.join(ROOT, "bin", "trace_run")
    cmd = [sys.executable, exe, "--model", folder, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens)]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    r = subprocess.run(cmd, input=text, capture_output=True, text=True, env=env, cwd=cwd, timeout=900)
    assert r.returncode == 0, f"trace_run failed ({r.returncode}):\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    done = [line for line in r.stdout.splitlines() if line.startswith("done ")]
    assert [d.split()[1] for d in done] == [str(s["step"]) for s in steps], r.stdout[-2000:]
    with open(os.path.join(folder, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    out = {}
    for s in steps:
        n_want = sum(len(e.get("want", [])) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if n_want:
            arr = np.fromfile(path, dtype="<f4")
            assert arr.size == n_want * vocab, (arr.size, n_want, vocab)
            out[s["step"]] = torch.from_numpy(arr.reshape(n_want, vocab).copy())
        else:
            assert not os.path.exists(path)
    return out
