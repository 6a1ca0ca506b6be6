"""Each part alone: built from its kind and parameters through the registries, given weights,
driven with a hand-made step context, and compared with the plain function of the same part.
Sizes differ from the tiny models' (width 88, 4 q / 2 kv heads of 48, inner 136)."""
import math

import pytest
import torch

from helpers import rel_err
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def setup(dtype):
    from builderforce_inference_b200.engine.context import Workspace
    from builderforce_inference_b200.engine.decoder import Runtime
    return Runtime(DEV, dtype), Workspace(DEV)


def rand_params(part, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, ps in part.all_param_specs().items():
        t = torch.randn(ps.shape, generator=g)
        t = 1 + 0.1 * t if ps.role == "norm" else 0.08 * t
        out[name] = t.to(dtype)
    return out


def ctx_for(seqs, dtype, ws):
    from builderforce_inference_b200.engine.context import build_context
    return build_context(seqs, dtype, ws, DEV)


def tolerance(dtype):
    return 5e-6 if dtype == torch.float32 else 1.5e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from builderforce_inference_b200.parts import NORMS, PartSpec
    rt, ws = setup(dtype)
    norm = NORMS.build(PartSpec("rms", {"width": 88, "eps": 2e-5}))
    w = rand_params(norm, dtype)
    norm.load_all({k: v.to(DEV) for k, v in w.items()}, rt)
    x = torch.randn(6, 88)
    ctx = ctx_for([(0, 0, [1] * 6)], dtype, ws)
    h = norm.forward(ctx, x.to(DEV))
    assert h.dtype == dtype
    assert rel_err(h.float(), P.rms_norm(x, w["weight"].float(), 2e-5)) < tolerance(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from builderforce_inference_b200.parts import FEED_FORWARDS, PartSpec
    rt, ws = setup(dtype)
    ffn = FEED_FORWARDS.build(PartSpec("gated_mlp", {"width": 88, "inner": 136}))
    w = rand_params(ffn, dtype, 1)
    ffn.load_all({k: v.to(DEV) for k, v in w.items()}, rt)
    for rows in (1, 5, 40):                       # few rows and many rows take different kernels
        h = torch.randn(rows, 88).to(dtype)
        res = torch.randn(rows, 88)
        ctx = ctx_for([(0, 0, [1] * rows)], dtype, ws)
        out = res.clone().to(DEV)
        ffn.forward(ctx, h.to(DEV), out)
        f = {k: v.float() for k, v in w.items()}
        ref = res + P.linear(f["down_proj"], P.swiglu(P.linear(f["gate_proj"], h.float()),
                                                      P.linear(f["up_proj"], h.float())))
        assert rel_err(out, ref) < tolerance(dtype)


def make_kv_cache(n_kv, d, dtype, window=None):
    from builderforce_inference_b200.cache import SequenceCache
    from builderforce_inference_b200.parts import KVNeed
    return SequenceCache([KVNeed(n_kv, d, window)], [None], 64 * 8, 512, dtype, DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_prefill_then_decode(dtype, window):
    from builderforce_inference_b200.parts import MIXERS, PartSpec
    rt, ws = setup(dtype)
    n_q, n_kv, d, width, theta, eps = 4, 2, 48, 88, 3e4, 1e-5
    att = MIXERS.build(PartSpec("attention", {
        "width": width, "n_heads": n_q, "n_kv_heads": n_kv, "head_dim": d, "qk_norm": True, "eps": eps,
        "window": window, "position": PartSpec("rotary", {"theta": theta, "rot_dim": d})}))
    w = rand_params(att, dtype, 2)
    att.load_all({k: v.to(DEV) for k, v in w.items()}, rt)
    att.prepare(rt, 512)
    cache = make_kv_cache(n_kv, d, dtype, window)
    f = {k: v.float() for k, v in w.items()}
    n = 70
    h = torch.randn(n, width).to(dtype)

    def plain(hh):
        t = hh.shape[0]
        q = P.linear(f["q_proj"], hh).reshape(t, n_q, d)
        k = P.linear(f["k_proj"], hh).reshape(t, n_kv, d)
        v = P.linear(f["v_proj"], hh).reshape(t, n_kv, d)
        q = P.rope_neox(P.rms_norm(q, f["q_norm"], eps), range(t), theta)
        k = P.rope_neox(P.rms_norm(k, f["k_norm"], eps), range(t), theta)
        return P.linear(f["o_proj"], P.attention(q, k, v, window).reshape(t, n_q * d))

    ref = plain(h.float())
    slot = cache.acquire()
    cache.begin_step([slot], [66])
    res = torch.zeros(66, width, device=DEV)
    att.forward(ctx_for([(slot, 0, [0] * 66)], dtype, ws), h[:66].to(DEV), res, cache.run_cache(0))
    cache.end_step([slot], [66])
    assert rel_err(res, ref[:66]) < tolerance(dtype)
    for t in range(66, n):
        cache.begin_step([slot], [1])
        res = torch.zeros(1, width, device=DEV)
        att.forward(ctx_for([(slot, t, [0])], dtype, ws), h[t:t + 1].to(DEV), res, cache.run_cache(0))
        cache.end_step([slot], [1])
        assert rel_err(res, ref[t:t + 1]) < tolerance(dtype), t


def test_attention_options_no_norm_no_rotation_custom_scale():
    from builderforce_inference_b200.parts import MIXERS, PartSpec
    dtype = torch.float32
    rt, ws = setup(dtype)
    n_q, n_kv, d, width = 3, 3, 16, 40
    att = MIXERS.build(PartSpec("attention", {"width": width, "n_heads": n_q, "n_kv_heads": n_kv, "head_dim": d,
                                              "scale": 0.3}))
    assert sorted(att.all_param_specs()) == ["k_proj", "o_proj", "q_proj", "v_proj"]
    w = rand_params(att, dtype, 3)
    att.load_all({k: v.to(DEV) for k, v in w.items()}, rt)
    att.prepare(rt, 64)
    cache = make_kv_cache(n_kv, d, dtype)
    h = torch.randn(20, width)
    q = P.linear(w["q_proj"], h).reshape(20, n_q, d) * (0.3 * math.sqrt(d))
    k = P.linear(w["k_proj"], h).reshape(20, n_kv, d)
    v = P.linear(w["v_proj"], h).reshape(20, n_kv, d)
    ref = P.linear(w["o_proj"], P.attention(q, k, v).reshape(20, n_q * d))
    slot = cache.acquire()
    cache.begin_step([slot], [20])
    res = torch.zeros(20, width, device=DEV)
    att.forward(ctx_for([(slot, 0, [0] * 20)], dtype, ws), h.to(DEV), res, cache.run_cache(0))
    assert rel_err(res, ref) < 5e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_part(dtype):
    from builderforce_inference_b200.parts import BLOCKS, PartSpec
    rt, ws = setup(dtype)
    n_q, n_kv, d, width, inner, theta, eps = 4, 1, 32, 72, 100, 1e4, 1e-6
    norm = PartSpec("rms", {"width": width, "eps": eps})
    block = BLOCKS.build(PartSpec("prenorm", {
        "norm1": norm, "norm2": norm,
        "mixer": PartSpec("attention", {"width": width, "n_heads": n_q, "n_kv_heads": n_kv, "head_dim": d,
                                        "qk_norm": True, "eps": eps,
                                        "position": PartSpec("rotary", {"theta": theta, "rot_dim": d})}),
        "ffn": PartSpec("gated_mlp", {"width": width, "inner": inner})}))
    w = rand_params(block, dtype, 4)
    assert "mixer.q_norm" in w and "norm2.weight" in w and "ffn.down_proj" in w
    block.load_all({k: v.to(DEV) for k, v in w.items()}, rt)
    block.mixer().prepare(rt, 128)
    cache = make_kv_cache(n_kv, d, dtype)
    x = torch.randn(37, width)
    names = {"input_layernorm.weight": "norm1.weight", "post_attention_layernorm.weight": "norm2.weight",
             "self_attn.q_proj.weight": "mixer.q_proj", "self_attn.k_proj.weight": "mixer.k_proj",
             "self_attn.v_proj.weight": "mixer.v_proj", "self_attn.o_proj.weight": "mixer.o_proj",
             "self_attn.q_norm.weight": "mixer.q_norm", "self_attn.k_norm.weight": "mixer.k_norm",
             "mlp.gate_proj.weight": "ffn.gate_proj", "mlp.up_proj.weight": "ffn.up_proj",
             "mlp.down_proj.weight": "ffn.down_proj"}
    pw = {"L." + k: w[v].float() for k, v in names.items()}
    pc = P.PlainConfig(1, width, inner, 10, 128, n_q, n_kv, d, eps, theta, True, [None])
    ref = P.mlp_half(P.attention_half(x, pw, "L.", pc, range(37), None), pw, "L.", pc)
    slot = cache.acquire()
    cache.begin_step([slot], [37])
    res = x.clone().to(DEV)
    block.forward(ctx_for([(slot, 0, [0] * 37)], dtype, ws), res, cache.run_cache(0))
    assert rel_err(res, ref) < tolerance(dtype)


def test_unknown_kinds_and_bad_sizes_are_refused():
    from builderforce_inference_b200.parts import MIXERS, NORMS, PartSpec
    with pytest.raises(KeyError, match="registered"):
        NORMS.build(PartSpec("layernorm", {"width": 8}))
    with pytest.raises(ValueError, match="steps of 16"):
        MIXERS.build(PartSpec("attention", {"width": 8, "n_heads": 2, "n_kv_heads": 1, "head_dim": 24}))
    with pytest.raises(ValueError, match="GQA"):
        MIXERS.build(PartSpec("attention", {"width": 8, "n_heads": 3, "n_kv_heads": 2, "head_dim": 16}))
