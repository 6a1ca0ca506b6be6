"""The plain implementation checked against closed forms the reference's own unit tests use
(crates/bfi-core/src/cpu.rs:834-1047) and against its core invariant: a prefix's logits do not
depend on what follows (crates/bfi-models/src/lib.rs:480-543)."""
import math

import torch

from helpers import TINY_A, TINY_B, TINY_C, model_folder, plain_logits
from plain import qwen3_plain as P


def test_rms_norm_of_ones_is_ones():
    x = torch.ones(3, 8)
    y = P.rms_norm(x, torch.ones(8), 0.0)
    assert torch.allclose(y, torch.ones(3, 8))


def test_rms_norm_weight_multiplies_as_stored_and_eps_inside_sqrt():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    eps = 0.5
    s = 1.0 / math.sqrt((9 + 16) / 2 + eps)
    assert torch.allclose(P.rms_norm(x, w, eps), torch.tensor([[3 * s * 2, 4 * s * 0.5]]))


def test_rope_position_zero_is_identity_and_pairs_i_with_half():
    x = torch.arange(8, dtype=torch.float32).reshape(1, 1, 8)
    assert torch.equal(P.rope_neox(x, [0], 10000.0), x)
    # position 1, first pair (x0, x4) turns by 1 rad (theta^0 = 1)
    y = P.rope_neox(x, [1], 10000.0)
    c, s = math.cos(1.0), math.sin(1.0)
    assert abs(float(y[0, 0, 0]) - (0 * c - 4 * s)) < 1e-6
    assert abs(float(y[0, 0, 4]) - (0 * s + 4 * c)) < 1e-6


def test_rope_preserves_norm():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 3, 16, generator=g)
    y = P.rope_neox(x, [0, 3, 17, 100, 1000], 1e6)
    assert torch.allclose(x.norm(dim=-1), y.norm(dim=-1), atol=1e-5)


def test_attention_single_key_returns_v():
    q = torch.randn(1, 4, 8)
    k = torch.randn(1, 2, 8)
    v = torch.randn(1, 2, 8)
    out = P.attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 1], v[0, 0])
    assert torch.allclose(out[0, 2], v[0, 1]) and torch.allclose(out[0, 3], v[0, 1])


def test_attention_is_causal_and_window_drops_old_keys():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(6, 2, 4, generator=g) for _ in range(3))
    full = P.attention(q, k, v)
    # changing a later key/value must not change an earlier output
    k2, v2 = k.clone(), v.clone()
    k2[5] += 1.0
    v2[5] += 1.0
    assert torch.equal(P.attention(q, k2, v2)[:5], full[:5])
    # window 2: token 4 sees keys 3 and 4 only
    w = P.attention(q, k, v, window=2)
    ref = P.attention(q[3:5], k[3:5], v[3:5])
    assert torch.allclose(w[4], ref[1], atol=1e-6)
    assert torch.allclose(P.attention(q, k, v, window=6), full)


def test_silu_values():
    x = torch.tensor([0.0, 1.0, -1.0, 20.0, -20.0])
    y = P.silu(x)
    assert abs(float(y[0])) < 1e-7
    assert abs(float(y[1]) - 0.7310586) < 1e-6
    assert abs(float(y[2]) + 0.26894143) < 1e-6
    assert abs(float(y[3]) - 20.0) < 1e-4 and abs(float(y[4])) < 1e-6


def test_prefix_logits_do_not_depend_on_what_follows():
    for name in ("A", "B", "C"):
        folder = model_folder(name, torch.float32)
        toks = list(range(3, 60))
        whole = plain_logits(folder, toks)
        part = plain_logits(folder, toks[:21])
        assert float((whole[:21] - part).abs().max()) < 1e-5


def test_plain_float64_agrees_with_float32():
    folder = model_folder("B", torch.float32)
    cfg, w32 = P.load_folder(folder, torch.float32)
    _, w64 = P.load_folder(folder, torch.float64)
    toks = list(range(40))
    a = P.forward_each(w32, cfg, toks)
    b = P.forward_each(w64, cfg, toks)
    assert float((a.double() - b).abs().max() / b.abs().max()) < 1e-5


def test_window_config_reaches_the_plain_model():
    cfg = P.PlainConfig.from_dict(TINY_C)
    assert cfg.windows == [None, None, 40, 40]
    assert P.PlainConfig.from_dict(TINY_A).windows == [None, None]
    assert P.PlainConfig.from_dict(TINY_B).n_head_kv == 3


def test_sampler_greedy_first_maximum_and_penalties():
    logits = [0.1, 2.0, 2.0, -1.0]
    assert P.target(logits, [], P.PlainSampleParams()) == ("token", 1)
    # repeat penalty divides positive logits of seen ids: id 1 drops below id 2
    assert P.target(logits, [1], P.PlainSampleParams(repeat_penalty=2.0)) == ("token", 2)
    assert P.target(logits, [1, 2], P.PlainSampleParams(presence_penalty=3.0)) == ("token", 0)


def test_sampler_draw_in_list_order():
    pairs = [(5, 0.2), (9, 0.5), (2, 0.3)]
    assert P.draw(pairs, 0.0) == 5
    assert P.draw(pairs, 0.19) == 5
    assert P.draw(pairs, 0.21) == 9
    assert P.draw(pairs, 0.71) == 2
    assert P.draw(pairs, 0.999999) == 2


def test_sampler_top_k_top_p_min_p():
    logits = [math.log(p) for p in (0.5, 0.3, 0.15, 0.05)]
    kind, pairs = P.target(logits, [], P.PlainSampleParams(temperature=1.0, top_k=2))
    assert kind == "weights" and [i for i, _ in pairs] == [0, 1]
    kind, pairs = P.target(logits, [], P.PlainSampleParams(temperature=1.0, top_p=0.75))
    assert [i for i, _ in pairs] == [0, 1]
    kind, pairs = P.target(logits, [], P.PlainSampleParams(temperature=1.0, min_p=0.5))
    assert [i for i, _ in pairs] == [0, 1]


def test_xorshift_unit_matches_hand_computation():
    x = 1
    x ^= (x << 13) & ((1 << 64) - 1)
    x ^= x >> 7
    x ^= (x << 17) & ((1 << 64) - 1)
    assert P.xorshift_unit(1) == (x >> 40) / float(1 << 24)
    assert 0.0 <= P.xorshift_unit(0) < 1.0
