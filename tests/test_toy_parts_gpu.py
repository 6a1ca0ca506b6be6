"""A model the framework has never heard of, defined entirely in this file: a mixer with a state of
its own (fixed size per sequence), registered as a part; an architecture registered by name whose
layer order is a list that names layers twice and lets one run read another run's cache.  It is
written to a folder, loaded, and stepped whole, token by token and in unequal batches through the
unchanged engine, and compared with a plain restatement below."""
import json
import os
import tempfile

import pytest
import torch

from helpers import rel_err
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

WIDTH, HEADS, KV, D, INNER, VOCAB, EPS, THETA = 48, 4, 2, 16, 80, 97, 1e-5, 1e4
TOY_CONFIG = {"architectures": ["ToyStateLM"], "model_type": "toy_state", "vocab_size": VOCAB, "width": WIDTH,
              "decay": 0.75, "max_position_embeddings": 256}


def register():
    """Registers the toy mixer and the toy architecture; returns a function that removes them."""
    from builderforce_inference_b200 import Architecture, register_architecture, unregister_architecture
    from builderforce_inference_b200.parts import (MIXERS, LayerSpec, Mixer, ModelSpec, ParamSpec, PartSpec, RunSpec,
                                                   StateNeed)

    class RunningStateMixer(Mixer):
        """s_t = decay * s_{t-1} + h_t (per sequence, float32 state of ``width``); adds s_t @ mix^T."""

        def __init__(self, width, decay):
            self.width, self.decay = width, decay

        def param_specs(self):
            return {"mix": ParamSpec((self.width, self.width))}

        def load(self, tensors, runtime):
            self.mix = tensors["mix"].float()

        def cache_need(self):
            return StateNeed((self.width,), "float32")

        def forward(self, ctx, h, residual, run):
            row = 0
            for slot, n in zip(ctx.host_seq_slot, ctx.host_seq_tokens):
                s = run.state[slot]
                for t in range(n):
                    s.mul_(self.decay).add_(h[row + t].float())
                    residual[row + t] += s @ self.mix.t()
                row += n

    MIXERS.register("running_state", RunningStateMixer)

    def describe(config):
        norm = PartSpec("rms", {"width": WIDTH, "eps": EPS})
        ffn = PartSpec("gated_mlp", {"width": WIDTH, "inner": INNER})
        rot = PartSpec("rotary", {"theta": THETA, "rot_dim": D})

        def att(own_kv):
            return PartSpec("attention", {"width": WIDTH, "n_heads": HEADS, "n_kv_heads": KV, "head_dim": D,
                                          "position": rot, "own_kv": own_kv})

        def layer(i, mixer, mixer_names):
            names = {"norm1.weight": f"blocks.{i}.n1", "norm2.weight": f"blocks.{i}.n2",
                     "ffn.gate_proj": f"blocks.{i}.gate", "ffn.up_proj": f"blocks.{i}.up",
                     "ffn.down_proj": f"blocks.{i}.down"}
            names.update({f"mixer.{k}": f"blocks.{i}.{k}" for k in mixer_names})
            return LayerSpec(PartSpec("prenorm", {"norm1": norm, "mixer": mixer, "norm2": norm, "ffn": ffn}), names)

        layers = (layer(0, att(True), ["q_proj", "k_proj", "v_proj", "o_proj"]),
                  layer(1, PartSpec("running_state", {"width": WIDTH, "decay": config["decay"]}), ["mix"]),
                  layer(2, att(False), ["q_proj", "o_proj"]))
        # layer 0 runs twice (two caches of its own), the state layer twice (two states), and the
        # last run has no keys of its own: it reads the cache the first run wrote
        schedule = (RunSpec(0), RunSpec(1), RunSpec(0), RunSpec(1), RunSpec(2, cache_of=0))
        return ModelSpec(vocab_size=config["vocab_size"], width=WIDTH, embedding_name="emb", layers=layers,
                         schedule=schedule, final_norm=norm, final_norm_names={"weight": "out_norm"},
                         head_name="head", max_positions=config["max_position_embeddings"])

    register_architecture(("toy_state", "ToyStateLM"), Architecture("toy_state", dict, describe))

    def undo():
        unregister_architecture("toy_state", "ToyStateLM")
        MIXERS.unregister("running_state")
    return undo


def plain_toy(w, tokens, decay):
    """Whole-sequence restatement of the toy model."""
    t = len(tokens)
    pos = list(range(t))
    x = P.embedding(w["emb"], tokens)

    def ffn(x, i):
        h = P.rms_norm(x, w[f"blocks.{i}.n2"], EPS)
        return x + P.linear(w[f"blocks.{i}.down"], P.swiglu(P.linear(w[f"blocks.{i}.gate"], h),
                                                           P.linear(w[f"blocks.{i}.up"], h)))

    def kv(h, i):
        k = P.rope_neox(P.linear(w[f"blocks.{i}.k_proj"], h).reshape(t, KV, D), pos, THETA)
        return k, P.linear(w[f"blocks.{i}.v_proj"], h).reshape(t, KV, D)

    def attend(x, i, h, k, v):
        q = P.rope_neox(P.linear(w[f"blocks.{i}.q_proj"], h).reshape(t, HEADS, D), pos, THETA)
        return x + P.linear(w[f"blocks.{i}.o_proj"], P.attention(q, k, v).reshape(t, HEADS * D))

    def state_layer(x):
        h = P.rms_norm(x, w["blocks.1.n1"], EPS)
        s = torch.zeros(WIDTH)
        ys = []
        for r in range(t):
            s = decay * s + h[r]
            ys.append(s @ w["blocks.1.mix"].t())
        return x + torch.stack(ys)

    h = P.rms_norm(x, w["blocks.0.n1"], EPS)
    k0, v0 = kv(h, 0)
    x = ffn(attend(x, 0, h, k0, v0), 0)
    x = ffn(state_layer(x), 1)
    h = P.rms_norm(x, w["blocks.0.n1"], EPS)
    k, v = kv(h, 0)
    x = ffn(attend(x, 0, h, k, v), 0)
    x = ffn(state_layer(x), 1)
    h = P.rms_norm(x, w["blocks.2.n1"], EPS)
    x = ffn(attend(x, 2, h, k0, v0), 2)
    return P.linear(w["head"], P.rms_norm(x, w["out_norm"], EPS))


def test_toy_architecture_with_state_repeated_layers_and_a_shared_cache():
    from builderforce_inference_b200 import write_model_folder
    from builderforce_inference_b200.engine.engine import Engine, SequenceStep as S
    undo = register()
    try:
        folder = tempfile.mkdtemp(prefix="bfi_toy_")
        write_model_folder(TOY_CONFIG, 3, folder, torch.float32)
        assert json.load(open(os.path.join(folder, "config.json")))["model_type"] == "toy_state"
        w = {k: v.float() for k, v in P.read_safetensors(os.path.join(folder, "model.safetensors")).items()}
        assert "blocks.1.mix" in w and "blocks.2.k_proj" not in w
        eng = Engine.load(folder, dtype="float32", max_tokens=1024)
        # the toy mixer is not graph-safe: its two runs stay as written, the attention layers around
        # them are replayed from CUDA graphs
        assert eng.use_graphs and [safe for safe, _ in eng.decoder.stages()] == [True, False, True, False, True]
        assert len(eng.cache.kv_groups) == 1 and eng.cache.kv_groups[0].runs == [0, 2]
        assert len(eng.cache.state_groups) == 1 and eng.cache.state_groups[0].runs == [1, 3]
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, VOCAB, (n,), generator=g).tolist() for n in (70, 9, 33)]
        refs = [plain_toy(w, p, TOY_CONFIG["decay"]) for p in prompts]
        # whole
        for p, r in zip(prompts, refs):
            s = eng.acquire()
            assert rel_err(eng.step([S(s, p, list(range(len(p))))]).cpu(), r) < 1e-4
            eng.release(s)
        # an unequal batch: prefixes together, then one token each; slots reused from above, so a
        # state that is not reset on acquire would show
        slots = [eng.acquire() for _ in prompts]
        pre = [40, 5, 30]
        lg = eng.step([S(s, p[:k], list(range(k))) for s, p, k in zip(slots, prompts, pre)]).cpu().clone()
        got, o = [[] for _ in prompts], 0
        for i, k in enumerate(pre):
            got[i].append(lg[o:o + k])
            o += k
        pos = list(pre)
        live = [0, 1, 2]
        while live:
            lg = eng.step([S(slots[i], [prompts[i][pos[i]]], [0]) for i in live]).cpu().clone()
            for j, i in enumerate(live):
                got[i].append(lg[j:j + 1])
                pos[i] += 1
            for i in list(live):
                if pos[i] == len(prompts[i]):
                    eng.release(slots[i])
                    live.remove(i)
        for i, r in enumerate(refs):
            assert rel_err(torch.cat(got[i]), r) < 1e-4, i
        eng.cache.check()
        # the same token by token without any graph gives the same logits
        plain = Engine.load(folder, dtype="float32", max_tokens=1024, use_graphs=False)
        a, b = eng.acquire(), plain.acquire()
        for t in prompts[2][:12]:
            assert torch.equal(eng.step([S(a, [t], [0])]), plain.step([S(b, [t], [0])]))
    finally:
        undo()
    from builderforce_inference_b200 import registered_architectures
    assert registered_architectures() == ["Qwen3ForCausalLM", "qwen3"]


# ------------------------------------------------------------------------------------------------
# A second unknown model: a feed-forward with routing (one of several experts per token, weighted
# by the router's probability), a position encoding with code of its own (adjacent pairs instead
# of rotate-half, so the attention kernels cannot fuse it), and a norm that subtracts the mean.
# All three are defined here and registered as parts; nothing in the framework's files changes.
# ------------------------------------------------------------------------------------------------
R_WIDTH, R_HEADS, R_KV, R_D, R_INNER, R_EXPERTS, R_VOCAB, R_EPS, R_THETA = 40, 5, 1, 16, 24, 3, 61, 1e-6, 500.0
ROUTED_CONFIG = {"architectures": ["ToyRoutedLM"], "model_type": "toy_routed", "vocab_size": R_VOCAB,
                 "n_experts": R_EXPERTS, "max_position_embeddings": 128}


def register_routed():
    from builderforce_inference_b200 import Architecture, register_architecture, unregister_architecture
    from builderforce_inference_b200.parts import (FEED_FORWARDS, NORMS, POSITION_ENCODINGS, FeedForward, LayerSpec, ModelSpec,
                                                   Norm, ParamSpec, PartSpec, PositionEncoding, RunSpec)

    class RoutedFeedForward(FeedForward):
        """Top-1 routing: expert e = argmax(router h); x += p_e * down_e(silu(gate_e h) * up_e h)."""

        def __init__(self, width, inner, n_experts):
            self.width, self.inner, self.n_experts = width, inner, n_experts

        def param_specs(self):
            specs = {"router": ParamSpec((self.n_experts, self.width))}
            for e in range(self.n_experts):
                specs[f"experts.{e}.gate"] = ParamSpec((self.inner, self.width))
                specs[f"experts.{e}.up"] = ParamSpec((self.inner, self.width))
                specs[f"experts.{e}.down"] = ParamSpec((self.width, self.inner))
            return specs

        def load(self, tensors, runtime):
            self.w = {k: v.float() for k, v in tensors.items()}

        def forward(self, ctx, h, residual):
            n = ctx.n_tokens
            x = h[:n].float()
            probs = torch.softmax(x @ self.w["router"].t(), dim=-1)           # router logits and softmax in float32
            top_p, top_e = probs.max(dim=-1)
            for e in range(self.n_experts):
                rows = (top_e == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                xe = x[rows]
                g, u = xe @ self.w[f"experts.{e}.gate"].t(), xe @ self.w[f"experts.{e}.up"].t()
                y = (torch.nn.functional.silu(g) * u) @ self.w[f"experts.{e}.down"].t()
                residual[rows] += top_p[rows, None] * y

    class AdjacentPairRotary(PositionEncoding):
        """Pairs (2i, 2i+1) turn by pos * theta^(-2i/d): not a rotate-half rotation, so it is applied
        by its own code between the norms and the cache write."""

        def __init__(self, theta, rot_dim):
            self.theta, self.rot_dim = theta, rot_dim

        def prepare(self, runtime, max_positions):
            i = torch.arange(self.rot_dim // 2, dtype=torch.float64)
            inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.rot_dim)
            ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv[None, :]
            self.cos, self.sin = ang.cos().float().to(runtime.device), ang.sin().float().to(runtime.device)

        def apply(self, ctx, q, k):
            pos = ctx.token_pos[:ctx.n_tokens].long()
            c, s = self.cos[pos][:, None, :], self.sin[pos][:, None, :]
            for t in (q, k):
                x = t[:ctx.n_tokens].float()
                a, b = x[..., 0::2], x[..., 1::2]
                out = torch.stack([a * c - b * s, a * s + b * c], dim=-1).reshape(x.shape)
                t[:ctx.n_tokens] = out.to(t.dtype)

    class CenteredNorm(Norm):
        """y = (x - mean) * rsqrt(var + eps) * w."""

        def __init__(self, width, eps):
            self.width, self.eps = width, eps

        def param_specs(self):
            return {"weight": ParamSpec((self.width,), "norm")}

        def load(self, tensors, runtime):
            self.weight = tensors["weight"].float()

        def forward(self, ctx, x, rows=None, tag="norm.out"):
            src = x if rows is None else x[rows.long()]
            out = ctx.rows(tag, self.width, n_rows=src.shape[0])
            v = src.float()
            v = v - v.mean(dim=-1, keepdim=True)
            out.copy_((v * torch.rsqrt(v.pow(2).mean(dim=-1, keepdim=True) + self.eps) * self.weight).to(out.dtype))
            return out

    FEED_FORWARDS.register("routed_mlp", RoutedFeedForward)
    POSITION_ENCODINGS.register("adjacent_rotary", AdjacentPairRotary)
    NORMS.register("centered", CenteredNorm)

    def describe(config):
        rms = PartSpec("rms", {"width": R_WIDTH, "eps": R_EPS})
        centered = PartSpec("centered", {"width": R_WIDTH, "eps": R_EPS})
        att = PartSpec("attention", {"width": R_WIDTH, "n_heads": R_HEADS, "n_kv_heads": R_KV, "head_dim": R_D,
                                     "position": PartSpec("adjacent_rotary", {"theta": R_THETA, "rot_dim": R_D})})
        routed = PartSpec("routed_mlp", {"width": R_WIDTH, "inner": R_INNER, "n_experts": config["n_experts"]})
        dense = PartSpec("gated_mlp", {"width": R_WIDTH, "inner": R_INNER})

        def layer(i, norm, ffn, ffn_names):
            names = {"norm1.weight": f"l{i}.n1", "norm2.weight": f"l{i}.n2"}
            names.update({f"mixer.{k}": f"l{i}.att.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj")})
            names.update({f"ffn.{k}": f"l{i}.ffn.{k}" for k in ffn_names})
            return LayerSpec(PartSpec("prenorm", {"norm1": norm, "mixer": att, "norm2": norm, "ffn": ffn}), names)

        routed_names = ["router"] + [f"experts.{e}.{m}" for e in range(config["n_experts"]) for m in ("gate", "up", "down")]
        layers = (layer(0, centered, routed, routed_names), layer(1, rms, dense, ["gate_proj", "up_proj", "down_proj"]))
        return ModelSpec(vocab_size=config["vocab_size"], width=R_WIDTH, embedding_name="emb", layers=layers,
                         schedule=(RunSpec(0), RunSpec(1)), final_norm=centered, final_norm_names={"weight": "out_norm"},
                         head_name="head", max_positions=config["max_position_embeddings"])

    register_architecture(("toy_routed", "ToyRoutedLM"), Architecture("toy_routed", dict, describe))

    def undo():
        unregister_architecture("toy_routed", "ToyRoutedLM")
        FEED_FORWARDS.unregister("routed_mlp")
        POSITION_ENCODINGS.unregister("adjacent_rotary")
        NORMS.unregister("centered")
    return undo


ROUTED_TO = set()


def plain_routed(w, tokens):
    t = len(tokens)
    x = P.embedding(w["emb"], tokens)

    def centered(v, weight):
        v = v - v.mean(dim=-1, keepdim=True)
        return v * torch.rsqrt(v.pow(2).mean(dim=-1, keepdim=True) + R_EPS) * weight

    def adjacent(v):                                     # [t, heads, d]
        i = torch.arange(R_D // 2, dtype=torch.float64)
        ang = torch.arange(t, dtype=torch.float64)[:, None] * torch.pow(torch.tensor(R_THETA, dtype=torch.float64), -2.0 * i / R_D)
        c, s = ang.cos().float()[:, None, :], ang.sin().float()[:, None, :]
        a, b = v[..., 0::2], v[..., 1::2]
        return torch.stack([a * c - b * s, a * s + b * c], dim=-1).reshape(v.shape)

    def attend(x, i, norm):
        h = norm(x, w[f"l{i}.n1"])
        q = adjacent(P.linear(w[f"l{i}.att.q_proj"], h).reshape(t, R_HEADS, R_D))
        k = adjacent(P.linear(w[f"l{i}.att.k_proj"], h).reshape(t, R_KV, R_D))
        v = P.linear(w[f"l{i}.att.v_proj"], h).reshape(t, R_KV, R_D)
        return x + P.linear(w[f"l{i}.att.o_proj"], P.attention(q, k, v).reshape(t, R_HEADS * R_D))

    x = attend(x, 0, centered)
    h = centered(x, w["l0.n2"])
    probs = torch.softmax(P.linear(w["l0.ffn.router"], h), dim=-1)
    rows = []
    for r in range(t):
        e = int(probs[r].argmax())
        ROUTED_TO.add(e)
        hr = h[r:r + 1]
        y = P.linear(w[f"l0.ffn.experts.{e}.down"], P.swiglu(P.linear(w[f"l0.ffn.experts.{e}.gate"], hr),
                                                              P.linear(w[f"l0.ffn.experts.{e}.up"], hr)))
        rows.append(probs[r, e] * y)
    x = x + torch.cat(rows)
    rms = lambda v, weight: P.rms_norm(v, weight, R_EPS)
    x = attend(x, 1, rms)
    h = rms(x, w["l1.n2"])
    x = x + P.linear(w["l1.ffn.down_proj"], P.swiglu(P.linear(w["l1.ffn.gate_proj"], h), P.linear(w["l1.ffn.up_proj"], h)))
    return P.linear(w["head"], centered(x, w["out_norm"]))


def test_toy_architecture_with_routing_another_position_encoding_and_another_norm():
    from builderforce_inference_b200 import write_model_folder
    from builderforce_inference_b200.engine.engine import Engine, SequenceStep as S
    undo = register_routed()
    try:
        folder = tempfile.mkdtemp(prefix="bfi_toy_routed_")
        write_model_folder(ROUTED_CONFIG, 5, folder, torch.float32)
        w = {k: v.float() for k, v in P.read_safetensors(os.path.join(folder, "model.safetensors")).items()}
        assert "l0.ffn.experts.2.down" in w and "l1.ffn.gate_proj" in w
        eng = Engine.load(folder, dtype="float32", max_tokens=512)
        assert not eng.use_graphs                      # the toy parts are not graph-safe
        g = torch.Generator().manual_seed(2)
        prompts = [torch.randint(0, R_VOCAB, (n,), generator=g).tolist() for n in (66, 7, 21)]
        refs = [plain_routed(w, p) for p in prompts]
        assert len(ROUTED_TO) >= 2, "the prompts must reach more than one expert, or the routing is not tested"
        for p, r in zip(prompts, refs):
            s = eng.acquire()
            assert rel_err(eng.step([S(s, p, list(range(len(p))))]).cpu(), r) < 1e-4
            eng.release(s)
        # unequal batch, then token by token
        slots = [eng.acquire() for _ in prompts]
        pre = [50, 3, 20]
        lg = eng.step([S(s, p[:k], [k - 1]) for s, p, k in zip(slots, prompts, pre)]).cpu().clone()
        for i, k in enumerate(pre):
            assert rel_err(lg[i:i + 1], refs[i][k - 1:k]) < 1e-4
        pos = list(pre)
        live = [0, 1, 2]
        while live:
            lg = eng.step([S(slots[i], [prompts[i][pos[i]]], [0]) for i in live]).cpu().clone()
            for j, i in enumerate(live):
                assert rel_err(lg[j:j + 1], refs[i][pos[i]:pos[i] + 1]) < 1e-4, (i, pos[i])
                pos[i] += 1
            for i in list(live):
                if pos[i] == len(prompts[i]):
                    eng.release(slots[i])
                    live.remove(i)
        eng.cache.check()
    finally:
        undo()
    from builderforce_inference_b200 import registered_architectures
    assert registered_architectures() == ["Qwen3ForCausalLM", "qwen3"]


# ------------------------------------------------------------------------------------------------
# A third unknown model: a mixer that keeps keys and values AND a fixed-size state (attention
# whose output is joined by a running sum of its input).  Its cache need is a pair; the run's
# cache then carries both entries.  The layer runs twice, so there are two such pairs.
# ------------------------------------------------------------------------------------------------
H_WIDTH, H_HEADS, H_KV, H_D, H_INNER, H_VOCAB, H_EPS, H_THETA, H_DECAY = 56, 3, 3, 32, 72, 83, 1e-6, 3e3, 0.6
HYBRID_CONFIG = {"architectures": ["ToyHybridLM"], "model_type": "toy_hybrid", "vocab_size": H_VOCAB,
                 "max_position_embeddings": 192}


def register_hybrid():
    from builderforce_inference_b200 import Architecture, register_architecture, unregister_architecture
    from builderforce_inference_b200.parts import KVNeed, LayerSpec, MIXERS, ModelSpec, ParamSpec, PartSpec, RunSpec, StateNeed
    from builderforce_inference_b200.parts.attention import Attention

    class AttentionWithRunningSum(Attention):
        """out = attention(h) + s_t @ mix^T with s_t = decay * s_{t-1} + h_t: keys and values in
        pages, s in a per-sequence state of ``width`` floats."""
        graph_safe = False

        def __init__(self, decay, **kw):
            super().__init__(**kw)
            self.decay = decay

        def param_specs(self):
            specs = dict(super().param_specs())
            specs["mix"] = ParamSpec((self.width, self.width))
            return specs

        def load(self, tensors, runtime):
            super().load(tensors, runtime)
            self.mix = tensors["mix"].float()

        def cache_need(self):
            return (KVNeed(self.n_kv_heads, self.head_dim, self.window), StateNeed((self.width,), "float32"))

        def forward(self, ctx, h, residual, run):
            assert isinstance(run.entries[1], torch.Tensor) and run.entries[0] is run.kv and run.entries[1] is run.state
            super().forward(ctx, h, residual, run)
            row = 0
            for slot, n in zip(ctx.host_seq_slot, ctx.host_seq_tokens):
                s = run.state[slot]
                for t in range(n):
                    s.mul_(self.decay).add_(h[row + t].float())
                    residual[row + t] += s @ self.mix.t()
                row += n

    MIXERS.register("attention_running_sum", AttentionWithRunningSum)

    def describe(config):
        norm = PartSpec("rms", {"width": H_WIDTH, "eps": H_EPS})
        ffn = PartSpec("gated_mlp", {"width": H_WIDTH, "inner": H_INNER})
        rot = PartSpec("rotary", {"theta": H_THETA, "rot_dim": H_D})
        att = {"width": H_WIDTH, "n_heads": H_HEADS, "n_kv_heads": H_KV, "head_dim": H_D, "position": rot}

        def layer(i, mixer, extra):
            names = {"norm1.weight": f"b{i}.n1", "norm2.weight": f"b{i}.n2", "ffn.gate_proj": f"b{i}.gate",
                     "ffn.up_proj": f"b{i}.up", "ffn.down_proj": f"b{i}.down"}
            names.update({f"mixer.{k}": f"b{i}.{k}" for k in ["q_proj", "k_proj", "v_proj", "o_proj"] + extra})
            return LayerSpec(PartSpec("prenorm", {"norm1": norm, "mixer": mixer, "norm2": norm, "ffn": ffn}), names)

        layers = (layer(0, PartSpec("attention_running_sum", dict(att, decay=H_DECAY)), ["mix"]),
                  layer(1, PartSpec("attention", att), []))
        return ModelSpec(vocab_size=config["vocab_size"], width=H_WIDTH, embedding_name="emb", layers=layers,
                         schedule=(RunSpec(0), RunSpec(1), RunSpec(0)), final_norm=norm,
                         final_norm_names={"weight": "out_norm"}, head_name=None,
                         max_positions=config["max_position_embeddings"])

    register_architecture(("toy_hybrid", "ToyHybridLM"), Architecture("toy_hybrid", dict, describe))

    def undo():
        unregister_architecture("toy_hybrid", "ToyHybridLM")
        MIXERS.unregister("attention_running_sum")
    return undo


def plain_hybrid(w, tokens):
    t = len(tokens)
    pos = list(range(t))
    x = P.embedding(w["emb"], tokens)

    def block(x, i, running_sum):
        h = P.rms_norm(x, w[f"b{i}.n1"], H_EPS)
        q = P.rope_neox(P.linear(w[f"b{i}.q_proj"], h).reshape(t, H_HEADS, H_D), pos, H_THETA)
        k = P.rope_neox(P.linear(w[f"b{i}.k_proj"], h).reshape(t, H_KV, H_D), pos, H_THETA)
        v = P.linear(w[f"b{i}.v_proj"], h).reshape(t, H_KV, H_D)
        x = x + P.linear(w[f"b{i}.o_proj"], P.attention(q, k, v).reshape(t, H_HEADS * H_D))
        if running_sum:
            s = torch.zeros(H_WIDTH)
            ys = []
            for r in range(t):
                s = H_DECAY * s + h[r]
                ys.append(s @ w[f"b{i}.mix"].t())
            x = x + torch.stack(ys)
        h = P.rms_norm(x, w[f"b{i}.n2"], H_EPS)
        return x + P.linear(w[f"b{i}.down"], P.swiglu(P.linear(w[f"b{i}.gate"], h), P.linear(w[f"b{i}.up"], h)))

    x = block(block(block(x, 0, True), 1, False), 0, True)
    return P.linear(w["emb"], P.rms_norm(x, w["out_norm"], H_EPS))


def test_toy_mixer_with_keys_and_values_and_a_state_of_its_own():
    from builderforce_inference_b200 import write_model_folder
    from builderforce_inference_b200.engine.engine import Engine, SequenceStep as S, StepError
    undo = register_hybrid()
    try:
        folder = tempfile.mkdtemp(prefix="bfi_toy_hybrid_")
        write_model_folder(HYBRID_CONFIG, 8, folder, torch.float32)
        w = {k: v.float() for k, v in P.read_safetensors(os.path.join(folder, "model.safetensors")).items()}
        eng = Engine.load(folder, dtype="float32", max_tokens=1024)
        assert eng.use_graphs and [safe for safe, _ in eng.decoder.stages()] == [True, False, True, False, True]
        # the three runs' keys and values share one group; the two hybrid runs' states another
        assert [g.keys for g in eng.cache.kv_groups] == [[(0, 0), (1, 0), (2, 0)]]
        assert [g.keys for g in eng.cache.state_groups] == [[(0, 1), (2, 1)]]
        assert eng.cache.state_bytes_per_slot() == 2 * H_WIDTH * 4
        g = torch.Generator().manual_seed(4)
        prompts = [torch.randint(0, H_VOCAB, (n,), generator=g).tolist() for n in (90, 13, 41)]
        refs = [plain_hybrid(w, p) for p in prompts]
        for p, r in zip(prompts, refs):
            s = eng.acquire()
            assert rel_err(eng.step([S(s, p, list(range(len(p))))]).cpu(), r) < 1e-4
            eng.release(s)
        slots = [eng.acquire() for _ in prompts]
        pre = [70, 4, 30]
        lg = eng.step([S(s, p[:k], [k - 1]) for s, p, k in zip(slots, prompts, pre)]).cpu().clone()
        for i, k in enumerate(pre):
            assert rel_err(lg[i:i + 1], refs[i][k - 1:k]) < 1e-4
        pos = list(pre)
        live = [0, 1, 2]
        while live:
            lg = eng.step([S(slots[i], [prompts[i][pos[i]]], [0]) for i in live]).cpu().clone()
            for j, i in enumerate(live):
                assert rel_err(lg[j:j + 1], refs[i][pos[i]:pos[i] + 1]) < 1e-4, (i, pos[i])
                pos[i] += 1
            for i in list(live):
                if pos[i] == len(prompts[i]):
                    if i == 0:
                        with pytest.raises(StepError, match="rewind unsupported.*fixed size"):
                            eng.rewind(slots[i], 5)          # a state cannot be wound back
                    eng.release(slots[i])
                    live.remove(i)
        eng.cache.check()
    finally:
        undo()
    from builderforce_inference_b200 import registered_architectures
    assert registered_architectures() == ["Qwen3ForCausalLM", "qwen3"]
