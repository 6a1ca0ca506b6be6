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
        assert not eng.use_graphs                      # the toy mixer is not graph-safe: never captured
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
    finally:
        undo()
    from builderforce_inference_b200 import registered_architectures
    assert registered_architectures() == ["Qwen3ForCausalLM", "qwen3"]
