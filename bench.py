"""Benchmark: decode and prefill throughput of the Qwen3-4B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B]

Prints ONE JSON line.  ``value`` is decoded tokens per second at the default batch (8), timed on
the device over K single-token steps after W warm-up steps; ``e2e`` is the same through
``Model.generate_batch`` with host token ids in and out (``e2e_b1``: at batch 1); ``prefill`` is a
2,048-token prompt, with a breakdown of one instrumented step by kernel class; ``points`` holds
decode at batch 1 and 64; ``decode_points`` holds, for batch 1, 8 and 64, a point right after the
prompts (lengths uniform in [128, 2048]) and a point with every sequence at 4,080 to 4,096 tokens,
the end of the benchmark's context, each with its step time, mean context, bytes and fraction of
the memory bandwidth; ``roofline`` relates the main decode step to the memory bandwidth.  The model
has the layer sizes of the benchmark configuration with random weights and synthetic token ids;
``--layers`` runs fewer layers of the same sizes (``config`` names both).

``--model 8b`` and ``--model 32b`` run the workloads named for those shapes instead (an unequal
batch of 16 prompts of 64 to 4,096 tokens with 256 decode steps and an 8,192-token prompt; decode
at batch 1 and 32 behind 2,048-token prompts and a 2,048-token prompt) and print one line each.

The work is one GPU's: for ``--gpus`` above 1 it says so and exits with 2.  The reference arm
(``--impl reference``) is unavailable: the reference is a Rust workspace, there is no Rust
toolchain or network here to build it, and its CUDA path runs none of its kernels for bfloat16
weights.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# layer sizes of the benchmark configuration (Qwen3-4B shape)
CONFIG_4B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=2560,
                 num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=9728,
                 vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                 max_position_embeddings=40960)
# the other shapes of the same architecture, for runs beside the benchmark (``--model``)
SHAPES = {
    "4b": CONFIG_4B,
    "8b": dict(CONFIG_4B, hidden_size=4096, intermediate_size=12288, tie_word_embeddings=False),
    "32b": dict(CONFIG_4B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600,
                tie_word_embeddings=False),
}
FULL_LAYERS = 36
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS)
    src = "fallback"
    if os.path.isfile(path):
        try:
            with open(path) as f:
                data = json.load(f)
            for k in out:
                if isinstance(data.get(k), (int, float)) and data[k] > 0:
                    out[k] = float(data[k])
            src = "measured"
        except (OSError, ValueError):
            pass
    out["source"] = src
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], 0, set()
        for p in self.samples:
            try:
                sm.append(int(float(p[0])))
                mx = max(mx, int(float(p[1])))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def decode_run(model, batch, steps, warmup, seed, lens=None):
    """One varlen prefill (untimed), then warm-up and timed single-token steps; device-timed.
    ``lens``: the prompts' lengths (default: uniform in [128, 2048])."""
    import torch
    from builderforce_inference_b200.engine.engine import SequenceStep
    eng = model.engine
    g = torch.Generator().manual_seed(seed)
    vocab = eng.spec.vocab_size
    if lens is None:
        lens = torch.randint(128, 2049, (batch,), generator=g).tolist()
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]
    slots = [eng.acquire() for _ in range(batch)]
    eng.step([SequenceStep(s, p, ()) for s, p in zip(slots, prompts)], check=False)
    toks = [int(t) for t in torch.randint(0, vocab, (batch,), generator=g).tolist()]

    def one():
        return eng.step([SequenceStep(s, (t,), (0,)) for s, t in zip(slots, toks)], check=False)

    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    bytes_before = eng.decode_step_bytes()
    launches0 = eng.kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches = eng.kernel_launches() - launches0
    step_bytes = (bytes_before + eng.decode_step_bytes()) / 2.0
    eng.check_status()
    ctx_mean = sum(eng.length(s) for s in slots) / batch
    for s in slots:
        eng.release(s)
    return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launches,
            "step_bytes": step_bytes, "ctx_mean": ctx_mean}


def point(run, pk):
    """A decode point as it goes into the line: rate, step time, mean context at the end of the
    timed steps, the bytes a step has to read and their rate as a fraction of the copy bandwidth."""
    gbs = run["step_bytes"] / (run["ms_per_step"] / 1e3) / 1e9
    return {"tok_s": round(run["tok_s"], 1), "ms_per_step": round(run["ms_per_step"], 4),
            "ctx_mean": round(run["ctx_mean"], 1), "step_bytes": int(run["step_bytes"]),
            "gb_s": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 4)}


def e2e_run(model, batch, steps, warmup, seed):
    """The same through ``Model.generate_batch``: host ids in, host ids out, every step."""
    import torch
    from builderforce_inference_b200 import SampleParams
    g = torch.Generator().manual_seed(seed)
    vocab = model.n_vocab()
    lens = torch.randint(128, 2049, (batch,), generator=g).tolist()
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]
    stamps = []
    model.stepper.on_tokens = lambda n: stamps.append((time.perf_counter(), n))
    try:
        model.generate_batch(prompts, SampleParams(max_tokens=warmup + steps + 1), ignore_eos=True)
    finally:
        model.stepper.on_tokens = None
    # stamps[0] follows the prefill; stamps[i] follows decode step i
    t0, t1 = stamps[warmup][0], stamps[warmup + steps][0]
    tokens = sum(n for _, n in stamps[warmup + 1:warmup + steps + 1])
    return {"tok_s": tokens / (t1 - t0), "h2d": model.stepper.h2d_bytes, "d2h": model.stepper.d2h_bytes}


def prefill_flops(c, layers, lens):
    """Floating-point operations of one prompt step over sequences of ``lens`` tokens, logits at
    each sequence's last token."""
    h, d, nq, nkv, inter = c["hidden_size"], c["head_dim"], c["num_attention_heads"], c["num_key_value_heads"], \
        c["intermediate_size"]
    tokens = sum(lens)
    per_layer = 2 * tokens * (h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * inter)
    attn = sum(4 * nq * d * n * (n + 1) / 2 for n in lens)
    return layers * (per_layer + attn) + 2 * h * c["vocab_size"] * len(lens)


KERNEL_CLASSES = (("products", ("gemm", "skinny")), ("attention", ("attention",)))


def prefill_breakdown(eng, step):
    """One instrumented prompt step: a CUDA event before and after every kernel, so the kernels run
    strictly one after the other (an event between two launches ends their overlap).  Returns the
    milliseconds by kernel class, the time between kernels (the GPU waiting for the host), and the
    whole of the instrumented step, which is therefore longer than a plain one."""
    import torch
    from builderforce_inference_b200.kernels import library as L
    marks, open_ = [], []

    def watch(name, what):
        if what == "begin":
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            open_.append(e)
        else:
            e0 = open_.pop()
            if what == "end":
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record()
                marks.append((name, e0, e1))

    torch.cuda.synchronize()
    L.set_call_observer(watch)
    try:
        step()
    finally:
        L.set_call_observer(None)
    torch.cuda.synchronize()
    out = {"products_ms": 0.0, "attention_ms": 0.0, "other_ms": 0.0}
    for name, e0, e1 in marks:
        cls = next((c for c, keys in KERNEL_CLASSES if any(k in name for k in keys)), "other")
        out[cls + "_ms"] += e0.elapsed_time(e1)
    whole = marks[0][1].elapsed_time(marks[-1][2]) if marks else 0.0
    out["gaps_ms"] = max(0.0, whole - sum(out.values()))
    out = {k: round(v, 3) for k, v in out.items()}
    out["instrumented_ms"] = round(whole, 3)
    out["kernels"] = len(marks)
    return out


def prefill_run(model, tokens, reps, layers, c=None, lens=None, breakdown=False):
    import torch
    from builderforce_inference_b200.engine.engine import SequenceStep
    eng = model.engine
    g = torch.Generator().manual_seed(99)
    lens = lens or [tokens]
    prompts = [torch.randint(0, eng.spec.vocab_size, (n,), generator=g).tolist() for n in lens]
    times = []

    def run_once():
        slots = [eng.acquire() for _ in prompts]
        try:
            eng.step([SequenceStep(s, p, (len(p) - 1,)) for s, p in zip(slots, prompts)], check=False)
        finally:
            torch.cuda.synchronize()
            for s in slots:
                eng.release(s)

    for i in range(reps + 2):
        slots = [eng.acquire() for _ in prompts]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        eng.step([SequenceStep(s, p, (len(p) - 1,)) for s, p in zip(slots, prompts)], check=False)
        e1.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(e0.elapsed_time(e1))
        for s in slots:
            eng.release(s)
    ms = statistics.median(times)
    out = {"ms": ms, "tok_s": sum(lens) / (ms / 1e3), "flops": prefill_flops(c or CONFIG_4B, layers, lens)}
    if breakdown:
        out["breakdown"] = prefill_breakdown(eng, run_once)
    return out


def side_run(a, model, shape_cfg, pk) -> dict:
    """The workloads named for the 8B and 32B shapes, beside the benchmark: one line of numbers."""
    layers = a.layers
    out = {}
    if a.shape_name == "8b":
        lens = [64 + round(i * (4096 - 64) / 15) for i in range(16)]            # 64 .. 4,096, then 256 more each
        pf = prefill_run(model, 0, 3, layers, shape_cfg, lens=lens)
        out["unequal16_prefill"] = {"tokens": sum(lens), "ms": round(pf["ms"], 3), "tok_s": round(pf["tok_s"], 1),
                                    "frac": round(pf["flops"] / (pf["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
        decode_run(model, 16, 2, 3, seed=3, lens=lens)
        out["unequal16_decode256"] = point(decode_run(model, 16, 256, 3, seed=4, lens=lens), pk)
        pf = prefill_run(model, 8192, 3, layers, shape_cfg)
        out["prefill_8192"] = {"tokens": 8192, "ms": round(pf["ms"], 3), "tok_s": round(pf["tok_s"], 1),
                               "frac": round(pf["flops"] / (pf["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    else:
        for b in (1, 32):
            decode_run(model, b, 2, 3, seed=3, lens=[2048] * b)
            out[f"decode_b{b}_prompt2048"] = point(decode_run(model, b, 32, 3, seed=4, lens=[2048] * b), pk)
        pf = prefill_run(model, 2048, 3, layers, shape_cfg)
        out["prefill_2048"] = {"tokens": 2048, "ms": round(pf["ms"], 3), "tok_s": round(pf["tok_s"], 1),
                               "frac": round(pf["flops"] / (pf["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    return out


KERNEL_SHAPES = {"qkv": (6144, 2560, 0), "o": (2560, 4096, 1), "gateup": (19456, 2560, 2), "down": (2560, 9728, 1),
                 "head": (151936, 2560, 0)}


def kernel_run(a) -> int:
    """Times ONE kernel on one workload (for profiling under ncu and for the files in profiles/):
    ``--kernel skinny_gemm|gemm_tcgen05 --shape qkv|o|gateup|down|head --rows M`` or
    ``--kernel attention_decode|attention_prefill|attention_prefill_tcgen05 --rows B_or_T --ctx C``
    (``--seqs N``: N prompts of --rows tokens each),
    ``--kernel qk_norm_rope --rows T``, ``--kernel weight_stream --shape S [--stages R] [--ksplit Z]`` (the
    matrix read once through the few-row products' TMA rings and nothing else: the floor under
    them).  Weights rotate over enough copies to exceed L2.  Prints one JSON line."""
    import torch
    from builderforce_inference_b200.kernels import fast_ops
    dev = torch.device("cuda:0")
    reps = a.steps
    if a.kernel == "weight_stream":
        # the floor under the few-row products: the matrix read once through their TMA rings, nothing else
        n, k, _ = KERNEL_SHAPES[a.shape]
        copies = max(2, int(400e6 // (n * k * 2)) + 1)
        ws = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]

        stages = a.stages
        # K split as the few-row product plans it: enough blocks for two per SM, at least 8 k blocks each
        tiles, kblocks, n_sm = (n + 127) // 128, (k + 63) // 64, fast_ops.sm_count(dev)
        ksplit = a.ksplit or (max(1, min(8, 2 * n_sm // tiles, kblocks // 8)) if tiles * 2 <= 2 * n_sm else 1)

        def one(i):
            if not fast_ops.weight_stream(ws[i % copies], stages=stages, ksplit=ksplit):
                raise SystemExit("weight_stream does not take this matrix")
        bytes_moved, flops = n * k * 2, 0.0
        what = {"shape": a.shape, "N": n, "K": k, "stages": stages, "ksplit": ksplit}
    elif a.kernel in ("skinny_gemm", "gemm_tcgen05"):
        n, k, epi = KERNEL_SHAPES[a.shape]
        m = a.rows
        copies = max(2, int(400e6 // (n * k * 2)) + 1)
        ws = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
        out = torch.zeros(m, n // 2 if epi == 2 else n, device=dev, dtype=torch.float32 if epi == 1 else torch.bfloat16)
        fn = fast_ops.skinny_gemm if a.kernel == "skinny_gemm" else fast_ops.gemm_tcgen05

        def one(i):
            if not fn(x, ws[i % copies], out, epi):
                raise SystemExit(f"{a.kernel} does not take M={m} N={n} K={k}")
        bytes_moved, flops = n * k * 2, 2.0 * m * n * k
        what = {"shape": a.shape, "M": m, "N": n, "K": k, "epilogue": epi}
    elif a.kernel == "qk_norm_rope":
        # q/k norm + rotation + cache write of one prompt of --rows tokens
        from builderforce_inference_b200.cache import KVView
        from builderforce_inference_b200.kernels import ops
        from builderforce_inference_b200.parts.rotary import rotary_table
        c = CONFIG_4B
        nq, nkv, d = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        t = a.rows
        blocks = (t + 63) // 64
        table = torch.arange(blocks, dtype=torch.int32, device=dev).reshape(1, blocks)
        copies = 4
        kvs = [KVView(torch.zeros(blocks, nkv, 64, d, device=dev, dtype=torch.bfloat16),
                      torch.zeros(blocks, nkv, 64, d, device=dev, dtype=torch.bfloat16), table, nkv, d, None)
               for _ in range(copies)]
        qkvs = [torch.randn(t, (nq + 2 * nkv) * d, device=dev, dtype=torch.bfloat16) for _ in range(copies)]
        norm_w = torch.ones(d, device=dev, dtype=torch.bfloat16)
        rope = rotary_table(c["rope_theta"], d, t, dev)
        pos = torch.arange(t, dtype=torch.int32, device=dev)
        slot = torch.zeros(t, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)

        def one(i):
            ops.qk_norm_rope_cache(qkvs[i % copies], nq, nkv, d, norm_w, norm_w, c["rms_norm_eps"], rope, d, pos, slot,
                                   kvs[i % copies], ops.FLAG_WRITE_CACHE, status)
        bytes_moved = t * (2 * nq + 3 * nkv) * d * 2          # q read and written, k and v read and written to the cache
        flops = 0.0
        what = {"tokens": t, "q_heads": nq, "kv_heads": nkv, "head_dim": d}
    else:
        from builderforce_inference_b200.cache import KVView
        c = CONFIG_4B
        nq, nkv, d = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        decode = a.kernel == "attention_decode"
        n_seq = a.rows if decode else a.seqs
        t_new = 1 if decode else a.rows
        ctx_len = a.ctx if decode else t_new
        blocks = (ctx_len + 63) // 64
        n_pages = n_seq * blocks
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).reshape(n_seq, blocks)
        cache_bytes = n_pages * nkv * 64 * d * 2 * 2
        copies = max(2, int(400e6 // cache_bytes) + 1) if decode else 1
        kvs = [KVView(torch.randn(n_pages, nkv, 64, d, device=dev, dtype=torch.bfloat16),
                      torch.randn(n_pages, nkv, 64, d, device=dev, dtype=torch.bfloat16), table, nkv, d, None)
               for _ in range(copies)]
        q = torch.randn(n_seq * t_new, (nq + 2 * nkv) * d, device=dev, dtype=torch.bfloat16)
        out = torch.empty(n_seq * t_new, nq * d, device=dev, dtype=torch.bfloat16)

        class Ctx:
            pass
        ctx = Ctx()
        from builderforce_inference_b200.engine.context import Workspace
        ctx.workspace = Workspace(dev)
        ctx.n_seqs, ctx.n_tokens, ctx.max_seq_tokens = n_seq, n_seq * t_new, t_new
        ctx.seq_slot = torch.arange(n_seq, dtype=torch.int32, device=dev)
        ctx.seq_start = torch.full((n_seq,), ctx_len - t_new, dtype=torch.int32, device=dev)
        ctx.cu_seqlens = torch.arange(0, (n_seq + 1) * t_new, t_new, dtype=torch.int32, device=dev)
        ctx.total_pages = torch.tensor([n_seq * blocks], dtype=torch.int32, device=dev)
        fn = {"attention_decode": fast_ops.attention_decode_bf16, "attention_prefill": fast_ops.attention_prefill_bf16,
              "attention_prefill_tcgen05": fast_ops.attention_prefill_tcgen05_bf16}[a.kernel]
        def one(i):
            if not fn(ctx, q, out, kvs[i % copies], nq, d ** -0.5):
                raise SystemExit(f"{a.kernel} does not take this shape")
        bytes_moved = n_seq * ctx_len * 2 * nkv * d * 2
        flops = 4.0 * nq * d * n_seq * (ctx_len if decode else t_new * (t_new + 1) / 2)
        what = {"seqs": n_seq, "new_tokens": t_new, "context": ctx_len, "q_heads": nq, "kv_heads": nkv, "head_dim": d}
    for i in range(3):
        one(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if a.eager:                             # plain launches (for captures under ncu)
        e0.record()
        for i in range(reps):
            one(i)
        e1.record()
    else:
        graph = torch.cuda.CUDAGraph()      # one graph of all launches: no host gaps between short kernels
        with torch.cuda.graph(graph):
            for i in range(reps):
                one(i)
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / reps
    pk = peaks()
    print(json.dumps({"kernel": a.kernel, **what, "us": round(us, 2), "launches": reps,
                      "GB_s": round(bytes_moved / us / 1e3, 1), "TFLOP_s": round(flops / us / 1e6, 1),
                      "frac_hbm": round(bytes_moved / us / 1e3 / pk["hbm_gbs"], 3),
                      "frac_bf16": round(flops / us / 1e6 / pk["bf16_tflops"], 3), "peaks": pk["source"],
                      "note": ("plain launches: short kernels include launch gaps" if a.eager else
                               "launches replayed from one CUDA graph") + ", operands rotating over more than L2"}))
    return 0


TRACE_UNITS = [("core", "elementwise"), ("core", "sampling"), ("core", "gemm_simt"), ("fast", "gemm_tcgen05"),
               ("fast", "attention_decode"), ("fast", "attention_prefill_tcgen05")]


def timeline_run(a) -> int:
    """``--timeline``: one decode step's kernels on the GPU's own clock.  The libraries are built
    with time stamps in the kernels (BFI_B200_TRACE=1, set below before the package loads): the first
    thread of every block records when it starts, when its wait for the kernel before it returns and
    (products and attention) when it ends.  Prints, for the kernels of ``--timeline-layer``, the
    first and last of each stamp in microseconds from the step's start: where the step's time goes
    between the kernels, which no serialised profile shows."""
    import ctypes

    import numpy as np
    import torch
    from builderforce_inference_b200 import Model
    from builderforce_inference_b200.engine.engine import SequenceStep
    from builderforce_inference_b200.kernels.library import library
    layers = a.layers or 12
    cfg = dict(SHAPES[a.shape_name], num_hidden_layers=layers)
    model = Model.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=a.batch * CONTEXT, max_seq_len=CONTEXT, max_batch=a.batch)
    eng = model.engine
    g = torch.Generator().manual_seed(2)
    lens = torch.randint(128, 2049, (a.batch,), generator=g).tolist()
    slots = [eng.acquire() for _ in lens]
    eng.step([SequenceStep(s, torch.randint(0, 1000, (n,), generator=g).tolist(), ()) for s, n in zip(slots, lens)], check=False)

    def one():
        eng.step([SequenceStep(s, (5,), (0,)) for s in slots], check=False)

    if a.timeline_prompt:
        # a prompt step instead: --timeline-prompt tokens, eager launches
        for s in slots:
            eng.release(s)
        prompt = torch.randint(0, 1000, (a.timeline_prompt,), generator=g).tolist()

        def one():                                                     # noqa: F811
            s = eng.acquire()
            eng.step([SequenceStep(s, prompt, (len(prompt) - 1,))], check=False)
            torch.cuda.synchronize()
            eng.release(s)

    for _ in range(6):
        one()
    torch.cuda.synchronize()
    cap = 1 << 18

    def read_all():
        recs = []
        for libname, unit in TRACE_UNITS:
            fn = getattr(library(libname).lib, f"bfi_trace_read_{unit}")
            fn.restype = ctypes.c_long
            buf = np.zeros(2 * cap, dtype=np.uint64)
            n = fn(buf.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(cap))
            for i in range(n):
                key, t = int(buf[2 * i]), int(buf[2 * i + 1])
                recs.append((key >> 32, (key >> 28) & 0xF, t, unit))
        return recs

    read_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    one()
    e1.record()
    torch.cuda.synchronize()
    recs = read_all()
    grids = {}
    for gid, what, t, unit in recs:
        d = grids.setdefault(gid, {"unit": unit, "t": {0: [], 1: [], 2: []}})
        d["t"][what].append(t)
    order = sorted(grids)
    t00 = min(t for _, _, t, _ in recs)
    per_layer = (len(order) - 3) // layers if layers else 9     # beside the layers: embedding, final norm, head
    first = 1 + a.timeline_layer * per_layer
    what = f"one prompt step of {a.timeline_prompt} tokens" if a.timeline_prompt else f"one decode step, batch {a.batch}"
    print(f"{what}, {layers} layers of the {a.shape_name} shape: {e0.elapsed_time(e1):.3f} ms with the stamps; "
          f"{len(order)} kernels, {per_layer} per layer; layer {a.timeline_layer}:")
    print("| # | source file | blocks | first start | last start | first wait over | last wait over | first end | last end |")
    print("|---|---|---|---|---|---|---|---|---|")

    def us(xs, fn):
        return f"{(fn(xs) - t00) / 1e3:.2f}" if xs else "-"

    for i, gid in enumerate(order):
        if not first <= i < first + per_layer + 1:
            continue
        d = grids[gid]
        print(f"| {i} | {d['unit']} | {len(d['t'][0])} | {us(d['t'][0], min)} | {us(d['t'][0], max)} | {us(d['t'][1], min)} | "
              f"{us(d['t'][1], max)} | {us(d['t'][2], min)} | {us(d['t'][2], max)} |")
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--timeline", action="store_true", help="print one decode step's kernels on the GPU's clock (see timeline_run)")
    ap.add_argument("--timeline-layer", type=int, default=6)
    ap.add_argument("--timeline-prompt", type=int, default=0, help="with --timeline: a prompt step of this many tokens instead")
    ap.add_argument("--seqs", type=int, default=1, help="kernel mode, prompt attention: prompts of --rows tokens each")
    ap.add_argument("--kernel", default=None, choices=["skinny_gemm", "gemm_tcgen05", "weight_stream", "qk_norm_rope", "attention_decode",
                                                       "attention_prefill", "attention_prefill_tcgen05"],
                    help="time one kernel instead of the model (see kernel_run)")
    ap.add_argument("--shape", default="qkv", choices=sorted(KERNEL_SHAPES))
    ap.add_argument("--eager", action="store_true", help="with --kernel: plain launches instead of one CUDA graph")
    ap.add_argument("--stages", type=int, default=6, help="--kernel weight_stream: 16 KB tiles in a block's ring (1..12)")
    ap.add_argument("--ksplit", type=int, default=0, help="--kernel weight_stream: ranges of K (0: as the product plans it)")
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", dest="shape_name", default="4b", choices=sorted(SHAPES),
                    help="layer sizes: the benchmark's Qwen3-4B shape, or the 8B / 32B shapes for runs beside it")
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers of the same sizes")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace: no Rust toolchain or network here to build it, "
                          "pip cannot install it, and its CUDA backend runs no kernel for bf16 weights"}))
        return 0
    if a.timeline:
        os.environ["BFI_B200_TRACE"] = "1"
        return timeline_run(a)
    if a.kernel is not None:
        return kernel_run(a)
    if a.gpus != 1:
        print(f"bench.py measures one GPU: this library has no multi-GPU path (asked for --gpus {a.gpus})")
        return 2
    warmup = max(3, a.warmup)

    import torch
    from builderforce_inference_b200 import Model
    pk = peaks()
    shape_cfg = SHAPES[a.shape_name]
    full_layers = shape_cfg["num_hidden_layers"]
    if a.layers is None:
        a.layers = full_layers
    cfg = dict(shape_cfg, num_hidden_layers=a.layers)
    max_batch = a.batch if a.no_points else max(64, a.batch)
    t_load = time.time()
    model = Model.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=max(max_batch * CONTEXT, 16384),
                              max_seq_len=max(CONTEXT, 8192) if a.shape_name == "8b" else CONTEXT, max_batch=max_batch)
    print(f"[bench] model ready in {time.time() - t_load:.1f} s", file=sys.stderr, flush=True)

    if a.shape_name != "4b":
        clocks = ClockSampler()
        clocks.start()
        numbers = side_run(a, model, shape_cfg, pk)
        print(json.dumps({"workloads": f"qwen3-{a.shape_name}-shape, builder-run beside the benchmark", "dtype": "bf16",
                          "layers": a.layers, "layers_full": full_layers, "peaks": pk["source"], **numbers,
                          "clocks": clocks.stop()}))
        return 0

    # untimed: compile, capture graphs, size workspaces
    decode_run(model, a.batch, 2, 3, seed=1)
    clocks = ClockSampler()
    clocks.start()
    main_run = decode_run(model, a.batch, a.steps, warmup, seed=2)
    e2e = e2e_run(model, a.batch, a.steps, warmup, seed=2)
    points, prefill, decode_points, e2e_b1 = {}, None, {}, None
    if not a.no_points:
        deep_steps = 12                                   # 3 warm-up + 12 timed steps end at 4,095 of 4,096
        deep_start = CONTEXT - (3 + deep_steps) - 1    # 4,080
        for b in sorted({1, a.batch, 64}):
            if b == a.batch:
                after = main_run
            else:
                decode_run(model, b, 2, 3, seed=3)         # untimed: graph capture for this batch size
                after = decode_run(model, b, min(a.steps, 32), warmup, seed=4)
            if b in (1, 64):
                points[f"decode_b{b}"] = round(after["tok_s"], 1)
            decode_points[f"b{b}_after_prompt"] = point(after, pk)
            deep = decode_run(model, b, deep_steps, 3, seed=5, lens=[deep_start] * b)
            decode_points[f"b{b}_ctx{CONTEXT}"] = point(deep, pk)
        e1 = e2e_run(model, 1, min(a.steps, 32), warmup, seed=4)          # the prompt of the batch-1 point above
        e2e_b1 = {"value": round(e1["tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e1["h2d"],
                  "d2h_bytes_per_step": e1["d2h"]}
        pf = prefill_run(model, PREFILL_TOKENS, 10, a.layers, shape_cfg, breakdown=True)          # median of 10
        prefill = {"value": round(pf["tok_s"], 1), "tokens": PREFILL_TOKENS, "ms": round(pf["ms"], 3),
                   "frac": round(pf["flops"] / (pf["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                   "breakdown": pf["breakdown"]}
    clk = clocks.stop()

    achieved = main_run["step_bytes"] / (main_run["ms_per_step"] / 1e3) / 1e9
    c = shape_cfg
    line = {
        "metric": f"Qwen3-{a.shape_name.upper()} bf16 decode tok/s at batch {a.batch} (batch 1/64 in points; prefill tok/s at 2,048 tokens)",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights",
        "config": {"model": f"qwen3-{a.shape_name}-shape", "layers": a.layers, "layers_full": full_layers,
                   "hidden": c["hidden_size"], "q_heads": c["num_attention_heads"],
                   "kv_heads": c["num_key_value_heads"], "head_dim": c["head_dim"],
                   "intermediate": c["intermediate_size"], "vocab": c["vocab_size"], "tied_head": bool(c["tie_word_embeddings"]),
                   "global_batch": a.batch, "seq_len": CONTEXT, "prompt_len": "uniform[128,2048]",
                   "ctx_mean": round(main_run["ctx_mean"], 1), "parallelism": "single-gpu",
                   "l2": "weights read per step exceed L2", "peaks": pk["source"]},
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "clocks": clk,
    }
    if prefill is not None:
        line["prefill"] = prefill
        line["points"] = points
        line["decode_points"] = decode_points
        line["e2e_b1"] = e2e_b1
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
