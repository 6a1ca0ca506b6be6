"""Command line, in the manner of the reference's ``bfi`` (crates/bfi/src/cli.rs:31-125):

    python -m builderforce_inference_b200 run   <model> [prompt]      one-shot, or a prompt loop without [prompt]
    python -m builderforce_inference_b200 bench <model> --pp 512 --tg 128 [--batch B --ctx C --reps R]
    python -m builderforce_inference_b200 random <config.json> <folder> --seed N
    python -m builderforce_inference_b200 replay --model DIR --dtype D --out DIR --max-tokens N

``<model>`` is a folder with config.json and model.safetensors, or, with ``--random-weights SEED``,
a config.json whose model is made from that seed in device memory.  A prompt is a list of token ids
separated by spaces or commas (tokenizers are outside this library), given on the command line or
in a file (``--prompt-ids FILE``: one prompt per line, served as one batch); generated ids are
printed the same way.  Stop ids come from the folder (generation_config.json, then config.json)
unless ``--stop-id`` names them.  The cache is sized in tokens (``--max-tokens-cached``) or from a
byte budget (``--cache-gib``).  ``run`` samples with the reference's defaults (greedy, 256 tokens:
crates/bfi/src/commands.rs:79, crates/bfi-runtime/src/sample.rs:33-49) unless told otherwise.
``bench`` reports ``pp{N}`` and ``tg{N}`` tokens per second as a table
(crates/bfi/src/commands.rs:250-294), timed on the device after a warm-up; ``--batch`` runs that many
sequences together, ``--ctx`` starts the generation test from prompts of that length and ``--reps``
repeats each test and reports the median.  ``replay`` is trace replay, the same code as
``bin/trace_run``.
"""
from __future__ import annotations

import argparse
import json
import re
import sys


def _ids(text: str):
    parts = [p for p in re.split(r"[,\s]+", text.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit(f"a prompt is a list of token ids, got {text!r}")


def _engine_flags(p: argparse.ArgumentParser) -> None:
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--max-seq-len", type=int, default=None, help="cap on one sequence's context")
    p.add_argument("--max-tokens-cached", type=int, default=65536,
                   help="tokens the cache holds over all live sequences")
    p.add_argument("--cache-gib", type=float, default=None,
                   help="size the cache from this many GiB instead (keys, values and per-sequence state)")
    p.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="<model> is a config.json; make its weights from this seed instead of loading a folder")
    p.add_argument("--max-batch", type=int, default=64)
    p.add_argument("--device", default="cuda:0")


def _sample_flags(p: argparse.ArgumentParser) -> None:
    p.add_argument("--max-tokens", "--max-new-tokens", dest="max_tokens", type=int, default=256,
                   help="tokens to generate per prompt; 0: until the context is full")
    p.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--min-p", type=float, default=0.0)
    p.add_argument("--repeat-penalty", type=float, default=1.0)
    p.add_argument("--presence-penalty", type=float, default=0.0)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--stop-id", type=int, action="append", default=None,
                   help="stop token id (repeatable); default: eos_token_id of config.json")
    p.add_argument("--ignore-eos", action="store_true")


def _params(a):
    from .sampling import SampleParams
    return SampleParams(max_tokens=a.max_tokens, temperature=a.temperature, top_k=a.top_k, top_p=a.top_p,
                        min_p=a.min_p, repeat_penalty=a.repeat_penalty, presence_penalty=a.presence_penalty,
                        seed=a.seed)


def _load(a):
    from .engine.api import Model
    kw = dict(dtype=a.dtype, max_tokens=a.max_tokens_cached, max_seq_len=a.max_seq_len, max_batch=a.max_batch,
              device=a.device)
    if a.cache_gib is not None:
        kw.update(cache_bytes=int(a.cache_gib * (1 << 30)), cache_slots=a.max_batch)
    if a.random_weights is not None:
        from .config import read_json
        print(f"random weights for {a.model}, seed {a.random_weights}", file=sys.stderr, flush=True)
        return Model.from_random(read_json(a.model), a.random_weights, **kw)
    print(f"loading {a.model}", file=sys.stderr, flush=True)
    return Model.load(a.model, **kw)


def _prompts_of_file(path: str):
    with open(path, "r", encoding="utf-8") as f:
        prompts = [_ids(line) for line in f if line.strip()]
    if not prompts:
        raise SystemExit(f"{path}: no prompt (one list of token ids per line)")
    return prompts


def cmd_run(a) -> int:
    if a.prompt is not None and a.prompt_ids is not None:
        raise SystemExit("give a prompt on the command line or --prompt-ids FILE, not both")
    model = _load(a)
    params = _params(a)
    if a.prompt_ids is not None:
        for out in model.generate_batch(_prompts_of_file(a.prompt_ids), params, a.stop_id, a.ignore_eos):
            print(" ".join(str(t) for t in out))
        return 0
    if a.prompt is not None:
        out = model.generate(_ids(a.prompt), params, a.stop_id, a.ignore_eos)
        print(" ".join(str(t) for t in out))
        return 0
    print("token ids per line; an empty line, /bye or /exit quits", file=sys.stderr)
    while True:
        sys.stdout.write("> ")
        sys.stdout.flush()
        line = sys.stdin.readline()
        if not line:
            break
        t = line.strip()
        if not t or t in ("/bye", "/exit"):
            break
        out = model.generate(_ids(t), params, a.stop_id, a.ignore_eos)
        print(" ".join(str(x) for x in out))
    return 0


def cmd_bench(a) -> int:
    import statistics

    import torch
    from .sampling import SampleParams
    model = _load(a)
    vocab = model.n_vocab()
    g = torch.Generator().manual_seed(0)
    batch, reps = max(a.batch, 1), max(a.reps, 1)

    def prompts(n):
        return [torch.randint(0, vocab, (max(n, 1),), generator=g).tolist() for _ in range(batch)]

    pp_prompts = prompts(a.pp)
    if a.prompt_len_max:
        lens = torch.randint(max(a.prompt_len_min, 1), a.prompt_len_max + 1, (batch,), generator=g).tolist()
        tg_prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]
    else:
        tg_prompts = prompts(a.ctx if a.ctx else 2)

    def timed(ps, n_new):
        model.generate_batch(ps, SampleParams(max_tokens=n_new), ignore_eos=True)       # warm-up
        times = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            model.generate_batch(ps, SampleParams(max_tokens=n_new), ignore_eos=True)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / 1e3)
        return statistics.median(times)

    pp_s = timed(pp_prompts, 1)
    # generation is timed without its prompts: the same prompts with one new token are taken off
    tg_s = timed(tg_prompts, a.tg + 1) - timed(tg_prompts, 1)
    label = f"B200 sm_100a {a.dtype}" + (f" b{batch}" if batch > 1 else "") + (f" ctx{a.ctx}" if a.ctx else "")
    rows = [("pp%d" % a.pp, batch * a.pp / pp_s), ("tg%d" % a.tg, batch * a.tg / max(tg_s, 1e-9))]
    if a.json:
        print(json.dumps({name: ts for name, ts in rows}))
        return 0
    print("| model | backend | test | t/s |")
    print("|---|---|---|---|")
    for name, ts in rows:
        print(f"| {a.model} | {label} | {name} | {ts:.2f} |")
    return 0


def cmd_replay(a) -> int:
    from .engine.replay import replay
    return replay(a)


def cmd_random(a) -> int:
    import torch
    from .config import read_json
    from .weights import write_model_folder
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[a.store_dtype]
    write_model_folder(read_json(a.config), a.seed, a.folder, dt)
    print(a.folder)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="builderforce_inference_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run", help="generate for one prompt, or read prompts line by line")
    r.add_argument("model")
    r.add_argument("prompt", nargs="?", default=None)
    r.add_argument("--prompt-ids", default=None, metavar="FILE",
                   help="prompts from a file, one list of token ids per line, served as one batch")
    _engine_flags(r)
    _sample_flags(r)
    r.set_defaults(fn=cmd_run)
    b = sub.add_parser("bench", help="pp/tg tokens per second")
    b.add_argument("model")
    b.add_argument("--pp", type=int, default=512)
    b.add_argument("--tg", type=int, default=128)
    b.add_argument("--json", action="store_true")
    b.add_argument("--batch", type=int, default=1, help="sequences run together")
    b.add_argument("--ctx", type=int, default=0, help="generate from prompts of this many tokens (0: two tokens)")
    b.add_argument("--reps", type=int, default=1, help="timed repetitions of each test (the median is reported)")
    b.add_argument("--prompt-len-min", type=int, default=0,
                   help="with --prompt-len-max: the generation test starts from prompts of unequal lengths, uniform between the two")
    b.add_argument("--prompt-len-max", type=int, default=0)
    _engine_flags(b)
    b.set_defaults(fn=cmd_bench)
    w = sub.add_parser("random", help="write a model folder with random weights")
    w.add_argument("config")
    w.add_argument("folder")
    w.add_argument("--seed", type=int, default=0)
    w.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    w.set_defaults(fn=cmd_random)
    t = sub.add_parser("replay", help="trace replay: token ids step by step from standard input, logits to files")
    from .engine.replay import add_arguments
    add_arguments(t)
    t.set_defaults(fn=cmd_replay)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
