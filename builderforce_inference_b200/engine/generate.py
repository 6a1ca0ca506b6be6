"""The generation loop above the step function.

Requests (prompts as token ids) are served in batches, one batch after another until none is
left.  The prompts of a batch run in ONE step, whatever their lengths; then every live sequence
takes one token per shared step.  A sequence that ends (stop token, token budget, context
limit) gives its slot and pages back at once and the others go on, so the shared step count of a
batch is the longest sequence's, not the sum (crates/bfi-runtime/src/engine/mod.rs:297-337,
560-580).

Rules kept from the reference (engine/mod.rs:349-462): the first token is sampled from the
prompt's last-position logits; a stop token ends the sequence and is not appended; the budget is
``max_tokens``, or what the context still holds when that is 0.  One difference: a token that
exhausts the budget is not forwarded, since nothing would read its logits.

The loop talks to the model only through ``acquire / release / step / sample``, so its decisions
are tested on the CPU against a toy stepper.

A stepper that can feed a step with the ids the sampler left on the device (``pipelined``) is driven
one step ahead: step k+1 is launched before the host has read token k, so the host's work (the
copy back, the stop test, packing the next step) runs beside the GPU instead of between its
steps.  What the host then learns about token k (a stop token) can only end a sequence, and a
sequence that ended takes at most one step too many, whose token is dropped; the results are
those of the plain loop, token for token.  Penalties need the host's history of every sequence
before sampling, so they keep the plain loop.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..sampling.params import SampleParams

MAX_SHARED_STEPS = 1_000_000     # the reference's safety cap (engine/mod.rs:323-325)


@dataclass
class Generated:
    tokens: List[int]
    finish_reason: str            # "stop" | "length"


@dataclass
class BatchReport:
    results: List[Generated]
    shared_steps: int = 0         # single-token steps summed over the batches
    generated_tokens: int = 0
    batches: int = 0


@dataclass
class _Live:
    request: int
    slot: int
    prompt_len: int
    budget: int
    history: List[int]
    generated: List[int] = field(default_factory=list)
    alive: bool = True


def token_budget(prompt_len: int, max_tokens: int, max_seq_len: int) -> int:
    """How many tokens a request may generate: ``max_tokens`` (0 = no limit of its own), capped by
    the room the context leaves after the prompt."""
    room = max_seq_len - prompt_len
    if room < 0:
        raise ValueError(f"context_exceeded: a prompt of {prompt_len} tokens passes the limit of {max_seq_len}")
    return room if max_tokens == 0 else min(max_tokens, room)


def plan_batches(prompt_lens: Sequence[int], budgets: Sequence[int], max_batch: int, page_tokens: int,
                 n_pages: int) -> List[List[int]]:
    """Cut the queue of requests into batches, in order: at most ``max_batch`` requests each, and
    no more than the cache can hold if every request of the batch runs to its budget."""
    batches: List[List[int]] = []
    cur: List[int] = []
    pages = 0
    for i, (p, b) in enumerate(zip(prompt_lens, budgets)):
        need = (p + max(b - 1, 0) + page_tokens - 1) // page_tokens
        need = max(need, 1)
        if need > n_pages:
            raise ValueError(f"request {i} needs {need} cache pages of {page_tokens} tokens; the cache has {n_pages}")
        if cur and (len(cur) == max_batch or pages + need > n_pages):
            batches.append(cur)
            cur, pages = [], 0
        cur.append(i)
        pages += need
    if cur:
        batches.append(cur)
    return batches


def _run_pipelined(stepper, live: List[_Live], prompts, params: SampleParams, stop, results, on_step) -> int:
    """One batch, one step ahead of the host.  The stepper provides, beside the plain interface:

    ``sample_start(handle, params, requests, steps) -> ticket``: launch the sampling and the copy of
    the ids to the host, without waiting;
    ``sample_wait(ticket) -> list[int]``: the ids, once they have arrived;
    ``decode_sampled(slots, ticket, rows) -> handle``: one step in which sequence ``i`` takes the id
    the ticket holds at ``rows[i]``, fed on the device.

    Returns the number of shared single-token steps whose tokens were used."""
    handle = stepper.prefill([s.slot for s in live], [prompts[s.request] for s in live])
    ticket = stepper.sample_start(handle, params, [s.request for s in live], [0] * len(live))
    members = list(live)              # the sequences whose ids the ticket holds, row by row
    launched = shared = 0
    first = True
    while True:
        # the step after the ids in flight, for everyone those ids cannot be the last of
        go = [(i, s) for i, s in enumerate(members) if s.alive and len(s.generated) + 1 < s.budget]
        nxt = None
        if go and launched < MAX_SHARED_STEPS - 1:
            handle = stepper.decode_sampled([s.slot for _, s in go], ticket, [i for i, _ in go])
            launched += 1
            nxt = stepper.sample_start(handle, params, [s.request for _, s in go],
                                       [len(s.generated) + 1 for _, s in go])
        picked = stepper.sample_wait(ticket)
        used = 0
        for s, tok in zip(members, picked):
            if not s.alive:
                continue                       # ended a step ago: this id belongs to nobody
            used += 1
            tok = int(tok)
            if tok in stop:
                results[s.request] = Generated(s.generated, "stop")
            else:
                s.generated.append(tok)
                s.history.append(tok)
                if len(s.generated) < s.budget:
                    continue
                results[s.request] = Generated(s.generated, "length")
            s.alive = False
            stepper.release(s.slot)
        if not first and used:
            shared += 1
            if on_step is not None:
                on_step(shared, used)
        first = False
        if nxt is None:
            break
        members, ticket = [s for _, s in go], nxt
    for s in live:                             # the cap on shared steps was reached
        if s.alive:
            results[s.request] = Generated(s.generated, "length")
            s.alive = False
            stepper.release(s.slot)
    return shared


def generate_batch(stepper, prompts: Sequence[Sequence[int]], params: SampleParams,
                   stop_ids: Sequence[int] = (), max_batch: int = 64,
                   on_step: Optional[Callable[[int, int], None]] = None) -> BatchReport:
    """Generate for every prompt.  ``stepper`` provides:

    ``max_seq_len``, ``page_tokens``, ``n_pages``;
    ``acquire() -> slot``, ``release(slot)``;
    ``prefill(slots, prompts) -> handle`` and ``decode(slots, tokens) -> handle``: run a step and
    return something ``sample`` understands (logits at each sequence's last position);
    ``sample(handle, params, requests, steps, histories) -> list[int]``.
    """
    params.validate()
    stop = set(int(s) for s in stop_ids)
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"request {i}: empty prompt")
    budgets = [token_budget(len(p), params.max_tokens, stepper.max_seq_len) for p in prompts]
    results: List[Optional[Generated]] = [None] * len(prompts)
    report = BatchReport(results=[])
    order = plan_batches([len(p) for p in prompts], budgets, max_batch, stepper.page_tokens, stepper.n_pages)
    for batch in order:
        report.batches += 1
        live: List[_Live] = []
        for i in batch:
            if budgets[i] == 0:
                results[i] = Generated([], "length")
                continue
            live.append(_Live(request=i, slot=stepper.acquire(), prompt_len=len(prompts[i]),
                              budget=budgets[i], history=list(prompts[i])))
        if not live:
            continue
        try:
            if getattr(stepper, "pipelined", False) and not params.has_penalties:
                report.shared_steps += _run_pipelined(stepper, live, prompts, params, stop, results, on_step)
                continue
            handle = stepper.prefill([s.slot for s in live], [prompts[s.request] for s in live])
            shared = 0
            while live:
                hist = [s.history for s in live] if params.has_penalties else None
                picked = stepper.sample(handle, params, [s.request for s in live],
                                        [len(s.generated) for s in live], hist)
                still: List[_Live] = []
                for s, tok in zip(live, picked):
                    tok = int(tok)
                    if tok in stop:
                        results[s.request] = Generated(s.generated, "stop")
                        s.alive = False
                        stepper.release(s.slot)
                        continue
                    s.generated.append(tok)
                    s.history.append(tok)
                    if len(s.generated) >= s.budget:
                        results[s.request] = Generated(s.generated, "length")
                        s.alive = False
                        stepper.release(s.slot)
                        continue
                    still.append(s)
                live = still
                if not live:
                    break
                shared += 1
                if shared >= MAX_SHARED_STEPS:
                    for s in live:
                        results[s.request] = Generated(s.generated, "length")
                        s.alive = False
                        stepper.release(s.slot)
                    live = []
                    break
                handle = stepper.decode([s.slot for s in live], [s.generated[-1] for s in live])
                if on_step is not None:
                    on_step(shared, len(live))
            report.shared_steps += shared
        except BaseException:
            for s in live:
                if not s.alive:
                    continue
                try:
                    stepper.release(s.slot)
                except Exception:
                    pass
            raise
    report.results = [r if r is not None else Generated([], "length") for r in results]
    report.generated_tokens = sum(len(r.tokens) for r in report.results)
    return report
