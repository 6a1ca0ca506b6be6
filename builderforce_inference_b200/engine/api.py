"""The Python entry point, in the manner of the reference's ``Engine``
(crates/bfi-runtime/src/engine/mod.rs:195-337): ``load``, ``generate``, ``generate_batch``,
``generate_greedy_trace`` and the counters of the last call — on token ids, since tokenizers
are outside this library.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..cache.pages import PAGE_TOKENS
from ..sampling.params import SampleParams
from ..sampling.sampler import Sampler
from .engine import Engine, SequenceStep
from .generate import BatchReport, generate_batch


@dataclass
class GreedyTrace:
    """Greedy ids plus the logits the last step produced (engine/mod.rs:269-290)."""

    token_ids: List[int]
    last_logits: torch.Tensor


@dataclass
class _SampleTicket:
    """Ids the sampler left on the device, on their way to a pinned host buffer."""

    ids: torch.Tensor             # int32 [n] on the device
    host: torch.Tensor            # pinned int32, at least n
    n: int
    arrived: torch.cuda.Event


class EngineStepper:
    """What the generation loop needs from an engine: slots, steps and sampling, with host token
    ids in and out.  Every step copies its inputs from pinned host memory and reads the chosen
    ids back into pinned host memory.  ``pipelined``: a single-token step can take its ids straight
    from the sampler's device buffer, so the loop may launch it before the host has read them."""

    pipelined = True

    def __init__(self, engine: Engine):
        self.engine = engine
        self.max_seq_len = engine.max_seq_len
        self.page_tokens = PAGE_TOKENS
        self.n_pages = engine.cache.n_pages
        self.sampler = Sampler(engine.device, engine.spec.vocab_size)
        self._host_ids = torch.empty(1024, dtype=torch.int32, pin_memory=True)
        self._ticket_bufs = [torch.empty(1024, dtype=torch.int32, pin_memory=True) for _ in range(3)]
        self._ticket_turn = 0
        self.last_logits: Optional[torch.Tensor] = None
        self.on_tokens = None          # called with the number of ids after each read-back
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def acquire(self) -> int:
        return self.engine.acquire()

    def release(self, slot: int) -> None:
        self.engine.release(slot)

    def prefill(self, slots: Sequence[int], prompts: Sequence[Sequence[int]]):
        seqs = [SequenceStep(s, p, (len(p) - 1,)) for s, p in zip(slots, prompts)]
        self.last_logits = self.engine.step(seqs, check=False)
        return self.last_logits

    def decode(self, slots: Sequence[int], tokens: Sequence[int]):
        seqs = [SequenceStep(s, (t,), (0,)) for s, t in zip(slots, tokens)]
        self.last_logits = self.engine.step(seqs, check=False)
        self.h2d_bytes = self.engine.last_h2d_bytes
        return self.last_logits

    def sample(self, handle, params: SampleParams, requests, steps, histories) -> List[int]:
        ids = self.sampler.sample(handle, params, requests, steps, histories)
        n = ids.numel()
        if n > self._host_ids.numel():
            self._host_ids = torch.empty(2 * n, dtype=torch.int32, pin_memory=True)
        host = self._host_ids[:n]
        host.copy_(ids, non_blocking=True)
        torch.cuda.current_stream(self.engine.device).synchronize()
        self.d2h_bytes = n * 4
        if self.on_tokens is not None:
            self.on_tokens(n)
        return host.tolist()


    # ---- one step ahead of the host ----------------------------------------------------
    def sample_start(self, handle, params: SampleParams, requests, steps) -> _SampleTicket:
        ids = self.sampler.sample(handle, params, requests, steps, None)
        n = ids.numel()
        i = self._ticket_turn
        self._ticket_turn = (i + 1) % len(self._ticket_bufs)
        if self._ticket_bufs[i].numel() < n:
            self._ticket_bufs[i] = torch.empty(2 * n, dtype=torch.int32, pin_memory=True)
        host = self._ticket_bufs[i]
        host[:n].copy_(ids, non_blocking=True)
        arrived = torch.cuda.Event()
        arrived.record(torch.cuda.current_stream(self.engine.device))
        return _SampleTicket(ids, host, n, arrived)

    def sample_wait(self, ticket: _SampleTicket) -> List[int]:
        ticket.arrived.synchronize()
        self.d2h_bytes = ticket.n * 4
        if self.on_tokens is not None:
            self.on_tokens(ticket.n)
        return ticket.host[:ticket.n].tolist()

    def decode_sampled(self, slots: Sequence[int], ticket: _SampleTicket, rows: Sequence[int]):
        ids = ticket.ids
        if list(rows) != list(range(ticket.n)):
            # some sequences of the ticket ended: the others' ids, gathered on the device
            index = torch.tensor(list(rows), dtype=torch.long, device=ids.device)
            ids = ids.index_select(0, index)
        self.last_logits = self.engine.step_sampled(slots, ids, check=False)
        self.h2d_bytes = self.engine.last_h2d_bytes
        return self.last_logits


class Model:
    """A loaded model ready to generate.  ``Model.load(folder)`` mirrors ``Engine::load``."""

    def __init__(self, engine: Engine, max_batch: int = 64):
        self.engine = engine
        self.max_batch = max_batch
        self.stepper = EngineStepper(engine)
        self.stop_ids = tuple(engine.stop_ids)
        self.last_generated_tokens = 0
        self.last_batch_decode_steps = 0
        self.last_finish_reasons: List[str] = []

    @classmethod
    def load(cls, folder: str, dtype="bfloat16", max_tokens: int = 16384, max_seq_len: Optional[int] = None,
             max_batch: int = 64, device="cuda:0", **kw) -> "Model":
        return cls(Engine.load(folder, dtype=dtype, max_tokens=max_tokens, max_seq_len=max_seq_len,
                               device=device, **kw), max_batch)

    @classmethod
    def from_random(cls, config, seed: int, dtype="bfloat16", max_tokens: int = 16384,
                    max_seq_len: Optional[int] = None, max_batch: int = 64, device="cuda:0", **kw) -> "Model":
        return cls(Engine.from_random(config, seed, dtype=dtype, max_tokens=max_tokens,
                                      max_seq_len=max_seq_len, device=device, **kw), max_batch)

    def _run(self, prompts, params: SampleParams, stop_ids, ignore_eos: bool) -> BatchReport:
        stop = () if ignore_eos else (self.stop_ids if stop_ids is None else tuple(stop_ids))
        report = generate_batch(self.stepper, prompts, params, stop, self.max_batch)
        self.engine.check_status()
        self.last_generated_tokens = report.generated_tokens
        self.last_batch_decode_steps = report.shared_steps
        self.last_finish_reasons = [r.finish_reason for r in report.results]
        return report

    def generate(self, prompt: Sequence[int], params: Optional[SampleParams] = None,
                 stop_ids: Optional[Sequence[int]] = None, ignore_eos: bool = False) -> List[int]:
        """Generated ids for one prompt (``Engine::generate``)."""
        return self._run([prompt], params or SampleParams(), stop_ids, ignore_eos).results[0].tokens

    def generate_batch(self, prompts: Sequence[Sequence[int]], params: Optional[SampleParams] = None,
                       stop_ids: Optional[Sequence[int]] = None, ignore_eos: bool = False) -> List[List[int]]:
        """Generated ids for every prompt; unequal prompts share steps (``Engine::generate_batch``)."""
        if not prompts:
            self.last_batch_decode_steps = 0
            self.last_generated_tokens = 0
            return []
        return [r.tokens for r in self._run(prompts, params or SampleParams(), stop_ids, ignore_eos).results]

    def generate_greedy_trace(self, prompt: Sequence[int], max_tokens: int) -> GreedyTrace:
        params = SampleParams(max_tokens=max_tokens, temperature=0.0, top_k=0, top_p=1.0)
        ids = self._run([prompt], params, None, False).results[0].tokens
        last = self.stepper.last_logits
        return GreedyTrace(ids, last[-1].detach().clone() if last is not None and last.shape[0] else torch.empty(0))

    # ---- the step function and the slots, for callers that drive the model themselves ------------
    def step(self, seqs: Sequence[SequenceStep], check: bool = True) -> torch.Tensor:
        """``Engine.step``: the given tokens of the given sequences as one batch, float32 logits at
        the wanted places."""
        return self.engine.step(seqs, check=check)

    def alloc_slot(self) -> int:
        return self.engine.acquire()

    def free_slot(self, slot: int) -> None:
        self.engine.release(slot)

    @property
    def config(self):
        """The configuration the model was built from, as its architecture's typed, read-only object
        (None for a model whose architecture registered no configuration class)."""
        from ..registry import architecture_for
        if self.engine.config is None:
            return None
        cls = architecture_for(self.engine.config).config_class
        return cls.from_dict(self.engine.config) if hasattr(cls, "from_dict") else self.engine.config

    # accessors in the reference's names (engine/mod.rs:477-503)
    def n_layer(self) -> int:
        return len(self.engine.spec.layers)

    def n_vocab(self) -> int:
        return self.engine.spec.vocab_size

    def n_ctx(self) -> int:
        return self.engine.max_seq_len

    def n_embd(self) -> int:
        return self.engine.spec.width
