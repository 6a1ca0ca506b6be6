"""A decoder built from a ``ModelSpec``: embedding, the blocks in the order the schedule names
them, final norm and head.  It owns the weights; the cache and the step function live beside it.

The decoder corresponds to ``Qwen3Model`` of the reference (crates/bfi-models/src/qwen3.rs:40-63,
assembly :101-174, layer loop :190-255, head :258-266) but knows no architecture: everything
specific arrives in the spec.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from ..kernels import ops
from ..kernels.linear import EPI_STORE, linear
from ..parts.base import BLOCKS, NORMS, Block, ModelSpec, ParamSpec


class Runtime:
    """What parts may ask of their surroundings while loading: the device, the run dtype and a
    place for tables that several parts share."""

    def __init__(self, device: torch.device, dtype: torch.dtype):
        self.device = torch.device(device)
        self.dtype = dtype
        self.shared: Dict[Any, Any] = {}


def _validate_schedule(spec: ModelSpec) -> None:
    for i, run in enumerate(spec.schedule):
        if not 0 <= run.layer < len(spec.layers):
            raise ValueError(f"schedule entry {i} names layer {run.layer}; the model has {len(spec.layers)}")
        if run.cache_of is not None and not 0 <= run.cache_of < i:
            raise ValueError(f"schedule entry {i} reads the cache of entry {run.cache_of}, which does not run before it")


def expected_tensors(spec: ModelSpec) -> Dict[str, ParamSpec]:
    """Every checkpoint tensor the model wants: checkpoint name -> ParamSpec."""
    out: Dict[str, ParamSpec] = {spec.embedding_name: ParamSpec((spec.vocab_size, spec.width), "table")}
    for i, layer in enumerate(spec.layers):
        block = BLOCKS.build(layer.block)
        for local, ps in block.all_param_specs().items():
            if local not in layer.names:
                raise ValueError(f"layer {i}: no checkpoint name for parameter '{local}'")
            out[layer.names[local]] = ps
    norm = NORMS.build(spec.final_norm)
    for local, ps in norm.all_param_specs().items():
        out[spec.final_norm_names[local]] = ps
    if spec.head_name is not None:
        out[spec.head_name] = ParamSpec((spec.vocab_size, spec.width), "matrix")
    return out


class Decoder:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        _validate_schedule(spec)
        self.spec = spec
        self.runtime = runtime
        self.blocks: List[Block] = [BLOCKS.build(layer.block) for layer in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.n_weight_bytes = 0

    # ---- what the cache has to provide -----------------------------------------------
    def run_needs(self) -> List[Any]:
        return [self.blocks[r.layer].mixer().cache_need() for r in self.spec.schedule]

    def run_cache_of(self) -> List[Optional[int]]:
        return [r.cache_of for r in self.spec.schedule]

    # ---- weights ---------------------------------------------------------------------
    def load(self, tensors: Dict[str, torch.Tensor], max_positions: int) -> None:
        """``tensors``: checkpoint name -> device tensor, as checked by the loader."""
        spec = self.spec
        self.embedding = tensors[spec.embedding_name]
        self.head = self.embedding if spec.head_name is None else tensors[spec.head_name]
        for layer, block in zip(spec.layers, self.blocks):
            local = {name: tensors[ckpt] for name, ckpt in layer.names.items() if ckpt in tensors}
            block.load_all(local, self.runtime)
            block.mixer().prepare(self.runtime, max_positions)
        self.final_norm.load_all({k: tensors[v] for k, v in spec.final_norm_names.items()}, self.runtime)
        self.n_weight_bytes = self._count_weight_bytes()

    def _count_weight_bytes(self) -> int:
        """Bytes of every weight a decode step reads once (each shared tensor counted once)."""
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            for k, v in vars(obj).items():
                if k == "table":       # position tables are not weights
                    continue
                if isinstance(v, torch.Tensor) and v.is_floating_point() and v.dim() >= 1:
                    if v.data_ptr() not in seen:
                        seen.add(v.data_ptr())
                        total += v.numel() * v.element_size()
            for c in getattr(obj, "children", lambda: {})().values():
                visit(c)

        used = {r.layer for r in self.spec.schedule}
        for i, b in enumerate(self.blocks):
            if i in used:
                visit(b)
        visit(self.final_norm)
        if self.head is not None and self.head.data_ptr() not in seen:
            total += self.head.numel() * self.head.element_size()
        return total

    def graph_safe(self) -> bool:
        return all(b.all_graph_safe() for b in self.blocks) and self.final_norm.all_graph_safe()

    def stages(self) -> List[tuple]:
        """A single-token step as stages that may (True) or may not be captured in a CUDA graph:
        ``("embed",)``, ``("runs", first, last)`` for schedule entries ``first .. last-1``, and
        ``("logits",)``, each with its flag; neighbours with the same flag are one stage.  A model
        whose parts are all graph-safe is one stage."""
        ops: List[tuple] = [(True, ("embed",))]
        for i, run in enumerate(self.spec.schedule):
            ops.append((self.blocks[run.layer].all_graph_safe(), ("runs", i, i + 1)))
        ops.append((self.final_norm.all_graph_safe(), ("logits",)))
        out: List[tuple] = []
        for safe, op in ops:
            if out and out[-1][0] == safe:
                last = out[-1][1]
                if op[0] == "runs" and last and last[-1][0] == "runs":
                    last[-1] = ("runs", last[-1][1], op[2])
                else:
                    last.append(op)
            else:
                out.append((safe, [op]))
        return out

    # ---- compute ---------------------------------------------------------------------
    def embed(self, ctx) -> torch.Tensor:
        x = ctx.rows("residual", self.spec.width, torch.float32)
        ops.embed_rows(self.embedding, ctx.token_ids[:ctx.n_tokens], x, ctx.status)
        return x

    def run_layers(self, ctx, x: torch.Tensor, cache, first: int = 0, last: Optional[int] = None) -> None:
        """Schedule entries ``first .. last-1`` (all of them by default)."""
        last = len(self.spec.schedule) if last is None else last
        for i in range(first, last):
            self.blocks[self.spec.schedule[i].layer].forward(ctx, x, cache.run_cache(i))

    def logits(self, ctx, x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
        """Final norm and head at the given rows of ``x``; ``out`` is float32 ``[len(rows), vocab]``."""
        h = self.final_norm.forward(ctx, x, rows, tag="head.norm")
        linear(h, self.head, out, EPI_STORE)
