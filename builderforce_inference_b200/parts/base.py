"""Interfaces of the parts a decoder is put together from, and their registries.

A model is described by data (``ModelSpec``): which part stands where, with which sizes and
constants, under which tensor names its weights are stored, and in which order the layers run.
Parts are looked up by kind in the registries below and built from their ``params`` alone; no
part knows which model it is in, and a new kind is added by registering a class, not by
editing this package.

Contracts (all tensors live on the GPU):

``Norm.forward(ctx, x, rows=None) -> h``
    ``x`` is the float32 residual stream ``[tokens, width]``; ``h`` is in the activation dtype.
    With ``rows`` (int32 indices) only those rows are normalised, in that order.
``Mixer.forward(ctx, h, residual, run)``
    adds the mixer's output for every token of the step into ``residual`` (float32) in place.
    ``run`` gives the run's cache (``run.kv`` pages or ``run.state`` rows) and whether this run
    writes it (``run.writes_cache``) or reads another run's.
``FeedForward.forward(ctx, h, residual)``
    adds its output into ``residual`` in place.
``PositionEncoding``
    either exposes a rotary table that the attention kernels consume in the same pass as the
    q/k norms and the cache write (``fused_rotary()``), or transforms q and k itself in
    ``apply(ctx, q, k)``.
``Block.forward(ctx, residual, run)``
    arranges norms, mixer and feed-forward around the residual stream.

Every part lists the tensors it wants in ``param_specs()`` under local names; the model's
``names`` maps them to checkpoint tensor names.  ``load(tensors)`` receives them on the device,
may fuse or re-lay them and keeps what it needs.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple


@dataclass(frozen=True)
class PartSpec:
    """A part by kind, with its sizes and constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part wants: its shape and what it is (which decides its random init)."""

    shape: Tuple[int, ...]
    role: str = "matrix"        # "matrix" | "table" | "norm"
    optional: bool = False


@dataclass(frozen=True)
class KVNeed:
    """A mixer that keeps keys and values of earlier tokens: all of them, or a window."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps a state of fixed size per sequence."""

    shape: Tuple[int, ...]
    dtype: str = "float32"


class Part:
    """Base of every part: parameters by local name."""

    # A part is graph-safe if its forward launches only work whose shapes and addresses are
    # fixed by the step's padded size and reads lengths, positions and slots from the device
    # arrays of the context.  Steps through parts that are not are never captured in a graph.
    graph_safe = False

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def load(self, tensors: Dict[str, Any], runtime: Any) -> None:
        for k, v in tensors.items():
            setattr(self, k.replace(".", "_"), v)

    def children(self) -> Dict[str, "Part"]:
        """Sub-parts by local prefix; their parameters appear as ``prefix.name``."""
        return {}

    def all_param_specs(self) -> Dict[str, ParamSpec]:
        out = dict(self.param_specs())
        for prefix, child in self.children().items():
            for k, v in child.all_param_specs().items():
                out[f"{prefix}.{k}"] = v
        return out

    def load_all(self, tensors: Dict[str, Any], runtime: Any) -> None:
        own = {k: v for k, v in tensors.items() if k in self.param_specs()}
        self.load(own, runtime)
        for prefix, child in self.children().items():
            sub = {k[len(prefix) + 1:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}
            child.load_all(sub, runtime)

    def all_graph_safe(self) -> bool:
        return self.graph_safe and all(c.all_graph_safe() for c in self.children().values())


class Norm(Part):
    def forward(self, ctx, x, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    def prepare(self, runtime, max_positions: int) -> None:
        """Build tables for positions ``0 .. max_positions-1``."""

    def fused_rotary(self):
        """``(table, rot_dim)`` if the encoding is a rotate-half rotation that the attention
        kernels apply themselves, else None."""
        return None

    def apply(self, ctx, q, k):
        """Transform q ``[tokens, heads, d]`` and k ``[tokens, kv_heads, d]`` in place."""
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self):
        """What the mixer keeps per sequence: ``KVNeed``, ``StateNeed``, None, or a tuple of several
        (keys and values beside a fixed-size state, say).  The run's cache then carries one entry
        per need, in this order, in ``run.entries``."""
        return None

    def prepare(self, runtime, max_positions: int) -> None:
        pass

    def forward(self, ctx, h, residual, run) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h, residual) -> None:
        raise NotImplementedError


class Block(Part):
    def mixer(self) -> Mixer:
        raise NotImplementedError

    def forward(self, ctx, residual, run) -> None:
        raise NotImplementedError


class Registry:
    """Kind name -> class, for one family of parts."""

    def __init__(self, family: str):
        self.family = family
        self._kinds: Dict[str, Callable[..., Part]] = {}

    def register(self, kind: str, cls: Optional[Callable[..., Part]] = None):
        def put(c):
            if kind in self._kinds and self._kinds[kind] is not c:
                raise ValueError(f"{self.family} kind '{kind}' is already registered")
            self._kinds[kind] = c
            return c
        return put(cls) if cls is not None else put

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def build(self, spec: PartSpec) -> Part:
        if spec.kind not in self._kinds:
            raise KeyError(
                f"unknown {self.family} kind '{spec.kind}'; registered: {sorted(self._kinds)}")
        return self._kinds[spec.kind](**dict(spec.params))

    def kinds(self) -> List[str]:
        return sorted(self._kinds)


NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its block and the checkpoint names of the block's tensors."""

    block: PartSpec
    names: Mapping[str, str]          # local parameter name -> checkpoint tensor name


@dataclass(frozen=True)
class RunSpec:
    """One entry of the order in which layers run.  ``layer`` may appear in several entries;
    ``cache_of`` names an earlier entry whose cache this run reads instead of keeping one."""

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder as data."""

    vocab_size: int
    width: int
    embedding_name: str
    layers: Sequence[LayerSpec]
    schedule: Sequence[RunSpec]
    final_norm: PartSpec
    final_norm_names: Mapping[str, str]
    head_name: Optional[str]          # None: the head is the embedding table (tied)
    ignored_names: Sequence[str] = ()  # tensors a checkpoint may carry that are not used
    max_positions: int = 0
    stop_ids: Tuple[int, ...] = ()
