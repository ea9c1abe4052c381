"""The description of a model as data: which parts, with which parameters, fed by which tensors,
run in which order.  An architecture's builder produces a ``ModelSpec`` from its configuration; the
generic ``DecoderModel`` (``pulse_infer_b200.parts.model``) instantiates it.  Nothing in here knows
an architecture by name.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class PartSpec:
    """One part: ``kind`` selects the class in the part registry, ``params`` are its constructor
    arguments (every size and constant), ``prefix`` is prepended to the tensor names it asks for."""
    kind: str
    params: dict = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One block: the arrangement (how norms, mixer, feed-forward and the residual are wired) and
    its four parts.  Different layers of one model may name different kinds."""
    arrangement: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  ``cache`` names the cache its mixer uses (an index into the model's
    caches).  A layer may appear in several entries (it runs again, normally with another cache), and
    two entries may name the same cache: the one whose mixer writes fills it, a mixer built with
    ``writes_cache=False`` only reads what an earlier entry wrote."""
    layer: int
    cache: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    embedding: PartSpec
    layers: tuple            # of LayerSpec
    order: tuple             # of ScheduleEntry: the sequence in which layers run
    final_norm: PartSpec
    lm_head: PartSpec
    positions: dict = field(default_factory=dict)   # name -> PartSpec of a position encoding
    hidden_size: int = 0
    vocab_size: int = 0
    max_position: int = 0

    @property
    def num_caches(self) -> int:
        used = [e.cache for e in self.order if e.cache is not None]
        return (max(used) + 1) if used else 0
