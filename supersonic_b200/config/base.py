"""Architecture-neutral description of a model: what the engine builds from.

An architecture's typed configuration (read from its own ``config.json`` keys)
is turned by its builder into a :class:`ModelSpec`: a list of blocks, each
naming its mixer, feed-forward, norms and position encoding with all sizes and
constants as parameters, plus the order in which the blocks run.  Nothing below
this file knows which architecture it serves.

The reference keeps one geometry struct per family and marks every Llama layer
``"full_attention"`` (crates/runner/src/llama31_engine.rs:78-105); here the
per-layer choice is first-class data instead.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that is missing a key, or holds a value the engine refuses."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a block: the registered ``kind`` and its parameters.

    ``params`` holds every size and constant the part needs; ``weights`` maps
    the part's own weight roles (``"q"``, ``"gate"``, ``"weight"`` ...) to
    tensor names in the model folder.
    """

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    weights: Dict[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class BlockSpec:
    """One layer: an arrangement (``kind``) of a mixer and a feed-forward."""

    kind: str                      # registered block arrangement, e.g. "pre_norm"
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    position: Optional[PartSpec] = None   # position encoding used by the mixer


@dataclass(frozen=True)
class ScheduleEntry:
    """One stop of the forward pass.

    ``layer`` indexes ``ModelSpec.blocks``.  ``cache`` names the cache entry
    the mixer reads; two stops with the same ``cache`` share storage.
    ``writes_cache`` is False for a stop that only reads what an earlier stop
    of the same step wrote (a layer that borrows another layer's keys).
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    blocks: List[BlockSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: List[int] = field(default_factory=list)

    def validate(self) -> None:
        if not self.blocks:
            raise ConfigError("a model needs at least one block")
        written = set()
        for i, stop in enumerate(self.schedule):
            if not 0 <= stop.layer < len(self.blocks):
                raise ConfigError(f"schedule[{i}] names layer {stop.layer}, "
                                  f"but there are {len(self.blocks)} blocks")
            if stop.writes_cache:
                written.add(stop.cache)
            elif stop.cache not in written:
                raise ConfigError(f"schedule[{i}] reads cache {stop.cache} "
                                  "before any stop has written it")


def default_schedule(num_layers: int) -> List[ScheduleEntry]:
    """Every layer once, in order, each with a cache entry of its own."""
    return [ScheduleEntry(layer=i, cache=i) for i in range(num_layers)]
