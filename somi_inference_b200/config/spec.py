"""Architecture-neutral description of a decoder: parts, layers and their order.

A model is data: a list of `LayerSpec` (which mixer, which feed-forward, which
norm, which arrangement, each with its own numbers) and a `schedule`, the list
of runs that one forward pass makes.  A run names a layer and, optionally, an
earlier run whose cache it reads instead of keeping one of its own.  Nothing in
this file knows an architecture; an architecture's config class produces a
`ModelSpec` (see `config/qwen2.py`).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered kind and its parameters.

    `kind` is looked up in the matching registry of `parts/registry.py`;
    `params` are passed to the part's constructor unchanged, so every size and
    constant a part uses is stated here and nowhere else.
    """

    kind: str
    params: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: weight-name prefix, its parts and their arrangement.

    A layer has at most one mixer and at most one feed-forward (either may be None) and any
    number of norms, each under the name by which the layer's arrangement asks for it: the
    pre-norm arrangement wants "mixer" and "feed_forward"; an arrangement that also normalises
    what its parts return can name four.  The arrangement's constructor is called with
    `(mixer, feed_forward, norms)`, `norms` being a dict from those names to built norms.

    `extras` are further parts of the layer that are neither of these (a gate on a residual
    branch, a short convolution in front of the mixer, ...), each under the name by which the
    arrangement asks for it and looked up in the registry of layer extras; an arrangement of a
    layer that has some is built with `(mixer, feed_forward, norms, extras)`.
    """

    prefix: str  # e.g. "model.layers.3"
    mixer: PartSpec | None
    feed_forward: PartSpec | None
    norms: Mapping[str, PartSpec] = field(default_factory=dict)
    arrangement: str = "pre_norm"
    extras: Mapping[str, PartSpec] = field(default_factory=dict)


@dataclass(frozen=True)
class RunSpec:
    """One entry of the schedule: run `layer`; read the cache of run `cache_of`.

    `cache_of is None` means the run owns a cache (and writes it).  Otherwise it
    is the index, in the schedule, of an earlier run whose cache this run reads
    without writing.  `add_embedding`: the embedding's output (the residual stream as it was
    before the first run) is added to the stream once more right in front of this run.
    `remix`: the name of one of the model's `stream_parts`; right in front of this run the
    stream is replaced by what that part makes of the stream and the embedding's output.
    """

    layer: int
    cache_of: int | None = None
    add_embedding: bool = False
    remix: str | None = None


@dataclass(frozen=True)
class ModelSpec:
    """Everything the generic decoder needs to be built."""

    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[RunSpec, ...]
    final_norm: PartSpec
    head: PartSpec
    # parts that act on the residual stream between runs (see `RunSpec.remix`), by name
    stream_parts: Mapping[str, PartSpec] = field(default_factory=dict)

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.schedule:
            raise ValueError("a model needs a non-empty schedule")
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule[{i}] names layer {run.layer}, "
                                 f"but there are {len(self.layers)} layers")
            if run.remix is not None and run.remix not in self.stream_parts:
                raise ValueError(f"schedule[{i}].remix names {run.remix!r}, which is none of the "
                                 f"model's stream parts {sorted(self.stream_parts)}")
            if run.add_embedding and i == 0:
                raise ValueError("schedule[0] cannot add the embedding's output again")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < i:
                    raise ValueError(f"schedule[{i}].cache_of={run.cache_of} must "
                                     "name an earlier run")
                if self.schedule[run.cache_of].cache_of is not None:
                    raise ValueError(f"schedule[{i}].cache_of={run.cache_of} names "
                                     "a run that owns no cache")
