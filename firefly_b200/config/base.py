"""Typed model configuration and the data form of a model (its "spec").

Two levels live here:

* ``ModelConfig`` — a typed view of an architecture's own ``config.json``.  Every
  architecture subclasses it, names its keys and defaults, and validates them.
* ``ModelSpec`` — what the generic decoder is built from: a list of layers, each
  put together from named parts (mixer, feed-forward, norms, position encoding)
  with their sizes as parameters, plus the *schedule*: the order in which the
  layers run, as data.  No size and no constant that ``config.json`` gives is
  written anywhere else.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, ClassVar, Dict, List, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A configuration is missing a key, has an invalid value, or asks for a
    feature this engine does not implement."""


# --------------------------------------------------------------------------- #
# config.json level
# --------------------------------------------------------------------------- #
_MISSING = object()


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's typed configuration.

    Subclasses are frozen dataclasses whose field names are the architecture's
    own ``config.json`` keys.  ``architecture`` is the string found in
    ``config.json["architectures"][0]``.
    """

    architecture: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architectures": [self.architecture]}
        for f in fields(self):
            out[f.name] = getattr(self, f.name)
        return out

    def validate(self) -> None:
        raise NotImplementedError

    # helpers for subclasses -------------------------------------------------
    @staticmethod
    def _get(raw: Mapping[str, Any], key: str, typ, default=_MISSING):
        if key not in raw or raw[key] is None:
            if default is _MISSING:
                raise ConfigError(f"config.json: required key '{key}' is missing")
            return default
        v = raw[key]
        if typ is bool:
            if not isinstance(v, bool):
                raise ConfigError(f"config.json: '{key}' must be true/false, got {v!r}")
            return v
        if typ is int:
            if isinstance(v, bool) or not isinstance(v, int):
                if isinstance(v, float) and v == int(v):
                    return int(v)
                raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
            return v
        if typ is float:
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
            return float(v)
        if typ is str:
            if not isinstance(v, str):
                raise ConfigError(f"config.json: '{key}' must be a string, got {v!r}")
            return v
        return v


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in model folder '{model_dir}'")
    with open(path, "r", encoding="utf-8") as fh:
        try:
            raw = json.load(fh)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from e
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw


# --------------------------------------------------------------------------- #
# spec level: the model as data
# --------------------------------------------------------------------------- #
@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered ``kind`` of the part, its sizes and
    constants (``params``), and the prefix of its tensor names."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""

    def with_params(self, **kw) -> "PartSpec":
        p = dict(self.params)
        p.update(kw)
        return PartSpec(self.kind, p, self.prefix)


@dataclass(frozen=True)
class LayerSpec:
    """A block: which arrangement joins the parts, and the parts themselves.

    ``position`` is the position encoding the mixer applies (rotary) or None.
    """

    arrangement: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Tuple[PartSpec, ...]
    position: Optional[PartSpec] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    ``layer``  index into ``ModelSpec.layers`` (a layer may be named twice).
    ``cache``  index of the cache slot the mixer uses; by default the entry's own
               place in the schedule, so that a layer that runs twice keeps two
               caches.  Pointing it at an earlier entry's slot makes this run
               read that entry's cache.
    ``write_cache``  False when the run only reads the (other layer's) cache.
    """

    layer: int
    cache: Optional[int] = None
    write_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    # position encoding applied to the embedding output (learned / absolute), or None
    embedding_position: Optional[PartSpec] = None

    def resolved_schedule(self) -> List[Tuple[int, int, bool]]:
        """(layer, cache slot, write) for every run, with defaults filled in,
        checked for consistency."""
        out: List[Tuple[int, int, bool]] = []
        writers: Dict[int, int] = {}
        for pos, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ConfigError(f"schedule[{pos}] names layer {e.layer}, "
                                  f"model has {len(self.layers)}")
            slot = pos if e.cache is None else e.cache
            if e.write_cache:
                if slot in writers:
                    raise ConfigError(
                        f"schedule[{pos}] and schedule[{writers[slot]}] both write cache slot {slot}")
                writers[slot] = pos
            out.append((e.layer, slot, e.write_cache))
        for pos, (layer, slot, write) in enumerate(out):
            if not write:
                if slot not in writers or writers[slot] >= pos:
                    raise ConfigError(
                        f"schedule[{pos}] reads cache slot {slot}, which no earlier run writes")
        return out
