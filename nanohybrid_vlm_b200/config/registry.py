"""One registry from the architecture's name (``architectures[0]`` of config.json, or its ``architecture``
string) to its model.

The reference keeps ``model_type -> (architectures, module, class)`` and checks both
(nanovllm/models/registry.py:36-149).  Here the key is the architecture name; the entry
gives the configuration class, the function that turns a configuration into a
:class:`~nanohybrid_vlm_b200.parts.spec.ModelSpec` (layers as data) and the allowed
``model_type`` values.  Everything else in the engine works from the spec.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .model_config import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    model_types: tuple[str, ...]
    parse_config: Callable[[dict], ModelConfig]
    build_spec: Callable[[ModelConfig], "ModelSpec"]  # noqa: F821
    # (raw config.json, shape_of) -> raw config.json completed by sizes that only a checkpoint tensor's shape gives;
    # shape_of(name) is the shape of that tensor in the model folder, or None.  None: config.json says everything.
    complete_config: Callable[[dict, Callable], dict] | None = None


class ArchitectureRegistry:
    def __init__(self):
        self._entries: dict[str, ArchitectureEntry] = {}

    def register(self, name: str, *, model_types, parse_config, build_spec, replace: bool = False,
                 complete_config=None) -> None:
        if not name:
            raise ValueError("an architecture needs a name")
        if name in self._entries and not replace:
            raise ValueError(f"architecture {name!r} is already registered")
        if not callable(parse_config) or not callable(build_spec):
            raise TypeError(f"architecture {name!r}: parse_config and build_spec must be callable")
        if complete_config is not None and not callable(complete_config):
            raise TypeError(f"architecture {name!r}: complete_config must be callable")
        self._entries[name] = ArchitectureEntry(name, tuple(model_types), parse_config, build_spec, complete_config)

    def unregister(self, name: str) -> None:
        self._entries.pop(name, None)

    def names(self) -> list[str]:
        return sorted(self._entries)

    def resolve(self, raw_config: dict) -> ArchitectureEntry:
        archs = raw_config.get("architectures") or raw_config.get("architecture") or ()
        if isinstance(archs, str):
            archs = (archs,)
        if not archs:
            raise ConfigError("config.json: key 'architectures' (or 'architecture') is missing or empty; "
                              f"supported architectures: {self.names()}")
        known = [a for a in archs if a in self._entries]
        if not known:
            raise ConfigError(f"unsupported architectures {tuple(archs)!r}; supported: {self.names()}")
        entry = self._entries[known[0]]
        model_type = raw_config.get("model_type")
        if model_type is not None and entry.model_types and model_type not in entry.model_types:
            raise ConfigError(f"architecture {entry.name!r} does not go with model_type {model_type!r} "
                              f"(expected one of {entry.model_types})")
        return entry


ARCHITECTURES = ArchitectureRegistry()


def register_architecture(name: str, *, model_types=(), parse_config, build_spec, replace=False,
                          complete_config=None) -> None:
    ARCHITECTURES.register(name, model_types=model_types, parse_config=parse_config,
                           build_spec=build_spec, replace=replace, complete_config=complete_config)


def checkpoint_shapes(model_dir: str) -> dict[str, tuple[int, ...]]:
    """Name -> shape of every tensor in the folder's ``*.safetensors`` files, from their headers alone (8 bytes of
    little-endian length, then that many bytes of JSON).  A folder without such files gives an empty table."""
    import glob
    import json
    import os
    import struct
    shapes: dict[str, tuple[int, ...]] = {}
    for path in sorted(glob.glob(os.path.join(model_dir, "*.safetensors"))):
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise ConfigError(f"{path}: too short for a safetensors file")
            (n,) = struct.unpack("<Q", head)
            try:
                table = json.loads(f.read(n))
            except (json.JSONDecodeError, UnicodeDecodeError) as e:
                raise ConfigError(f"{path}: the header is not valid JSON: {e}") from e
        for name, info in table.items():
            if name != "__metadata__" and isinstance(info, dict) and "shape" in info:
                shapes[name] = tuple(int(x) for x in info["shape"])
    return shapes


def load_model_config(model_dir: str) -> tuple[ArchitectureEntry, ModelConfig]:
    """Read ``model_dir/config.json``, pick the architecture, parse its typed configuration."""
    from .. import models  # noqa: F401  (registers the built-in architecture)
    raw = read_config_json(model_dir)
    entry = ARCHITECTURES.resolve(raw)
    if entry.complete_config is not None:
        shapes = checkpoint_shapes(model_dir)
        raw = entry.complete_config(raw, shapes.get)
    return entry, entry.parse_config(raw)
