"""One registry from an architecture's name to the code that builds its model.

Mirrors the reference's provider registry (crates/model/package/src/providers/
registry.rs:22-37 hint order, :91-110 duplicate claims rejected, :116-135 resolve):
hints are collected most specific first -- `architectures`, then `model_type`, then
the nested `text_config` -- and the first registered entry that claims any of them
wins.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Mapping, Sequence

from .errors import ConfigError, UnsupportedConfig
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    """What an architecture must bring: names it claims, a typed config reader and a
    function from that config to a :class:`ModelSpec`."""

    name: str
    claims: Sequence[str]
    read_config: Callable[[Mapping[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]


class ArchitectureRegistry:
    def __init__(self) -> None:
        self._entries: List[Architecture] = []

    def register(self, arch: Architecture) -> None:
        if not arch.claims:
            raise ConfigError("architecture claims no name")
        for claimed in arch.claims:
            for existing in self._entries:
                if claimed in existing.claims:
                    raise ConfigError(
                        f"model architecture {claimed} is already provided by {existing.name}")
        self._entries.append(arch)

    def unregister(self, name: str) -> None:
        self._entries = [e for e in self._entries if e.name != name]

    @staticmethod
    def hints(raw: Mapping[str, Any]) -> List[str]:
        out: List[str] = []

        def collect(d: Mapping[str, Any]) -> None:
            names = d.get("architectures") or ()
            if isinstance(names, str):
                names = (names,)
            elif not isinstance(names, (list, tuple)):
                raise ConfigError(f"architectures must be a list of names, found {names!r}")
            for name in names:
                if not isinstance(name, str):
                    raise ConfigError(f"architectures must be a list of names, found {names!r}")
                if name not in out:
                    out.append(name)
            mt = d.get("model_type")
            if mt is not None and not isinstance(mt, str):
                raise ConfigError(f"model_type must be a name, found {mt!r}")
            if mt is not None and mt not in out:
                out.append(mt)
            tc = d.get("text_config")
            if isinstance(tc, Mapping):
                collect(tc)

        collect(raw)
        return out

    def resolve(self, raw: Mapping[str, Any]) -> Architecture:
        if not isinstance(raw, Mapping):
            raise ConfigError("config.json must hold a JSON object")
        names = self.hints(raw)
        for entry in self._entries:
            if any(n in entry.claims for n in names):
                return entry
        raise UnsupportedConfig(
            f"no model architecture registered for {names}; register an Architecture "
            "with inferloop_b200.config.registry.default_registry().register(...)")

    def names(self) -> List[str]:
        return [e.name for e in self._entries]


_DEFAULT: ArchitectureRegistry | None = None


def default_registry() -> ArchitectureRegistry:
    global _DEFAULT
    if _DEFAULT is None:
        _DEFAULT = ArchitectureRegistry()
        from ..models.qwen3 import ARCHITECTURE
        _DEFAULT.register(ARCHITECTURE)
    return _DEFAULT


def read_model_config(text: str, registry: ArchitectureRegistry | None = None):
    """Parse config.json text; return (architecture entry, typed config, ModelSpec)."""
    try:
        raw = json.loads(text)
    except (json.JSONDecodeError, RecursionError) as e:      # (brackets nested thousands deep end the parser's recursion)
        raise ConfigError(f"config.json is not valid JSON: {e}") from None
    reg = registry or default_registry()
    arch = reg.resolve(raw)
    cfg = arch.read_config(raw)
    return arch, cfg, arch.build_spec(cfg)
