"""Plug-ins, lazily registered first-party defaults, and kind tables with option schemas.

``IdrakPlugin``        what a plug-in module exposes: ``name`` and ``register(api)``; ``load_plugins()`` imports the modules
                       named in ``IDRAK_PLUGINS`` (comma separated) and the ``idrak_b200.plugins`` entry-point group and
                       hands each the ``PluginApi`` (the registries it may add to: operations' kernels, device providers,
                       model families, tokenizers, losses, kinds)
``LibraryDefaults``    ``ensure(name)``: the first-party entries of a registry are registered the first time the registry is
                       asked, not at import (import stays cheap; a plug-in registered earlier is not overwritten because
                       defaults use the ``fallback`` policy)
``KindTable`` / ``OptionSchema``  named kinds (of layer, optimizer, schedule, ...) each with a schema of options: type,
                       default, choices, range; ``create(kind, **options)`` validates and fills defaults, and an unknown
                       kind or option is refused with the list of known ones

Reference: IIdrakPlugin (src/Idrak.Abstraction/Plugins), LibraryDefaults.Ensure (LibraryDefaults.cs:18-30), KindTable /
OptionSchema (src/Idrak.Abstraction/Kinds).
"""
from __future__ import annotations

import dataclasses
import importlib
import os
from typing import Any, Callable, Dict, List, Optional, Sequence

from .registry import SlotTable


# --------------------------------------------------------------------------- option schemas and kind tables
@dataclasses.dataclass(frozen=True)
class Option:
    name: str
    type: type = float
    default: Any = None
    choices: Optional[Sequence[Any]] = None
    minimum: Optional[float] = None
    maximum: Optional[float] = None
    required: bool = False
    doc: str = ""


class OptionSchema:
    def __init__(self, *options: Option):
        self.options: Dict[str, Option] = {o.name: o for o in options}

    def validate(self, given: Dict[str, Any], owner: str = "") -> Dict[str, Any]:
        """Defaults filled in, values converted to the declared type; unknown names, wrong types, values outside the
        choices or the range are refused with a message that names the option and what is allowed."""
        unknown = [k for k in given if k not in self.options]
        if unknown:
            raise KeyError(f"{owner}: unknown option '{unknown[0]}'. Known: {', '.join(sorted(self.options))}")
        out = {}
        for name, o in self.options.items():
            if name not in given:
                if o.required:
                    raise KeyError(f"{owner}: option '{name}' is required")
                out[name] = o.default
                continue
            v = given[name]
            if o.type is bool and isinstance(v, str):
                if v.lower() not in ("true", "false", "1", "0", "yes", "no"):
                    raise ValueError(f"{owner}: option '{name}' wants true or false, got '{v}'")
                v = v.lower() in ("true", "1", "yes")
            elif o.type in (int, float) and isinstance(v, str):
                try:
                    v = o.type(v)
                except ValueError:
                    raise ValueError(f"{owner}: option '{name}' wants {o.type.__name__}, got '{v}'")
            elif o.type is float and isinstance(v, int) and not isinstance(v, bool):
                v = float(v)
            elif v is not None and not isinstance(v, o.type):
                raise ValueError(f"{owner}: option '{name}' wants {o.type.__name__}, got {type(v).__name__}")
            if o.choices is not None and v not in o.choices:
                raise ValueError(f"{owner}: option '{name}' must be one of {list(o.choices)}, got {v!r}")
            if o.minimum is not None and v < o.minimum or o.maximum is not None and v > o.maximum:
                raise ValueError(f"{owner}: option '{name}' = {v} is outside [{o.minimum}, {o.maximum}]")
            out[name] = v
        return out

    def describe(self) -> List[Dict[str, Any]]:
        return [dataclasses.asdict(o) | {"type": o.type.__name__} for o in self.options.values()]


class KindTable:
    """Named kinds with a factory and an option schema each."""

    def __init__(self, what: str, defaults: Optional[Callable[["KindTable"], None]] = None):
        self.what = what
        self._table: SlotTable = SlotTable(what, (lambda t: defaults(self)) if defaults else None)

    def register(self, kind: str, factory: Callable[..., Any], schema: Optional[OptionSchema] = None,
                 policy: str = "shadow"):
        return self._table.register(kind, (factory, schema or OptionSchema()), policy)

    def kinds(self) -> List[str]:
        return self._table.keys()

    def schema(self, kind: str) -> OptionSchema:
        return self._entry(kind)[1]

    def _entry(self, kind: str):
        e = self._table.get(kind)
        if e is None:
            raise KeyError(f"{self.what} '{kind}' is not registered. Known: {', '.join(self.kinds())}")
        return e

    def create(self, kind: str, *args, **options):
        factory, schema = self._entry(kind)
        return factory(*args, **schema.validate(options, f"{self.what} '{kind}'"))


# --------------------------------------------------------------------------- lazily registered first-party defaults
class LibraryDefaults:
    """``LibraryDefaults.add(name, fn)`` notes how to fill a registry; ``ensure(name)`` runs it once, on first need."""
    _pending: Dict[str, List[Callable[[], None]]] = {}
    _done: set = set()

    @classmethod
    def add(cls, name: str, fill: Callable[[], None]) -> None:
        if name in cls._done:
            fill()
        else:
            cls._pending.setdefault(name, []).append(fill)

    @classmethod
    def ensure(cls, name: str) -> None:
        if name in cls._done:
            return
        cls._done.add(name)
        for fill in cls._pending.pop(name, []):
            fill()

    @classmethod
    def ensured(cls) -> List[str]:
        return sorted(cls._done)


# --------------------------------------------------------------------------- plug-ins
class PluginApi:
    """What a plug-in may touch."""

    def __init__(self):
        from . import backend, device
        self.operations = backend.OPERATIONS
        self.register_kernel = backend.register_kernel
        self.device_providers = device.DEVICE_PROVIDERS
        self.kind_tables: Dict[str, KindTable] = KIND_TABLES

    def registry(self, name: str):
        """First-party registries by name (model families, preference losses, tokenizers ...), imported on demand."""
        if name == "model_families":
            from ..models import families
            return families.FAMILIES if hasattr(families, "FAMILIES") else families
        if name == "preference_losses":
            from ..text.finetuning import PREFERENCE_LOSSES
            return PREFERENCE_LOSSES
        if name == "contract_suites":
            from ..testing.contracts import SUITES
            return SUITES
        raise KeyError(f"registry '{name}' is not known. Known: model_families, preference_losses, contract_suites")


KIND_TABLES: Dict[str, KindTable] = {}
_LOADED: Dict[str, Any] = {}


def load_plugins(names: Optional[Sequence[str]] = None) -> List[str]:
    """Imports every plug-in module once and calls its ``register(api)``. Returns the names loaded by this call."""
    wanted = list(names) if names is not None else [n.strip() for n in os.environ.get("IDRAK_PLUGINS", "").split(",") if n.strip()]
    if names is None:
        try:
            from importlib.metadata import entry_points
            wanted += [ep.value.split(":")[0] for ep in entry_points(group="idrak_b200.plugins")]
        except Exception:          # no metadata available: environment variable only
            pass
    api, new = PluginApi(), []
    for mod_name in wanted:
        if mod_name in _LOADED:
            continue
        module = importlib.import_module(mod_name)
        register = getattr(module, "register", None)
        if register is None:
            raise AttributeError(f"plug-in '{mod_name}' has no register(api) function")
        register(api)
        _LOADED[mod_name] = module
        new.append(getattr(module, "name", mod_name))
    return new


def loaded_plugins() -> List[str]:
    return sorted(_LOADED)
