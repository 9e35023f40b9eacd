"""Machine-readable description of an operator package and its lazily resolved public surface.

Mirrors the reference's operator header (``b12x/_lib/meta.py:17-64``: ``Provenance``, ``OpMeta``
with the same field names, and ``install_lazy_api``), so that tooling written against the
reference's ``META`` objects reads these as well.  Standard library only: an operator package is
imported for its ``META`` without pulling in torch or loading the CUDA library."""

from __future__ import annotations

import importlib
from dataclasses import dataclass, field
from typing import Any, Literal


@dataclass(frozen=True, kw_only=True)
class Provenance:
    """Which upstream files an operator answers to."""

    repo: str
    commit: str
    paths: tuple[str, ...]


def _no_provenance() -> Provenance:
    return Provenance(repo="", commit="", paths=())


@dataclass(frozen=True, kw_only=True)
class OpMeta:
    """Header of one operator (keyword-only, so the field order carries no meaning).

    ``api_style``: "planned" = ``Caps -> plan() -> bind() -> run()`` (``plan`` on the host, ``bind``
    views only, ``run`` safe under CUDA-graph capture); "oneshot" = plain functions; "stateful" =
    long-lived objects."""

    # identity
    group: str
    name: str
    # what the package exports and how it is driven
    entry_points: tuple[str, ...]
    api_style: Literal["planned", "oneshot", "stateful"]
    # what it runs on and with
    archs: tuple[str, ...] = ("sm100a",)
    recipes: tuple[str, ...] = ()
    dtypes: tuple[str, ...] = ()
    requires: tuple[str, ...] = ()
    # bookkeeping
    status: Literal["experimental"] = "experimental"
    since: str = ""
    test_path: str = ""
    notes: str = ""
    provenance: Provenance = field(default_factory=_no_provenance)

    @property
    def qualname(self) -> str:
        return self.group + "." + self.name


class _LazySurface:
    """PEP 562 hooks for one operator package: names listed in ``META.entry_points`` are fetched
    from the package's ``api`` module the first time they are asked for, then cached in the
    package's globals (so a test can replace one with ``setattr`` like any module attribute)."""

    def __init__(self, namespace: dict[str, Any], meta: OpMeta):
        self.namespace = namespace
        self.meta = meta
        self.package = namespace["__name__"]

    def getattr(self, name: str) -> Any:
        if name not in self.meta.entry_points:
            raise AttributeError(f"module {self.package!r} has no attribute {name!r}")
        value = getattr(importlib.import_module(self.package + ".api"), name)
        self.namespace[name] = value
        return value

    def dir(self) -> list[str]:
        return sorted(set(self.meta.entry_points) | {"META"})


def install_lazy_api(module_globals: dict[str, Any], meta: OpMeta) -> None:
    """Give the operator package ``__getattr__`` / ``__dir__`` / ``__all__`` derived from ``meta``."""
    surface = _LazySurface(module_globals, meta)
    module_globals["__getattr__"] = surface.getattr
    module_globals["__dir__"] = surface.dir
    module_globals["__all__"] = [*meta.entry_points, "META"]


__all__ = ["OpMeta", "Provenance", "install_lazy_api"]
