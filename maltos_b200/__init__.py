"""maltos_b200 — a Blackwell-native (sm_100a) modular LLM training runtime.

Sub-packages mirror the flat top-level layout of the reference project so that user code written for it
keeps working: ``runtime`` (core, mesh, plugins, layers, step runners), ``parallel`` (plans/specs/planners),
``state`` (checkpoints), ``data``, ``train``, ``models``, ``utils``, ``tools``. The hot ops live in ``ops``
(Python wrappers) and ``csrc`` (hand-written CUDA for sm_100a).

Importing this package also makes those sub-packages importable under their short names (``import runtime``,
``from runtime.plugins.zero3 import Zero3Plugin`` ...) unless a real top-level module of that name is already
importable. Sharded checkpoints pickle ``runtime.types.PpStatus`` by that path, so the alias is part of the
on-disk format (reference ``state/checkpoint.py:278-279``).
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import importlib.util
import sys

__version__ = "0.1.0"

_ALIASED = ("runtime", "parallel", "state", "data", "train", "models", "utils", "tools")


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, real_name: str) -> None:
        self.real_name = real_name

    def create_module(self, spec):
        return importlib.import_module(self.real_name)

    def exec_module(self, module) -> None:  # the real module is already initialised
        return None


class _AliasFinder(importlib.abc.MetaPathFinder):
    """Resolve ``runtime[.x]`` & co. to ``maltos_b200.runtime[.x]`` (same module objects, not copies)."""

    def __init__(self) -> None:
        self.enabled: set[str] = set()

    def find_spec(self, fullname, path=None, target=None):
        top = fullname.split(".", 1)[0]
        if top not in self.enabled:
            return None
        real = f"{__name__}.{fullname}"
        try:
            real_spec = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            return None
        if real_spec is None:
            return None
        spec = importlib.machinery.ModuleSpec(fullname, _AliasLoader(real), is_package=real_spec.submodule_search_locations is not None)
        if real_spec.submodule_search_locations is not None:
            spec.submodule_search_locations = list(real_spec.submodule_search_locations)
        return spec


_finder = _AliasFinder()


def install_aliases(force: bool = False) -> list[str]:
    """Enable the short import names. Names already provided by another distribution are left alone."""
    installed = []
    for name in _ALIASED:
        if name in _finder.enabled:
            installed.append(name)
            continue
        if not force:
            if name in sys.modules and not getattr(sys.modules[name], "__name__", "").startswith(__name__):
                continue
            try:
                other = importlib.machinery.PathFinder.find_spec(name, None)
            except (ImportError, ValueError):
                other = None
            if other is not None:
                continue
        _finder.enabled.add(name)
        installed.append(name)
    if _finder not in sys.meta_path:
        # In front of the path finder: `runtime.types` must resolve to the SAME module object as
        # `maltos_b200.runtime.types`, not to a second copy loaded from the aliased package's __path__.
        sys.meta_path.insert(0, _finder)
    return installed


install_aliases()
