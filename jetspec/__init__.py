"""Import alias: ``jetspec`` resolves to :mod:`jetspec_b200`.

Code written against the reference package's import names (``from jetspec import LLM``,
``from jetspec.inference_engine import JetSpecEngine``, ``from jetspec.tree import get_algorithm``,
``from jetspec.draft_head_adapter import GraphedDraftHead`` ...) runs on this framework unchanged.
Module names that differ are mapped one to one below; everything else under ``jetspec.`` is looked up
under ``jetspec_b200.`` with the same dotted tail.

The alias steps aside when another ``jetspec`` package is importable from a later ``sys.path`` entry
(a checkout or install of the reference itself): that package is loaded under the name instead, so a
process that put the reference on its path keeps getting the reference.
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))

# reference module name -> module of this framework that provides the same public names
_RENAMED = {
    "jetspec.inference_engine": "jetspec_b200.engine",
    "jetspec.inference_engine.engine": "jetspec_b200.engine.engine",
    "jetspec.inference_engine.scheduler": "jetspec_b200.runtime.scheduler",
    "jetspec.inference_engine.paged_kv_cache": "jetspec_b200.runtime.kv_pool",
    "jetspec.inference_engine.attn_metadata": "jetspec_b200.runtime.attn_metadata",
    "jetspec.draft": "jetspec_b200.drafters",
    "jetspec.draft_head_adapter": "jetspec_b200.drafters",
    "jetspec.core.sampler": "jetspec_b200.sampling",
    "jetspec.models.draft_head": "jetspec_b200.models.draft_head",
    "jetspec.models.qwen3": "jetspec_b200.models.qwen3",
}


def _other_jetspec():
    """``__init__.py`` of a different ``jetspec`` package further along ``sys.path``, if there is one."""
    for entry in sys.path:
        cand = os.path.join(entry or os.getcwd(), "jetspec", "__init__.py")
        if os.path.isfile(cand) and os.path.dirname(os.path.abspath(cand)) != _HERE:
            return cand
    return None


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if fullname == "jetspec" or not fullname.startswith("jetspec."):
            return None
        return importlib.util.spec_from_loader(fullname, self)

    def create_module(self, spec):
        real = _RENAMED.get(spec.name, "jetspec_b200." + spec.name[len("jetspec."):])
        return importlib.import_module(real)

    def exec_module(self, module):       # the real module is already initialised
        return None


_ref = _other_jetspec()
if _ref is not None:
    _spec = importlib.util.spec_from_file_location("jetspec", _ref, submodule_search_locations=[os.path.dirname(_ref)])
    _mod = importlib.util.module_from_spec(_spec)
    sys.modules["jetspec"] = _mod
    _spec.loader.exec_module(_mod)
else:
    import jetspec_b200 as _impl
    if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
        sys.meta_path.insert(0, _AliasFinder())
    sys.modules["jetspec"] = _impl
