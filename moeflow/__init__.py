"""Import alias for call sites written against the reference's package name.

``import moeflow``, ``from moeflow.fixed import FixedEPLayer``, ``import moeflow.integrations.vllm_plugin`` and
so on resolve to the modules of :mod:`moeflow_b200` — the very same module objects, not copies, so classes
and module-level state (the runner's buffer pool, the plugin's registration flags) are shared whichever name
is used.  Nothing is imported eagerly; a submodule is loaded when it is first asked for.
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

import moeflow_b200 as _impl
from moeflow_b200 import *  # noqa: F401,F403  (MoEConfig, GLM53_FLASH, ...)

_PREFIX = __name__ + "."
_TARGET = _impl.__name__


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """Maps ``moeflow.<x>`` onto the already importable ``moeflow_b200.<x>``."""

    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        real = _TARGET + fullname[len(__name__):]
        if importlib.util.find_spec(real) is None:
            return None
        return importlib.util.spec_from_loader(fullname, self)

    def create_module(self, spec):
        module = importlib.import_module(_TARGET + spec.name[len(__name__):])
        self._real_spec = getattr(self, "_real_spec", {})
        self._real_spec[spec.name] = module.__spec__
        return module

    def exec_module(self, module):
        # The real module has been executed under its own name already; the import machinery has just stamped the
        # alias spec on it, so put its own spec back (reload and pickling keep working under the real name).
        for alias, real in getattr(self, "_real_spec", {}).items():
            if sys.modules.get(alias) is module:
                module.__spec__ = real


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

__path__ = []  # a package without files of its own: every submodule comes from the finder above
__all__ = list(getattr(_impl, "__all__", []))
