"""Import alias: lets code that imports the package name ``flexkv`` find ``flexkv_b200``.

Serving engines ship connector shims that import the reference's module paths, for instance vLLM's
``FlexKVConnectorV1`` does ``from flexkv.integration.vllm.vllm_v1_adapter import FlexKVConnectorV1Impl``.
With this directory's parent on ``PYTHONPATH`` (``export PYTHONPATH=<repo>/compat:<repo>``) those imports
resolve to the very same module objects as ``flexkv_b200.…``: nothing is loaded twice and no engine needs a
patch. Do not install it beside the reference package itself.
"""
import importlib
import importlib.abc
import importlib.machinery
import sys

_REAL = "flexkv_b200"
_ALIAS = __name__


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, name, path=None, target=None):
        if name == _ALIAS or name.startswith(_ALIAS + "."):
            real = _REAL + name[len(_ALIAS):]
            try:
                found = importlib.util.find_spec(real)
            except (ImportError, ValueError):
                found = None
            if found is None:
                return None
            return importlib.machinery.ModuleSpec(name, self, is_package=found.submodule_search_locations is not None)
        return None

    def create_module(self, spec):
        return importlib.import_module(_REAL + spec.name[len(_ALIAS):])      # the one and only module object

    def exec_module(self, module):
        pass


import importlib.util  # noqa: E402

if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())
sys.modules[_ALIAS] = importlib.import_module(_REAL)
