"""Import-compatibility alias: ``monarch`` and every ``monarch.<submodule>`` resolve to
``monarch_b200`` and ``monarch_b200.<submodule>``.

Programs written against the reference's package name keep their imports:

    from monarch.actor import Actor, endpoint, this_host
    from monarch.tensor_engine import RDMABuffer
    import monarch; monarch.remote, monarch.DeviceMesh, monarch.timer ...

The alias adds no code of its own: a meta-path finder hands out the very module objects of
``monarch_b200`` (so ``monarch.actor.Actor is monarch_b200.actor.Actor``).  Names that exist
only in the reference (legacy mesh constructors for its older back ends, scheduler-specific
helpers) are not provided; looking one up raises ``AttributeError`` naming the gap.
"""
import importlib
import importlib.abc
import importlib.machinery
import importlib.util
import sys

import monarch_b200 as _impl

_PREFIX = __name__ + "."
_TARGET = _impl.__name__ + "."


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str):
        self._target = target

    def create_module(self, spec):
        return importlib.import_module(self._target)

    def exec_module(self, module):      # the target module is already initialised
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        real = _TARGET + fullname[len(_PREFIX):]
        try:
            found = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            found = None
        if found is None:
            return None
        spec = importlib.machinery.ModuleSpec(fullname, _AliasLoader(real),
                                              is_package=found.submodule_search_locations is not None)
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

__version__ = _impl.__version__


def __getattr__(name):
    try:
        return getattr(_impl, name)
    except AttributeError:
        raise AttributeError(f"monarch (monarch_b200) has no attribute {name!r}") from None


def __dir__():
    return dir(_impl)
