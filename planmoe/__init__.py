"""Import alias: ``planmoe.X`` is ``planmoe_b200.X`` (same module objects).

``planmoe`` is the name used by the reference's README; ``schemoe`` is the name its code and its
Megatron / fairseq patches import (``from schemoe.moe import moe_layer``)."""

import importlib
import importlib.abc
import importlib.util
import sys

import planmoe_b200 as _impl
from planmoe_b200 import *  # noqa: F401,F403
from planmoe_b200 import moe, net, system, jit  # noqa: F401

_PREFIX = __name__ + '.'


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        real = 'planmoe_b200.' + fullname[len(_PREFIX):]
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except ModuleNotFoundError:
            return None
        return importlib.util.spec_from_loader(fullname, self, origin=real)

    def create_module(self, spec):
        return importlib.import_module(spec.origin)

    def exec_module(self, module):
        pass


sys.meta_path.insert(0, _AliasFinder())
for _name in ('moe', 'net', 'system', 'jit'):
    sys.modules[_PREFIX + _name] = getattr(_impl, _name)
__version__ = _impl.__version__
