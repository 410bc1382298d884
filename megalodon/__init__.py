"""`megalodon` import paths of the reference (`megalodon.model.mega`, `megalodon.distributed`,
`megalodon.modules`, `megalodon.optim`, `megalodon.utils`, `megalodon.reloading`, ...) served by the
`megalodon_b200` implementation.  `import megalodon.x.y` returns the very same module object as
`import megalodon_b200.x.y`, so code written against the reference runs unchanged and both spellings
share one state (process groups, kernel extension, caches)."""
import importlib
import importlib.abc
import importlib.machinery
import sys

import megalodon_b200 as _impl

_PREFIX = __name__ + "."
_REAL = _impl.__name__ + "."


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        real = _REAL + fullname[len(_PREFIX):]
        try:
            module = importlib.import_module(real)
        except ModuleNotFoundError as e:
            if e.name == real:
                return None
            raise
        is_pkg = hasattr(module, "__path__")
        return importlib.machinery.ModuleSpec(fullname, self, is_package=is_pkg)

    def create_module(self, spec):
        return sys.modules[_REAL + spec.name[len(_PREFIX):]]

    def exec_module(self, module):
        pass


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

__version__ = _impl.__version__
__path__ = []          # sub-modules come from the finder above, never from the file system
