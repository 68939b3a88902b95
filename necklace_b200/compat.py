"""Run a script written for the reference without editing its imports.

    import necklace_b200.compat; necklace_b200.compat.install()
    from necklace.trainer import tndszd            # -> necklace_b200.trainer.tndszd
    import necklace; necklace.init(0)              # -> necklace_b200.init

Or, with no edit at all (also covers processes the script spawns):

    PYTHONPATH=$(python -m necklace_b200.compat --path):$PYTHONPATH python their_script.py ...

``install()`` puts a finder on ``sys.meta_path`` that resolves ``necklace`` and every
``necklace.<sub>`` to the module of the same path under ``necklace_b200`` (the same module
object, not a copy).  It is opt-in: nothing is aliased unless a script asks for it, and a real
``necklace`` package that is already imported is left alone."""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

ALIAS, TARGET = "necklace", "necklace_b200"


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target):
        self.target = target

    def create_module(self, spec):
        return importlib.import_module(self.target)

    def exec_module(self, module):
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if fullname != ALIAS and not fullname.startswith(ALIAS + "."):
            return None
        real = TARGET + fullname[len(ALIAS):]
        try:
            found = importlib.util.find_spec(real)
        except ModuleNotFoundError:
            return None
        if found is None:
            return None
        return importlib.util.spec_from_loader(fullname, _AliasLoader(real),
                                               is_package=found.submodule_search_locations
                                               is not None)


def install(force: bool = False) -> bool:
    """Returns False (and does nothing) when another ``necklace`` is already imported, unless
    ``force`` (used by the stand-in package of ``alias_path()`` while it is being imported)."""
    mod = sys.modules.get(ALIAS)
    if mod is not None and getattr(mod, "__name__", "") != TARGET and not force:
        return False
    if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
        sys.meta_path.insert(0, _AliasFinder())
    return True


def alias_path() -> str:
    """Directory to put on ``PYTHONPATH`` so that ``import necklace`` works with no edit at all
    (it holds a one-file stand-in package that installs the alias when imported)."""
    import os
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "_alias")


def uninstall() -> None:
    sys.meta_path[:] = [f for f in sys.meta_path if not isinstance(f, _AliasFinder)]
    for name in [n for n in sys.modules if n == ALIAS or n.startswith(ALIAS + ".")]:
        if getattr(sys.modules[name], "__name__", "").startswith(TARGET):
            del sys.modules[name]


if __name__ == "__main__":
    if "--path" in sys.argv:
        print(alias_path())
    else:
        print(__doc__)
