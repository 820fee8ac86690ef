"""Import name of the package that lives in the folder ``mormot2-ai_b200/``.

The folder's name carries a hyphen and so cannot stand in an ``import`` statement.
This module loads that folder as the package ``mormot2_ai_b200`` (one copy, under this one
name) and puts it in its own place in ``sys.modules``; ``import mormot2_ai_b200`` and
``import mormot2_ai_b200.config`` then work as for any package, and
``python -m mormot2_ai_b200 ...`` runs its command line.
"""
import importlib.util
import os
import sys

_NAME = "mormot2_ai_b200"
_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mormot2-ai_b200")


def _load():
    if _NAME in sys.modules and hasattr(sys.modules[_NAME], "__path__"):
        return sys.modules[_NAME]
    spec = importlib.util.spec_from_file_location(
        _NAME, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
    pkg = importlib.util.module_from_spec(spec)
    sys.modules[_NAME] = pkg
    spec.loader.exec_module(pkg)
    return pkg


_pkg = _load()
if __name__ == "__main__":
    from mormot2_ai_b200.cli import main
    sys.exit(main())
