"""Import name of the package that lives in the folder ``mormot2-ai_b200/``.

The folder's name carries a hyphen and so cannot stand in an ``import`` statement.
This module loads that folder as the package ``mormot2_ai_b200`` (one copy, under this one
name) and puts it in its own place in ``sys.modules``; ``import mormot2_ai_b200`` and
``import mormot2_ai_b200.config`` then work as for any package.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mormot2-ai_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_pkg = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _pkg
_spec.loader.exec_module(_pkg)
