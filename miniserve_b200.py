"""Import name of the package that lives in ``miniserve-llm-nv_b200/``.

The folder's name is not a Python identifier, so ``import miniserve_b200`` loads
this file, which registers the folder as the package ``miniserve_b200`` and
stands aside: afterwards ``miniserve_b200.config`` and the other subpackages
import as usual.
"""

import importlib.util as _util
import pathlib as _pathlib
import sys as _sys

_root = _pathlib.Path(__file__).resolve().parent / "miniserve-llm-nv_b200"
_spec = _util.spec_from_file_location(
    "miniserve_b200", _root / "__init__.py", submodule_search_locations=[str(_root)])
_package = _util.module_from_spec(_spec)
_sys.modules["miniserve_b200"] = _package
_spec.loader.exec_module(_package)
