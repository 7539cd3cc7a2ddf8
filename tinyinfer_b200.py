"""Import alias for the package that lives in the folder ``tinyinfer.cpp_b200``.

The folder carries the project's name, which is not a Python identifier, so it
cannot be imported by that name.  ``import tinyinfer_b200`` finds this file,
which loads the folder as a regular package under the name ``tinyinfer_b200``
(sub-modules such as ``tinyinfer_b200.config`` resolve inside the folder).
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tinyinfer.cpp_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_module = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
