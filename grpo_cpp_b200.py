"""Import alias: ``import grpo_cpp_b200`` loads the package directory ``grpo.cpp_b200/``.

The package directory carries the reference's name, which has a dot in it and so is not a
valid Python identifier; this one-file alias registers it under an importable name.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "grpo.cpp_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
