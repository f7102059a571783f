"""Import shim: the package lives in the folder ``vllm-cpp_b200`` (the project's
name, which is not a Python identifier); ``import vllm_cpp_b200`` loads it."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "vllm-cpp_b200")
_spec = importlib.util.spec_from_file_location(
    "vllm_cpp_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["vllm_cpp_b200"] = _mod
_spec.loader.exec_module(_mod)
