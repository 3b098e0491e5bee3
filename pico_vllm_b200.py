"""Import shim for the package whose source folder is ``pico-vllm_b200/``.

A folder name with a hyphen cannot be written in an ``import`` statement, so this
module loads ``pico-vllm_b200/__init__.py`` under the importable name
``pico_vllm_b200`` and replaces itself with that package in ``sys.modules``.
After ``import pico_vllm_b200`` every submodule (``pico_vllm_b200.config`` …)
resolves inside the hyphenated folder.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "pico-vllm_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir]
)
_pkg = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _pkg
_spec.loader.exec_module(_pkg)
