"""Import alias: ``import mps_bitsandbytes_b200`` loads the package in ``mps-bitsandbytes_b200/``.

A directory name with a hyphen cannot be imported directly; this module loads that
directory as the package ``mps_bitsandbytes_b200`` and replaces itself with it in
``sys.modules``, so submodules (``mps_bitsandbytes_b200.functional``, ``.nn``) resolve.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mps-bitsandbytes_b200")
_spec = importlib.util.spec_from_file_location(
    "mps_bitsandbytes_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["mps_bitsandbytes_b200"] = _mod
_spec.loader.exec_module(_mod)
