"""Import shim: ``import fairseq_apollo_b200`` loads the package that lives in the
directory ``fairseq-apollo_b200/`` (a hyphen is not a valid Python identifier)."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fairseq-apollo_b200")
_spec = importlib.util.spec_from_file_location(
    "fairseq_apollo_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["fairseq_apollo_b200"] = _mod
_spec.loader.exec_module(_mod)
