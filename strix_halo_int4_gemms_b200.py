"""Import alias: ``import strix_halo_int4_gemms_b200`` loads the package directory
``strix-halo-int4-gemms_b200/`` (whose name is not a Python identifier)."""
import importlib.util
import os
import sys

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "strix-halo-int4-gemms_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_DIR, "__init__.py"), submodule_search_locations=[_DIR]
)
_module = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
