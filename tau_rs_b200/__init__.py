"""Import name of the library whose sources live in the folder `tau.rs_b200/`.

A folder name with a dot in it cannot be imported, so this module loads that folder's
`__init__.py` under the name `tau_rs_b200` and lets every submodule
(`tau_rs_b200.config`, `tau_rs_b200.engine`, ...) resolve inside it.
"""
import importlib.util
import os
import sys

_sources = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tau.rs_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_sources, "__init__.py"), submodule_search_locations=[_sources]
)
_module = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
