"""Import name of the package in the folder `ember.cpp_b200/` (a dot cannot be part of a module
name): `import ember_cpp_b200` loads that folder as a package under this name."""
import importlib.util
import os
import sys

_here = os.path.dirname(os.path.abspath(__file__))
_pkg = os.path.join(_here, "ember.cpp_b200")
_spec = importlib.util.spec_from_file_location(__name__, os.path.join(_pkg, "__init__.py"),
                                               submodule_search_locations=[_pkg])
_module = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
