"""Import alias for the package directory ``turboquant.cpp_b200``.

The package directory carries a dot in its name, which the import statement
cannot spell.  Importing this module loads that directory as the package
``turboquant_cpp_b200`` (sub-packages included), so

    import turboquant_cpp_b200 as tq
    from turboquant_cpp_b200.engine import Engine

work from the repository root or from anywhere once the root is on sys.path.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "turboquant.cpp_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
