"""Import name of the package in ``go-tinygrad_b200/``.

A hyphen cannot appear in a Python module name, so this module loads the
package from its folder and installs it as ``go_tinygrad_b200``:
``import go_tinygrad_b200`` and ``from go_tinygrad_b200.engine import Model``
then work as for any package.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "go-tinygrad_b200")
_spec = importlib.util.spec_from_file_location(
    "go_tinygrad_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_module = importlib.util.module_from_spec(_spec)
sys.modules["go_tinygrad_b200"] = _module
_spec.loader.exec_module(_module)
