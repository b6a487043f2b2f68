"""Import shim: ``import bitnet_c_b200`` loads the package that lives in ``bitnet.c_b200/``.

The package folder carries the project's name, which holds a dot and so cannot be
written in an ``import`` statement.  This module loads that folder as a regular
package under the importable name ``bitnet_c_b200`` and replaces itself with it
in ``sys.modules``; submodules (``bitnet_c_b200.config`` and so on) then resolve
through the package's ``__path__`` like those of any other package.
"""
import importlib.util as _ilu
import os as _os
import sys as _sys

_dir = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "bitnet.c_b200")
_spec = _ilu.spec_from_file_location(
    __name__, _os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir]
)
_pkg = _ilu.module_from_spec(_spec)
_sys.modules[__name__] = _pkg
_spec.loader.exec_module(_pkg)
