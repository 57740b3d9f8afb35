"""Import alias for the package that lives in ``p4app-switchML_b200/``.

The project directory carries the name of the project it re-implements, and that name
holds a hyphen, which ``import`` cannot spell. This module gives it an importable name:
``import switchml_b200`` runs the real ``__init__`` and every submodule
(``switchml_b200.ops``, ``switchml_b200.parallel`` ...) resolves inside that directory.
"""
import os as _os

_real = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))),
                      "p4app-switchML_b200")
__path__ = [_real]
with open(_os.path.join(_real, "__init__.py")) as _f:
    exec(compile(_f.read(), _os.path.join(_real, "__init__.py"), "exec"))
del _f
