"""Import name of the package whose sources live in the folder
``semantic-aware_adaptive_kv_cache_precision_b200/``.

The folder carries the project's name, which has a hyphen and so cannot be
written in an ``import`` statement. This module stands in for it: it points
``__path__`` at the folder, so that every sub-package is found there, and runs
the folder's ``__init__.py`` in its own namespace. Run with ``python -m`` it is
the command line (``cli.py`` of the package).
"""

import os as _os

if __name__ == "__main__":
    import sys as _sys
    from importlib import import_module as _import
    _sys.path.insert(0, _os.path.dirname(_os.path.abspath(__file__)))
    _sys.exit(_import("semantic_aware_adaptive_kv_cache_precision_b200.cli").main())

_HOME = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)),
                      "semantic-aware_adaptive_kv_cache_precision_b200")
__path__ = [_HOME]
__package__ = __name__
if __spec__ is not None:
    __spec__.submodule_search_locations = __path__

with open(_os.path.join(_HOME, "__init__.py"), encoding="utf-8") as _f:
    exec(compile(_f.read(), _os.path.join(_HOME, "__init__.py"), "exec"))
del _f
