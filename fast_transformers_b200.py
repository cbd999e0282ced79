"""Import shim: the package sources live in the directory ``fast-transformers_b200/`` (a
name Python cannot import directly).  Importing ``fast_transformers_b200`` executes that
directory's ``__init__.py`` under this module name and lets sub-modules resolve there."""
import os as _os

__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)),
                          "fast-transformers_b200")]
__package__ = __name__
if __spec__ is not None:
    __spec__.submodule_search_locations = __path__
__file__ = _os.path.join(__path__[0], "__init__.py")
with open(__file__) as _f:
    exec(compile(_f.read(), __file__, "exec"))
del _f, _os
