"""Import door for the package directory `renderformer-cuda_b200/` (a hyphen is not a valid
Python identifier). Importing this module yields that package: it turns itself into a
package whose `__path__` is the directory, then runs the directory's `__init__.py`, so
`import renderformer_cuda_b200.ops` resolves to `renderformer-cuda_b200/ops.py`."""
import os as _os

__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "renderformer-cuda_b200")]
__package__ = __name__
if __spec__ is not None:
    __spec__.submodule_search_locations = __path__
with open(_os.path.join(__path__[0], "__init__.py")) as _f:
    exec(compile(_f.read(), _os.path.join(__path__[0], "__init__.py"), "exec"))
del _f
