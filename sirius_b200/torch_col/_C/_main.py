"""torch_col._C._main: the module path of the reference's Cython extension (pytorch/setup.py:101-114,
cython/main.pyx). The implementation lives in the package's __init__; this module re-exports every public
name, so `from torch_col._C._main import X` keeps working."""
import sys as _sys

_impl = _sys.modules[__name__.rsplit('.', 1)[0]]
globals().update({k: v for k, v in vars(_impl).items() if not k.startswith('_') or k in ('_DynamicBatchDistirbutor', '_PerfModel')})
__all__ = [k for k in globals() if not k.startswith('_')]
