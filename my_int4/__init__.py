"""Drop-in ``my_int4`` package: same import surface as rib12316/WUSH_int4_kernel.

``my_int4._C`` is the compiled operator module of ``wush_int4_kernel_b200`` (sm_100a kernels);
``my_int4.rtn_int4`` and ``my_int4.wush_transform`` are the torch-level semantics and the
offline transform pipeline.  As in the reference (``my_int4/__init__.py:4-6``) importing the
package requires the compiled extension: there is no CPU fallback.
"""
import sys as _sys

import torch  # noqa: F401  (torch first: it owns the CUDA runtime libraries the extension links to)

from wush_int4_kernel_b200 import _C, rtn_int4, wush_transform

_sys.modules[__name__ + "._C"] = _C
_sys.modules[__name__ + ".rtn_int4"] = rtn_int4
_sys.modules[__name__ + ".wush_transform"] = wush_transform

quant_int4 = _C.quant_int4

# The reference's scripts also import `block_transform` / `compute_gram` by name once
# `my_int4.wush_transform` has put an external WUSH checkout on sys.path
# (my_int4/wush_transform.py:15-24, tests/test_sw1.py:30).  With no such checkout importable,
# this package's own implementations answer to those names.
import importlib.util as _ilu  # noqa: E402

for _name in ("block_transform", "compute_gram"):
    if _name not in _sys.modules and _ilu.find_spec(_name) is None:
        from wush_int4_kernel_b200 import block_compat as _compat

        _sys.modules[_name] = _compat
