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
