"""B200 (sm_100a) implementation of the INT4 W4A4 linear-layer path.

Layout
    csrc/                  CUDA kernels, the C ABI (``include/wush_int4.h``) and the torch binding
    capi.py                ctypes view of the C ABI (what a foreign-language binding would call)
    _C                     compiled torch-facing operator module (same surface as the reference's ``my_int4._C``)
    rtn_int4.py            torch reference semantics of the quantiser (mirrors ``my_int4/rtn_int4.py``)
    wush_transform.py      offline transform solve / weight transform (mirrors ``my_int4/wush_transform.py``)
    linear.py              M-dispatching W4A4 linear layer and its N-sharded variant

The compiled pieces are required: importing ``_C`` (or ``my_int4``) without them raises
ImportError -- there is no CPU fallback.  ``python -m wush_int4_kernel_b200.build`` builds them.
"""
__version__ = "0.1.0"
