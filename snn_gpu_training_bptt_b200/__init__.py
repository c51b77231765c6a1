"""B200-native LIF fire / BPTT hot path behind the reference's ``snnlib`` operator API.

Layout
    csrc/             hand-written sm_100a kernels + the C ABI (libsnn_b200.so, include/snn_b200.h)
    _capi.py          ctypes binding of that C ABI (raises if the library is missing)
    snnlib/           drop-in for the reference's compiled ``snnlib`` module (function table)
    snnlib_func.py    autograd Functions + hyper-parameter globals (mirror of the reference's)
    snnlib_op.py      nn.Module layers (mirror of the reference's)
    build.py          in-tree nvcc build
"""
import sys

__version__ = "0.1.0"


def install_as_snnlib():
    """Register this package's op table, Functions and layers under the reference's
    top-level module names (``snnlib``, ``snnlib_func``, ``snnlib_op``) so code written
    against the reference (``import snnlib_op as sop``) imports them unchanged."""
    from . import snnlib, snnlib_func, snnlib_op
    sys.modules.setdefault("snnlib", snnlib)
    sys.modules.setdefault("snnlib_func", snnlib_func)
    sys.modules.setdefault("snnlib_op", snnlib_op)
    return snnlib
