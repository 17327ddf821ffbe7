"""nncase_b200 -- B200 (sm_100a) kernels behind nncase's `cuda` module.

The product is the C-ABI library ``libnncase_b200.so`` (declared in ``include/nncase_b200.h``);
this package is its Python host side: a ctypes binding (``nncase_b200.lib``) and wrappers
named after the reference's ``kernels::stackvm`` operators (``nncase_b200.kernels``), the
kmodel writer / reader for the ``cuda`` module kind (``nncase_b200.kmodel``) and a ``Simulator``
with the surface of the reference's Python interpreter binding (``nncase_b200.simulator``).
There is no CPU fallback: without the built library, or without a B200, calls raise.
"""
from . import lib  # noqa: F401
from .lib import NncbError, load  # noqa: F401

__all__ = ["lib", "kernels", "kmodel", "simulator", "load", "NncbError"]
