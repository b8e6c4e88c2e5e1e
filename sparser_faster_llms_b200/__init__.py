"""B200-native (sm_100a) activation-sparse gated-FFN kernels behind the module
surface of SakanaAI/sparser-faster-llms.

* :mod:`.twell` - replacement for ``custom_models.twell_modules.twell``
  (TwELL / TwELL-flex inference modules and functions).
* :mod:`.dropin` - registers the replacements under the reference's module names
  so the reference's scripts run unchanged.
* :mod:`._lib` - ctypes binding of the C-ABI library declared in
  ``include/b200_sparse_ffn.h``.

Importing the package does not load the CUDA library; the first operator call
does, and raises if it is missing (there is no CPU fallback).
"""
from . import _lib  # noqa: F401
from ._lib import B200Error, load_library  # noqa: F401

__all__ = ["B200Error", "load_library", "twell", "dropin"]
__version__ = "0.1.0"
