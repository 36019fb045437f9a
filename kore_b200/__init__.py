"""kore_b200 — B200-native (sm_100a) BitLinear / QuatLinear forward for KORE.

The package is a thin host layer over ``libkore_b200.so`` (C ABI in
``include/kore_b200.h``): ``nn`` mirrors KORE's module API, ``kernels`` mirrors the
kore-kernels function API.  There is no CPU implementation in this package.
"""
from . import _cabi
from ._cabi import KoreError
from .nn import BitLinear, QLoraLinear, QuatLinear

__all__ = ["BitLinear", "QuatLinear", "QLoraLinear", "KoreError", "_cabi"]
__version__ = "0.1.0"
