"""B200-native Mixture-of-Experts layer behind the Mixture-of-Kittens Python API.

`mok.ops` holds the ten `mok::*` custom operators, `mok.functional` the workspace / schedule /
forward / backward layer on top of them.  The kernels live in libmok_b200.so (sm_100a only);
importing this package fails if that library has not been built.
"""
import torch  # noqa: F401

from . import _lib as _lib
from . import ops as ops
from . import _fake_impls as _fake_impls
from . import functional as functional
from . import nn as nn
from ._lib import last_status, raise_for_status

__version__ = "0.1.0"

__all__ = ["__version__", "functional", "nn", "ops", "last_status", "raise_for_status"]
