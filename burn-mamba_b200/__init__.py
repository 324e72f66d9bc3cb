"""B200-native (sm_100a) implementation of burn-mamba's SSM hot path.

The product is ``libbm_b200.so`` (hand-written CUDA behind the C ABI of ``include/bm_b200.h``);
this package is the host-side mirror of the reference crate's interface for that path.  The
directory name contains a hyphen, so it is loaded with ``__graft_entry__.load_package()`` (or any
``importlib`` spec loader) under the module name ``burn_mamba_b200``.
"""
from . import _ffi, mamba2, mamba3, ops, shard  # noqa: F401
from ._ffi import BmError, lib  # noqa: F401
from .mamba2 import Mamba2, Mamba2Cache, Mamba2SsdInput, Mamba2SsdPath  # noqa: F401
from .mamba3 import Mamba3  # noqa: F401
