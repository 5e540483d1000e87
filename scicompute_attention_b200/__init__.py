"""B200-native attention runtime: hand-written sm_100a kernels behind a C ABI
(include/sca_b200.h), a C++ host layer with the reference's public API, and this thin Python
harness (device memory, streams and torch.distributed come from PyTorch; the math does not)."""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
__version__ = "0.1.0"
