"""B200-native INT8 quantized linear: hand-written sm_100a CUDA behind the fwd_32 / bwd_33
operator surface of jiaoch/Triton-INT8.  Host code is Python/torch; all compute goes through the
C ABI of libi8linear.so (see include/i8linear.h).  There is no CPU or eager fallback."""
from . import _lib
from ._lib import I8LError

__all__ = ["_lib", "I8LError", "block_channel", "double_channel", "fused", "kernels", "linear"]


def __getattr__(name):
    if name in ("block_channel", "double_channel", "fused", "kernels", "linear", "tp"):
        import importlib
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
