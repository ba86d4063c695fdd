"""mlx_rs_b200 - B200-native quantized mixture-of-experts path behind the mlx-rs op surface.

The directory is named `mlx-rs_b200`; import it as `mlx_rs_b200` through
`__graft_entry__.load_package()` (or any importlib loader pointing at this file).

Everything here drives `libb200moe.so` (hand-written sm_100a CUDA behind the C ABI of
`include/b200_moe.h`) through ctypes.  torch is used for device memory and streams only.
There is no CPU fallback: without the library, or without a B200, calls raise.
"""
from ._lib import B200Error, Context, default_context, lib, library_path  # noqa: F401
from . import ops, nn  # noqa: F401

__all__ = ["B200Error", "Context", "default_context", "lib", "library_path", "ops", "nn"]
