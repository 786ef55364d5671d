"""kaio_b200: sm_100a (B200) implementation of KAIO's quantized-inference ops.

``kaio_b200.ops`` mirrors the ``kaio-ops`` entry points over the C ABI of
``libkaio_b200.so`` (``include/kaio_b200.h``); ``kaio_b200.build`` compiles the library.
"""
from .errors import (CudaError, DeviceTimeout, InvalidConfig, KaioError,  # noqa: F401
                     UnsupportedArch)

__all__ = ["KaioError", "InvalidConfig", "CudaError", "UnsupportedArch", "DeviceTimeout"]
