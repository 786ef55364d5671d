"""Error type mirroring ``KaioError`` (kaio-runtime/src/error.rs:4-37)."""
from __future__ import annotations

OK = 0
ERR_INVALID_CONFIG = 1
ERR_CUDA = 2
ERR_UNSUPPORTED_ARCH = 3
ERR_TIMEOUT = 4


class KaioError(Exception):
    """Base class; ``code`` is the C-ABI status code."""

    code = -1

    def __init__(self, message: str):
        super().__init__(message)
        self.message = message


class InvalidConfig(KaioError):
    """``KaioError::InvalidConfig``: the message text is the reference's."""
    code = ERR_INVALID_CONFIG


class CudaError(KaioError):
    """``KaioError::Cuda``."""
    code = ERR_CUDA


class UnsupportedArch(KaioError):
    """Analogue of ``ValidationError::SmTooLow``: the device is not sm_100."""
    code = ERR_UNSUPPORTED_ARCH


class DeviceTimeout(KaioError):
    """A bounded device-side wait gave up; the context stays usable."""
    code = ERR_TIMEOUT


_BY_CODE = {c.code: c for c in (InvalidConfig, CudaError, UnsupportedArch, DeviceTimeout)}


def from_code(code: int, message: str) -> KaioError:
    return _BY_CODE.get(code, KaioError)(message)
