"""Error taxonomy of the scan path, one class per variant of the reference's
`Error` enum that this path can raise (src/error.rs:9-48), plus the two that only
exist on this side of the C ABI (a CUDA failure, a bounded device wait giving up).
"""
from __future__ import annotations


class Mamba3Error(Exception):
    """Base of every failure that is not a programming bug."""


class ConfigError(Mamba3Error):
    """Error::Config - a configuration is internally inconsistent."""


class ShapeError(Mamba3Error):
    """Error::Shape - extents that cannot be reconciled."""


class RankError(Mamba3Error):
    """Error::Rank { expected, got, shape }."""

    def __init__(self, expected: int, got: int, shape):
        self.expected, self.got, self.shape = expected, got, tuple(shape)
        super().__init__(f"expected rank {expected}, got {got} (shape {list(shape)})")


class AutodiffError(Mamba3Error):
    """Error::Autodiff - a gradient that does not exist was asked for."""


class UnsupportedError(Mamba3Error):
    """Error::Unsupported - recognised but not served by this path."""


class CudaError(Mamba3Error):
    """A CUDA runtime call failed inside the library."""


class DeviceTimeout(Mamba3Error):
    """A bounded device-side wait gave up (the context stays usable)."""


class NullError(Mamba3Error):
    """A required buffer was not supplied."""


_BY_STATUS = {1: ShapeError, 3: ConfigError, 4: UnsupportedError, 5: CudaError,
              6: DeviceTimeout, 7: NullError}


def from_status(code: int, message: str) -> Mamba3Error:
    """Map an m3_status (include/m3scan.h) and its message to an exception."""
    cls = _BY_STATUS.get(code, Mamba3Error)
    return cls(message or f"m3scan status {code}")
