"""Error types of the attention path, one per `PotError` variant that the path
can raise (reference: src/error.rs:7-40)."""
from __future__ import annotations

BP_OK = 0
BP_ERR_CONFIG = 1
BP_ERR_CONTEXT_OVERFLOW = 2
BP_ERR_PREFILL_TOO_LARGE = 3
BP_ERR_DEVICE_LOST = 4
BP_ERR_CUDA = 5
BP_ERR_TIMEOUT = 6
BP_ERR_NULL = 7
BP_ERR_IO = 8


class PotError(Exception):
    """Base class; `status` is the C-ABI status code."""

    status = -1

    def __init__(self, message: str, **fields):
        super().__init__(message)
        self.fields = fields
        for k, v in fields.items():
            setattr(self, k, v)


class ConfigError(PotError):
    """`PotError::Config(&str)`."""
    status = BP_ERR_CONFIG


class ContextOverflow(PotError):
    """`PotError::ContextOverflow { pos, n, max }`."""
    status = BP_ERR_CONTEXT_OVERFLOW


class PrefillTooLarge(PotError):
    """`PotError::PrefillTooLarge { n, max }`."""
    status = BP_ERR_PREFILL_TOO_LARGE


class DeviceLost(PotError):
    """`PotError::DeviceLost`."""
    status = BP_ERR_DEVICE_LOST


class CudaError(PotError):
    """A CUDA call failed, or no CUDA device / extension is present. There is no CPU path."""
    status = BP_ERR_CUDA


class IoError(PotError):
    """`PotError::Io { path, source }`: a file of the model directory could not be read."""
    status = BP_ERR_IO


class DeviceTimeout(PotError):
    """A bounded device-side wait gave up."""
    status = BP_ERR_TIMEOUT


_BY_STATUS = {cls.status: cls for cls in (ConfigError, ContextOverflow, PrefillTooLarge, DeviceLost, CudaError, DeviceTimeout, IoError)}


def raise_for_status(status: int, message: str, **fields):
    if status == BP_OK:
        return
    cls = _BY_STATUS.get(status, PotError)
    raise cls(message or f"status {status}", **fields)
