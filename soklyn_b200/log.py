"""Error types of the host mirror, one per variant of the reference's
`soklyn::log::Error` that the DenseBlock path can raise (src/util/log.rs:15-99)."""
from __future__ import annotations


class Error(Exception):
    """Base class (the reference's `Error` enum)."""


class DriverError(Error):
    pass


class MismatchedDimensions(Error):
    def __init__(self, reason: str, expected: int, found: int):
        super().__init__(f"Dimension mismatch: {reason}: expected {expected}, found {found}.")
        self.reason, self.expected, self.found = reason, expected, found


class AllocationLimitExceeded(Error):
    def __init__(self, received: int, max: int, reason: str):
        super().__init__(f"Allocation limit exceeded: {reason}: items received ({received}) exceeds maximum "
                         f"allowed allocation ({max}).")
        self.received, self.max, self.reason = received, max, reason


class InvalidConfiguration(Error):
    def __init__(self, reason: str):
        super().__init__(f"Invalid network configuration: {reason}")
        self.reason = reason


class InvalidBatchSize(Error):
    def __init__(self, reason: str):
        super().__init__(f"Batch size constraint violation: {reason}")
        self.reason = reason


class TrainingModeRequired(Error):
    def __init__(self, reason: str):
        super().__init__(f"Invalid operation: {reason}: Action requires the network to be in training mode.")
        self.reason = reason


class HardwareConstraintViolation(Error):
    def __init__(self, precision, expected: int, found: int):
        super().__init__(f"Hardware acceleration constraint violation: Precision is {precision}, which requires a "
                         f"tile dimension of {expected}, but found {found}.")
        self.precision, self.expected, self.found = precision, expected, found


class UnsupportedTypeCast(Error):
    def __init__(self, src, dst):
        super().__init__(f"Unsupported precision cast operation: Cannot convert data from {src} to {dst}")


class NativeError(Error):
    """A status code of the C ABI that has no counterpart in the reference."""


_BY_STATUS = {1: DriverError, 2: MismatchedDimensions, 3: AllocationLimitExceeded, 4: InvalidConfiguration,
              5: InvalidBatchSize, 6: TrainingModeRequired, 7: HardwareConstraintViolation, 8: UnsupportedTypeCast}


def raise_status(status: int, detail: str):
    """Turn a non-zero status of the C ABI into the matching exception. The host mirror
    checks arguments itself first (with the reference's messages); this is the net for
    anything only the native side sees."""
    if status == 0:
        return
    cls = _BY_STATUS.get(status, NativeError)
    err = cls.__new__(cls)
    Exception.__init__(err, f"[status {status}] {detail}")
    raise err
