"""Exception classes named after the reference's (tfcc/core/exceptions/)."""


class TFCCError(Exception):
    """Base of every error this package raises (tfcc::Exception)."""


class InvalidArgumentError(TFCCError):
    """Shape or argument rejected before any launch (tfcc::InvalidArgumentError)."""


class NotImplementedError(TFCCError):  # noqa: A001 - mirrors the reference's name
    """dtype or feature the backend does not provide (tfcc::NotImplementedError)."""


class ResourceExhaustedError(TFCCError):
    """Device allocation failed (tfcc::ResourceExhaustedError)."""


class RuntimeError(TFCCError):  # noqa: A001 - mirrors the reference's name
    """CUDA failure or a device-side give-up reported by the kernel library."""

    def __init__(self, status: int, message: str):
        super().__init__(f"tfcc_b200 status {status}: {message}")
        self.status = status
