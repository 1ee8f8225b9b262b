"""Exception classes, with the names and bases of the reference's
python/quabla/_errors.py so that `except ValueError` handlers keep working."""

__all__ = ["QuablaError", "TracerError", "UnsupportedOperationError"]


class QuablaError(Exception):
    """Base class of the errors specific to this backend."""


class UnsupportedOperationError(QuablaError, ValueError, NotImplementedError):
    """An operation, transform or composition the B200 backend does not
    implement.  `op` names it and `device` is the target device."""

    def __init__(self, message, *, op=None, device=None):
        super().__init__(message)
        self.op = op
        self.device = device


class TracerError(QuablaError, TypeError):
    """A traced value was used where a concrete value is required."""
