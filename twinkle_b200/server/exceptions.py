"""Exception hierarchy of the server. Handlers map these to HTTP status codes in one place
(:func:`status_code_of`) instead of every route guessing.

Parity: reference ``src/twinkle/server/exceptions.py`` (``TwinkleServerError``, ``StateBackendError``, ``ConfigError``,
``ConfigParseError``, ``ResourceExhaustedError``) and ``server/state/backend/base.py`` (``ConcurrencyError``)."""
from __future__ import annotations

from typing import Optional, Sequence


class TwinkleServerError(Exception):
    """Base of every error the server raises on purpose."""
    status_code = 500


class StateBackendError(TwinkleServerError):
    """The shared state store failed: unreachable, timed out, unreadable document."""
    status_code = 503


class ConcurrencyError(StateBackendError):
    """An optimistic update kept losing against concurrent writers and gave up."""
    status_code = 409


class ConfigError(TwinkleServerError, ValueError):
    """A known configuration field holds a value outside its permitted set. Carries the field, the value and the
    permitted values so that the operator can fix the YAML entry without another start attempt."""
    status_code = 400

    def __init__(self, field: str, value: object, allowed: Optional[Sequence[str]] = None, message: Optional[str] = None):
        self.field, self.value, self.allowed = field, value, list(allowed) if allowed is not None else None
        if message is None:
            message = f'Invalid value for {field}: {value!r}' + (f', allowed: {self.allowed}' if self.allowed is not None else '')
        super().__init__(message)


class ConfigParseError(TwinkleServerError, ValueError):
    """The configuration source is not parseable (malformed YAML, a document that is not a mapping). Different from a
    validation error (parsed, but a rule is violated) and from ``FileNotFoundError`` (not readable at all)."""
    status_code = 400


class ResourceExhaustedError(TwinkleServerError, PermissionError):
    """A bounded resource is used up: adapter slots, per-token model quota, queue capacity."""
    status_code = 429


def status_code_of(exc: BaseException) -> int:
    """HTTP status for an exception: its ``status_code`` when it has one, 404 / 400 / 403 / 504 for the built-in lookup,
    value, permission and timeout errors, else 500."""
    code = getattr(exc, 'status_code', None)
    if isinstance(code, int):
        return code
    if isinstance(exc, (KeyError, FileNotFoundError)):
        return 404
    if isinstance(exc, TimeoutError):
        return 504
    if isinstance(exc, PermissionError):
        return 403
    if isinstance(exc, (ValueError, TypeError)):
        return 400
    return 500
