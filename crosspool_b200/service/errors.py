"""Typed errors of the control plane and their HTTP mapping (reference: src/xpool/service/errors.py)."""

from __future__ import annotations


class DaemonError(Exception):
    """An error the daemon answers with; ``code`` decides the HTTP status."""

    STATUS = {"conflict": 409, "not_ready": 503, "not_found": 404, "invalid": 422, "mismatch": 409, "gone": 410}

    def __init__(self, code: str, message: str):
        super().__init__(message)
        self.code, self.message = code, message

    @property
    def http_status(self) -> int:
        return self.STATUS.get(self.code, 400)

    @property
    def is_recoverable(self) -> bool:
        """True when retrying later can succeed (the daemon is merely not there yet)."""
        return self.code == "not_ready"


class ClientError(Exception):
    """Transport-level failure talking to the daemon (unreachable, timeout, bad payload)."""
