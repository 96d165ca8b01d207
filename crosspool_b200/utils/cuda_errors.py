"""Classification of CUDA failures.

A *terminal* device error poisons the context: no later call can succeed, so the owning process
reports the failure and leaves with ``os._exit`` instead of unwinding through destructors that would
touch the device again (reference: src/xpool/utils/cuda.py, src/xpool/runtime/agent.py:595-620).
"""

from __future__ import annotations

TERMINAL_MARKERS = (
    "illegal memory access", "illegal instruction", "misaligned address", "unspecified launch failure",
    "device-side assert", "hardware stack error", "uncorrectable ecc", "launch timed out", "invalid program counter",
    "cudaerrorlaunchfailure", "cudaerrorillegaladdress", "context is destroyed", "gpu has fallen off the bus",
)
RECOVERABLE_MARKERS = ("out of memory", "cudaerrormemoryallocation", "invalid argument", "not ready",
                       "operation not permitted when stream is capturing")


class CudaDriverError(RuntimeError):
    def __init__(self, call: str, code: int, name: str = ""):
        super().__init__(f"{call} failed with {code}{' (' + name + ')' if name else ''}")
        self.call, self.code, self.name = call, code, name


def is_terminal_device_error(exc: BaseException) -> bool:
    text = f"{type(exc).__name__}: {exc}".lower()
    if any(m in text for m in RECOVERABLE_MARKERS):
        return False
    if isinstance(exc, CudaDriverError):
        return exc.code in (700, 701, 702, 709, 710, 715, 716, 717, 718, 719, 720)
    return any(m in text for m in TERMINAL_MARKERS)
