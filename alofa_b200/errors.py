"""Named errors.  Every refusal of the engine is an :class:`AlofaError` whose
``code`` is one of a short list of names, after the reference's error codes
(src/alofa/core/error.mojo:25-108), so that callers can tell a capacity
refusal from a malformed file without parsing the message."""
from __future__ import annotations

CODES = (
    "invalid_argument",
    "out_of_range",
    "capacity",
    "parse",
    "unsupported",
    "io",
    "state",
    "build",
)


class AlofaError(RuntimeError):
    """An engine refusal: ``code`` names the kind, ``message`` says what, and
    ``detail`` carries the offending values."""

    def __init__(self, code: str, message: str, detail: str = ""):
        if code not in CODES:
            raise ValueError(f"unknown error code {code!r}")
        self.code = code
        self.message = message
        self.detail = detail
        text = f"[{code}] {message}"
        if detail:
            text += f" ({detail})"
        super().__init__(text)
