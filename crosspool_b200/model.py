"""Model identifiers: ``namespace/name`` as on the Hugging Face hub, with a URI-safe form for paths
and query strings (reference: src/xpool/model.py)."""

from __future__ import annotations

import re
from dataclasses import dataclass
from urllib.parse import quote, unquote

_PART = r"[A-Za-z0-9][A-Za-z0-9._-]*"
_RE = re.compile(rf"^(?:({_PART})/)?({_PART})$")


@dataclass(frozen=True)
class ModelId:
    namespace: str
    name: str

    def __lt__(self, other: "ModelId") -> bool:
        """Identifiers sort as their text does (``a-/x`` before ``a/z``), the order every listing and the placement
        search use, so two processes that sort the same set agree whatever the components are."""
        if not isinstance(other, ModelId):
            return NotImplemented
        return str(self) < str(other)

    @classmethod
    def parse(cls, text: str) -> "ModelId":
        m = _RE.match(text)
        if m is None:
            raise ValueError(f"invalid model id {text!r}: expected 'namespace/name' or 'name'")
        return cls(m.group(1) or "", m.group(2))

    def __str__(self) -> str:
        return f"{self.namespace}/{self.name}" if self.namespace else self.name

    def uri(self) -> str:
        return quote(str(self), safe="")

    @classmethod
    def from_uri(cls, text: str) -> "ModelId":
        return cls.parse(unquote(text))

    def resolve(self, base_uri: str) -> str:
        """Path or URL of the checkpoint under ``vendor.model_base_uri``."""
        return f"{base_uri.rstrip('/')}/{self}" if base_uri else str(self)
