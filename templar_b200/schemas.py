"""Typed records shared by the storage and chain layers.

Parity: src/tplr/schemas.py:24-65 of the reference (``Bucket`` is hashable over all four
fields; ``CommsGetResult.success`` means status OK *and* data present).
"""

from __future__ import annotations

from typing import Any, Literal

from pydantic import BaseModel, ConfigDict, Field


class Bucket(BaseModel):
    """An object-store bucket plus the credentials used to reach it."""

    model_config = ConfigDict(str_strip_whitespace=True)

    name: str = Field(..., min_length=1)
    account_id: str = Field(..., min_length=1)
    access_key_id: str = Field(..., min_length=1)
    secret_access_key: str = Field(..., min_length=1)

    def _key(self):
        return (self.name, self.account_id, self.access_key_id, self.secret_access_key)

    def __hash__(self):
        return hash(self._key())

    def __eq__(self, other):
        return isinstance(other, Bucket) and self._key() == other._key()


class CommsGetResult(BaseModel):
    """Outcome of ``Comms.get``: payload, the sender's global step and a status code."""

    data: None | dict[str, Any] = None
    global_step: None | int = None
    status: Literal["OK", "TOO_EARLY", "TOO_LATE", "NOT_FOUND", "ERROR"] = "OK"

    @property
    def success(self) -> bool:
        return self.status == "OK" and self.data is not None
