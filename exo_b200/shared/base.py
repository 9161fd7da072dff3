"""Foundations of the wire model: camelCase frozen models, class-name tagged unions, id newtypes,
byte quantities.

JSON produced here is what the dashboard, the macOS app and other exo nodes decode, so it keeps
the reference's conventions (``src/exo/utils/pydantic_ext.py:11-36``: camelCase aliases, unknown
keys rejected, a union member serialised as ``{"ClassName": {...}}``;
``src/exo/shared/types/common.py:9-70``: ids are strings defaulting to a fresh UUID4;
``src/exo/shared/types/memory.py``: ``{"inBytes": n}``).
"""
from __future__ import annotations

import math
from typing import Any, ClassVar, Self
from uuid import uuid4

from pydantic import BaseModel, ConfigDict, GetCoreSchemaHandler, field_validator, model_serializer, model_validator
from pydantic.alias_generators import to_camel
from pydantic_core import core_schema


class FrozenModel(BaseModel):
    model_config = ConfigDict(alias_generator=to_camel, validate_by_name=True, extra="forbid", strict=True, frozen=True,
                              serialize_by_alias=True)


class TaggedModel(FrozenModel):
    """Serialises as ``{ClassName: fields}`` so that unions decode without a discriminator field."""

    @classmethod
    def tag(cls) -> str:
        """Wire name of the class (``__tag__`` overrides the Python class name)."""
        return cls.__dict__.get("__tag__") or cls.__name__

    @model_serializer(mode="wrap")
    def _tag(self, inner):
        return {type(self).tag(): inner(self)}

    @model_validator(mode="wrap")
    @classmethod
    def _untag(cls, value: Any, inner) -> Self:
        if isinstance(value, dict) and len(value) == 1 and cls.tag() in value:
            return inner(value[cls.tag()])
        return inner(value)

    def __str__(self) -> str:
        return f"{type(self).__name__}({super().__str__()})"


class Id(str):
    """String newtype; ``Id()`` draws a random UUID4."""

    def __new__(cls, value: str | None = None) -> Self:
        return super().__new__(cls, value if value else str(uuid4()))

    @classmethod
    def __get_pydantic_core_schema__(cls, _src: type, _h: GetCoreSchemaHandler) -> core_schema.CoreSchema:
        return core_schema.no_info_after_validator_function(cls, core_schema.str_schema())


class NodeId(Id): ...
class SystemId(Id): ...
class CommandId(Id): ...
class TaskId(Id): ...
class EventId(Id): ...
class InstanceId(Id): ...
class RunnerId(Id): ...
class InstanceLinkId(Id): ...


class ModelId(Id):
    def normalize(self) -> str:
        return self.replace("/", "--")

    def short(self) -> str:
        return self.rsplit("/", 1)[-1]


CANCEL_ALL_TASKS = TaskId("CANCEL_ALL_TASKS")


class SessionId(FrozenModel):
    master_node_id: NodeId
    election_clock: int


class Host(FrozenModel):
    ip: str
    port: int

    @field_validator("port")
    @classmethod
    def _port(cls, v: int) -> int:
        if not 0 <= v <= 65535:
            raise ValueError("Port must be between 0 and 65535")
        return v

    def __str__(self) -> str:
        return f"{self.ip}:{self.port}"


class Memory(FrozenModel):
    in_bytes: int = 0

    @classmethod
    def from_bytes(cls, n: int) -> Self:
        return cls(in_bytes=int(n))

    @classmethod
    def from_kb(cls, n: float) -> Self:
        return cls(in_bytes=round(n * 1024))

    @classmethod
    def from_mb(cls, n: float) -> Self:
        return cls(in_bytes=round(n * 1024 ** 2))

    @classmethod
    def from_gb(cls, n: float) -> Self:
        return cls(in_bytes=round(n * 1024 ** 3))

    @property
    def in_kb(self) -> int:
        return math.ceil(self.in_bytes / 1024)

    @property
    def in_mb(self) -> int:
        return round(self.in_bytes / 1024 ** 2)

    @property
    def in_gb(self) -> float:
        return self.in_bytes / 1024 ** 3

    def __add__(self, o: object) -> "Memory":
        return Memory.from_bytes(self.in_bytes + o.in_bytes) if isinstance(o, Memory) else NotImplemented

    def __radd__(self, o: object) -> "Memory":
        return self if o == 0 else NotImplemented

    def __sub__(self, o: object) -> "Memory":
        return Memory.from_bytes(self.in_bytes - o.in_bytes) if isinstance(o, Memory) else NotImplemented

    def __mul__(self, k: float) -> "Memory":
        return Memory.from_bytes(round(self.in_bytes * k))

    __rmul__ = __mul__

    def __truediv__(self, o: object):
        if isinstance(o, Memory):
            return self.in_bytes / o.in_bytes
        return Memory.from_bytes(round(self.in_bytes / o)) if isinstance(o, (int, float)) else NotImplemented

    def __lt__(self, o: "Memory") -> bool:
        return self.in_bytes < o.in_bytes

    def __le__(self, o: "Memory") -> bool:
        return self.in_bytes <= o.in_bytes

    def __gt__(self, o: "Memory") -> bool:
        return self.in_bytes > o.in_bytes

    def __ge__(self, o: "Memory") -> bool:
        return self.in_bytes >= o.in_bytes

    def __hash__(self) -> int:
        return hash(self.in_bytes)

    def __str__(self) -> str:
        for unit, div in (("GiB", 1024 ** 3), ("MiB", 1024 ** 2), ("KiB", 1024)):
            if self.in_bytes > 2 * div:
                return f"{self.in_bytes / div:.2f} {unit}"
        return f"{self.in_bytes} B"
