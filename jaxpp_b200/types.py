"""Core enums and id types shared by schedules, compiler and runtime.

``TaskType`` mirrors the reference's task kinds and integer latencies used for list
scheduling (src/jaxpp/types.py:79-96): FWD 1, BWD 2, BWD_I 1, BWD_W 1.
"""
from __future__ import annotations

import enum
import itertools
from typing import NewType

MpmdIdx = NewType("MpmdIdx", int)
ScalarUid = NewType("ScalarUid", int)

_uid_counter = itertools.count()


def fresh_scalar_uid() -> ScalarUid:
    return ScalarUid(next(_uid_counter))


class TaskType(enum.Enum):
    FWD = 1
    BWD = 2
    BWD_I = 3  # activation-gradient half of a split backward
    BWD_W = 4  # weight-gradient half of a split backward

    def __repr__(self) -> str:
        return f"TaskType.{self.name}"

    @property
    def default_latency(self) -> int:
        return 2 if self is TaskType.BWD else 1

    @property
    def is_bwd(self) -> bool:
        return self is not TaskType.FWD
