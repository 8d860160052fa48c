"""Position-id generation for packed data (reference ``astrai/preprocessing/position_id.py:15-46``)."""

from __future__ import annotations

from typing import List

from astrai_b200.factory import BaseFactory


class PositionIdStrategy:
    def generate(self, sequences: List[List[int]]) -> List[int]:
        raise NotImplementedError


class PositionIdStrategyFactory(BaseFactory["PositionIdStrategy"]):
    pass


@PositionIdStrategyFactory.register("none")
class NoPositionId(PositionIdStrategy):
    def generate(self, sequences):
        return []


@PositionIdStrategyFactory.register("doc_reset")
class DocResetPositionId(PositionIdStrategy):
    """Positions restart at 0 at every document: the trainer recovers document boundaries from them."""

    def generate(self, sequences):
        return [p for s in sequences for p in range(len(s))]


@PositionIdStrategyFactory.register("continuous")
class ContinuousPositionId(PositionIdStrategy):
    def generate(self, sequences):
        return list(range(sum(len(s) for s in sequences)))
