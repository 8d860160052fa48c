from astrai_b200.preprocessing.builder import (
    BaseMaskBuilder, MaskBuilderFactory, MultiOutputMaskBuilder, SectionedMaskBuilder, SectionRenderer,
    SingleOutputMaskBuilder,
)
from astrai_b200.preprocessing.packing import PackingStrategy, PackingStrategyFactory, plan_bfd
from astrai_b200.preprocessing.pipeline import Pipeline, filter_by_length
from astrai_b200.preprocessing.position_id import PositionIdStrategy, PositionIdStrategyFactory
from astrai_b200.preprocessing.transform import TokenizeTransform
from astrai_b200.preprocessing.writer import StoreWriter, StoreWriterFactory

__all__ = [
    "BaseMaskBuilder", "MaskBuilderFactory", "MultiOutputMaskBuilder", "PackingStrategy", "PackingStrategyFactory",
    "Pipeline", "PositionIdStrategy", "PositionIdStrategyFactory", "SectionRenderer", "SectionedMaskBuilder",
    "SingleOutputMaskBuilder", "StoreWriter", "StoreWriterFactory", "TokenizeTransform", "filter_by_length", "plan_bfd",
]
