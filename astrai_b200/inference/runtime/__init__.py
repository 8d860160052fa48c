from astrai_b200.inference.runtime.executor import Executor, SamplingBatchInfo, build_sampling_info, timed
from astrai_b200.inference.runtime.graph import CudaGraphContext
from astrai_b200.inference.runtime.sample import (
    BaseSamplingStrategy, FrequencyPenaltyStrategy, SamplingPipeline, TemperatureStrategy, TopKStrategy, TopPStrategy, sample,
)

__all__ = [
    "BaseSamplingStrategy", "CudaGraphContext", "Executor", "FrequencyPenaltyStrategy", "SamplingBatchInfo",
    "SamplingPipeline", "TemperatureStrategy", "TopKStrategy", "TopPStrategy", "build_sampling_info", "sample", "timed",
]
