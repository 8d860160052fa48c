from astrai_b200.optim.base import CompositeOptimizer, OptimizerFactory
from astrai_b200.optim.fused_adamw import FusedAdamW

__all__ = ["CompositeOptimizer", "FusedAdamW", "OptimizerFactory"]
