from astrai_b200.optim.base import (
    CompositeOptimizer, OptimizerFactory, composite_state_dict, composite_step, composite_zero_grad, refresh_param_groups,
)
from astrai_b200.optim.fused_adamw import FusedAdamW
from astrai_b200.optim.matrix import (
    Mano, ManoAdamW, Muon, MuonAdamW, NAdamW, Nora, NoraNAdamW, OptimizerParameterGroups, newton_schulz, nora_direction,
    nora_lr_scale, partition_optimizer_parameters,
)

__all__ = [
    "CompositeOptimizer", "FusedAdamW", "Mano", "ManoAdamW", "Muon", "MuonAdamW", "NAdamW", "Nora", "NoraNAdamW",
    "OptimizerFactory", "OptimizerParameterGroups", "composite_state_dict", "composite_step", "composite_zero_grad", "newton_schulz", "nora_direction", "nora_lr_scale",
    "partition_optimizer_parameters", "refresh_param_groups",
]
