from astrai_b200.parallel.executor import (
    AccumOptimizer, AccumScheduler, BaseExecutor, DDPExecutor, ExecutorFactory, FSDPExecutor, GradientState,
    NoneExecutor, broadcast_state_dict, create_ref_model,
)
from astrai_b200.parallel.flat import FlatParamEngine, FlatUnit
from astrai_b200.parallel.mesh import ParallelMesh, build_mesh, data_parallel_size, model_parallel_size
from astrai_b200.parallel.model_parallel import (
    ContextParallelExecutor, ExpertParallelExecutor, ModelParallelExecutor, PipelineParallelExecutor, TensorParallelExecutor,
)
from astrai_b200.parallel.setup import (
    LaunchStrategy, LocalStrategy, TorchrunStrategy, find_free_port, get_current_device, get_rank, get_world_size, launch_strategy,
    only_on_rank, setup_parallel, spawn_parallel_fn,
)

__all__ = [
    "AccumOptimizer", "AccumScheduler", "BaseExecutor", "ContextParallelExecutor", "DDPExecutor", "ExecutorFactory",
    "ExpertParallelExecutor", "FSDPExecutor", "ModelParallelExecutor", "ParallelMesh", "PipelineParallelExecutor", "TensorParallelExecutor",
    "build_mesh", "data_parallel_size", "model_parallel_size",
    "FlatParamEngine", "FlatUnit", "GradientState", "NoneExecutor", "broadcast_state_dict", "create_ref_model",
    "find_free_port", "get_current_device", "get_rank", "get_world_size", "only_on_rank", "setup_parallel",
    "spawn_parallel_fn", "LaunchStrategy", "LocalStrategy", "TorchrunStrategy", "launch_strategy",
]
