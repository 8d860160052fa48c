from astrai_b200.inference.cache import KVCache, PagePool, TaskCacheManager
from astrai_b200.inference.engine import GenerateResult, InferenceEngine
from astrai_b200.inference.metrics import MetricsCollector
from astrai_b200.inference.runtime.executor import Executor
from astrai_b200.inference.runtime.sample import SamplingPipeline, sample
from astrai_b200.inference.scheduler import InferenceScheduler
from astrai_b200.inference.task import STOP, Task, TaskManager, TaskStatus


def get_app(*args, **kwargs):
    from astrai_b200.inference.network import get_app as _get_app

    return _get_app(*args, **kwargs)


def run_server(*args, **kwargs):
    from astrai_b200.inference.network import run_server as _run_server

    return _run_server(*args, **kwargs)


__all__ = [
    "Executor", "GenerateResult", "InferenceEngine", "InferenceScheduler", "KVCache", "MetricsCollector", "PagePool", "STOP",
    "SamplingPipeline", "Task", "TaskCacheManager", "TaskManager", "TaskStatus", "get_app", "run_server", "sample",
]
