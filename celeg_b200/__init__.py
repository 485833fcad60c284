"""celeg_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a).

    from celeg_b200 import Engine
    engine = Engine("model_folder", dtype="bfloat16")
    tokens = engine.generate([1, 5, 17], max_new_tokens=16, temperature=0.0)
"""
__version__ = "0.1.0"

_LAZY = {
    "Engine": ("celeg_b200.engine.engine", "Engine"),
    "EngineOptions": ("celeg_b200.engine.scheduler", "EngineOptions"),
    "RequestOptions": ("celeg_b200.engine.scheduler", "RequestOptions"),
    "RequestStatus": ("celeg_b200.engine.scheduler", "RequestStatus"),
    "SchedulerPolicy": ("celeg_b200.engine.scheduler", "SchedulerPolicy"),
    "SamplingParams": ("celeg_b200.sampling.params", "SamplingParams"),
    "KernelOptions": ("celeg_b200.parts.options", "KernelOptions"),
    "StepEntry": ("celeg_b200.engine.step", "StepEntry"),
    "load_model": ("celeg_b200.engine.loading", "load_model"),
    "write_random_model": ("celeg_b200.weights.random_init", "write_random_model"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        module, attribute = _LAZY[name]
        return getattr(importlib.import_module(module), attribute)
    raise AttributeError(f"module 'celeg_b200' has no attribute '{name}'")
