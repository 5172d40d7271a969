"""cuca_b200: a small, whole Llama inference engine for one NVIDIA B200 (sm_100a).

    from cuca_b200 import LocalModel, LocalModelConfig, generate
    model = LocalModel.load(LocalModelConfig(source="path/to/model"))
    out = model.generate([1, 2, 3], max_tokens=16, temperature=0.0)
"""
from .config.engine_config import BatchingConfig, LocalModelConfig, RandomWeights, SamplingConfig  # noqa: F401


def __getattr__(name):
    # the engine imports torch and builds kernels; keep `import cuca_b200` light
    if name in ("LocalModel", "LocalGeneration", "GenerationReport", "generate"):
        from .engine import engine
        return getattr(engine, name)
    raise AttributeError(name)
