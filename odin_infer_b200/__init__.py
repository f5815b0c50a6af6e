"""odin_infer_b200: a small model library with generation of its own for one
NVIDIA B200 (sm_100a): everything between a request's token ids and its next
token, for the Qwen3 dense decoder, built from parts so that another
architecture can be added.

    from odin_infer_b200 import Engine, Engine_Opts
    e = Engine.load("model_dir", Engine_Opts(max_ctx=4096, dtype="bfloat16"))
    out = e.generate([[1, 2, 3], [4, 5]], max_new_tokens=16, temperature=0.0)
"""
from .config import ConfigError, ModelConfig, Qwen3Config, load_config, register_architecture
from .engine import (Engine, Engine_Opts, GenerationResult, GenerationStats, StepEntry, StepError, engine_config,
                     engine_destroy, engine_forward, engine_load)
from .sampling import SamplingParams
from .weights import WeightError, write_random_model

__all__ = ["ConfigError", "Engine", "Engine_Opts", "GenerationResult", "GenerationStats", "ModelConfig", "Qwen3Config",
           "SamplingParams", "StepEntry", "StepError", "WeightError", "engine_config", "engine_destroy",
           "engine_forward", "engine_load", "load_config", "register_architecture", "write_random_model"]
