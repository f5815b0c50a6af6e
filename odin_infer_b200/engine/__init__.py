"""Engine: runtime, step function, model assembly, generation loop, library API."""
from .api import (DEFAULT_MAX_CONTEXT, Engine, Engine_Opts, engine_config, engine_destroy, engine_forward, engine_load)
from .generate import GenerationResult, GenerationStats, generate, plan_batches
from .model import DecoderModel
from .runtime import Runtime
from .step import StepBatch, StepEntry, StepError

__all__ = ["DEFAULT_MAX_CONTEXT", "DecoderModel", "Engine", "Engine_Opts", "GenerationResult", "GenerationStats",
           "Runtime", "StepBatch", "StepEntry", "StepError", "engine_config", "engine_destroy", "engine_forward",
           "engine_load", "generate", "plan_batches"]
