"""tokenweave_b200: a Blackwell-native tensor-parallel LLM inference engine with TokenWeave's
token-split compute/communication overlap and fused all-reduce + RMSNorm."""

__version__ = "0.1.0"

from .sampling_params import BeamSearchParams, SamplingParams  # noqa: E402,F401
from .outputs import (BeamSearchOutput, BeamSearchSequence, ClassificationOutput, CompletionOutput,  # noqa: E402,F401
                      PoolingOutput,
                      RequestOutput)


def __getattr__(name):
    if name == "LLM":
        from .entrypoints.llm import LLM
        return LLM
    if name == "LoRARequest":
        from .lora import LoRARequest
        return LoRARequest
    if name == "EngineArgs":
        from .config import EngineArgs
        return EngineArgs
    raise AttributeError(name)
