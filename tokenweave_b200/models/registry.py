"""Architecture name -> model class, and model construction + weight loading."""
from __future__ import annotations

import torch

from ..config import EngineConfig


def get_model_class(architecture: str):
    from .llama import LlamaForCausalLM
    from .mistral import MistralForCausalLM
    from .mixtral import MixtralForCausalLM
    from .phi3 import Phi3ForCausalLM
    from .qwen2 import Qwen2ForCausalLM
    from .qwen3 import Qwen3ForCausalLM
    table = {"llama": LlamaForCausalLM, "qwen2": Qwen2ForCausalLM, "mixtral": MixtralForCausalLM,
             "qwen3": Qwen3ForCausalLM, "mistral": MistralForCausalLM, "phi3": Phi3ForCausalLM}
    if architecture not in table:
        raise ValueError(f"unsupported architecture {architecture!r} (supported: {sorted(table)})")
    return table[architecture]


def build_model(config: EngineConfig, device: torch.device, embedding_parallel: bool = False):
    """Instantiate on ``device`` and fill the weights (checkpoint or random init)."""
    from .loader import load_model_weights
    cls = get_model_class(config.model.architecture)
    model = cls(config.model, device=device, embedding_parallel=embedding_parallel)
    load_model_weights(model, config)
    return model
