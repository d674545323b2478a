"""Model families: Llama-3.x, Qwen2.5 and Mixtral share one decoder implementation."""
from .registry import get_model_class, build_model  # noqa: F401
