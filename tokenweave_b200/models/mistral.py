"""Mistral dense family (Mistral-7B, Mistral-Nemo, Mistral-Large): the Llama decoder layout with its own
configuration defaults (vllm/model_executor/models/llama.py serves ``MistralForCausalLM`` with the same
class). Checkpoints whose configuration asks for sliding-window attention get it: the attention kernels mask
keys older than the window (``ModelConfig.sliding_window``)."""
from .decoder import DecoderModel


class MistralForCausalLM(DecoderModel):
    architecture = "mistral"
    overlap_threshold = 1024
