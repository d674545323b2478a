"""Mistral dense family (Mistral-7B, Mistral-Nemo, Mistral-Large): the Llama decoder layout with its own
configuration defaults (vllm/model_executor/models/llama.py serves ``MistralForCausalLM`` with the same
class). Checkpoints whose configuration asks for sliding-window attention are served up to the window
length, where windowed and full attention coincide."""
from .decoder import DecoderModel


class MistralForCausalLM(DecoderModel):
    architecture = "mistral"
    overlap_threshold = 1024
