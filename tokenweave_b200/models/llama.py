"""Llama-3.x family (vllm/model_executor/models/llama.py in the reference)."""
from .decoder import DecoderModel


class LlamaForCausalLM(DecoderModel):
    architecture = "llama"
    overlap_threshold = 1024      # tokens per step from which the overlap schedule is used (llama.py:512)
