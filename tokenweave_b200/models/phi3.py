"""Phi-3 family (mini / medium, 4k-context variants): the Llama decoder whose checkpoints store the fused
``qkv_proj`` and ``gate_up_proj`` tensors (vllm/model_executor/models/phi3.py); the loader cuts them at the
full-model boundaries and shards the pieces. The LongRoPE variants (128k) are refused by the rotary table
builder."""
from .decoder import DecoderModel


class Phi3ForCausalLM(DecoderModel):
    architecture = "phi3"
    overlap_threshold = 1024
