"""Phi-3 family (mini / medium): the Llama decoder whose checkpoints store the fused ``qkv_proj`` and
``gate_up_proj`` tensors (vllm/model_executor/models/phi3.py); the loader cuts them at the full-model
boundaries and shards the pieces. The 128k variants' LongRoPE (short and long per-frequency factors) lives in
the rotary table builder (``ops/reference.py``) and a per-step position shift in the model runner."""
from .decoder import DecoderModel


class Phi3ForCausalLM(DecoderModel):
    architecture = "phi3"
    overlap_threshold = 1024
