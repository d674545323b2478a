"""Qwen2 / Qwen2.5 family: the Llama decoder plus a bias on the QKV projection and rope_theta 1e6
(vllm/model_executor/models/qwen2.py:147,494 in the reference)."""
from .decoder import DecoderModel


class Qwen2ForCausalLM(DecoderModel):
    architecture = "qwen2"
    overlap_threshold = 1024
