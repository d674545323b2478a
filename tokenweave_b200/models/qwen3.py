"""Qwen3 dense family: the Qwen2 decoder without the QKV bias and with an RMSNorm over ``head_dim`` on every
query and key head before the rotary embedding (vllm/model_executor/models/qwen3.py ``Qwen3Attention``:
``q_norm`` / ``k_norm``). Here the per-head norm is part of the rope + KV-write kernel, so the layer has no
extra launch."""
from .decoder import DecoderModel


class Qwen3ForCausalLM(DecoderModel):
    architecture = "qwen3"
    overlap_threshold = 1024
