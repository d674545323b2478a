"""Mixtral family: the MLP of every layer is a top-2 mixture of 8 tensor-sharded experts whose output
is written in place and reduced by the fused collective that follows
(vllm/model_executor/models/mixtral.py:103-110,457 in the reference)."""
from .decoder import DecoderModel


class MixtralForCausalLM(DecoderModel):
    architecture = "mixtral"
    overlap_threshold = 2048      # below this the split costs more than it hides (mixtral.py:457)
