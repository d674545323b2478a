"""tokenweave_b200: a Blackwell-native tensor-parallel LLM inference engine with TokenWeave's
token-split compute/communication overlap and fused all-reduce + RMSNorm."""

__version__ = "0.1.0"
