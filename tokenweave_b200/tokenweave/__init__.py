"""TokenWeave scheduling: per-model split/SM-budget configs, the split planner and the layer
schedules (fuse-only, overlap, baselines)."""
from .config import SplitPlan, TokenWeavePlanner, load_config, default_config_path  # noqa: F401
