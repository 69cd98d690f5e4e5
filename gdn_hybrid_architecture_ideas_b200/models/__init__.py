from .hybrid import ControlCache, HybridLM, ModelOutput, build_model, lm_head  # noqa: F401
