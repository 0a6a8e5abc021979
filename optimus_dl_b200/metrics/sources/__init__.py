"""Metric sources: causal_lm, generation, model_info."""
