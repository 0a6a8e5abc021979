"""Recipes: train, eval, metrics, serve, pretokenize, grpo."""
