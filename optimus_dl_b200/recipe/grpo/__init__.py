"""GRPO recipe (placeholder until the trainer lands in this package)."""
