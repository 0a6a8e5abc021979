"""Model presets that take their shape (and optionally weights) from Hugging Face checkpoints."""

from . import hf_llama, hf_olmo3, hf_qwen3  # noqa: F401
