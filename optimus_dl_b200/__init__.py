"""B200-native LLM training framework with the capabilities of Optimus-DL."""

__version__ = "0.1.0"
