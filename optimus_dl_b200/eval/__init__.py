from .model import LLMBaselinesModel

__all__ = ["LLMBaselinesModel"]
