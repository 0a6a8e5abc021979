"""Concrete tokenizers."""
