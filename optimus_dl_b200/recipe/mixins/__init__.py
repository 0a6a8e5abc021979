"""Pieces shared between recipes."""
