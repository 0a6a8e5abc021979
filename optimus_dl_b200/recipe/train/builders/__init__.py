"""Builders for the criterion, data, optimizer and scheduler; each is a registry entry named ``base``."""
