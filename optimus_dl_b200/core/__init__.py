"""Core runtime: config tree, registries, bootstrap, logging, device/dtype helpers."""
