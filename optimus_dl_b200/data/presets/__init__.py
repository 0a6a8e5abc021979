"""Dataset presets (``preset_*`` keys of the ``dataset`` registry)."""
