"""Mixed precision: autocast contexts and the FP8 recipe objects."""
