"""Stand-in for `lm_eval`: base classes only, so the reference's eval adapter module imports."""
