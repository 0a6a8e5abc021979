"""Mix-ins of the train recipe."""
