"""Execution mix-ins: context, iteration, interruption."""
