"""Managers: logger fan-out and periodic evaluation."""
