"""Callers of the codec that keep optimizer state compressed between steps
(the reference's ``LCT/components``; only the optimizers are provided here)."""
