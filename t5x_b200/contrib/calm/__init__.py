"""Confident Adaptive Language Modeling: early-exit decoding (role of t5x/contrib/calm)."""
