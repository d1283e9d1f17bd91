"""Utilities: FLOP accounting, clocks sampling, misc helpers."""
