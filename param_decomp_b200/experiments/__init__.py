"""Composition roots: YAML -> target + CI function + data -> engine."""
