"""Targets: frozen networks exposed to the engine through the `DecomposedModel` protocol."""
