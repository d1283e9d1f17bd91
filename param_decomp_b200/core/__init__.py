"""Algorithm core: components, masking, losses, adversaries, CI functions, optimizers, the train
step and the engine loop. Imports nothing from `models` or `experiments`."""
