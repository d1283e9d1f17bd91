"""B200-native stochastic/variational parameter decomposition (SPD/VPD) training framework.

Layers, bottom up: `formats` (artifact schemas) -> `config` (YAML run schema) -> `core`
(numerics, CI functions, train step, engine) -> `models` (targets) -> `ops` (sm_100a kernels) /
`parallel` (mesh, placement, fused collectives) -> `experiments` (CLI composition roots).
"""

__version__ = "0.1.0"
