"""kohakumosstrainer_b200: a Blackwell-native (sm_100a) finetuning and inference framework
for the MOSS-Image DiT.

Layers (bottom-up): `utils` (no torch) -> `ops` (+ `csrc` CUDA kernels) -> `types`,
`models` -> `quant`, `memory`, `adapters`, `diffusion`, `optim` -> `parallel` ->
`training`, `inference` -> `cli`, `scripts/`, `configs/`.
"""

__version__ = "0.1.0"
