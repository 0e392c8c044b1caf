"""Base layer of sampling runs: 32 Euler steps, CFG 3 packed with the block-22 skip, 1024 x 1024."""
STEPS = 32
CFG = 3.0
SHIFT = 5.0
SKIP_LAYERS = "default"
CFG_MODE = "packed"
SIZE = (1024, 1024)
BATCH = 4
