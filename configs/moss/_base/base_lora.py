"""Base layer of adapter runs (defaults of the reference's `configs/moss/_base/base_lora.py`)."""
ALGO = "lora"
PRESET = "attn-mlp"
DIM = 32
ALPHA = 32.0
LR = 1e-4
BETAS = (0.9, 0.95)
WEIGHT_DECAY = 0.01
GRAD_CLIP = 1.0
SCHEDULE = {"mode": "cosine", "warmup": 100, "end": -1}
