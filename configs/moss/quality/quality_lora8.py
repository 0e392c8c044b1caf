"""Small-rank LoRA quality setting: r8 on attention + MLP, cosine schedule, EMA off."""
use_config("../_base/base_lora.py")
DIM = 8
ALPHA = 8.0
LR = 2e-4
