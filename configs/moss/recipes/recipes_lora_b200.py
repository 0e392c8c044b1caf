"""LoRA r8, fp8 per-tensor base, ~20k joint tokens per step on one B200."""
use_config("../_base/base_lora.py")
use_config("../algo/algo_lora.py")
use_config("../precision/precision_fp8.py")
use_config("../data/data_synthetic.py")
DIM = 8
ALPHA = 8.0
MEMORY_PROFILE = "speed"
CHECKPOINT = "none"
