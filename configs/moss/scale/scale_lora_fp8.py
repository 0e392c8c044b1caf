"""LoRA at scale, fp8 per-tensor base GEMMs (the headline configuration), data parallel x 8."""
use_config("../_base/base_lora.py")
use_config("../precision/precision_fp8.py")
use_config("../parallel/parallel_ddp.py")
MAX_TOKENS = 20480
DEVICES = (0, 1, 2, 3, 4, 5, 6, 7)
