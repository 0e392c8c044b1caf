"""LoRA at scale, bf16 base: data-parallel over every GPU of the node, ~20k joint tokens per rank."""
use_config("../_base/base_lora.py")
use_config("../precision/precision_bf16.py")
use_config("../parallel/parallel_ddp.py")
MAX_TOKENS = 20480
DEVICES = (0, 1, 2, 3, 4, 5, 6, 7)
