"""LoRA r8 fp8-base DDP over the eight B200 of a node."""
use_config("recipes_lora_b200.py")
use_config("../parallel/parallel_ddp.py")
