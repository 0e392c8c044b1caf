"""Full finetune at scale: FSDP over 8 GPUs, Muon + EMA, bf16 compute with fp32 master shards."""
use_config("../_base/base_full.py")
use_config("../precision/precision_bf16.py")
use_config("../parallel/parallel_fsdp.py")
OPTIMIZER = "muon"
EMA = 0.999
MAX_TOKENS = 16384
DEVICES = (0, 1, 2, 3, 4, 5, 6, 7)
