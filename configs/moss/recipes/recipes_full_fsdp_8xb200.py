"""Full finetune, Muon + AdamW + EMA 0.9999, sharded over eight B200."""
use_config("../_base/base_full.py")
use_config("../data/data_synthetic.py")
use_config("../parallel/parallel_fsdp.py")
DATASETS = [{"type": "synthetic", "fixed_size": (1024, 1024), "fixed_text": 256, "samples": 8}]
BASE_PRECISION = "mxfp8"
