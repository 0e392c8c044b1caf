"""Full finetune, 4 pipeline stages x 2 data-parallel replicas (1F1B, 8 micro-batches)."""
use_config("../_base/base_full.py")
use_config("../precision/precision_bf16.py")
use_config("../parallel/parallel_pipeline.py")
PIPELINE_STAGES = 4
PIPELINE_SCHEDULE = "1f1b"
MICROBATCHES = 8
DEVICES = (0, 1, 2, 3, 4, 5, 6, 7)
