"""LoKr factor 16 quality setting (the configuration the published throughput number uses)."""
use_config("../_base/base_lora.py")
use_config("../algo/algo_lokr.py")
ALGO_KWARGS = {"factor": 16}
LR = 1e-4
