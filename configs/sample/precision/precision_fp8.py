"""fp8 sampling: e4m3 weights with per-row scales, fp8 tensor-core products."""
PRECISION = "bf16"
BASE_PRECISION = "fp8_compute"
FP8_RECIPE = "row"
