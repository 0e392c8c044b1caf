"""fp8 per-tensor base GEMMs under a bf16 adapter."""
PRECISION = "bf16"
BASE_PRECISION = "fp8_compute"
FP8_RECIPE = "tensor"
