"""bf16 sampling (dense weights)."""
PRECISION = "bf16"
BASE_PRECISION = "auto"
