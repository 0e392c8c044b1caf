"""bf16 compute."""
PRECISION = "bf16"
