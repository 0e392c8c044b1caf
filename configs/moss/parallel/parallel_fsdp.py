"""FSDP2-style sharding."""
PARALLEL = "fsdp"
DEVICES = (0, 1, 2, 3, 4, 5, 6, 7)
FSDP_REDUCE = "step"
FSDP_RESHARD = "forward"
