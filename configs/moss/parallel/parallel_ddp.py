"""Data parallel over every GPU of the node; gradients reduced by the peer-memory kernel."""
PARALLEL = "ddp"
DEVICES = (0, 1, 2, 3, 4, 5, 6, 7)
DDP_BACKEND = "kohakumoss"
DDP_REDUCE_DTYPE = "fp32"
DDP_BUCKET_MB = 25
