"""Process-group pipeline."""
PARALLEL = "pipeline"
DEVICES = (0, 1, 2, 3)
PIPELINE_SCHEDULE = "1f1b"
MICROBATCHES = 16
