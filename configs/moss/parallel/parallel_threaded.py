"""Threaded pipeline (one process, stages on several devices)."""
PARALLEL = "threaded"
DEVICES = (0, 1, 2, 3)
PIPELINE_SCHEDULE = "gpipe"
MICROBATCHES = 16
