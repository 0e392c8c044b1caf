"""Data knobs for the cache passes and the inspector on a kohya-style folder."""
DATASETS = [{"source": "kohya", "path": "data/train"}]
TARGET_AREA = 1024 * 1024
CACHE_DTYPE = "bf16"
