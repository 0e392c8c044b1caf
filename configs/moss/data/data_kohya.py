"""Kohya-style folders: `<repeats>_<name>/image + .txt tags`; repeats become row weight."""
DATASETS = [{"source": "kohya", "path": "data/train", "repeat_prefix": "first", "txt_as": "tags"}]
CAPTION = {"template": "tags", "shuffle": True, "keep_first": 1}
RESOLUTION_MODE = "resize"
LATENT_CACHE = "online"
TEXT_CACHE = "online"
