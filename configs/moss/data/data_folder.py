"""A plain image folder with `.txt` tag sidecars."""
DATASETS = [{"source": "folder", "path": "data/train", "txt_as": "tags"}]
CAPTION = {"template": "tags"}
