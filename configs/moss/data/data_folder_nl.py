"""A plain image folder whose `.txt` sidecars are natural-language captions."""
DATASETS = [{"source": "folder", "path": "data/train", "txt_as": "nl"}]
CAPTION = {"template": "nl"}
