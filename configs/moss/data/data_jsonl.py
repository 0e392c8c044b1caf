"""A JSON-lines manifest: `{"image": "rel/path.png", "tags": ..., "caption": ..., "weight": ...}`."""
DATASETS = [{"source": "jsonl", "path": "data/train.jsonl"}]
CAPTION = {"template": "mix", "p_nl": 0.5}
