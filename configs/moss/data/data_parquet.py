"""A parquet table with image paths (`image`) or embedded bytes (`bytes_col`)."""
DATASETS = [{"source": "parquet", "path": "data/train.parquet", "image_col": "image"}]
CAPTION = {"template": "nl"}
