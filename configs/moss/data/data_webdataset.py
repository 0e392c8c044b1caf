"""WebDataset tar shards (uncompressed): `<key>.jpg + <key>.txt + <key>.json`."""
DATASETS = [{"source": "webdataset", "path": "data/shards/*.tar", "txt_as": "tags"}]
NUM_WORKERS = 8
