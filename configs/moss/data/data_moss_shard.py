"""A dataset imported into packed image shards (`scripts/data/catalog_build.py` with `import_to`)."""
DATASETS = [{"source": "moss_shard", "path": "data/packed"}]
LATENT_CACHE = "offline"
TEXT_CACHE = "offline"
TOKEN_BUDGET = "exact"
