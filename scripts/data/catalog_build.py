"""Scan the datasets into catalog files, or import them into packed shards.

Each `DATASETS` entry is scanned (incrementally when its catalog file exists; `DATA_RESCAN="full"`
starts over) and its catalog written to `catalog` of the entry, or to the catalog cache dir.
An entry with `import_to` is copied into packed image shards there (a `moss_shard` dataset).
Role of `scripts/data/catalog_build.py` in the reference.
"""

DATASETS = []
CACHE_DIR = ""
DATA_RESCAN = True
DATA_SCAN_WORKERS = 8
SHARD_BYTES = 1 << 30

globals().update(globals().pop("__kmoss_overrides__", {}))


def main():
    from kohakumosstrainer_b200.data.catalog import Catalog, is_catalog, merge_scan
    from kohakumosstrainer_b200.data.dataset import DataConfig, scan_source
    from kohakumosstrainer_b200.data.sources import build_source, import_to_shards

    cfg = DataConfig(datasets=list(DATASETS), cache_dir=CACHE_DIR, data_rescan=DATA_RESCAN, data_scan_workers=DATA_SCAN_WORKERS,
                     latent_cache="off", text_cache="off")
    out = []
    for entry in DATASETS:
        src = build_source(entry)
        if hasattr(src, "workers"):
            src.workers = DATA_SCAN_WORKERS
        target = entry.get("catalog")
        if entry.get("import_to"):
            cat = import_to_shards(src, src.scan(), entry["import_to"], SHARD_BYTES)
            print(f"imported {len(cat)} images into {entry['import_to']}")
        elif target:
            old = Catalog.load(target) if is_catalog(target) and DATA_RESCAN != "full" else None
            cat, stats = merge_scan(old, src.scan())
            cat.save(target)
            print(f"{target}: {len(cat)} rows {stats}")
        else:
            cat = scan_source(entry, src, cfg, writer=True)
            print(f"{entry.get('path')}: {len(cat)} rows ({int(cat.live.sum())} live) -> {cat.path or 'memory'}")
        out.append(len(cat))
    return out


if __name__ == "__main__":
    main()
