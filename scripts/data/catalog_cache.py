"""List or clear the catalog files of a cache dir (`list` | `clear`). Role of
`scripts/data/catalog_cache.py` in the reference."""

CACHE_DIR = ""
ACTION = "list"

globals().update(globals().pop("__kmoss_overrides__", {}))


def main():
    import glob
    import os

    from kohakumosstrainer_b200.data.catalog import Catalog

    if ACTION not in ("list", "clear"):
        raise SystemExit("ACTION must be 'list' or 'clear'")
    files = sorted(glob.glob(os.path.join(CACHE_DIR, "catalog-*.kmc")))
    for path in files:
        if ACTION == "clear":
            os.remove(path)
            print(f"removed {path}")
        else:
            cat = Catalog.load(path)
            print(f"{path}: {len(cat)} rows, {int(cat.live.sum())} live, {os.path.getsize(path) / 1e6:.1f} MB")
    return files


if __name__ == "__main__":
    main()
