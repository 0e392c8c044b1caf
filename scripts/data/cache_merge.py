"""Fold the per-rank shards written by online caches (`<stem>.r<rank>.kmts`) into the main
cache files. Run it while no trainer is writing. Role of `scripts/data/cache_merge.py` there."""

CACHE_DIR = ""
CACHE_DTYPE = "bf16"
KEEP_SHARDS = False

globals().update(globals().pop("__kmoss_overrides__", {}))


def main():
    import os

    from kohakumosstrainer_b200.data.store import merge_shards

    if not CACHE_DIR:
        raise SystemExit("set CACHE_DIR")
    out = {}
    for stem in ("latents", "text"):
        out[stem] = merge_shards(os.path.join(CACHE_DIR, stem), CACHE_DTYPE, remove=not KEEP_SHARDS)
        print(f"{stem}: merged {out[stem]} values")
    return out


if __name__ == "__main__":
    main()
