"""Loader throughput: batches per second and MB/s of the stateless loader over a dataset config, per worker count
(role of `scripts/bench/data/loader.py`). With no DATASETS it measures the synthetic dataset.

    python -m kohakumosstrainer_b200.cli.run scripts/bench/data/loader.py --config configs/moss/data/data_kohya.py --set WORKERS="(0, 4, 8)"
"""

DATASETS = []
MAX_TOKENS = 16384
TARGET_AREA = 1024 * 1024
LATENT_CACHE = "off"
TEXT_CACHE = "off"
CACHE_DIR = ""
WORKERS = (0, 4)
BATCHES = 32
SEED = 0

globals().update(globals().pop("__kmoss_overrides__", {}))


def main():
    import json
    import time

    from kohakumosstrainer_b200.config import collect
    from kohakumosstrainer_b200.data import SyntheticConfig, SyntheticDataset, build_loader
    from kohakumosstrainer_b200.data.scripting import open_dataset

    k = collect(globals())
    rows = []
    for workers in WORKERS:
        if DATASETS:
            ds = open_dataset(k, num_workers=int(workers))
            it = iter(build_loader(ds))
            fetch = lambda: next(it)     # noqa: E731
        else:
            ds = SyntheticDataset(SyntheticConfig(max_tokens=int(MAX_TOKENS), seed=int(SEED)))
            state = {"i": 0}

            def fetch():
                state["i"] += 1
                return ds.materialize(state["i"] - 1)

        fetch()
        t0 = time.perf_counter()
        nbytes = 0
        for _ in range(int(BATCHES)):
            hb = fetch()
            nbytes += hb.nbytes() if hb.encoded else sum(p.numel() for p in hb.pixels or [])
        dt = time.perf_counter() - t0
        rows.append({"workers": int(workers), "batches_per_s": round(BATCHES / dt, 2), "mb_per_s": round(nbytes / dt / 1e6, 1)})
        print(json.dumps(rows[-1]), flush=True)
    return rows


if __name__ == "__main__":
    main()
