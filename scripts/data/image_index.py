"""Build the locator -> byte-offset index of a GBC records file (`<records>.index.json`), so loader
workers seek to a record instead of loading the manifest. Role of `scripts/data/image_index.py`."""

RECORDS = ""

globals().update(globals().pop("__kmoss_overrides__", {}))


def main():
    import json

    from kohakumosstrainer_b200.data.sources import build_record_index

    if not RECORDS:
        raise SystemExit("set RECORDS")
    index = build_record_index(RECORDS)
    with open(RECORDS + ".index.json", "w", encoding="utf-8") as f:
        json.dump(index, f)
    print(f"{RECORDS}: {len(index)} records indexed")
    return len(index)


if __name__ == "__main__":
    main()
