"""Measure this card and the block ops once and store the per-card JSON (same as
`python -m kohakumosstrainer_b200.cli.tune`; role of `scripts/bench/tune/tune.py`).

    python scripts/bench/tune/tune.py --sizes 1024x1024 832x1216 --batch 4 --out runs/tune/card.json
"""

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))
from kohakumosstrainer_b200.cli.tune import main  # noqa: E402

if __name__ == "__main__":
    raise SystemExit(main())
