"""`python -m kohakumosstrainer_b200.cli.run SCRIPT [--config CFG] [--set KEY=VALUE ...]`:
the equivalent of `kogine run` for this repository's knob scripts."""

from __future__ import annotations

import argparse

from ..config import run_script


def main(argv=None):
    ap = argparse.ArgumentParser(prog="kmoss-run", description=__doc__)
    ap.add_argument("script")
    ap.add_argument("--config", default=None)
    ap.add_argument("--set", dest="sets", action="append", default=[], metavar="KEY=VALUE")
    args = ap.parse_args(argv)
    run_script(args.script, args.config, args.sets)


if __name__ == "__main__":
    main()
