"""Counter-based seeds: every random draw is a pure function of (tag, seed, counters).

Same construction as the reference (`src/kohakumoss_data/seeds.py:8-17`): a blake2b digest
of the tag and integers, so batch i of rank r never depends on what was drawn before it
and a resumed run replays exactly.
"""

from __future__ import annotations

import hashlib
import struct


def seed_of(tag: str, *counters: int) -> int:
    h = hashlib.blake2b(digest_size=8)
    h.update(tag.encode())
    for c in counters:
        h.update(struct.pack("<q", int(c)))
    return int.from_bytes(h.digest(), "little") & 0x7FFF_FFFF_FFFF_FFFF
