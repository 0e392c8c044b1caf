"""MEMORY_PROFILE=low (see `kohakumosstrainer_b200/memory/plan.py` for what the profile resolves to on a 180 GB B200)."""
MEMORY_PROFILE = "low"
