"""A 48 GB card of the same family: block checkpointing, streamed optimiser state, 16 resident blocks."""
MEMORY_PROFILE = "low"
MAX_TOKENS = 8192
