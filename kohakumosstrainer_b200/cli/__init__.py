"""Command-line tools: `run` (kogine-style script runner), `doctor`, `config`."""
