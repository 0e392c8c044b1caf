"""kogine-style configuration: UPPER_CASE script globals are the knobs, config files are Python
files assigning them, `use_config` composes layers, `--set KEY=VALUE` overrides, and one
validation pass reports every problem at once."""

from .engine import ConfigError, apply_sets, check, collect, load_config, run_script, script_knobs

__all__ = ["ConfigError", "apply_sets", "check", "collect", "load_config", "run_script", "script_knobs"]
