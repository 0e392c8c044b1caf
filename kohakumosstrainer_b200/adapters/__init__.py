"""LyCORIS-format adapters (LoRA / LoCon / LoHa / LoKr / DoRA / OFT / IA3 / dense diff)."""

from .apply import AdapterConfig, AdapterSet, apply, resolve_preset
from .modules import MODULES, AdapterModule, LoRAModule

__all__ = ["AdapterConfig", "AdapterSet", "apply", "resolve_preset", "MODULES", "AdapterModule", "LoRAModule"]
