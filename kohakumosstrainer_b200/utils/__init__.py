"""Shared utilities with no dependency on torch or on the rest of the package.

Counterpart of the reference's `kohakumoss_common` package
(`src/kohakumoss_common/__init__.py`): logging, registries, knob collection, retry,
atomic JSON, unit constants.
"""
