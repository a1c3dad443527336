"""Operator layer: thin Python wrappers over the C ABI, named like ``equitorch.ops``."""
