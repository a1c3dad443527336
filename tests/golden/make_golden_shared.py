"""Helpers shared by the fixture generator and the tests (no reference import)."""


def flatten(obj, prefix=""):
    """NamedTuple tree -> ``{dotted path: leaf}``."""
    out = {}
    if hasattr(obj, "_fields"):
        for f in obj._fields:
            out.update(flatten(getattr(obj, f), f"{prefix}.{f}" if prefix else f))
    elif isinstance(obj, (tuple, list)):
        for n, v in enumerate(obj):
            out.update(flatten(v, f"{prefix}[{n}]"))
    else:
        out[prefix] = obj
    return out
