"""B200-native permutohedral-lattice hash encoding with the Python surface of
RaduAlexandru/permutohedral_encoding (reference: src/__init__.py:6-8).

The public names are resolved on first use, so that ``python -m permutohedral_encoding_b200.build``
can run before the CUDA extension exists.  Using any of them without the built library raises an
ImportError that names the build command; there is no CPU fallback.
"""
import importlib

__all__ = ["PermutoEncoding", "Coarse2Fine", "map_range_val", "cosine_easing_window"]

_HOME = {"PermutoEncoding": ".modules", "Coarse2Fine": ".modules", "map_range_val": ".utils",
         "cosine_easing_window": ".utils"}


def __getattr__(name):
    home = _HOME.get(name)
    if home is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(importlib.import_module(home, __name__), name)
    globals()[name] = value
    return value


def __dir__():
    return sorted(set(globals()) | set(__all__))
