"""B200-native permutohedral-lattice hash encoding with the Python surface of
RaduAlexandru/permutohedral_encoding (reference: src/__init__.py:6-8)."""
from .modules import Coarse2Fine, PermutoEncoding
from .utils import cosine_easing_window, map_range_val

__all__ = ["PermutoEncoding", "Coarse2Fine", "map_range_val", "cosine_easing_window"]
