"""B200 (sm_100a) triangle attention and triangle multiplicative update."""
from . import _cabi  # noqa: F401

__all__ = ["_cabi"]
