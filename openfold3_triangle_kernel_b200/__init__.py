"""B200 (sm_100a) triangle attention and triangle multiplicative update.

Public operators: :func:`turbo_attention`, :func:`turbo_trimul` (same contracts as
the TurboPairFormer operators of the same names).  The device is reached only
through ``libtpf_b200.so`` (C ABI, ``include/tpf_b200.h``); there is no fallback.
"""
from . import _cabi
from .attention import is_turbo_attention_supported, turbo_attention
from .trimul import check_trimul_support, turbo_trimul

__all__ = ["turbo_attention", "turbo_trimul", "is_turbo_attention_supported", "check_trimul_support", "_cabi"]
