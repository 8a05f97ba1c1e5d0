"""chill_attention for NVIDIA B200 (sm_100a): masked flash attention with the API of
alexdremov/chill-attention (same export list as its chill_attention/__init__.py:1-13)."""
from .chill import (
    _chill_reference_naive,
    chill_attention,
    register_chill_mask,
)
from ._cabi import is_deterministic, set_deterministic
from .mask import (
    CausalChillMask,
    ChillMask,
    ChunkwiseChillMask,
    FullChillMask,
    PrefixLMChillMask,
    SlidingWindowChillMask,
)

__all__ = [
    "chill_attention", "register_chill_mask", "_chill_reference_naive", "ChillMask", "FullChillMask",
    "CausalChillMask", "SlidingWindowChillMask", "ChunkwiseChillMask", "PrefixLMChillMask",
    "set_deterministic", "is_deterministic",
]
