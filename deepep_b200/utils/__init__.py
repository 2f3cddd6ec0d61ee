"""Helper modules: numerics, gate generators, the pure-torch oracle, timing and environment probes."""
from .math import align, ceil_div, calc_diff, per_token_cast_to_fp8, per_token_cast_back, count_bytes  # noqa: F401
from .semantic import value_or, weak_lru  # noqa: F401
