"""nnabla_b200 — B200 (sm_100a) implementation of nnabla's quantized-layer forward
path. `functions` mirrors `nnabla.functions`; the C ABI is in include/nnabla_b200.h."""
from . import _capi  # noqa: F401

__all__ = ["functions", "_capi"]
