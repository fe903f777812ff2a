"""dilution-attention_b200: dilution attention for NVIDIA B200 (sm_100a).

A drop-in for the `dilution.kernels` entry points of
Royer-Research-Labs/Dilution-Attention backed by libdilution_b200.so
(hand-written CUDA, C ABI in include/dilution_b200.h).

The directory name carries a hyphen, so import it by name:

    import importlib
    pkg = importlib.import_module("dilution-attention_b200")
    out = pkg.kernels.dilution_attention(q, k, v)

After the first import it is also registered as `dilution_attention_b200`.
"""

import sys as _sys

from . import _lib, kernels, kernels_bid, layers, partition  # noqa: F401
from .kernels import (  # noqa: F401
    dilution_attention,
    dilution_attention_forward,
    dilution_attention_host,
    dilution_attention_reference,
    dilution_decode_append_step,
    dilution_decode_step,
    install,
    softmax_attention_forward,
    uninstall,
)
from .layers import (  # noqa: F401
    GraphedDecode,
    install_layers,
    softmax_decode_append_step,
    split_heads_rope,
    uninstall_layers,
)

_sys.modules.setdefault("dilution_attention_b200", _sys.modules[__name__])

__all__ = [
    "kernels", "kernels_bid", "partition", "dilution_attention", "dilution_attention_forward",
    "dilution_attention_reference", "dilution_attention_host", "dilution_decode_step",
    "dilution_decode_append_step", "softmax_attention_forward", "softmax_decode_append_step",
    "split_heads_rope", "install", "uninstall", "install_layers", "uninstall_layers", "layers", "GraphedDecode",
]
