"""ctypes binding of libdilution_b200.so (declarations: include/dilution_b200.h).

There is no fallback: if the library is missing or a call fails, an exception
is raised.  The library is looked up next to this file.
"""

from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libdilution_b200.so")

F32, BF16 = 0, 1
PREC = {"ieee": 0, "tf32": 1, "bf16": 2}
CARRY_ROWS = 32   # the fp32 kernels' checkpoint spacing; see carry_rows()

_P, _I, _L, _F, _Z = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_size_t

SIGNATURES = {
    "dilution_version": (ctypes.c_int, []),
    "dilution_last_error": (ctypes.c_char_p, []),
    "dilution_device_status": (_I, []),
    "dilution_selftest_bounded_wait": (_I, [_P, _P]),
    "dilution_launch_count": (ctypes.c_ulonglong, []),
    "dilution_profile_enable": (_I, [_I]),
    "dilution_profile_collect": (_I, [ctypes.c_char_p, _Z]),
    "dilution_rowstats": (_I, [_P, _P, _I, _I, _L, _L, _L, _L, _I, _F, _P, _P, _P]),
    "dilution_rowstats_pk": (_I, [_P, _P, _I, _I, _L, _L, _I, _F, _P, _P, _P, _P]),
    "dilution_softmax_forward": (_I, [_P, _P, _P, _I, _I, _L, _L, _L, _L, _I, _F, _P, _P, _P, _P]),
    "dilution_carry_rows": (_I, [_I, _I, _I, _I]),
    "dilution_colsum_scan": (_I, [_P, _P, _I, _I, _L, _L, _L, _L, _I, _F, _P, _P, _P, _I, _P, _P, _P]),
    "dilution_forward_main": (_I, [_P, _P, _P, _I, _I, _L, _L, _L, _L, _I, _F, _F,
                                   _P, _P, _P, _I, _P, _P, _P, _P, _P]),
    "dilution_forward_fused": (_I, [_P, _P, _P, _I, _I, _L, _L, _I, _F, _F, _P, _P, _P, _P, _P, _P, _P]),
    "dilution_backward_scratch_bytes": (_Z, [_L, _L, _I]),
    "dilution_backward": (_I, [_P, _P, _P, _I, _I, _L, _L, _I, _F, _F,
                               _P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _P, _P]),
    "dilution_decode_scratch_bytes": (_Z, [_L, _L, _I]),
    "dilution_decode": (_I, [_P, _P, _P, _I, _L, _L, _L, _I, _F, _F, _P, _P, _P, _P]),
    "dilution_decode_append": (_I, [_P, _P, _P, _P, _P, _I, _L, _L, _L, _I, _F, _F, _P, _P, _P, _P]),
    "dilution_softmax_decode_append": (_I, [_P, _P, _P, _P, _P, _I, _L, _L, _L, _I, _F, _P, _P, _P]),
    "dilution_split_heads_rope": (_I, [_P, _P, _P, _P, _P, _P, _L, _L, _I, _I, _I, _P]),
    "dilution_decode_static": (_I, [_P, _P, _P, _I, _L, _L, _L, _I, _F, _F, _P, _P, _P]),
    "dilution_decode_append_at": (_I, [_P, _P, _P, _P, _P, _I, _L, _L, _P, _I, _F, _F, _P, _P, _P, _P]),
    "dilution_softmax_decode_append_at": (_I, [_P, _P, _P, _P, _P, _I, _L, _L, _P, _I, _F, _P, _P, _P]),
    "dilution_split_heads_rope_at": (_I, [_P, _P, _P, _P, _P, _P, _L, _L, _I, _I, _P, _P]),
    "dilution_variant_forward": (_I, [_P, _P, _P, _I, _I, _L, _L, _I, _F, _F, _I, _I, _F,
                                      _P, _P, _P, _P, _P, _P, _P, _P]),
    "dilution_variant_backward": (_I, [_P, _P, _P, _I, _I, _L, _L, _I, _F, _F, _I, _I, _F,
                                       _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "dilution_variant_decode": (_I, [_P, _P, _P, _P, _P, _I, _L, _L, _L, _I, _F, _F, _I, _I, _F, _P, _P, _P, _P]),
}
# codes of the reference's BID_TYPES (kernels_bid.py:84) for the bids that are built
BID = {"softmax": 0, "relu": 1, "relu2": 2, "softplus": 3, "minshift": 4, "sigmoid": 5, "expshift": 6, "sigshift": 7}
ROW_SUM_BIDS = (0, 1, 2, 3, 4)      # bids with row statistics and a Jacobian correction in the backward

_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def load() -> ctypes.CDLL:
    """Load the shared library once; raise RuntimeError if it is not built."""
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError(
                f"{LIB_PATH} is not built; run `python dilution-attention_b200/build.py` "
                "(there is no CPU or Triton fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().dilution_last_error().decode()
        kind = ValueError if rc in (1, 2) else RuntimeError
        raise kind(f"{what} failed ({rc}): {msg}")


def launch_count() -> int:
    return int(load().dilution_launch_count())


def profile(enable: bool) -> None:
    load().dilution_profile_enable(1 if enable else 0)


def profile_collect() -> dict:
    """{kernel: (launches, total_ms)} of the launches recorded since the last call."""
    buf = ctypes.create_string_buffer(1 << 16)
    check(load().dilution_profile_collect(buf, len(buf)), "dilution_profile_collect")
    out = {}
    for line in buf.value.decode().splitlines():
        name, count, ms = line.split()
        out[name] = (int(count), float(ms))
    return out


def carry_rows(dtype_code: int, precision_code: int, head_dim: int, training: bool) -> int:
    """Query rows per demand checkpoint for this case (dilution_carry_rows of the C ABI)."""
    return int(load().dilution_carry_rows(dtype_code, precision_code, head_dim, 1 if training else 0))


def tensor_core_path(dtype_code: int, precision_code: int, head_dim: int) -> bool:
    """True when a call with these parameters runs on the tcgen05 kernels."""
    return dtype_code == BF16 and precision_code == PREC["bf16"] and head_dim == 64
