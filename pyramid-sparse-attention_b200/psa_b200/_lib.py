"""ctypes binding of the C-ABI CUDA library (include/psa_b200.h).

There is no CPU or eager-PyTorch fallback: if the shared library is missing or does not load, importing
this module raises, and every op raises if its tensors are not CUDA tensors.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpsa_b200.so")

PSA_OK, PSA_ERR_ARG, PSA_ERR_UNSUPPORTED, PSA_ERR_CUDA, PSA_ERR_TIMEOUT = 0, 1, 2, 3, 4
PSA_F32, PSA_F16, PSA_BF16 = 0, 1, 2

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} not found: the PSA CUDA library has not been built. Run "
        "`python pyramid-sparse-attention_b200/build.py` (needs nvcc with sm_100a support). "
        "This package has no CPU fallback.")

lib = C.CDLL(LIB_PATH)

_p, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); mirrors include/psa_b200.h declaration by declaration
SIGNATURES = {
    "psa_last_error_string": (C.c_char_p, []),
    "psa_build_info": (C.c_char_p, []),
    "psa_pyramid_kv": (_i, [_p] * 8 + [_i64, _i64, _i, _i, _i, _p]),
    "psa_kv_image_bytes": (_sz, [_i64, _i64, _i, _i]),
    "psa_pyramid_kv_images": (_i, [_p] * 4 + [_i64, _i64, _i, _i, _i, _p]),
    "psa_fwd_images": (_i, [_p] * 5 + [_i64, _i64, _i64, _i, _i, _i, _i, _i, _f, _i, _i, _p, _p]),
    "psa_gather_rows": (_i, [_p, _p, _p, _i64, _i64, _i, _i, _p]),
    "psa_pyramid_kv_images_perm": (_i, [_p] * 5 + [_i64, _i64, _i, _i, _i, _p]),
    "psa_block_scores_perm": (_i, [_p] * 8 + [_sz, _i64, _i64, _i64, _i, _i, _i, _i, _p]),
    "psa_fwd_images_perm": (_i, [_p] * 6 + [_i64, _i64, _i64, _i, _i, _i, _i, _i, _f, _i, _i, _p, _p]),
    "psa_gather_heads": (_i, [_p, _p, _p, _i, _i64, _i, _i, _p]),
    "psa_pyramid_kv_images_tm": (_i, [_p] * 5 + [_i, _i64, _i, _i, _i, _p]),
    "psa_block_scores_tm": (_i, [_p] * 7 + [_sz, _i, _i64, _i, _i, _i, _i, _p]),
    "psa_fwd_images_tm": (_i, [_p] * 6 + [_i, _i64, _i, _i, _i, _i, _i, _f, _i, _i, _p, _p]),
    "psa_gather_heads_rope": (_i, [_p, _p, _p, _p, _i64, _p, _i, _i64, _i, _i, _p]),
    "psa_pyramid_kv_images_tm_rope": (_i, [_p] * 5 + [_i64, _p, _p, _i, _i64, _i, _i, _i, _p]),
    "psa_block_scores_tm_rope": (_i, [_p] * 5 + [_i64] + [_p] * 4 + [_sz, _i, _i64, _i, _i, _i, _i, _p]),
    "psa_gather_rows_rope": (_i, [_p, _p, _p, _p, _i64, _p, _i64, _i64, _i, _i, _p]),
    "psa_pyramid_kv_images_perm_rope": (_i, [_p] * 5 + [_i64, _p, _p, _i64, _i64, _i, _i, _i, _p]),
    "psa_block_scores_perm_rope": (_i, [_p] * 5 + [_i64] + [_p] * 4 + [_sz, _i64, _i64, _i, _i, _i, _i, _p]),
    "psa_antidiag_scratch_bytes": (_sz, [_i64, _i64, _i, _i, _i, _i]),
    "psa_antidiag_scores": (_i, [_p, _p, _p, _p, _sz, _i64, _i64, _i, _i, _i, _i, _i, _i, _p]),
    "psa_antidiag_scores_impl": (_i, [_p, _p, _p, _p, _sz, _i64, _i64, _i, _i, _i, _i, _i, _i, _i, _p, _p]),
    "psa_assign_levels_causal": (_i, [_p, _p, _i64, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _i, _p]),
    "psa_legacy_index_bytes": (_sz, [_i64, _i64]),
    "psa_legacy_fwd_images": (_i, [_p] * 7 + [_i64, _i64, _i, _i, _f, _i, _i, _p, _p]),
    "psa_fwd_images_scatter": (_i, [_p] * 5 + [_i, _i64, _i, _i, _i64, _i64, _i64, _i, _i, _i, _i, _i, _f, _i, _i, _p, _p]),
    "psa_block_scores_peers": (_i, [_p, _p, _i, _i64, _i, _i, _p, _p, _p, _p, _sz, _i64, _i, _i, _i, _i, _p]),
    "psa_pyramid_kv_images_peers": (_i, [_p, _p, _i, _i64, _i, _i, _p, _p, _i64, _i, _i, _i, _i, _p]),
    "psa_sample_rows": (_i, [_i64, _i64, _i, _i, _p, _p, _p]),
    "psa_push_samples": (_i, [_p, _p, _p, _i, _i64, _i, _i, _i, _i, _i, _i64, _i64, _i, _p]),
    "psa_block_scores_samples": (_i, [_p, _p, _p, _p, _sz, _i64, _i64, _i64, _i, _i, _i, _i, _p]),
    "psa_push_heads": (_i, [_p, _p, _i, _i64, _i, _i, _i, _i, _i, _p]),
    "psa_peer_alloc": (_i, [_sz, _p, _p]),
    "psa_peer_open": (_i, [_p, _p]),
    "psa_peer_close": (_i, [_p]),
    "psa_peer_free": (_i, [_p]),
    "psa_pull_heads": (_i, [_p, _i, _p, _i64, _i, _i, _i, _i, _i, _i, _i, _p]),
    "psa_block_scores_scratch_bytes": (_sz, [_i64, _i64, _i64, _i, _i, _i]),
    "psa_block_scores": (_i, [_p] * 6 + [_sz, _i64, _i64, _i64, _i, _i, _i, _i, _i, _p]),
    "psa_block_scores_static_capacity": (_sz, []),
    "psa_block_scores_static": (_i, [_p] * 5 + [_i64, _i64, _i64, _i, _i, _i, _i, _i, _p]),
    "psa_assign_levels": (_i, [_p, _p, _i64, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _i, _i, _p]),
    "psa_density": (_i, [_p, _p, _i64, _i64, _i, _i, _p]),
    "psa_ksim": (_i, [_p, _p, _i64, _i64, _i, _i, _f, _f, _f, _i, _p]),
    "psa_ksim_perm": (_i, [_p, _p, _p, _i64, _i64, _i, _i, _f, _f, _f, _i, _p]),
    "psa_legacy_fwd_images_perm": (_i, [_p] * 7 + [_i64, _i64, _i, _i, _f, _i, _p, _p]),
    "psa_fwd": (_i, [_p] * 11 + [_i64, _i64, _i64, _i, _i, _i, _i, _i, _f, _i, _i, _i, _p, _p]),
    "psa_legacy_fwd": (_i, [_p] * 12 + [_i64, _i64, _i, _i, _f, _i, _i, _p]),
    "psa_legacy_bwd": (_i, [_p] * 17 + [_i64, _i64, _i, _i, _f, _i, _i, _p]),
    "psa_legacy_bwd_tc": (_i, [_p] * 17 + [_i64, _i64, _i, _i, _f, _i, _i, _p]),
    "psa_legacy_bwd_scratch_bytes": (_sz, [_i64, _i64, _i]),
    "psa_legacy_bwd_tcgen05": (_i, [_p] * 11 + [_sz, _i64, _i64, _i, _i, _f, _i, _i, _p, _p]),
}
for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)          # AttributeError here = the library does not export a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args


class PSAKernelError(RuntimeError):
    pass


def last_error() -> str:
    return lib.psa_last_error_string().decode()


def check(rc: int, what: str) -> None:
    """Turn a status code into the exception type the reference raises for the same condition
    (ValueError for bad arguments, RuntimeError otherwise)."""
    if rc == PSA_OK:
        return
    msg = f"{what}: {last_error()} (status {rc})"
    if rc in (PSA_ERR_ARG, PSA_ERR_UNSUPPORTED):
        raise ValueError(msg)
    raise PSAKernelError(msg)
