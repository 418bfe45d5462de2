"""CPU: the C-ABI library loads and exports every symbol include/psa_b200.h declares (no compute calls)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    src = open(os.path.join(ROOT, "include", "psa_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(psa_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_the_expected_entry_points():
    syms = declared_symbols()
    for s in ("psa_pyramid_kv", "psa_block_scores", "psa_assign_levels", "psa_fwd", "psa_legacy_fwd", "psa_legacy_bwd",
              "psa_ksim", "psa_density", "psa_last_error_string"):
        assert s in syms


def test_library_exports_every_declared_symbol():
    from psa_b200 import _lib
    for s in declared_symbols():
        assert hasattr(_lib.lib, s), f"{s} declared in include/psa_b200.h but not exported"
        assert s in _lib.SIGNATURES, f"{s} has no ctypes signature"
    assert b"sm_100a" in _lib.lib.psa_build_info()


def test_argument_errors_need_no_gpu():
    from psa_b200 import _lib
    rc = _lib.lib.psa_pyramid_kv(None, None, None, None, None, None, None, None, 1, 1, 64, 64, 0, None)
    assert rc == _lib.PSA_ERR_ARG and "null" in _lib.last_error()
    assert _lib.lib.psa_block_scores_scratch_bytes(2, 1000, 1000, 128, 48, 0) == 0     # block_n 48 unsupported


def test_config_validation_matches_reference_conditions():
    import pytest
    from psa_b200 import PSAConfig, legacy_sparse_attention_factory
    with pytest.raises(ValueError):
        PSAConfig(use_sim_mask=True)
    with pytest.raises(ValueError):
        PSAConfig(attn_impl="old_mask_type", block_n=64)
    with pytest.raises(ValueError):
        PSAConfig(block_n=48)
    with pytest.raises(ValueError):
        legacy_sparse_attention_factory(64, 32, 128)
    PSAConfig(attn_impl="old_mask_type", block_n=128, use_sim_mask=True)


def test_no_cpu_path():
    import pytest
    import torch
    from psa_b200 import ops
    x = torch.zeros(1, 1, 64, 64)
    with pytest.raises(RuntimeError):
        ops.pyramid_kv(x, x, 64)
