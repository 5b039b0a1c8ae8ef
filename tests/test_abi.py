"""The C-ABI library loads without a GPU and exports every symbol include/eisen_b200.h declares."""
import ctypes
import os

import eisen_b200 as eb
from eisen_b200 import _lib


def test_header_declares_entry_points():
    d = eb.declarations()
    for name in ("eisen_gemm_bf16", "eisen_attn_fwd", "eisen_attn_bwd", "eisen_rmsnorm_bwd", "eisen_ce_fwd",
                 "eisen_ce_bwd", "eisen_rope", "eisen_swiglu_bwd", "eisen_embedding_bwd", "eisen_adamw_step"):
        assert name in d, name
    assert len(d) >= 38


def test_library_exports_every_declared_symbol():
    assert os.path.exists(_lib.LIB_PATH), "build the library first (python eisen_b200/build.py)"
    raw = ctypes.CDLL(_lib.LIB_PATH)
    missing = [n for n in eb.declarations() if not hasattr(raw, n)]
    assert not missing, missing


def test_version_and_error_string():
    L = eb.lib()
    assert b"sm_100a" in L.eisen_version()
    assert isinstance(L.eisen_last_error(), bytes)


def test_workspace_queries_need_no_gpu():
    L = eb.lib()
    assert L.eisen_attn_bwd_workspace_bytes(2, 256, 4, 2, 64) >= 2 * 256 * 4 * 64 * 4
    assert L.eisen_embedding_bwd_workspace_bytes(100, 50) >= (2 * 50 + 2 * 100) * 4
