"""The C-ABI library loads and exports every symbol that include/pt_b200.h declares (no compute calls)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "pt_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pt_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_op_surface():
    syms = declared_symbols()
    for name in ["pt_int4_to_half", "pt_linear", "pt_norm_ce", "pt_rms_norm", "pt_softmax", "pt_kv_cache", "pt_kv_cache_pipeline", "pt_kv_cache_fp8", "pt_kv_cache_pipeline_fp8",
                 "pt_kv_append_attn", "pt_kv_export", "pt_kv_reorder_pages", "pt_kv_reorder_table", "pt_topk", "pt_beam_search",
                 "pt_cast_fp8", "pt_fp8_matmul", "pt_wkv", "pt_embedding", "pt_step_containers"]:
        assert name in syms


def test_library_exports_every_declared_symbol():
    from poptransformer_b200 import _lib, build
    build.build()
    handle = ctypes.CDLL(_lib.LIB_PATH)
    missing = [s for s in declared_symbols() if not hasattr(handle, s)]
    assert not missing, f"declared in pt_b200.h but not exported: {missing}"
    # the ctypes table mirrors the header one to one
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    assert handle.pt_version() >= 100


def test_argument_checks_run_without_a_gpu():
    """Shape violations are rejected before any launch, like the reference's setup()-time errors."""
    from poptransformer_b200 import _lib
    L = _lib.lib()
    rc = L.pt_norm_ce(ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16), 2, 770, 1e-5, ctypes.c_void_p(16), None)
    assert rc == -1 and b"4x a last dim" in L.pt_last_error()
    rc = L.pt_norm_ce(ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16), 2, 8192, 1e-5, ctypes.c_void_p(16), None)
    assert rc == -1 and b"8192" in L.pt_last_error()
    rc = L.pt_int4_to_half(ctypes.c_void_p(16), ctypes.c_void_p(16), 4, 4, 2, 0, ctypes.c_void_p(16), None)
    assert rc == -1 and b"axis" in L.pt_last_error()
    assert L.pt_linear_packed_bytes(0, 4096, 4096) == 256 * 32 * 1056     # 16-row x 128-k tiles: 1 KB of nibbles + 32 B of scales
    assert L.pt_linear_packed_bytes(1, 4096, 4096) == 4096 * 4096 * 2
    assert L.pt_linear_workspace_bytes(1, 4096, 4) >= 4 * 4096 * 4
