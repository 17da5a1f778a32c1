"""The one table of the kernel libraries' C entry points as ctypes sees them.

Each entry is `name: (result, arguments)` in one-letter codes; `apply` sets `restype` and
`argtypes` on a loaded library for the entries it exports, so a call with a wrong number or
kind of arguments fails in Python instead of corrupting a kernel's stack.  The table restates
csrc/sonicboom_b200.h (and csrc/no_alloc.h); a test parses the headers and compares.

    i int      f float     z size_t     u uint32_t     p any data pointer     s the CUDA stream
    c const char* (result only)          v void (result only)
"""
from __future__ import annotations

import ctypes

CODES = {"i": ctypes.c_int, "f": ctypes.c_float, "z": ctypes.c_size_t, "u": ctypes.c_uint32,
         "p": ctypes.c_void_p, "s": ctypes.c_void_p, "c": ctypes.c_char_p, "v": None}

_GEMM = "pipiiiiipippis"          # A, a_dtype, W, w_dtype, M, N, K, epilogue, bias, bias_dtype, residual, out, out_dtype, stream

EVERY_LIBRARY = {
    "sb_last_error": ("c", ""),
    "sb_pdl_enabled": ("i", ""),
    "sb_set_pdl": ("v", "i"),
}
CORE = {
    "sb_abi_version": ("i", ""),
    "sb_embed": ("i", "pipiiifps"),
    "sb_rmsnorm": ("i", "ppiipifpis"),
    "sb_softcap": ("i", "pzfs"),
    "sb_add_bias": ("i", "ppiiis"),
    "sb_cast": ("i", "pipizs"),
    "sb_rope_store": ("i", "piiiiipppppipipiis"),
    "sb_gemm_plain": ("i", _GEMM),
    "sb_gemm_skinny": ("i", _GEMM),
    "sb_gemm_tiled": ("i", _GEMM),
    "sb_gemm_tc5": ("i", _GEMM[:-1] + "pziis"),
    "sb_gemm_tc5_ex": ("i", _GEMM[:-1] + "pziips"),
    "sb_gemm_tc5_scratch_bytes": ("z", "iiii"),
    "sb_gemm_tc5_fuses_norm": ("i", "iiiiiii"),
    "sb_gemm_tc5_fuses_rope": ("i", "iiiiiiiii"),
    "sb_tc5_status": ("i", ""),
    "sb_gemm_tc5_pairs": ("v", "i"),
    "sb_gemm_tc5_tile_width": ("i", "iii"),
    "sb_gemm_tc5_force_width": ("v", "i"),
    "sb_attention_plain": ("i", "ppiippppipiiiiifs"),
    "sb_sample_params_size": ("i", ""),
    "sb_sample": ("i", "piippipps"),
    "sb_add_i32": ("i", "piis"),
    "sb_advance_rows": ("i", "ppis"),
    "sb_random_normal": ("i", "pizuuffs"),
}
ATTENTION = {
    "sb_attention_head_dim": ("i", ""),
    "sb_attention_force_mma": ("v", "i"),
    "sb_attention_status": ("i", ""),
    "sb_attention_last_launches": ("i", ""),
    "sb_attention_scratch_bytes": ("z", "iiiii"),
    "sb_attention": ("i", "ppiiippppipiiiifpzpiiiipzs"),
    "sb_attention_decode_static": ("i", "ppiiippppipiiiifis"),
    "sb_attention_static_scratch_bytes": ("z", ""),
}


def apply(lib: ctypes.CDLL, table: dict) -> ctypes.CDLL:
    """Types the entry points of `table` (and those every library has) on a loaded library."""
    for name, (result, args) in {**EVERY_LIBRARY, **table}.items():
        fn = getattr(lib, name)
        fn.restype = CODES[result]
        fn.argtypes = [CODES[a] for a in args]
    return lib
