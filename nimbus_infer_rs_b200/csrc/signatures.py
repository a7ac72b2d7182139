"""Argument types of the library's ``extern "C"`` entry points, one letter per argument:
``p`` pointer or stream, ``i`` int, ``l`` long long, ``f`` float, ``d`` double.  With these declared, the
callers pass plain Python numbers and addresses, which ctypes converts without a wrapper
object per argument (a prefill step makes about a hundred calls, and the host must keep ahead
of the GPU).  ``tests/test_signatures.py`` derives the same table from the CUDA sources."""
from __future__ import annotations

import ctypes

SIGNATURES = {
    "nb_attention_decode_supported": "iiiii",
    "nb_attention_decode_scratch": "iiiiippp",
    "nb_attention_decode": "piiipppppiiiiipiifiiipppiiip",
    "nb_attention_decode_static": "piiipppppiiiiipiifiiip",
    "nb_attention_decode_cluster_merge": "i",
    "nb_attention_decode_cluster_limit": "",
    "nb_attention_generic": "piiipppppiiiiipiifiip",
    "nb_attention_prefill_supported": "iiiiiii",
    "nb_attention_prefill_f32_supported": "iiii",
    "nb_attention_prefill_f32": "piiippppppiiiiipiifiiip",
    "nb_attention_prefill": "piiippppppiiiiipiifiiip",
    "nb_attention_prefill_tc_supported": "iiiiiiiii",
    "nb_attention_prefill_tc_error": "",
    "nb_attention_prefill_tc_set_wait_budget": "l",
    "nb_attention_prefill_tc": "piiiipppppipiiiiipiifiiiiippiiip",
    "nb_attention_prefill_tc_record": "i",
    "nb_gemm_simt": "pipipppiiiiip",
    "nb_gemm_skinny": "pippfpipppiiiiip",
    "nb_gemm_stream": "pippfppppiiiiip",
    "nb_gemm_stream_supported": "iiii",
    "nb_gemm_stream_plan": "iiiip",
    "nb_gemm_stream_tune": "i",
    "nb_gemm_stream_set_wait_budget": "l",
    "nb_gemm_skinny_norm_supported": "iii",
    "nb_gemm_tc_rows_supported": "iii",
    "nb_gemm_tc_rows_preferred": "iii",
    "nb_gemm_tc_rows_plan": "iiip",
    "nb_gemm_tc_rows_force_split": "i",
    "nb_gemm_tc_rows_set_wait_budget": "l",
    "nb_gemm_tc_rows": "pppppiiiiip",
    "nb_gemm_tcgen05_supported": "iiiii",
    "nb_gemm_tcgen05_error": "",
    "nb_gemm_tcgen05_set_wait_budget": "l",
    "nb_wait_probe": "pp",
    "nb_device_errors": "i",
    "nb_gemm_tcgen05_use_pairs": "i",
    "nb_gemm_tcgen05_tune": "ii",
    "nb_gemm_tcgen05": "pppppiiiiip",
    "nb_abi_version": "",
    "nb_set_overlap": "i",
    "nb_get_overlap": "",
    "nb_embed_pos": "ppppipiip",
    "nb_layernorm": "pppppiiifp",
    "nb_kv_append": "piiiipppppiiiiip",
    "nb_advance_decode": "ppppip",
    "nb_repetition_penalty": "piipipfp",
    "nb_history_append": "pipppip",
    "nb_top_candidates": "piiiidppppp",
    "nb_argmax_split": "piipppip",
    "nb_argmax": "piipp",
    "nb_sample_temperature": "piifppp",
    "nb_sample_top_k": "piiifppp",
    "nb_sample_top_p": "piiiffppp",
    "nb_sample_top_p_max_k": "",
}

_CTYPE = {"p": ctypes.c_void_p, "i": ctypes.c_int, "f": ctypes.c_float, "d": ctypes.c_double,
          "l": ctypes.c_longlong}


def declare(lib) -> None:
    """Set ``argtypes`` (and ``int`` results) on every entry point of the loaded library."""
    for name, letters in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = [_CTYPE[c] for c in letters]
        fn.restype = ctypes.c_int
    lib.nb_set_overlap.restype = None
    lib.nb_attention_decode_scratch.restype = None
    lib.nb_last_error.argtypes = []
    lib.nb_last_error.restype = ctypes.c_char_p
    lib.nb_attention_decode_static_capacity.argtypes = []
    lib.nb_attention_decode_static_capacity.restype = ctypes.c_longlong
