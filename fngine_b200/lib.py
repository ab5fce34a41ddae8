"""ctypes binding of libfngine_b200.so (the C ABI declared in include/fngine_b200.h).

There is no fallback path: if the library has not been built, or a compute entry point fails,
an exception is raised.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# FNGINE_B200_LIB names another build of the same library (A/B runs of kernel variants).
LIB_PATH = os.environ.get("FNGINE_B200_LIB") or os.path.join(HERE, "libfngine_b200.so")

FMT_IQ4_NL, FMT_IQ3_S = 20, 21
FMT_IQ3_XXS, FMT_IQ2_S, FMT_IQ4_XS, FMT_Q2_0 = 18, 22, 23, 42  # decode width only (plain kernels)
DT_F32, DT_BF16 = 0, 1
ACT_Q8_K, ACT_Q8_0 = 0, 1
HIDDEN, EXPERTS, TOPK, ROUTER_ROWS = 2560, 512, 10, 513
DECODE_MAX_TOKENS, DECODE_MAX_PAIRS = 16, 160
XQ_STRIDE, HQ_STRIDE = 2880, 720
STATUS_OK, STATUS_PIPELINE_TIMEOUT, STATUS_BAD_WORK = 0, 1, 2


class FbError(RuntimeError):
    pass


class ExpertLayout(C.Structure):
    _fields_ = [("slots", C.c_void_p), ("blob_stride", C.c_int64), ("gate_offset", C.c_int64),
                ("up_offset", C.c_int64), ("down_offset", C.c_int64), ("gate_up_format", C.c_int32),
                ("down_format", C.c_int32), ("inter", C.c_int32), ("reserved", C.c_int32)]


class DecodeWork(C.Structure):
    _fields_ = [("n_items", C.c_int32), ("n_pairs", C.c_int32), ("n_cold", C.c_int32), ("tokens", C.c_int32),
                ("item_slot", C.c_int32 * DECODE_MAX_PAIRS), ("item_pair_begin", C.c_int32 * (DECODE_MAX_PAIRS + 1)),
                ("pair_token", C.c_int32 * DECODE_MAX_PAIRS), ("pair_weight", C.c_float * DECODE_MAX_PAIRS),
                ("token_pair_count", C.c_int32 * DECODE_MAX_TOKENS),
                ("token_pairs", (C.c_int32 * TOPK) * DECODE_MAX_TOKENS),
                ("token_cold_count", C.c_int32 * DECODE_MAX_TOKENS),
                ("topk_expert", (C.c_int32 * TOPK) * DECODE_MAX_TOKENS),
                ("topk_weight", (C.c_float * TOPK) * DECODE_MAX_TOKENS)]


class DecodeWorkspace(C.Structure):
    _fields_ = [("work", C.c_void_p), ("xq", C.c_void_p), ("h", C.c_void_p), ("hq", C.c_void_p),
                ("partial", C.c_void_p), ("item_done", C.c_void_p), ("sched", C.c_void_p), ("status", C.c_void_p),
                ("gate_up_format", C.c_int32), ("down_format", C.c_int32), ("inter", C.c_int32),
                ("reserved", C.c_int32)]


class PrefillWorkspace(C.Structure):
    _fields_ = [("capacity", C.c_int32), ("inter", C.c_int32), ("max_units_gate_up", C.c_int32),
                ("max_units_down", C.c_int32), ("meta", C.c_void_p), ("expert_count", C.c_void_p),
                ("expert_offset", C.c_void_p), ("expert_cursor", C.c_void_p), ("topk_expert", C.c_void_p),
                ("topk_weight", C.c_void_p), ("pair_token", C.c_void_p), ("pair_weight", C.c_void_p),
                ("token_pair", C.c_void_p), ("units_gate_up", C.c_void_p), ("units_down", C.c_void_p),
                ("h", C.c_void_p), ("yp", C.c_void_p), ("status", C.c_void_p)]


_P = C.c_void_p
_I32, _I64 = C.c_int32, C.c_int64
EP_MAX_RANKS = 8


class LinearEpilogue(C.Structure):
    """fb_linear_epilogue: the output side of a decode-width projection."""
    _fields_ = [("kind", C.c_int32), ("gate_stride", C.c_int32), ("out", C.c_void_p), ("inj", C.c_void_p),
                ("gate_logit", C.c_void_p)]


EPI_STORE_BF16, EPI_STORE_F32, EPI_GR_WRITE, EPI_SWIGLU, EPI_SHARED_SCALE = range(5)
FP8_PATH_AUTO, FP8_PATH_A16, FP8_PATH_A8 = range(3)


class EpPeers(C.Structure):
    """fb_ep_peers: peer-mapped exchange buffers of an expert-parallel decode step."""
    _fields_ = [("rank", C.c_int32), ("n_ranks", C.c_int32), ("x_all", C.c_void_p * EP_MAX_RANKS),
                ("y_parts", C.c_void_p * EP_MAX_RANKS)]


_SIGNATURES = {
    # name: (restype, argtypes)
    "fb_last_error_string": (C.c_char_p, []),
    "fb_abi_version": (_I32, []),
    "fb_compiled_sm": (_I32, []),
    "fb_moe_row_bytes": (_I64, [_I32, _I32]),
    "fb_moe_act_format": (_I32, [_I32]),
    "fb_act_row_bytes": (_I64, [_I32, _I32]),
    "fb_moe_expert_layout_make": (_I32, [_P, _I64, _I32, _I32, _I32, C.POINTER(ExpertLayout)]),
    "fb_moe_blob_bytes": (_I64, [_I32, _I32, _I32]),
    "fb_moe_decode_workspace_bytes": (C.c_size_t, [_I32]),
    "fb_moe_decode_workspace_make": (_I32, [_P, C.POINTER(ExpertLayout), C.POINTER(DecodeWorkspace)]),
    "fb_router_logits": (_I32, [_P, _I32, _P, _I32, _I32, _P, _I32, _P]),
    "fb_moe_select_publish": (_I32, [_P, _I32, _P, _I32, _P, _I32, _P, _P, _I32, C.POINTER(DecodeWorkspace), _P, _P]),
    "fb_moe_hot_gate_up": (_I32, [C.POINTER(ExpertLayout), _I32, C.POINTER(DecodeWorkspace), _P]),
    "fb_moe_hot_down": (_I32, [C.POINTER(ExpertLayout), _I32, C.POINTER(DecodeWorkspace), _P]),
    "fb_moe_hot_experts": (_I32, [C.POINTER(ExpertLayout), _I32, C.POINTER(DecodeWorkspace), _P]),
    "fb_moe_combine": (_I32, [C.POINTER(DecodeWorkspace), _P, _P, _I32, _P, _P, _P, _P, _I32, C.c_longlong, _P,
                              C.c_float, _P]),
    "fb_moe_layer_decode": (_I32, [_P, C.POINTER(ExpertLayout), _P, _I32, _I32, C.POINTER(DecodeWorkspace), _P, _P, _P]),
    "fb_moe_layer_decode_host": (_I32, [_P, C.POINTER(ExpertLayout), _P, _I32, _I32, C.POINTER(DecodeWorkspace), _P,
                                        _P, _P, _P, _P]),
    "fb_moe_prefill_workspace_bytes": (C.c_size_t, [_I32, _I32]),
    "fb_moe_prefill_workspace_make": (_I32, [_P, _I32, _I32, C.POINTER(PrefillWorkspace)]),
    "fb_moe_route": (_I32, [_P, _I32, _P, _P, _I32, _P, _P, _I32, C.POINTER(PrefillWorkspace), _P]),
    "fb_moe_grouped_gate_up": (_I32, [C.POINTER(ExpertLayout), _P, _P, _I32, C.POINTER(PrefillWorkspace), _P]),
    "fb_moe_grouped_down": (_I32, [C.POINTER(ExpertLayout), _P, _I32, C.POINTER(PrefillWorkspace), _P]),
    "fb_moe_prefill_combine": (_I32, [C.POINTER(PrefillWorkspace), _P, _P, _I32, _P, _P, _P, _P, _I32, C.c_longlong, _P,
                                      C.c_float, _P]),
    "fb_moe_layer_decode_ep": (_I32, [_P, C.POINTER(ExpertLayout), _P, _P, _I32, _I32, C.POINTER(DecodeWorkspace), _P, _P,
                               _P]),
    "fb_ep_sum_ranks": (_I32, [_P, _I32, _I32, _P, _P]),
    "fb_ep_exchange_bytes": (C.c_size_t, [_I32]),
    "fb_ep_exchange_create": (_I32, [_P, _P, _P]),
    "fb_ep_exchange_open": (_I32, [_P, _P, _P]),
    "fb_ep_exchange_close": (_I32, [_P, _P, _I32]),
    "fb_moe_layer_decode_ep_p2p": (_I32, [_P, C.POINTER(ExpertLayout), _P, _P, _I32, C.POINTER(EpPeers), C.c_uint32,
                                          C.POINTER(DecodeWorkspace), _P, _P, _P]),
    "fb_moe_topk": (_I32, [_P, _I32, _I32, _P, _P, _P]),
    "fb_moe_route_ep": (_I32, [_P, _P, _I32, _I32, _I32, C.POINTER(PrefillWorkspace), _P]),
    "fb_moe_prefill_set_accumulation": (_I32, [_I32]),
    "fb_ep_prefill_scratch_bytes": (C.c_size_t, [_I32, _I32, _I32]),
    "fb_ep_prefill_layer": (_I32, [C.POINTER(ExpertLayout), _P, _P, _I32, _I32, _P, _I32, _P, _I32, _I32, _I32,
                                   C.POINTER(PrefillWorkspace), _P, _P, _P, _P]),
    "fb_moe_route_placed": (_I32, [_P, _P, _P, _I32, C.POINTER(PrefillWorkspace), _P]),
    "fb_ep_scatter_sum": (_I32, [_P, _P, _I32, _I32, _P, _P]),
    "fb_moe_layer_decode_static": (_I32, [_P, C.POINTER(ExpertLayout), _P, _I32, _I32, _P, _P]),
    "fb_moe_layer_decode_static_status": (_I32, [_P, _P]),
    "fb_ep_set_wait_limit": (None, [C.c_uint32]),
    "fb_linear_fp8_workspace_bytes": (C.c_size_t, [_I32, _I32, _I32]),
    "fb_linear_fp8": (_I32, [_P, _I32, _P, _P, _I32, _I32, _I32, C.POINTER(LinearEpilogue), _P, C.c_size_t, _P, _I32]),
    "fb_fp8_split_tokens": (_I32, [_P, _I32, _I32, _P, _P, _P, _P]),
    "fb_fp8_quantize_tokens": (_I32, [_P, _I32, _I32, _P, _P, _P]),
    "fb_linear_fp8_decode_workspace_bytes": (C.c_size_t, [_I32, _I32]),
    "fb_linear_fp8_decode": (_I32, [_P, _I32, _P, _P, _I32, _I32, _I32, C.POINTER(LinearEpilogue), _P, C.c_size_t, _P]),
    "fb_dequant_rows": (_I32, [_I32, _P, _I64, _I32, _I32, _P, _P]),
    "fb_quantize_act": (_I32, [_I32, _P, _I32, _I32, _I32, _P, _P]),
    "fb_synth_fill_blocks": (_I32, [_I32, _P, _I64, _I64, C.c_uint64, _P, _P]),
    "fb_synth_fill_experts": (_I32, [_I32, _P, _I64, _I32, _I32, _I64, C.c_uint64, _P, _P]),
}

_lib = None


def exported_names():
    """Every symbol include/fngine_b200.h declares (kept in step with the header by a test)."""
    return sorted(_SIGNATURES)


def load():
    """Loads the shared library and sets the prototypes. Raises FbError if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FbError("libfngine_b200.so is not built: run `python -m fngine_b200.build` "
                          "(or __graft_entry__.build()); there is no CPU fallback")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status, what=""):
    if status != 0:
        msg = load().fb_last_error_string().decode("utf-8", "replace")
        raise FbError("%s failed with status %d: %s" % (what or "fngine_b200 call", status, msg))
