"""ctypes binding of libmfb200.so (the C ABI declared in include/mfb200.h).

The library is built in-tree by ``python -m mference_b200.build``.  There is no fallback: if the shared
object is missing, loading raises, and every compute call reports the library's own error text.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libmfb200.so")

OK = 0
ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED_SHAPE, ERR_CUDA, ERR_CAPACITY, ERR_ALLOC = 1, 2, 3, 4, 5
ERR_DEVICE_STATUS, ERR_IO, ERR_NO_SLOT = 6, 7, 8
ERR_GROUP_BASE = 100
GROUP_ERROR_NAMES = {
    101: "invalidQueryCount", 102: "invalidTopK", 103: "invalidNumExperts", 104: "invalidTileExpertCount",
    105: "pairCountMismatch", 106: "tokenOutOfRange", 107: "rankOutOfRange", 108: "expertOutOfRange",
    109: "duplicateTokenRank", 110: "expertSortKeyCountMismatch",
}

DT_BF16, DT_F16, DT_F32 = 0, 1, 2
ACT_SILU, ACT_GELU_TANH = 0, 1
ROUTER_SOFTMAX_TOPK, ROUTER_SQRTSOFTPLUS = 0, 1
FLAG_PREFILL_TENSOR_CORE = 1


class MfbError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"mfb200 error {code}: {text}")
        self.code = code
        self.text = text


class ExpertOffsets(C.Structure):
    """MoEExpertOffsets: nine u32 byte offsets, 36 bytes."""
    _fields_ = [(n, C.c_uint32) for n in
                ("gate_w", "gate_s", "gate_b", "up_w", "up_s", "up_b", "down_w", "down_s", "down_b")]


class Pair(C.Structure):
    _fields_ = [("token", C.c_uint32), ("expert", C.c_uint32), ("rank", C.c_uint32), ("weight_bits", C.c_uint32)]


class Group(C.Structure):
    _fields_ = [("expert", C.c_uint32), ("pair_start", C.c_uint32), ("pair_count", C.c_uint32)]


class Tile(C.Structure):
    _fields_ = [("group_start", C.c_uint32), ("group_count", C.c_uint32), ("pair_start", C.c_uint32),
                ("pair_count", C.c_uint32)]


class MoEConfig(C.Structure):
    _fields_ = [("d", C.c_uint32), ("f", C.c_uint32), ("num_experts", C.c_uint32), ("top_k", C.c_uint32),
                ("bits", C.c_uint32), ("shared_bits", C.c_uint32), ("group_size", C.c_uint32),
                ("scale_dtype", C.c_uint32), ("x_dtype", C.c_uint32), ("activation", C.c_uint32),
                ("router_mode", C.c_uint32), ("swiglu_limit", C.c_float), ("route_scale", C.c_float),
                ("rms_eps", C.c_float), ("max_tokens", C.c_uint32), ("flags", C.c_uint32),
                ("max_layers", C.c_uint32)]


class LayerWeightsC(C.Structure):
    _fields_ = [("router_w", C.c_void_p), ("logit_bias", C.c_void_p), ("per_expert_scale", C.c_void_p),
                ("correction_bias", C.c_void_p), ("norm_w", C.c_void_p), ("pool", C.c_void_p),
                ("slot_stride", C.c_uint64), ("slot_of", C.c_void_p), ("shared_blob", C.c_void_p),
                ("routed_off", ExpertOffsets), ("shared_off", ExpertOffsets),
                ("router_scales", C.c_void_p), ("router_biases", C.c_void_p), ("router_effective_scale", C.c_void_p),
                ("shared_gate_w", C.c_void_p), ("shared_gate_s", C.c_void_p), ("shared_gate_b", C.c_void_p),
                ("gate_group_size", C.c_uint32)]


# name -> (restype, argtypes); every symbol include/mfb200.h declares
_V, _U32, _U64, _I32, _I64 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32, C.c_int64
SIGNATURES = {
    "mfb_last_error": (C.c_char_p, []),
    "mfb_version": (_I32, []),
    "mfb_launch_count": (_U64, []),
    "mfb_expert_layout": (_I32, [_U32, _U32, _U32, C.POINTER(ExpertOffsets), C.POINTER(_U64)]),
    "mfb_moe_prefill_accumulate_f32": (_I32, [_V, _V, C.POINTER(LayerWeightsC), _V, _U32, _U32, _V, _V, _V, _V, _V]),
    "mfb_expert_layout_gate": (_I32, [_U32, _U32, _U32, _U32, C.POINTER(ExpertOffsets), C.POINTER(_U64)]),
    "mfb_moe_create": (_I32, [C.POINTER(MoEConfig), C.POINTER(_V)]),
    "mfb_moe_destroy": (_I32, [_V]),
    "mfb_moe_set_generic": (_I32, [_V, _I32]),
    "mfb_moe_set_trace": (_I32, [_V, _V]),
    "mfb_moe_device_status": (_I32, [_V, _V, C.POINTER(_U32)]),
    "mfb_moe_partial_rows": (_I32, [_V, C.POINTER(_V)]),
    "mfb_moe_selftest_wait": (_I32, [_V, _V, _U64]),
    "mfb_router_logits": (_I32, [_V, _V, _V, _U32, _U32, _V, _V, _V]),
    "mfb_router_select": (_I32, [_V, _V, _V, _U32, _V, _V, _V, _V]),
    "mfb_router_topk": (_I32, [_V, _V, _V, _U32, _U32, C.POINTER(LayerWeightsC), _V, _V]),
    "mfb_slot_lookup": (_I32, [_V, _V, _V, _U32, _V, _U64, _V, _V]),
    "mfb_pool_create": (_I32, [_U32, _U64, _U32, _U32, _U32, C.POINTER(_V)]),
    "mfb_pool_destroy": (_I32, [_V]),
    "mfb_pool_info": (_I32, [_V, C.POINTER(_V), C.POINTER(_U64), C.POINTER(_V)]),
    "mfb_pool_plan": (_I32, [_V, _V, _U32, _V, _U32, _V, _V, C.POINTER(_U32)]),
    "mfb_pool_fill_async": (_I32, [_V, _V, _V, _V, _V, _U32, _V, _U64]),
    "mfb_pool_publish": (_I32, [_V, _V, _V, _V, _V, _U32]),
    "mfb_pool_reserve_speculative": (_I32, [_V, _V, _U32, _U32, _V, _V, C.POINTER(_U32)]),
    "mfb_pool_mark_in_flight": (_I32, [_V, _V, _U32]),
    "mfb_pool_finish_speculative": (_I32, [_V, _V, _V, _V, _V, _U32]),
    "mfb_pool_note_all_hit": (_I32, [_V, _V, _U32]),
    "mfb_pool_slot_of_host": (_I32, [_V, _V]),
    "mfb_ep_plan": (_I32, [_V, _V, _U32, _U32, _U32, _U32, _V, _V, _V, _V]),
    "mfb_ep_pack": (_I32, [_V, _V, _U32, _U32, _V, _U32, _U32, _V]),
    "mfb_ep_combine": (_I32, [_V, _V, _V, _V, _V, _V, _V, _U32, _U32, _U32, _U32]),
    "mfb_router_hash_weights": (_I32, [_V, _V, _V, _U32, _U32, _U32, C.c_float, _V]),
    "mfb_gemv_int8": (_I32, [_V, _V, _V, _V, _V, _U32, _U32, _U32, _V, _U32, _U32, _V]),
    "mfb_gemv_int4": (_I32, [_V, _V, _V, _V, _U32, _V, _U32, _U32, _U32, _U32, _U32, _V]),
    "mfb_ep_create": (_I32, [_U32, _U32, _U32, _U32, C.POINTER(_V)]),
    "mfb_ep_destroy": (_I32, [_V]),
    "mfb_ep_export": (_I32, [_V, _V]),
    "mfb_ep_import": (_I32, [_V, _V]),
    "mfb_ep_dispatch": (_I32, [_V, _V, _V, _U32, _V, _U32, _U32, _U32, _V]),
    "mfb_ep_receive": (_I32, [_V, _V, C.POINTER(_V), C.POINTER(_V), C.POINTER(_V), C.POINTER(_U32)]),
    "mfb_ep_return": (_I32, [_V, _V]),
    "mfb_ep_results": (_I32, [_V, _V, C.POINTER(_V)]),
    "mfb_ep_status": (_I32, [_V, _V, C.POINTER(_U32), _V]),
    "mfb_moe_prefill_grouped_rows": (_I32, [_V, _V, C.POINTER(LayerWeightsC), _V, _U32, _U32, _V, _V, _V, _V]),
    "mfb_router_topk_static": (_I32, [_V, _V, _U32, _U32, _U32, _U32, _V, _V, _U32, _U32, _U32, _V, _V, C.c_float, _V, _V]),
    "mfb_moe_decode": (_I32, [_V, _V, C.POINTER(LayerWeightsC), _V, _U32, _U32, _V, _V, _V, _V]),
    "mfb_moe_experts": (_I32, [_V, _V, C.POINTER(LayerWeightsC), _V, _U32, _U32, _V, _V, C.POINTER(_U32), _U32, _I32]),
    "mfb_moe_combine": (_I32, [_V, _V, _U32, _V, _I32, _V, _V]),
    "mfb_moe_layer": (_I32, [_V, _V, C.POINTER(LayerWeightsC), _V, _V, _U32]),
    "mfb_moe_stack": (_I32, [_V, _V, C.POINTER(LayerWeightsC), _U32, _V, _U32]),
    "mfb_moe_stack_rows": (_I32, [_V, _V, C.POINTER(LayerWeightsC), _U32, _V, _U64, _U32]),
    "mfb_moe_group": (_I32, [_V, _V, _V, _V, _U32, _V, _V, _V, _V, _V]),
    "mfb_moe_group_host": (_I32, [_V, _I64, _I64, _I64, _I64, _I64, _V, _I64, _V, _V, _V, _V, C.POINTER(_U32), _V,
                                  C.POINTER(_U32), C.POINTER(_U32), C.POINTER(_U32)]),
    "mfb_moe_prefill_grouped": (_I32, [_V, _V, C.POINTER(LayerWeightsC), _V, _U32, _U32, _V, _V, _V, _V]),
    "mfb_moe_reduce": (_I32, [_V, _V, _V, _V, _U32, _V, _V]),
    "mfb_moe_layer_prefill": (_I32, [_V, _V, C.POINTER(LayerWeightsC), _V, _V, _U32]),
    "mfb_rmsnorm": (_I32, [_V, _V, _V, _V, _U32, _V]),
    "mfb_residual_add": (_I32, [_V, _V, _V, _V, _U64, _V]),
    "mfb_synth_expert_pool": (_I32, [_V, _U64, _U32, _U32, _U32, _I32, _U32, _U32, _U32, _U32, _V, _U64]),
    "mfb_synth_normal": (_I32, [_V, _U64, C.c_char_p, _U64, C.c_double, C.c_double, _I32, _U32, _V]),
}

_lib = None


def load():
    """Load the shared library, binding every declared symbol.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m mference_b200.build` (there is no fallback path)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)   # AttributeError if the library does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc: int):
    if rc != OK:
        raise MfbError(rc, load().mfb_last_error().decode(errors="replace"))
