"""ctypes binding of ``libmoe_b200.so`` (the C ABI declared in ``include/moe_b200.h``).

There is no fallback: if the shared library is missing or a call fails, an
exception is raised.  Nothing here imports PyTorch or the CPU oracle.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmoe_b200.so")
HEADER_PATH = os.path.join(_HERE, "..", "include", "moe_b200.h")

MOE_OK = 0
ERR_INVALID, ERR_CUDA, ERR_STATE, ERR_INTERRUPTED, ERR_DEVICE_WAIT, ERR_UNSUPPORTED, ERR_IO = -1, -2, -3, -4, -5, -6, -7
SCHEME_BQ4, SCHEME_INT4 = 0, 1
DT_F32, DT_BF16, DT_INT4, DT_INT8 = 0, 1, 2, 3
H_EMBED, H_FINAL_NORM, H_LM_HEAD = 0, 1, 2
(M_PRE_FC_NORM_HIDDEN, M_PRE_FC_NORM_EMBEDDING, M_FC, M_INPUT_NORM, M_Q_PROJ, M_K_PROJ, M_V_PROJ, M_Q_NORM, M_K_NORM,
 M_O_PROJ, M_OUT_NORM) = range(11)
T_POST_NORM, T_ROUTER, T_SHARED_GATE, T_SHARED_UP, T_SHARED_DOWN, T_SHARED_SGATE = range(6)
EP_HANDLE_BYTES = 64


class MoeDims(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("hidden", "inter", "shared_inter", "num_experts", "top_k",
                                         "num_layers", "num_mtp_layers", "group", "vocab", "scheme")]


class ExpertLayout(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("gate_w", "gate_s", "gate_b", "up_w", "up_s", "up_b",
                                         "down_w", "down_s", "down_b", "expert_size")]


class AttnDims(C.Structure):
    _fields_ = [("num_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("rotary_dim", C.c_int32),
                ("max_seq", C.c_int32), ("rope_theta", C.c_float)]


class ModelAttnDims(C.Structure):
    _fields_ = [("full", AttnDims), ("lin_num_k_heads", C.c_int32), ("lin_num_v_heads", C.c_int32), ("lin_key_dim", C.c_int32),
                ("lin_value_dim", C.c_int32), ("conv_kernel", C.c_int32), ("full_attn_interval", C.c_int32)]


(A_INPUT_NORM, A_Q_PROJ, A_K_PROJ, A_V_PROJ, A_Q_NORM, A_K_NORM, A_O_PROJ, A_IN_PROJ_QKV, A_IN_PROJ_Z, A_IN_PROJ_B, A_IN_PROJ_A,
 A_CONV1D, A_A_LOG, A_DT_BIAS, A_LIN_NORM, A_OUT_PROJ) = range(16)
ST_K_CACHE, ST_V_CACHE, ST_CONV, ST_SSM = range(4)  # moe_state_tensor_t


class LayerPtrs(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("experts", "post_norm", "router_bf16", "router_w", "router_s", "router_b",
                                          "shared", "sgate_w", "sgate_s", "sgate_b")]


CHECK_FN = C.CFUNCTYPE(C.c_int, C.c_void_p)

_vp, _i, _i32, _i64, _sz = C.c_void_p, C.c_int, C.c_int32, C.c_int64, C.c_size_t
_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); must list every function the headers under include/ declare
SIGNATURES = {
    "moe_last_error": (C.c_char_p, []),
    "moe_version": (C.c_char_p, []),
    "moe_expert_layout": (_i, [_i32, _i32, _i32, C.POINTER(ExpertLayout)]),
    "moe_engine_create": (_i, [C.POINTER(MoeDims), _i, _pp]),
    "moe_engine_destroy": (None, [_vp]),
    "moe_engine_sync": (_i, [_vp]),
    "moe_engine_dims": (_i, [_vp, C.POINTER(MoeDims)]),
    "moe_store_load_layer": (_i, [_vp, _i, _vp, _sz]),
    "moe_store_layer_dev": (_i, [_vp, _i, _pp]),
    "moe_store_mark_loaded": (_i, [_vp, _i]),
    "moe_store_load_tensor": (_i, [_vp, _i, _i, _vp, _vp, _vp, _i]),
    "moe_store_bytes": (_i, [_vp, C.POINTER(_sz)]),
    "moe_pack_int4_dev": (_i, [_vp, _vp, _i, _i64, _i32, _vp, _vp, _vp]),
    "moe_pack_int4_host": (_i, [_vp, _vp, _i, _i64, _i32, _vp, _vp, _vp]),
    "moe_pack_int8_host": (_i, [_vp, _vp, _i, _i64, _i32, _vp, _vp]),
    "moe_pack_experts_dev": (_i, [_vp, _vp, _vp, _i, _i32, _vp]),
    "moe_pack_experts_host": (_i, [_vp, _vp, _vp, _i, _i32, _vp]),
    "moe_matvec_int4_dev": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32]),
    "moe_matvec_int4_host": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32]),
    "moe_layer_forward_host": (_i, [_vp, _i, _vp, _i32, _vp, _vp, _vp, _vp, _vp]),
    "moe_layer_forward_dev": (_i, [_vp, _i, _vp, _i32, _vp, _vp, _vp, _vp, _vp]),
    "moe_forward_hidden_host": (_i, [_vp, _vp, _i32, _i, _i, CHECK_FN, _vp, _vp]),
    "moe_forward_hidden_dev": (_i, [_vp, _vp, _i32, _i, _vp]),
    "moe_last_h_pre_norm": (_i, [_vp, _vp]),
    "moe_head_load_tensor": (_i, [_vp, _i, _vp, _vp, _vp, _i]),
    "moe_embed_lookup_host": (_i, [_vp, _vp, _i32, _vp]),
    "moe_embed_lookup_dev": (_i, [_vp, _vp, _i32, _vp]),
    "moe_logits_host": (_i, [_vp, _vp, _i32, _vp]),
    "moe_logits_dev": (_i, [_vp, _vp, _i32, _vp]),
    "moe_forward_host": (_i, [_vp, _vp, _i32, _i, _i, CHECK_FN, _vp, _vp]),
    "moe_mtp_forward_host": (_i, [_vp, _vp, _vp]),
    "moe_mtp_configure": (_i, [_vp, C.POINTER(AttnDims)]),
    "moe_mtp_load_tensor": (_i, [_vp, _i, _vp, _vp, _vp, _i]),
    "moe_mtp_step_host": (_i, [_vp, _vp, _i64, _vp]),
    "moe_attn_configure": (_i, [_vp, C.POINTER(ModelAttnDims)]),
    "moe_attn_load_tensor": (_i, [_vp, _i, _i, _vp, _vp, _vp, _i]),
    "moe_model_forward_hidden_host": (_i, [_vp, _vp, _i32, _vp]),
    "moe_model_forward_host": (_i, [_vp, _vp, _i32, _vp]),
    "moe_model_reset": (_i, [_vp]),
    "moe_model_pos": (_i, [_vp, C.POINTER(_i64)]),
    "moe_model_snapshot": (_i, [_vp, _pp]),
    "moe_model_restore": (_i, [_vp, _vp]),
    "moe_model_snapshot_free": (None, [_vp]),
    "moe_model_state_host": (_i, [_vp, _i32, _i32, _vp, _i64, _i32]),
    "moe_model_set_pos": (_i, [_vp, _i64]),
    "moe_mtp_reset": (_i, [_vp]),
    "moe_mtp_rollback": (_i, [_vp, _i64]),
    "moe_mtp_pos": (_i, [_vp, C.POINTER(_i64)]),
    "moe_set_record_telemetry": (None, [_i]),
    "moe_get_record_telemetry": (_i, []),
    "moe_telemetry_get": (_i, [_vp, C.POINTER(C.c_char_p), C.POINTER(C.c_double), C.POINTER(_i)]),
    "moe_decode_profile": (_i, [_vp, _i, C.POINTER(_i64), _i, C.POINTER(_i)]),
    "moe_ep_export": (_i, [_vp, _i, _i, _i32, _vp]),
    "moe_ep_init": (_i, [_vp, _vp]),
    "moe_ep_finalize": (_i, [_vp]),
    "moe_ep_layer_forward_dev": (_i, [_vp, _i, _vp, _i32, _vp]),
    "moe_ep_forward_hidden_dev": (_i, [_vp, _vp, _i32, _vp]),
    "moe_layer_decode_noalloc": (_i, [C.POINTER(MoeDims), _i, C.POINTER(LayerPtrs), _vp, _vp, _vp, _vp, _vp, _i]),
    "moe_layer_decode_noalloc_status": (_i, [_i, _vp, C.POINTER(C.c_uint)]),
    "moe_synth_normal_dev": (_i, [_vp, _vp, _i, _i64, C.c_uint64, C.c_float, C.c_float, C.c_float]),
    "moe_dev_alloc": (_i, [_vp, _sz, _pp]),
    "moe_dev_free": (_i, [_vp, _vp]),
    "moe_dev_upload": (_i, [_vp, _vp, _vp, _sz]),
    "moe_dev_download": (_i, [_vp, _vp, _vp, _sz]),
    "moe_dev_memset": (_i, [_vp, _vp, _i, _sz]),
    "moe_host_alloc_pinned": (_i, [_sz, _pp]),
    "moe_host_free_pinned": (_i, [_vp]),
    "moe_timer_start": (_i, [_vp]),
    "moe_timer_stop": (_i, [_vp, C.POINTER(C.c_float)]),
    "moe_launch_count": (_i, [_vp, C.POINTER(_i64)]),
}

_lib = None


class MoeError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def load():
    """Loads the shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m moe_infer_b200.build` "
                "(needs nvcc with sm_100a support). There is no CPU fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().moe_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Maps a status code to the exception class the reference binding raises."""
    if status == MOE_OK:
        return
    msg = last_error()
    if status == ERR_INVALID:
        raise ValueError(msg)
    if status == ERR_IO:
        raise IOError(msg)
    raise MoeError(status, msg)


def ptr(a: Optional[np.ndarray]):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "arrays crossing the C ABI must be C-contiguous"
    return a.ctypes.data_as(C.c_void_p)


def expert_layout(hidden: int, inter: int, group: int = 64) -> dict:
    L = ExpertLayout()
    check(load().moe_expert_layout(hidden, inter, group, C.byref(L)))
    return {n: getattr(L, n) for n, _ in ExpertLayout._fields_}
