"""Loader of libpcb200.so (include/pcb200.h).  There is no CPU fallback: if the library is
missing or a call fails, an exception is raised."""
from __future__ import annotations

import ctypes as C
import os

from .circuit import PcbCircuitDesc

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpcb200.so")
_lib = None


class PcbError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"pcb200 error {code}: {msg}")
        self.code = code


class PcbCircuitInfo(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "num_nodes", "num_edges", "num_sum_edges", "num_up_layers", "num_inner_params", "num_input_params",
        "num_param_groups", "num_dense_blocks", "num_sum_regions", "max_group_size", "max_num_cats")] + [
        ("num_dense_edges", C.c_uint64), ("device_bytes", C.c_uint64), ("num_heads", C.c_uint32), ("reserved", C.c_uint32)]


class PcbEvidence(C.Structure):
    """ctypes mirror of `pcb_evidence` (include/pcb200.h)."""
    _fields_ = [("data_dev", C.c_void_p), ("miss_dev", C.c_void_p), ("soft_dev", C.c_void_p), ("head_mask_dev", C.c_void_p),
                ("num_rows", C.c_uint64), ("row_ids_dev", C.c_void_p), ("row_start", C.c_uint32), ("B", C.c_uint32),
                ("soft_reg", C.c_float), ("soft_reg_width", C.c_uint32)]


_u32, _u64, _i32, _f32, _vp = C.c_uint32, C.c_uint64, C.c_int32, C.c_float, C.c_void_p

SIGNATURES = {
    "pcb_version": [],
    "pcb_circuit_create": [C.POINTER(PcbCircuitDesc), _i32, C.POINTER(_vp)],
    "pcb_circuit_destroy": [_vp],
    "pcb_circuit_get_info": [_vp, C.POINTER(PcbCircuitInfo)],
    "pcb_circuit_status": [_vp],
    "pcb_workspace_create": [_vp, _u32, _i32, C.POINTER(_vp)],
    "pcb_workspace_destroy": [_vp],
    "pcb_get_params": [_vp, _vp, _u64],
    "pcb_set_params": [_vp, _vp, _u64],
    "pcb_get_params_dev": [_vp, _vp, _u64, _vp],
    "pcb_set_params_dev": [_vp, _vp, _u64, _vp],
    "pcb_get_heap": [_vp, _vp, _u64],
    "pcb_get_edge_aggr": [_vp, _vp, _u64],
    "pcb_get_edge2param": [_vp, _vp, _u64],
    "pcb_get_sum_regions": [_vp, _vp, _u64],
    "pcb_forward": [_vp, _vp, _vp, _vp, _u64, _vp, _u32, _u32, _vp, _vp],
    "pcb_backward": [_vp, _vp, _vp, _vp],
    "pcb_clear_flows": [_vp, _f32, _vp],
    "pcb_em_update": [_vp, _f32, _f32, _vp],
    "pcb_em_step": [_vp, _vp, _vp, _vp, _u64, _vp, _u32, _u32, _vp, _f32, _f32, _f32, _vp, _vp],
    "pcb_forward_ex": [_vp, _vp, C.POINTER(PcbEvidence), _vp, _vp],
    "pcb_em_step_ex": [_vp, _vp, C.POINTER(PcbEvidence), _vp, _f32, _f32, _f32, _vp, _vp],
    "pcb_get_head_roots": [_vp, _vp, _u64],
    "pcb_normalize_params": [_vp, _vp, _u32, _i32, _vp],
    "pcb_map_param_columns": [_vp, _vp, _u32, _vp, _vp, _u32, _vp],
    "pcb_normalized_flows": [_vp, _vp, C.POINTER(PcbEvidence), _vp, _vp, _vp],
    "pcb_get_mars": [_vp, _vp, _vp, _u64],
    "pcb_get_flows": [_vp, _vp, _vp, _u64],
    "pcb_kld": [_vp, _vp, _vp, _vp, _u32, _vp, _vp],
    "pcb_kld_backward": [_vp, _vp, _vp, _vp, _u32, _vp, _vp, _vp],
    "pcb_get_klds": [_vp, _vp, _u32, _vp],
    "pcb_kld_edge_klds": [_vp, _vp, _vp, _vp, _u32, _vp, _vp],
    "pcb_adam_step": [_vp, _vp, _vp, _vp, _vp, _i32, _f32, _f32, _f32, _f32, _f32, _vp],
    "pcb_kld_adam_step": [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _f32, _f32, _f32, _f32, _vp, _vp],
    "pcb_sample_hard": [_vp, _vp, _vp, _u32, _vp, _vp, _u32, _vp, _vp],
    "pcb_sample_hard_static": [_vp, _vp, _u32, _vp, _vp, _u32, _vp, _vp],
    "pcb_sample_soft": [_vp, _vp, _vp, _u32, _vp, _f32, _u32, _vp, _vp],
    "pcb_cond_td_prob": [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _vp, _vp],
    "pcb_pairwise_mi": [_vp, _u64, _u32, _u32, _f32, _vp, _vp],
    "pcb_comm_unique_id": [_vp],
    "pcb_comm_init": [_vp, _vp, _i32, _i32],
    "pcb_comm_destroy": [_vp],
    "pcb_comm_set_enabled": [_vp, _i32],
    "pcb_selftest_wait_limit": [_i32, _u32, C.POINTER(_i32), C.POINTER(_i32), C.POINTER(_f32), C.POINTER(_u32)],
    "pcb_comm_poll": [_vp],
    "pcb_comm_wait": [_vp, _vp, _u32],
    "pcb_comm_abort": [_vp],
    "pcb_profile_num_classes": [],
    "pcb_profile_enable": [_vp, _i32],
    "pcb_profile_read": [_vp, _vp, _vp, _i32],
}


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise PcbError(-1, f"{LIB_PATH} is missing: build it with `python -m lvd_pg_b200.build` "
                               "(there is no CPU fallback)")
        _lib = C.CDLL(os.environ.get("PCB200_LIBRARY", LIB_PATH))   # override: a differently tuned build of the same sources
        _lib.pcb_last_error.restype = C.c_char_p
        for name, args in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.argtypes = args
            fn.restype = _i32
        _lib.pcb_profile_class_name.argtypes = [_i32]
        _lib.pcb_profile_class_name.restype = C.c_char_p
    return _lib


def check(code: int) -> None:
    if code != 0:
        raise PcbError(code, lib().pcb_last_error().decode("utf-8", "replace"))
