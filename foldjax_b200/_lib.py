"""ctypes binding of libb200tri.so (the C ABI declared in include/b200tri.h).

The structures below mirror the header field for field. Loading fails loudly:
there is no fallback implementation behind these calls.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

_HERE = Path(__file__).resolve().parent
# B200TRI_LIBRARY points at another build of the same library (kernel experiments).
LIB_PATH = Path(os.environ.get("B200TRI_LIBRARY", _HERE / "libb200tri.so"))

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_WORKSPACE = range(6)
DTYPE_BF16, DTYPE_F32 = 0, 1
TRIATT_CORE_STATIC_MAX_FLOATS = 1 << 20


class B200TriError(RuntimeError):
    """A libb200tri entry point returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libb200tri error {code}: {message}")
        self.code = code


class TrimulArgs(C.Structure):
    _fields_ = [
        ("n", C.c_int32), ("incoming", C.c_int32), ("eps", C.c_float),
        ("x", C.c_void_p), ("mask", C.c_void_p),
        ("norm_in_scale", C.c_void_p), ("norm_in_bias", C.c_void_p),
        ("p_in", C.c_void_p), ("g_in", C.c_void_p),
        ("norm_out_scale", C.c_void_p), ("norm_out_bias", C.c_void_p),
        ("p_out", C.c_void_p), ("g_out", C.c_void_p),
        ("residual", C.c_void_p), ("out", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("dtype", C.c_int32),
        ("c_z", C.c_int32), ("c_hidden", C.c_int32),
    ]


class TrimulProjectArgs(C.Structure):
    _fields_ = [
        ("n_outer", C.c_int32), ("n_inner", C.c_int32), ("eps", C.c_float),
        ("x", C.c_void_p), ("xs_outer", C.c_int64), ("xs_inner", C.c_int64),
        ("mask", C.c_void_p), ("ms_outer", C.c_int64), ("ms_inner", C.c_int64),
        ("norm_in_scale", C.c_void_p), ("norm_in_bias", C.c_void_p),
        ("p_in", C.c_void_p), ("g_in", C.c_void_p),
        ("a", C.c_void_p), ("b", C.c_void_p),
        ("ld", C.c_int64), ("chan_stride", C.c_int64), ("block_stride", C.c_int64),
        ("rows_per_block", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class TrimulContractArgs(C.Structure):
    _fields_ = [
        ("n_i", C.c_int32), ("n_j", C.c_int32), ("n_k", C.c_int32), ("n_src", C.c_int32),
        ("a", C.c_void_p), ("a_ld", C.c_int64), ("a_chan_stride", C.c_int64), ("a_src_stride", C.c_int64),
        ("b", C.c_void_p), ("b_ld", C.c_int64), ("b_chan_stride", C.c_int64), ("b_src_stride", C.c_int64),
        ("acc_in", C.c_void_p), ("out_f32", C.c_void_p), ("out_bf16", C.c_void_p),
        ("out_ld", C.c_int64), ("out_chan_stride", C.c_int64),
        ("a_rows_per_block", C.c_int32), ("b_rows_per_block", C.c_int32), ("out_rows_per_block", C.c_int32),
        ("a_block_stride", C.c_int64), ("b_block_stride", C.c_int64), ("out_block_stride", C.c_int64),
    ]


class TrimulFinishArgs(C.Structure):
    _fields_ = [
        ("n_i", C.c_int32), ("n_j", C.c_int32), ("eps", C.c_float),
        ("t", C.c_void_p), ("t_ld", C.c_int64), ("t_chan_stride", C.c_int64),
        ("x", C.c_void_p), ("xs_i", C.c_int64), ("xs_j", C.c_int64),
        ("norm_in_scale", C.c_void_p), ("norm_in_bias", C.c_void_p),
        ("norm_out_scale", C.c_void_p), ("norm_out_bias", C.c_void_p),
        ("p_out", C.c_void_p), ("g_out", C.c_void_p),
        ("residual", C.c_void_p), ("out", C.c_void_p),
        ("os_i", C.c_int64), ("os_j", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("t_rows_per_block", C.c_int32), ("t_block_stride", C.c_int64),
    ]


class TriattArgs(C.Structure):
    _fields_ = [
        ("n", C.c_int32), ("starting", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("inf", C.c_float), ("eps", C.c_float),
        ("x", C.c_void_p), ("mask", C.c_void_p),
        ("norm_scale", C.c_void_p), ("norm_bias", C.c_void_p), ("w_bias", C.c_void_p),
        ("w_q", C.c_void_p), ("w_k", C.c_void_p), ("w_v", C.c_void_p), ("w_g", C.c_void_p), ("w_o", C.c_void_p),
        ("residual", C.c_void_p), ("out", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("dtype", C.c_int32), ("c_z", C.c_int32),
    ]


class TriattProjectArgs(C.Structure):
    _fields_ = [
        ("n_outer", C.c_int32), ("n_inner", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("eps", C.c_float),
        ("x", C.c_void_p), ("xs_outer", C.c_int64), ("xs_inner", C.c_int64),
        ("norm_scale", C.c_void_p), ("norm_bias", C.c_void_p),
        ("w_q", C.c_void_p), ("w_k", C.c_void_p), ("w_v", C.c_void_p), ("w_bias", C.c_void_p),
        ("q", C.c_void_p), ("k", C.c_void_p), ("vt", C.c_void_p), ("bias", C.c_void_p),
        ("ld", C.c_int64), ("bias_head_stride", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class TriattCoreArgs(C.Structure):
    _fields_ = [
        ("n_i", C.c_int32), ("n_j", C.c_int32), ("n_k", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("vt", C.c_void_p), ("v_ld", C.c_int64),
        ("bias", C.c_void_p), ("bias_ld", C.c_int64), ("bias_head_stride", C.c_int64),
        ("mask", C.c_void_p), ("ms_i", C.c_int64), ("ms_k", C.c_int64), ("inf", C.c_float),
        ("o", C.c_void_p), ("row_max", C.c_void_p), ("row_sum", C.c_void_p), ("unnormalized", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("acc_o", C.c_void_p), ("resume", C.c_int32), ("mask_additive", C.c_int32),
    ]


class TriattFinishArgs(C.Structure):
    _fields_ = [
        ("n_outer", C.c_int32), ("n_inner", C.c_int32), ("eps", C.c_float),
        ("o", C.c_void_p), ("x", C.c_void_p), ("xs_outer", C.c_int64), ("xs_inner", C.c_int64),
        ("norm_scale", C.c_void_p), ("norm_bias", C.c_void_p), ("w_g", C.c_void_p), ("w_o", C.c_void_p),
        ("residual", C.c_void_p), ("out", C.c_void_p), ("os_outer", C.c_int64), ("os_inner", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class PairTransitionArgs(C.Structure):
    _fields_ = [
        ("rows", C.c_int64), ("channels", C.c_int32), ("hidden", C.c_int32), ("eps", C.c_float),
        ("x", C.c_void_p), ("norm_scale", C.c_void_p), ("norm_bias", C.c_void_p),
        ("fc1", C.c_void_p), ("fc2", C.c_void_p), ("fc3", C.c_void_p),
        ("residual", C.c_void_p), ("out", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("row_mask", C.c_void_p),
    ]


class AttentionPairBiasArgs(C.Structure):
    _fields_ = [
        ("n", C.c_int32), ("c_s", C.c_int32), ("c_z", C.c_int32), ("heads", C.c_int32),
        ("eps", C.c_float), ("inf", C.c_float),
        ("s", C.c_void_p), ("k_in", C.c_void_p), ("z", C.c_void_p), ("mask", C.c_void_p),
        ("proj_q", C.c_void_p), ("proj_q_bias", C.c_void_p), ("proj_k", C.c_void_p), ("proj_v", C.c_void_p),
        ("proj_g", C.c_void_p), ("proj_z_norm_scale", C.c_void_p), ("proj_z_norm_bias", C.c_void_p),
        ("proj_z", C.c_void_p), ("proj_o", C.c_void_p),
        ("out", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class CpEvent(C.Structure):
    _fields_ = [(k, C.c_int32) for k in ("kind", "group", "round", "src", "dst", "what", "block", "slot0", "slot1",
                                          "n_i", "n_j", "reserved")] + [
        ("src_off", C.c_int64), ("dst_off", C.c_int64), ("bytes", C.c_int64), ("off", C.c_int64 * 4)]


class CpMsg(C.Structure):
    _fields_ = [("src", C.c_int32), ("dst", C.c_int32), ("what", C.c_int32), ("block", C.c_int32),
                ("slot0", C.c_int32), ("slot1", C.c_int32)]


class TrimulCpArgs(C.Structure):
    _fields_ = [
        ("n", C.c_int32), ("incoming", C.c_int32), ("eps", C.c_float),
        ("x", C.c_void_p), ("mask", C.c_void_p),
        ("norm_in_scale", C.c_void_p), ("norm_in_bias", C.c_void_p),
        ("p_in", C.c_void_p), ("g_in", C.c_void_p),
        ("norm_out_scale", C.c_void_p), ("norm_out_bias", C.c_void_p),
        ("p_out", C.c_void_p), ("g_out", C.c_void_p),
        ("residual", C.c_void_p), ("out", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class TriattCpArgs(C.Structure):
    _fields_ = [
        ("n", C.c_int32), ("starting", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("inf", C.c_float), ("eps", C.c_float),
        ("x", C.c_void_p), ("mask", C.c_void_p),
        ("norm_scale", C.c_void_p), ("norm_bias", C.c_void_p), ("w_bias", C.c_void_p),
        ("w_q", C.c_void_p), ("w_k", C.c_void_p), ("w_v", C.c_void_p), ("w_g", C.c_void_p), ("w_o", C.c_void_p),
        ("residual", C.c_void_p), ("out", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class TrimulParams(C.Structure):
    _fields_ = [(k, C.c_void_p) for k in ("norm_in_scale", "norm_in_bias", "p_in", "g_in", "norm_out_scale",
                                          "norm_out_bias", "p_out", "g_out")]


class TriattParams(C.Structure):
    _fields_ = [(k, C.c_void_p) for k in ("norm_scale", "norm_bias", "w_bias", "w_q", "w_k", "w_v", "w_g", "w_o")]


class TransitionParams(C.Structure):
    _fields_ = [(k, C.c_void_p) for k in ("norm_scale", "norm_bias", "fc1", "fc2", "fc3")] + [("hidden", C.c_int32)]


class AttentionParams(C.Structure):
    _fields_ = [(k, C.c_void_p) for k in ("proj_q", "proj_q_bias", "proj_k", "proj_v", "proj_g", "proj_z_norm_scale",
                                          "proj_z_norm_bias", "proj_z", "proj_o")]


class PairformerBlockParams(C.Structure):
    _fields_ = [
        ("tri_mul_out", TrimulParams), ("tri_mul_in", TrimulParams),
        ("tri_att_start", TriattParams), ("tri_att_end", TriattParams),
        ("transition_z", TransitionParams),
        ("pre_norm_s_scale", C.c_void_p), ("pre_norm_s_bias", C.c_void_p),
        ("attention", AttentionParams), ("transition_s", TransitionParams),
    ]


class PairformerArgs(C.Structure):
    _fields_ = [
        ("n", C.c_int32), ("c_s", C.c_int32), ("heads_s", C.c_int32), ("n_blocks", C.c_int32), ("stacked", C.c_int32),
        ("eps", C.c_float), ("tri_inf", C.c_float), ("att_inf", C.c_float),
        ("params", C.POINTER(PairformerBlockParams)),
        ("z_in", C.c_void_p), ("z_out", C.c_void_p), ("s_in", C.c_void_p), ("s_out", C.c_void_p),
        ("pair_mask", C.c_void_p), ("mask", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("pair_gate", C.c_int32), ("mask_transition", C.c_int32), ("attention_first", C.c_int32),
    ]


COMM_ID_BYTES = 128
CP_TRIMUL_OUTGOING, CP_TRIMUL_INCOMING, CP_TRIATT_STARTING, CP_TRIATT_ENDING = range(4)

# C struct name -> ctypes mirror (tests compare sizeof on both sides)
STRUCTS = {
    "b200tri_trimul_args": TrimulArgs,
    "b200tri_trimul_project_args": TrimulProjectArgs,
    "b200tri_trimul_contract_args": TrimulContractArgs,
    "b200tri_trimul_finish_args": TrimulFinishArgs,
    "b200tri_triatt_args": TriattArgs,
    "b200tri_triatt_project_args": TriattProjectArgs,
    "b200tri_triatt_core_args": TriattCoreArgs,
    "b200tri_triatt_finish_args": TriattFinishArgs,
    "b200tri_pair_transition_args": PairTransitionArgs,
    "b200tri_attention_pair_bias_args": AttentionPairBiasArgs,
    "b200tri_cp_msg": CpMsg,
    "b200tri_cp_event": CpEvent,
    "b200tri_trimul_cp_args": TrimulCpArgs,
    "b200tri_triatt_cp_args": TriattCpArgs,
    "b200tri_pairformer_args": PairformerArgs,
}
# parameter containers of the block-level call (checked the same way)
PARAM_STRUCTS = {
    "b200tri_trimul_params": TrimulParams,
    "b200tri_triatt_params": TriattParams,
    "b200tri_transition_params": TransitionParams,
    "b200tri_attention_params": AttentionParams,
    "b200tri_pairformer_block_params": PairformerBlockParams,
}

# name -> (restype, argtypes); every symbol include/b200tri.h declares.
SIGNATURES = {
    "b200tri_version": (C.c_int, []),
    "b200tri_last_error": (C.c_char_p, []),
    "b200tri_device_status": (C.c_int, []),
    "b200tri_selftest_wait": (C.c_int, [C.c_int64, C.c_void_p]),
    "b200tri_launch_count": (C.c_uint64, []),
    "b200tri_set_sm_limit": (C.c_int, [C.c_int32]),
    "b200tri_timing_enable": (C.c_int, [C.c_int32]),
    "b200tri_timing_reset": (C.c_int, []),
    "b200tri_timing_read": (C.c_int, [C.c_char_p, C.POINTER(C.c_double), C.POINTER(C.c_int32)]),
    "b200tri_timing_list": (C.c_int, [C.c_char_p, C.POINTER(C.c_double), C.c_int32, C.POINTER(C.c_int32)]),
    "b200tri_trimul_workspace_bytes": (C.c_size_t, [C.c_int32]),
    "b200tri_trimul_workspace_bytes_dtype": (C.c_size_t, [C.c_int32, C.c_int32]),
    "b200tri_trimul_workspace_bytes_shape": (C.c_size_t, [C.c_int32] * 4),
    "b200tri_triatt_workspace_bytes_shape": (C.c_size_t, [C.c_int32] * 5),
    "b200tri_triatt_workspace_bytes_dtype": (C.c_size_t, [C.c_int32, C.c_int32]),
    "b200tri_trimul_forward": (C.c_int, [C.POINTER(TrimulArgs), C.c_void_p]),
    "b200tri_trimul_project_workspace_bytes": (C.c_size_t, []),
    "b200tri_trimul_project": (C.c_int, [C.POINTER(TrimulProjectArgs), C.c_void_p]),
    "b200tri_trimul_contract": (C.c_int, [C.POINTER(TrimulContractArgs), C.c_void_p]),
    "b200tri_trimul_finish_workspace_bytes": (C.c_size_t, []),
    "b200tri_trimul_finish": (C.c_int, [C.POINTER(TrimulFinishArgs), C.c_void_p]),
    "b200tri_triatt_workspace_bytes": (C.c_size_t, [C.c_int32]),
    "b200tri_triatt_forward": (C.c_int, [C.POINTER(TriattArgs), C.c_void_p]),
    "b200tri_triatt_project_workspace_bytes": (C.c_size_t, []),
    "b200tri_triatt_project": (C.c_int, [C.POINTER(TriattProjectArgs), C.c_void_p]),
    "b200tri_triatt_core_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32]),
    "b200tri_triatt_core": (C.c_int, [C.POINTER(TriattCoreArgs), C.c_void_p]),
    "b200tri_triatt_core_multi_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    "b200tri_triatt_core_multi": (C.c_int, [C.POINTER(TriattCoreArgs), C.c_int32, C.c_void_p]),
    "b200tri_triatt_core_static": (C.c_int, [C.POINTER(TriattCoreArgs), C.c_void_p]),
    "b200tri_triatt_finish_workspace_bytes": (C.c_size_t, []),
    "b200tri_triatt_finish": (C.c_int, [C.POINTER(TriattFinishArgs), C.c_void_p]),
    "b200tri_comm_unique_id": (C.c_int, [C.c_void_p]),
    "b200tri_comm_init": (C.c_int, [C.POINTER(C.c_void_p), C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "b200tri_comm_init_all": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(C.c_int32), C.c_int32, C.c_int32, C.c_int32]),
    "b200tri_comm_destroy": (C.c_int, [C.c_void_p]),
    "b200tri_comm_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                    C.POINTER(C.c_int32)]),
    "b200tri_comm_workspace": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "b200tri_comm_pulls": (C.c_int, [C.c_void_p]),
    "b200tri_comm_configure": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32]),
    "b200tri_comm_group_start": (C.c_int, []),
    "b200tri_comm_group_end": (C.c_int, []),
    "b200tri_comm_probe": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200tri_cp_plan": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.POINTER(CpMsg), C.c_int32]),
    "b200tri_cp_rounds": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.c_int32]),
    "b200tri_cp_dry_run": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                     C.POINTER(CpEvent), C.c_int32]),
    "b200tri_cp_layout": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int64)]),
    "b200tri_trimul_cp_workspace_bytes": (C.c_size_t, [C.c_void_p, C.c_int32]),
    "b200tri_trimul_cp": (C.c_int, [C.c_void_p, C.POINTER(TrimulCpArgs), C.c_void_p]),
    "b200tri_triatt_cp_workspace_bytes": (C.c_size_t, [C.c_void_p, C.c_int32]),
    "b200tri_triatt_cp": (C.c_int, [C.c_void_p, C.POINTER(TriattCpArgs), C.c_void_p]),
    "b200tri_pairformer_workspace_bytes": (C.c_size_t, [C.c_int32] * 5),
    "b200tri_pairformer_forward": (C.c_int, [C.POINTER(PairformerArgs), C.c_void_p]),
    "b200tri_pair_transition_workspace_bytes": (C.c_size_t, [C.c_int32]),
    "b200tri_pair_transition": (C.c_int, [C.POINTER(PairTransitionArgs), C.c_void_p]),
    "b200tri_attention_pair_bias_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    "b200tri_attention_pair_bias": (C.c_int, [C.POINTER(AttentionPairBiasArgs), C.c_void_p]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library (once) and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m foldjax_b200.build` "
            "(needs nvcc); foldjax_b200 has no fallback implementation"
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != OK:
        msg = load().b200tri_last_error()
        raise B200TriError(rc, msg.decode() if msg else "unknown error")


def device_status() -> int:
    """Synchronise and return the device status word (0 = fine); raises on timeout codes."""
    st = load().b200tri_device_status()
    if st != 0:
        msg = load().b200tri_last_error()
        raise B200TriError(ERR_TIMEOUT, msg.decode() if msg else f"device status {st}")
    return st


KERNELS = ("trimul_project", "trimul_contract", "trimul_finish", "triatt_project", "triatt_core", "triatt_finish",
           "pair_transition", "pair_bias", "cp_exchange", "cp_ready", "cp_copy")


def kernel_time_list(name: str, capacity: int = 4096) -> list[float]:
    """The recorded durations (ms) of one kernel name since the last timing reset, in launch order."""
    buf, n = (C.c_double * capacity)(), C.c_int32(0)
    check(load().b200tri_timing_list(name.encode(), buf, capacity, C.byref(n)))
    return [buf[i] for i in range(n.value)]


def kernel_times() -> dict[str, tuple[float, int]]:
    """{kernel: (total ms, launches)} since the last timing reset (synchronises)."""
    lib = load()
    out = {}
    for name in KERNELS:
        ms, n = C.c_double(0.0), C.c_int32(0)
        check(lib.b200tri_timing_read(name.encode(), C.byref(ms), C.byref(n)))
        out[name] = (ms.value, n.value)
    return out
