"""ctypes binding of libturbopi_b200.so (the C ABI declared in include/turbopi_b200.h).

There is no fallback: if the library is missing or a call returns a non-zero
status, an exception is raised.
"""
import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libturbopi_b200.so"

F32, F16, BF16 = 0, 1, 2
ACT_NONE, ACT_GELU, ACT_SILU, ACT_GEGLU = 0, 1, 2, 3
SCALE_F32, SCALE_E4M3, SCALE_F16, SCALE_BF16 = 0, 1, 2, 3
INT4_KBLOCK, INT4_ROWMAJOR, INT4_PLUGIN = 0, 1, 2
FLAG_NONE, FLAG_PDL = 0, 1
MAX_GROUP = 64

ACTIVATIONS = {"none": ACT_NONE, "gelu": ACT_GELU, "silu": ACT_SILU}


class TurboPiError(RuntimeError):
    pass


class GemvProblem(ctypes.Structure):
    _fields_ = [("x", c_void_p), ("weight_packed", c_void_p), ("weight_scales", c_void_p), ("bias", c_void_p),
                ("out", c_void_p), ("N", c_int), ("K", c_int), ("global_scale", c_float), ("out_stride", c_int)]


class GemmArgs(ctypes.Structure):
    _fields_ = [("a_packed", c_void_p), ("a_pitch", c_int), ("a_sf", c_void_p),
                ("a_pieces", c_int), ("a_piece_rows", c_int), ("a_row_scale", c_void_p),
                ("b_packed", c_void_p), ("b_pitch", c_int), ("b_sf", c_void_p),
                ("alpha", c_float), ("bias", c_void_p), ("activation", c_int),
                ("out", c_void_p), ("out_dtype", c_int), ("ldo", c_int),
                ("M", c_int), ("N", c_int), ("K", c_int),
                ("qkv_q_out", c_void_p), ("qkv_ldq", c_int), ("qkv_q_dim", c_int),
                ("qkv_k_rows", c_void_p), ("qkv_v_rows", c_void_p),
                ("qkv_positions", c_void_p), ("qkv_rope_cos", c_void_p), ("qkv_rope_sin", c_void_p),
                ("workspace", c_void_p), ("workspace_bytes", c_size_t), ("layout", c_int), ("flags", c_int)]


class GemvTcProblem(ctypes.Structure):
    _fields_ = [("w_image", c_void_p), ("x_image", c_void_p),
                ("x_row_scale", c_void_p), ("bias", c_void_p), ("out", c_void_p),
                ("N", c_int), ("K", c_int), ("ldo", c_int), ("global_scale", c_float)]


class GemvTcFusedProblem(ctypes.Structure):
    _fields_ = [("w_image", c_void_p), ("x", c_void_p), ("ldx", c_int), ("bias", c_void_p), ("out", c_void_p),
                ("N", c_int), ("K", c_int), ("ldo", c_int), ("global_scale", c_float)]


class GemvTcPlanInfo(ctypes.Structure):
    _fields_ = [("grid", c_int), ("units", c_int), ("max_load_stages", c_int), ("total_stages", c_int),
                ("cut_tiles", c_int), ("pool_units", c_int), ("workspace_bytes", c_size_t)]


class AttentionArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("out", c_void_p), ("key_bias", c_void_p),
                ("n_rows", c_int), ("n_keys", c_int), ("head_dim", c_int),
                ("ldq", c_int), ("ldk", c_int), ("ldv", c_int), ("ldo", c_int),
                ("groups_outer", c_int), ("groups_inner", c_int),
                ("q_stride", ctypes.c_longlong * 2), ("k_stride", ctypes.c_longlong * 2),
                ("v_stride", ctypes.c_longlong * 2), ("o_stride", ctypes.c_longlong * 2),
                ("scale", c_float), ("workspace", c_void_p), ("workspace_bytes", c_size_t), ("flags", c_int),
                ("quant_image", c_void_p), ("quant_row_scale", c_void_p), ("quant_pieces", c_int),
                ("quant_rows_per_token", c_int),
                ("quant_sf", c_void_p), ("quant_pitch", c_int), ("quant_piece_rows", c_int)]


class ActTc(ctypes.Structure):
    _fields_ = [("x", c_void_p), ("ldx", c_int), ("K", c_int), ("x_image", c_void_p), ("x_row_scale", c_void_p)]


class RowOpArgs(ctypes.Structure):
    _fields_ = [("mode", c_int), ("M", c_int), ("K", c_int), ("x", c_void_p), ("ldx", c_int),
                ("res_in", c_void_p), ("gate", c_void_p), ("h_out", c_void_p),
                ("w0", c_void_p), ("w1", c_void_p), ("eps", c_float), ("y_out", c_void_p),
                ("packed", c_void_p), ("pitch", c_int), ("sf", c_void_p), ("row_scale", c_void_p),
                ("pieces", c_int), ("piece_rows", c_int), ("layout", c_int), ("flags", c_int)]


ROW_NONE, ROW_RMSNORM, ROW_ADARMS, ROW_LAYERNORM, ROW_GELU_MUL, ROW_SILU_MUL = 0, 1, 2, 3, 4, 5

# name -> (restype, argtypes); every symbol include/turbopi_b200.h declares
SIGNATURES = {
    "tpb200_version": (c_int, []),
    "tpb200_status_string": (c_char_p, [c_int]),
    "tpb200_last_error": (c_int, []),
    "tpb200_device_error": (c_int, [c_int]),
    "tpb200_w4a16_gemv": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                                  c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "tpb200_nvfp4_gemv": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p,
                                  c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "tpb200_nvfp4_gemv_grouped": (c_int, [ctypes.POINTER(GemvProblem), c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_int, c_int, c_int, c_void_p]),
    "tpb200_nvfp4_sf_bytes": (c_size_t, [c_int, c_int]),
    "tpb200_nvfp4_gemm_workspace_size": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "tpb200_nvfp4_tiled_a_bytes": (c_size_t, [c_int, c_int, c_int]),
    "tpb200_nvfp4_tiled_b_bytes": (c_size_t, [c_int, c_int]),
    "tpb200_measure_fp4_mma_rate": (c_int, [c_int, c_void_p]),
    "tpb200_nvfp4_tile_weights": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "tpb200_nvfp4_quantize_act": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p]),
    "tpb200_nvfp4_gemm": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_float, c_void_p, c_int,
                                  c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "tpb200_nvfp4_gemm_ex": (c_int, [ctypes.POINTER(GemmArgs), c_void_p]),
    "tpb200_nvfp4_quantize_act_pieces": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                                 c_int, c_int, c_int, c_void_p]),
    "tpb200_nvfp4_gemv_tc_workspace_size": (c_size_t, [ctypes.POINTER(GemvTcProblem), c_int]),
    "tpb200_nvfp4_gemv_tc_x_image_bytes": (c_size_t, [c_int, c_int]),
    "tpb200_nvfp4_quantize_act_tc": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                             c_void_p]),
    "tpb200_nvfp4_quantize_acts_tc": (c_int, [ctypes.POINTER(ActTc), c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "tpb200_nvfp4_gemv_tc": (c_int, [ctypes.POINTER(GemvTcProblem), c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                     c_size_t, c_int, c_void_p]),
    "tpb200_nvfp4_gemv_tc_fused_workspace_size": (c_size_t, [ctypes.POINTER(GemvTcFusedProblem), c_int]),
    "tpb200_nvfp4_gemv_tc_fused": (c_int, [ctypes.POINTER(GemvTcFusedProblem), c_int, c_int, c_int, c_int, c_int, c_int,
                                           c_int, c_void_p, c_size_t, c_int, c_void_p]),
    "tpb200_nvfp4_gemv_tc_plan": (c_int, [ctypes.POINTER(c_int), ctypes.POINTER(c_int), c_int, c_int,
                                          ctypes.POINTER(GemvTcPlanInfo)]),
    "tpb200_attention_workspace_size": (c_size_t, [c_int, c_int, c_int, c_int]),
    "tpb200_attention": (c_int, [ctypes.POINTER(AttentionArgs), c_void_p]),
    "tpb200_w4a16_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                  c_int, c_int, c_int, c_float, c_float, c_int, c_void_p]),
    "tpb200_row_transform_quantize": (c_int, [ctypes.POINTER(RowOpArgs), c_void_p]),
    "tpb200_nvfp4_gemv_tc_static_capacity": (c_size_t, []),
    "tpb200_nvfp4_gemv_tc_static": (c_int, [ctypes.POINTER(GemvTcProblem), c_int, c_int, c_int, c_int, c_int, c_int,
                                            c_int, c_void_p]),
    "nvfp4_gemv_forward": (None, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                  c_int, c_int, c_void_p]),
    "nvfp4_gemv_workspace_size": (c_size_t, [c_int, c_int, c_int]),
    "w4a16GemmForward": (None, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float,
                                c_void_p, c_size_t, c_void_p]),
    "getW4A16GemmWorkspaceSize": (c_size_t, [c_int, c_int, c_int]),
    "w4a8GemmForward": (None, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p,
                               c_size_t, c_void_p]),
    "getW4A8GemmWorkspaceSize": (c_size_t, [c_int, c_int, c_int]),
    "quantizeWeightToINT4": (None, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "dequantizeINT4ToBF16": (None, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "quantizeActivationToFP8": (None, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "quantizeWeightToNVFP4": (None, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
}

_lib = None


def load():
    """Load the shared library once and attach signatures."""
    global _lib
    if _lib is not None:
        return _lib
    path = Path(os.environ.get("TURBOPI_B200_LIB", LIB_PATH))    # an alternative build (e.g. a diagnostic one)
    if not path.exists():
        raise TurboPiError(
            f"{path} is missing: build it with `python -m turbopi_b200.build` "
            "(there is no CPU or PyTorch fallback for these kernels)")
    lib = ctypes.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)      # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status, what):
    if status != 0:
        msg = load().tpb200_status_string(status).decode()
        raise TurboPiError(f"{what}: {msg} (status {status})")


def check_void(what):
    """After a void-returning (reference-signature) entry point."""
    check(load().tpb200_last_error(), what)
