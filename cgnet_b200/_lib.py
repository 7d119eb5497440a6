"""ctypes binding of libcgnet_b200.so (the C ABI declared in include/cgnet_b200.h).

There is no fallback: if the library is missing or a call fails, a RuntimeError is raised.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcgnet_b200.so")
_lib = None

c_i32p = ctypes.POINTER(ctypes.c_int32)
c_i64p = ctypes.POINTER(ctypes.c_int64)
vp = ctypes.c_void_p

# name -> (restype, argtypes); must list every symbol include/cgnet_b200.h declares
SIGNATURES = {
    "cgb200_last_error": (ctypes.c_char_p, []),
    "cgb200_version": (ctypes.c_int, []),
    "cgb200_max_lmax": (ctypes.c_int, []),
    "cgb200_cg_table_build": (ctypes.c_int, [vp, ctypes.c_int64, ctypes.c_int, c_i32p, ctypes.c_int, vp]),
    "cgb200_cg_table_length": (ctypes.c_int64, [ctypes.c_int, c_i32p, ctypes.c_int]),
    "cgb200_plan_create": (ctypes.c_int, [ctypes.POINTER(vp), ctypes.c_int, c_i32p, c_i32p, c_i32p, ctypes.c_int, ctypes.c_int]),
    "cgb200_plan_destroy": (None, [vp]),
    "cgb200_plan_query": (ctypes.c_int, [vp, ctypes.c_int, c_i64p]),
    "cgb200_plan_t_ff": (ctypes.c_int, [vp, c_i32p]),
    "cgb200_plan_status": (ctypes.c_int, [vp, c_i32p]),
    "cgb200_plan_set_option": (ctypes.c_int, [vp, ctypes.c_int, ctypes.c_int]),
    "cgb200_plan_get_option": (ctypes.c_int, [vp, ctypes.c_int, c_i32p]),
    "cgb200_plan_cg_table": (vp, [vp]),
    "cgb200_cg_product_fwd": (ctypes.c_int, [vp, vp, vp, ctypes.c_int64, vp]),
    "cgb200_cg_product_bwd": (ctypes.c_int, [vp, vp, vp, vp, ctypes.c_int64, vp]),
    "cgb200_fn_wmm_fwd": (ctypes.c_int, [vp, vp, vp, vp, ctypes.c_float, ctypes.c_float, ctypes.c_int, vp, ctypes.c_int64, vp]),
    "cgb200_fn_wmm_bwd": (ctypes.c_int, [vp, vp, vp, vp, vp, ctypes.c_float, ctypes.c_int, vp, vp, ctypes.c_int64, vp]),
    "cgb200_layer_fwd": (ctypes.c_int, [vp, vp, vp, vp, ctypes.c_float, ctypes.c_float, ctypes.c_int, vp, ctypes.c_int64, vp, ctypes.c_int64, vp]),
    "cgb200_layer_bwd": (ctypes.c_int, [vp, vp, vp, vp, ctypes.c_float, ctypes.c_int, vp, vp, vp, ctypes.c_int64, vp, ctypes.c_int64, vp]),
    "cgb200_layer_workspace_bytes": (ctypes.c_int64, [vp, ctypes.c_int64]),
    "cgb200_layer_fwd_workspace_bytes": (ctypes.c_int64, [vp, ctypes.c_int64]),
    "cgb200_layer_keeps_mid": (ctypes.c_int, [vp, ctypes.c_int64]),
    "cgb200_layer_packed_weights_bytes": (ctypes.c_int64, [vp]),
    "cgb200_layer_pack_weights": (ctypes.c_int, [vp, vp, vp, ctypes.c_float, ctypes.c_int, vp, ctypes.c_int64, vp]),
    "cgb200_layer_fwd_packed": (ctypes.c_int, [vp, vp, vp, vp, ctypes.c_int64, vp, ctypes.c_int64, vp]),
    "cgb200_layer_fwd_workspace_bytes_for": (ctypes.c_int64, [vp, ctypes.c_int64, ctypes.c_int]),
    "cgb200_layer_fwd_static": (ctypes.c_int, [vp, vp, vp, vp, ctypes.c_float, ctypes.c_float, ctypes.c_int, vp, ctypes.c_int64, vp]),
    "cgb200_sh_basis_bytes": (ctypes.c_int64, [ctypes.c_int64, ctypes.c_int]),
    "cgb200_sh_workspace_bytes": (ctypes.c_int64, [ctypes.c_int64, ctypes.c_int64]),
    "cgb200_sh_basis_pack": (ctypes.c_int, [vp, ctypes.c_int64, ctypes.c_int, vp, vp]),
    "cgb200_sh_project": (ctypes.c_int, [vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, vp, ctypes.c_float, vp, vp, ctypes.c_int64, vp, vp]),
    "cgb200_raycast_workspace_bytes": (ctypes.c_int64, [ctypes.c_int64]),
    "cgb200_raycast_sphere": (ctypes.c_int, [vp, ctypes.c_int64, vp, ctypes.c_int64, vp, ctypes.c_int64, vp, vp, ctypes.c_int64, vp, vp]),
    "cgb200_launch_count": (ctypes.c_int64, [ctypes.c_int]),
    "cgb200_kernel_count": (ctypes.c_int, []),
    "cgb200_kernel_name": (ctypes.c_char_p, [ctypes.c_int]),
    "cgb200_timing_enable": (None, [ctypes.c_int]),
    "cgb200_timing_read": (ctypes.c_int, [ctypes.POINTER(ctypes.c_double), c_i64p, ctypes.c_int]),
}

Q_N_F, Q_N_FF, Q_N_O, Q_W_LEN, Q_SUM_TFF, Q_CG_LEN, Q_N_TRIPLES, Q_TILE = range(8)
FN_PRESENT, FN_UPDATE, FN_KEEP_MID = 0x1, 0x2, 0x4
PLAN_DEPTHWISE = 0x1
AUTO = -1
(OPT_TC_FWD, OPT_TC_GRAD_W, OPT_TC_GRAD_F, OPT_TC_STAGES, OPT_FWD_SLAB, OPT_GRAD_F_SPLIT, OPT_STATS_SPLIT, OPT_BWD_SERIAL,
 OPT_WAIT_POLLS, OPT_TEST_IDLE_MMA, OPT_TC_STAGED, OPT_TC_ABUF, OPT_TC_FWD_SPLIT, OPT_GRAD_MID_GEMM,
 OPT_FWD_KEEP_MID, OPT_SHORT_GROUP) = range(16)


def plan_tile_flag(tile):
    """Plan-creation flag that forces the channel-tile edge (CGB200_PLAN_TILE in the header)."""
    return (int(tile) & 0xF) << 8


def load():
    """Load the shared library once and attach the signatures."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m cgnet_b200.build` (needs nvcc). "
                "cgnet_b200 has no CPU or PyTorch fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status, what):
    if status != 0:
        msg = load().cgb200_last_error()
        raise RuntimeError(f"{what} failed with status {status}: {msg.decode() if msg else '?'}")


def i32(seq):
    """A ctypes int32 array from any integer sequence (kept alive by the caller)."""
    seq = [int(x) for x in seq]
    return (ctypes.c_int32 * max(len(seq), 1))(*seq)
