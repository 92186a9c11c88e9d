"""ctypes binding of libanchor_attn_b200.so (the C ABI in include/anchor_attn_b200.h).

The library is built in-tree by ``anchor_attention_b200.build``.  There is no
fallback: if the library is missing or fails to load, importing the operator
raises."""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libanchor_attn_b200.so")

AA_OK = 0
AA_BF16 = 0

EXPORTS = [
    "aa_workspace_bytes", "aa_workspace_layout", "aa_id_row_offset", "aa_forward",
    "aa_step1_anchor", "aa_step2_stripes", "aa_step3_sparse", "aa_check_status",
    "aa_total_selected", "aa_strerror", "aa_last_cuda_error", "aa_version",
    "aa_launches_per_forward", "aa_forward_launches", "aa_step2_stripes_static", "aa_step3_sparse_push",
    "aa_selftest_wait_timeout", "aa_block_sparse_workspace_bytes", "aa_block_sparse_attend",
    "aa_block_sparse_check_status", "aa_validate_lists", "aa_step2_stripes_static_check_status",
    "aa_peer_barrier", "aa_dense_causal_attend", "aa_rope_dispatch",
]
MAX_PEERS = 8
STATIC_SCRATCH_BYTES = 8 << 20


class AAParams(ctypes.Structure):
    _fields_ = [
        ("B", ctypes.c_int32), ("H", ctypes.c_int32), ("Hkv", ctypes.c_int32),
        ("N", ctypes.c_int32), ("D", ctypes.c_int32),
        ("block_size", ctypes.c_int32), ("step", ctypes.c_int32), ("dtype", ctypes.c_int32),
        ("theta", ctypes.c_double), ("sm_scale", ctypes.c_double),
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("q_stride_b", ctypes.c_int64), ("q_stride_h", ctypes.c_int64), ("q_stride_n", ctypes.c_int64),
        ("k_stride_b", ctypes.c_int64), ("k_stride_h", ctypes.c_int64), ("k_stride_n", ctypes.c_int64),
        ("v_stride_b", ctypes.c_int64), ("v_stride_h", ctypes.c_int64), ("v_stride_n", ctypes.c_int64),
        ("o_stride_b", ctypes.c_int64), ("o_stride_h", ctypes.c_int64), ("o_stride_n", ctypes.c_int64),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
    ]


class AALayout(ctypes.Structure):
    _fields_ = [(n, ctypes.c_size_t) for n in (
        "m_off", "l_off", "acc_off", "qpool_off", "apool_off", "bitmap_off", "counts_off",
        "ids_off", "status_off", "total_bytes")] + [("ids_per_head", ctypes.c_int64)] + [
        (n, ctypes.c_size_t) for n in ("tile_slot_off", "gather_off", "gather_bytes", "min_bytes")]


class AAStripesStaticArgs(ctypes.Structure):
    _fields_ = [
        ("B", ctypes.c_int32), ("H", ctypes.c_int32), ("Hkv", ctypes.c_int32),
        ("N", ctypes.c_int32), ("D", ctypes.c_int32),
        ("block_size", ctypes.c_int32), ("step", ctypes.c_int32), ("dtype", ctypes.c_int32),
        ("theta", ctypes.c_double), ("sm_scale", ctypes.c_double),
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p),
        ("q_stride_b", ctypes.c_int64), ("q_stride_h", ctypes.c_int64), ("q_stride_n", ctypes.c_int64),
        ("k_stride_b", ctypes.c_int64), ("k_stride_h", ctypes.c_int64), ("k_stride_n", ctypes.c_int64),
        ("anchors", ctypes.c_void_p), ("counts", ctypes.c_void_p), ("ids", ctypes.c_void_p),
    ]


class AABlockSparse(ctypes.Structure):
    _fields_ = [
        ("B", ctypes.c_int32), ("H", ctypes.c_int32), ("Hkv", ctypes.c_int32),
        ("N", ctypes.c_int32), ("D", ctypes.c_int32),
        ("dtype", ctypes.c_int32), ("max_blocks", ctypes.c_int32),
        ("sm_scale", ctypes.c_double),
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("q_stride_b", ctypes.c_int64), ("q_stride_h", ctypes.c_int64), ("q_stride_n", ctypes.c_int64),
        ("k_stride_b", ctypes.c_int64), ("k_stride_h", ctypes.c_int64), ("k_stride_n", ctypes.c_int64),
        ("v_stride_b", ctypes.c_int64), ("v_stride_h", ctypes.c_int64), ("v_stride_n", ctypes.c_int64),
        ("o_stride_b", ctypes.c_int64), ("o_stride_h", ctypes.c_int64), ("o_stride_n", ctypes.c_int64),
        ("block_index", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
    ]


class AAPush(ctypes.Structure):
    _fields_ = [("n_peers", ctypes.c_int32), ("rows_per_peer", ctypes.c_int32), ("out", ctypes.c_void_p * MAX_PEERS)]


class AADenseCausal(ctypes.Structure):
    _fields_ = [
        ("B", ctypes.c_int32), ("H", ctypes.c_int32), ("Hkv", ctypes.c_int32),
        ("Nq", ctypes.c_int32), ("Nkv", ctypes.c_int32), ("D", ctypes.c_int32),
        ("dtype", ctypes.c_int32), ("sm_scale", ctypes.c_double),
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("q_stride_b", ctypes.c_int64), ("q_stride_h", ctypes.c_int64), ("q_stride_n", ctypes.c_int64),
        ("k_stride_b", ctypes.c_int64), ("k_stride_h", ctypes.c_int64), ("k_stride_n", ctypes.c_int64),
        ("v_stride_b", ctypes.c_int64), ("v_stride_h", ctypes.c_int64), ("v_stride_n", ctypes.c_int64),
        ("o_stride_b", ctypes.c_int64), ("o_stride_h", ctypes.c_int64), ("o_stride_n", ctypes.c_int64),
        ("status", ctypes.c_void_p),
    ]


class AARopeDispatch(ctypes.Structure):
    _fields_ = [
        ("n", ctypes.c_int32), ("H", ctypes.c_int32), ("Hkv", ctypes.c_int32), ("D", ctypes.c_int32),
        ("dtype", ctypes.c_int32), ("n_peers", ctypes.c_int32), ("token0", ctypes.c_int32),
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
        ("q_stride_n", ctypes.c_int64), ("k_stride_n", ctypes.c_int64), ("v_stride_n", ctypes.c_int64),
        ("cos", ctypes.c_void_p), ("sin", ctypes.c_void_p),
        ("dst", ctypes.c_void_p * MAX_PEERS),
    ]


class AAPeerBarrier(ctypes.Structure):
    _fields_ = [("n_peers", ctypes.c_int32), ("rank", ctypes.c_int32), ("epoch", ctypes.c_int32),
                ("timeout_ms", ctypes.c_uint32), ("flags", ctypes.c_void_p * MAX_PEERS), ("status", ctypes.c_void_p)]


_lib = None


def load():
    """Load the shared library once and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m anchor_attention_b200.build` "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(LIB_PATH)
    P = ctypes.POINTER(AAParams)
    lib.aa_workspace_bytes.argtypes = [P, ctypes.POINTER(ctypes.c_size_t)]
    lib.aa_workspace_layout.argtypes = [P, ctypes.POINTER(AALayout)]
    lib.aa_id_row_offset.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
    lib.aa_id_row_offset.restype = ctypes.c_int64
    for name in ("aa_forward", "aa_step1_anchor", "aa_step2_stripes", "aa_step3_sparse", "aa_check_status",
                 "aa_selftest_wait_timeout", "aa_validate_lists"):
        getattr(lib, name).argtypes = [P, ctypes.c_void_p]
        getattr(lib, name).restype = ctypes.c_int
    lib.aa_step2_stripes_static.argtypes = [ctypes.POINTER(AAStripesStaticArgs), ctypes.c_void_p]
    lib.aa_step2_stripes_static.restype = ctypes.c_int
    lib.aa_step2_stripes_static_check_status.argtypes = [ctypes.c_void_p]
    lib.aa_step2_stripes_static_check_status.restype = ctypes.c_int
    lib.aa_step3_sparse_push.argtypes = [P, ctypes.POINTER(AAPush), ctypes.c_void_p]
    lib.aa_step3_sparse_push.restype = ctypes.c_int
    lib.aa_dense_causal_attend.argtypes = [ctypes.POINTER(AADenseCausal), ctypes.c_void_p]
    lib.aa_dense_causal_attend.restype = ctypes.c_int
    lib.aa_rope_dispatch.argtypes = [ctypes.POINTER(AARopeDispatch), ctypes.c_void_p]
    lib.aa_rope_dispatch.restype = ctypes.c_int
    lib.aa_peer_barrier.argtypes = [ctypes.POINTER(AAPeerBarrier), ctypes.c_void_p]
    lib.aa_peer_barrier.restype = ctypes.c_int
    PB = ctypes.POINTER(AABlockSparse)
    lib.aa_block_sparse_workspace_bytes.argtypes = [PB, ctypes.POINTER(ctypes.c_size_t)]
    lib.aa_block_sparse_workspace_bytes.restype = ctypes.c_int
    for name in ("aa_block_sparse_attend", "aa_block_sparse_check_status"):
        getattr(lib, name).argtypes = [PB, ctypes.c_void_p]
        getattr(lib, name).restype = ctypes.c_int
    lib.aa_total_selected.argtypes = [P, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64)]
    lib.aa_forward_launches.argtypes = [P]
    lib.aa_forward_launches.restype = ctypes.c_int
    lib.aa_strerror.argtypes = [ctypes.c_int]
    lib.aa_strerror.restype = ctypes.c_char_p
    lib.aa_last_cuda_error.restype = ctypes.c_char_p
    _lib = lib
    return lib


def error_text(code: int) -> str:
    lib = load()
    msg = lib.aa_strerror(code).decode()
    if code == -10:
        msg += ": " + lib.aa_last_cuda_error().decode()
    return msg
