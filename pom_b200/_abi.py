"""ctypes binding of libpom_b200.so (see include/pom_b200.h for the contract).

The library is the only compute path of this package: if it cannot be loaded the
import of any operator fails loudly; there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpom_b200.so")

ABI_VERSION = 3
POM_BF16, POM_F32 = 0, 1
ROPE_NONE, ROPE_1D, ROPE_2D = 0, 1, 2
OUT_BF16, OUT_F32, OUT_F32_ACCUM = 0, 1, 2

ERR_UNSUPPORTED = -4
ERR_K_TOO_LARGE = -5
ERR_BAD_SHAPE = -1


class PomError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        super().__init__(f"{where}: {strerror(code)} (code {code})")


class Rope(C.Structure):
    _fields_ = [
        ("kind", C.c_int32),
        ("pos_stride", C.c_int32),
        ("cos0", C.c_void_p),
        ("sin0", C.c_void_p),
        ("cos1", C.c_void_p),
        ("sin1", C.c_void_p),
        ("pos", C.c_void_p),
        ("len0", C.c_int32), ("len1", C.c_int32),
        ("step0", C.c_int32), ("step1", C.c_int32),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("Bm", C.c_void_p), ("C", C.c_void_p),
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
        ("batches", C.c_int32), ("a_mn_major", C.c_int32), ("b_mn_major", C.c_int32),
        ("out_mode", C.c_int32), ("split_k", C.c_int32), ("alpha", C.c_float),
        ("act", C.c_int32), ("residual", C.c_void_p), ("ldr", C.c_int64),
        ("a_batch_stride", C.c_int64), ("b_batch_stride", C.c_int64), ("c_batch_stride", C.c_int64),
        ("b_batched", C.c_int32),
    ]


class CtxArgs(C.Structure):
    _fields_ = [
        ("X", C.c_void_p), ("Wpo", C.c_void_p), ("coeff", C.c_void_p), ("row_weight", C.c_void_p),
        ("hp_out", C.c_void_p), ("partial", C.c_void_p),
        ("ldx", C.c_int64), ("ldw", C.c_int64), ("ld_hp", C.c_int64),
        ("B", C.c_int32), ("N", C.c_int32), ("D", C.c_int32), ("P", C.c_int32), ("K", C.c_int32),
        ("tile_weight", C.c_void_p),
        ("rope", Rope),
        ("causal", C.c_int32), ("pre_out", C.c_void_p), ("ld_pre", C.c_int64), ("group_sums", C.c_void_p),
    ]


class GateArgs(C.Structure):
    _fields_ = [
        ("X", C.c_void_p), ("Wse", C.c_void_p), ("bias", C.c_void_p), ("H", C.c_void_p),
        ("z_out", C.c_void_p), ("sh_out", C.c_void_p),
        ("ldx", C.c_int64), ("ldw", C.c_int64), ("ld_z", C.c_int64), ("ld_sh", C.c_int64),
        ("h_batch_stride", C.c_int64), ("h_row_stride", C.c_int64),
        ("B", C.c_int32), ("T", C.c_int32), ("D", C.c_int32), ("P", C.c_int32),
        ("rope", Rope),
        ("causal", C.c_int32), ("pre", C.c_void_p), ("ld_pre", C.c_int64), ("carry", C.c_void_p),
        ("token_offset", C.c_int64),
    ]


class GateBwdArgs(C.Structure):
    _fields_ = [
        ("dY", C.c_void_p), ("Wo", C.c_void_p), ("bias", C.c_void_p), ("H", C.c_void_p),
        ("z", C.c_void_p), ("g_out", C.c_void_p), ("dh_partial", C.c_void_p), ("db_partial", C.c_void_p),
        ("ld_dy", C.c_int64), ("ldw", C.c_int64), ("ld_z", C.c_int64), ("ld_g", C.c_int64),
        ("h_batch_stride", C.c_int64),
        ("B", C.c_int32), ("T", C.c_int32), ("D", C.c_int32), ("P", C.c_int32),
        ("WoT", C.c_void_p), ("ldwt", C.c_int64),
        ("rope", Rope),
        ("causal", C.c_int32), ("pre", C.c_void_p), ("ld_pre", C.c_int64), ("carry", C.c_void_p),
        ("suf_out", C.c_void_p), ("ld_suf", C.c_int64), ("group_sums", C.c_void_p), ("token_offset", C.c_int64),
    ]


class AggArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("coeff", C.c_void_p), ("row_weight", C.c_void_p), ("carry", C.c_void_p),
        ("partial", C.c_void_p), ("out", C.c_void_p), ("total", C.c_void_p),
        ("ldx", C.c_int64), ("ld_out", C.c_int64), ("token_offset", C.c_int64),
        ("B", C.c_int32), ("N", C.c_int32), ("P", C.c_int32), ("K", C.c_int32),
        ("dtype", C.c_int32), ("causal", C.c_int32),
        ("rope", Rope),
    ]


class AggBwdArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("coeff", C.c_void_p), ("row_weight", C.c_void_p), ("denom", C.c_void_p),
        ("dH", C.c_void_p), ("dout", C.c_void_p), ("carry", C.c_void_p), ("partial", C.c_void_p),
        ("total", C.c_void_p), ("dx", C.c_void_p), ("dcoeff_partial", C.c_void_p),
        ("ldx", C.c_int64), ("ld_dx", C.c_int64), ("ld_dout", C.c_int64), ("token_offset", C.c_int64),
        ("scale", C.c_float),
        ("B", C.c_int32), ("N", C.c_int32), ("P", C.c_int32), ("K", C.c_int32),
        ("dtype", C.c_int32), ("causal", C.c_int32), ("phase", C.c_int32),
        ("rope", Rope),
    ]


class SelectArgs(C.Structure):
    _fields_ = [
        ("z", C.c_void_p), ("bias", C.c_void_p), ("H", C.c_void_p), ("sh", C.c_void_p),
        ("ld_z", C.c_int64), ("ld_h", C.c_int64), ("ld_sh", C.c_int64),
        ("B", C.c_int32), ("T", C.c_int32), ("P", C.c_int32),
        ("dtype", C.c_int32), ("h_per_token", C.c_int32), ("activated", C.c_int32),
        ("row_denom", C.c_void_p),
        ("rope", Rope),
    ]


class SelectBwdArgs(C.Structure):
    _fields_ = [
        ("dsh", C.c_void_p), ("z", C.c_void_p), ("bias", C.c_void_p), ("H", C.c_void_p),
        ("dz", C.c_void_p), ("dbias_partial", C.c_void_p), ("dh_partial", C.c_void_p), ("dh_tok", C.c_void_p),
        ("ld_dsh", C.c_int64), ("ld_z", C.c_int64), ("ld_h", C.c_int64), ("ld_dz", C.c_int64), ("ld_dh", C.c_int64),
        ("B", C.c_int32), ("T", C.c_int32), ("P", C.c_int32),
        ("dtype", C.c_int32), ("h_per_token", C.c_int32), ("activated", C.c_int32),
        ("row_denom", C.c_void_p),
        ("rope", Rope),
    ]


class SelectHeadsArgs(C.Structure):
    _fields_ = [
        ("s", C.c_void_p), ("H", C.c_void_p), ("dsh", C.c_void_p), ("sh", C.c_void_p), ("ds", C.c_void_p),
        ("dh_partial", C.c_void_p), ("dh_tok", C.c_void_p),
        ("ld_h", C.c_int64), ("ld_sh", C.c_int64), ("ld_dsh", C.c_int64), ("ld_dh", C.c_int64),
        ("B", C.c_int32), ("T", C.c_int32), ("P", C.c_int32), ("heads", C.c_int32),
        ("dtype", C.c_int32), ("h_per_token", C.c_int32),
    ]


class HeadsArgs(C.Structure):
    _fields_ = [
        ("H", C.c_void_p), ("Wo", C.c_void_p), ("s", C.c_void_p), ("Mb", C.c_void_p), ("y", C.c_void_p),
        ("residual", C.c_void_p), ("dy", C.c_void_p), ("ds", C.c_void_p), ("dMb_partial", C.c_void_p),
        ("dMb", C.c_void_p), ("dH", C.c_void_p), ("dWo", C.c_void_p),
        ("ldw", C.c_int64),
        ("B", C.c_int32), ("T", C.c_int32), ("D", C.c_int32), ("P", C.c_int32), ("heads", C.c_int32),
        ("dtype", C.c_int32),
    ]


class LayerArgs(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("T", C.c_int32), ("N", C.c_int32), ("D", C.c_int32), ("P", C.c_int32), ("K", C.c_int32),
        ("self_mixing", C.c_int32), ("frames", C.c_int32), ("save", C.c_int32), ("n_past", C.c_float),
        ("xq", C.c_void_p), ("xc", C.c_void_p), ("w_qc", C.c_void_p), ("w_ag", C.c_void_p),
        ("se_bias", C.c_void_p), ("coeff", C.c_void_p), ("mask", C.c_void_p), ("h_past", C.c_void_p),
        ("residual", C.c_void_p),
        ("y", C.c_void_p), ("hp", C.c_void_p), ("z", C.c_void_p), ("sh", C.c_void_p),
        ("H", C.c_void_p), ("denom", C.c_void_p),
        ("dy", C.c_void_p), ("dh_state", C.c_void_p), ("G", C.c_void_p), ("dxq", C.c_void_p), ("dxc", C.c_void_p),
        ("grads", C.c_void_p), ("d_hpast", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_uint64),
        ("rope_c", Rope), ("rope_q", Rope), ("w_ag_t", C.c_void_p),
        ("causal", C.c_int32), ("reserved0", C.c_int32), ("token_offset", C.c_int64),
        ("pre", C.c_void_p), ("carry", C.c_void_p),
    ]


PEER_MAX_RANKS = 16
PEER_HANDLE_BYTES = 64
PEER_SUM_ALL, PEER_SUM_BEFORE, PEER_SUM_AFTER = 0, 1, 2


class PeerComm(C.Structure):
    _fields_ = [
        ("base", C.c_void_p * PEER_MAX_RANKS),
        ("rank", C.c_int32), ("world", C.c_int32),
        ("slot_floats", C.c_ulonglong), ("flat_floats", C.c_ulonglong),
        ("wait_ns", C.c_ulonglong),
    ]


class PeerXchgArgs(C.Structure):
    _fields_ = [
        ("partial", C.c_void_p), ("out", C.c_void_p), ("denom", C.c_void_p),
        ("scale", C.c_float),
        ("B", C.c_int32), ("chunks", C.c_int32), ("P", C.c_int32), ("mode", C.c_int32),
    ]


# Every exported symbol with its signature; test_abi_exports checks the list against the header.
_SIGNATURES = {
    "pom_abi_version": (C.c_int, []),
    "pom_strerror": (C.c_char_p, [C.c_int]),
    "pom_device_check": (C.c_int, []),
    "pom_launch_count": (C.c_longlong, []),
    "pom_gemm_bf16": (C.c_int, [C.POINTER(GemmArgs), C.c_void_p, C.c_void_p]),
    "pom_set_gemm_mode": (C.c_int, [C.c_int]),
    "pom_gemm_f32": (C.c_int, [C.POINTER(GemmArgs), C.c_void_p]),
    "pom_ctx_gemm": (C.c_int, [C.POINTER(CtxArgs), C.c_void_p, C.c_void_p]),
    "pom_reduce_partials": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "pom_gate_gemm": (C.c_int, [C.POINTER(GateArgs), C.c_void_p, C.c_void_p]),
    "pom_gate_bwd_gemm": (C.c_int, [C.POINTER(GateBwdArgs), C.c_void_p, C.c_void_p]),
    "pom_agg_chunks": (C.c_int32, [C.c_int32]),
    "pom_poly_agg_fwd": (C.c_int, [C.POINTER(AggArgs), C.c_void_p]),
    "pom_poly_agg_mean_noalloc": (C.c_int, [C.POINTER(AggArgs), C.c_void_p, C.c_float, C.c_void_p, C.c_void_p]),
    "pom_poly_agg_bwd": (C.c_int, [C.POINTER(AggBwdArgs), C.c_void_p]),
    "pom_poly_agg_bwd_slots": (C.c_int32, [C.POINTER(AggBwdArgs)]),
    "pom_ops_status": (C.c_int, [C.POINTER(C.c_int32)]),
    "pom_select_fwd": (C.c_int, [C.POINTER(SelectArgs), C.c_void_p]),
    "pom_select_bwd": (C.c_int, [C.POINTER(SelectBwdArgs), C.c_void_p]),
    "pom_select_heads_fwd": (C.c_int, [C.POINTER(SelectHeadsArgs), C.c_void_p]),
    "pom_select_heads_bwd": (C.c_int, [C.POINTER(SelectHeadsArgs), C.c_void_p]),
    "pom_state_merge": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int64, C.c_void_p]),
    "pom_tile_weights": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "pom_frame_prefix_mean": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "pom_fill_zero": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p]),
    "pom_group_scan": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                C.c_void_p]),
    "pom_rope_pos_info": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p]),
    "pom_transpose_bf16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "pom_cast_f32_to_bf16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "pom_cast_bf16_to_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "pom_heads_supported": (C.c_int, [C.c_int32, C.c_int32, C.c_int32]),
    "pom_heads_mix": (C.c_int, [C.POINTER(HeadsArgs), C.c_void_p]),
    "pom_heads_out_fwd": (C.c_int, [C.POINTER(HeadsArgs), C.c_void_p]),
    "pom_heads_out_bwd": (C.c_int, [C.POINTER(HeadsArgs), C.c_void_p]),
    "pom_heads_mix_bwd": (C.c_int, [C.POINTER(HeadsArgs), C.c_void_p]),
    "pom_layer_workspace_bytes": (C.c_uint64, [C.POINTER(LayerArgs)]),
    "pom_layer_fwd": (C.c_int, [C.POINTER(LayerArgs), C.c_void_p, C.c_void_p]),
    "pom_layer_bwd": (C.c_int, [C.POINTER(LayerArgs), C.c_void_p, C.c_void_p]),
    "pom_peer_layout": (C.c_int, [C.c_int, C.c_ulonglong, C.c_ulonglong, C.POINTER(C.c_ulonglong)]),
    "pom_peer_export": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_ulonglong)]),
    "pom_peer_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "pom_peer_close": (C.c_int, [C.c_void_p]),
    "pom_peer_exchange": (C.c_int, [C.POINTER(PeerComm), C.POINTER(PeerXchgArgs), C.c_void_p, C.c_void_p]),
    "pom_peer_allreduce_flat": (C.c_int, [C.POINTER(PeerComm), C.c_ulonglong, C.c_void_p, C.c_void_p]),
    "pom_peer_allreduce_flat_bf16": (C.c_int, [C.POINTER(PeerComm), C.c_ulonglong, C.c_void_p, C.c_void_p]),
    "pom_copy_bytes": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
}

_lib = None


def lib() -> C.CDLL:
    """Load the shared library once. Raises if it is missing: there is no fallback path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m pom_b200._build` "
                "(the package has no CPU or PyTorch fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        if handle.pom_abi_version() != ABI_VERSION:
            raise ImportError("libpom_b200.so ABI version mismatch; rebuild it")
        _lib = handle
    return _lib


def strerror(code: int) -> str:
    return lib().pom_strerror(code).decode()


def check(code: int, where: str) -> None:
    if code != 0:
        raise PomError(code, where)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr() -> C.c_void_p:
    """The current device's current stream as the library's ``void* stream`` argument."""
    if _raw_stream is not None:  # one C call instead of building a torch.cuda.Stream object
        return C.c_void_p(_raw_stream(torch.cuda.current_device()))
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t) -> C.c_void_p | None:
    return None if t is None else C.c_void_p(t.data_ptr())


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return POM_BF16
    if dt == torch.float32:
        return POM_F32
    raise TypeError(f"pom_b200 supports bfloat16 and float32 tensors, got {dt}")


_status = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 word the GEMM kernels write when a bounded wait expires."""
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def read_status(device) -> int:
    """Synchronising read of the status words (tests and debugging only): the GEMM / exchange word, else the
    operator kernels' word."""
    word = int(status_word(device).item())
    if word:
        return word
    v = C.c_int32(0)
    with torch.cuda.device(device):
        check(lib().pom_ops_status(C.byref(v)), "pom_ops_status")
    return int(v.value)
