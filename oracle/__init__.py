"""TEST INFRASTRUCTURE: ctypes binding of oracle/liboracle.so (the CPU restatement in efa_oracle.c).

Only tests, the smoke check and the CPU-baseline leg of bench.py import this module. The product
package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")


def build() -> None:
    subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, stdout=subprocess.DEVNULL)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        h = C.CDLL(LIB_PATH)
        h.oracle_ref_inputs.restype = C.c_int
        h.oracle_ref_inputs.argtypes = [C.c_int] * 6 + [_f32p, _f32p, _f32p, _f32p]
        h.oracle_round_f16.argtypes = [_f32p, _u16p, C.c_size_t]
        h.oracle_widen_f16.argtypes = [_u16p, _f32p, C.c_size_t]
        h.oracle_attention_rows.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int,
                                            C.c_void_p, C.c_int, _f32p]
        h.oracle_project_rows.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p]
        h.oracle_block_rows.restype = C.c_int
        h.oracle_block_rows.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                        C.c_void_p, C.c_int, C.c_int, _f32p]
        h.oracle_compare.argtypes = [_f32p, _f32p, C.c_size_t, C.POINTER(C.c_float), C.POINTER(C.c_float)]
        _lib = h
    return _lib


def ref_inputs(S, d, H, R, rank, seed):
    """fp32 Q, K, V [H_local][S][d_h] and W_O [d_local][d] of the reference recipe."""
    H_local, d_h = H // R, d // H
    Q = np.empty((H_local, S, d_h), np.float32)
    K = np.empty_like(Q)
    V = np.empty_like(Q)
    W = np.empty((H_local * d_h, d), np.float32)
    rc = lib().oracle_ref_inputs(S, d, H, R, rank, seed, Q, K, V, W)
    if rc:
        raise ValueError(f"oracle_ref_inputs: bad shape ({rc})")
    return Q, K, V, W


def round_f16(x):
    """fp32 array -> uint16 fp16 bit patterns (round to nearest even)."""
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().oracle_round_f16(x, out, x.size)
    return out


def widen_f16(u):
    u = np.ascontiguousarray(u, np.uint16)
    out = np.empty(u.shape, np.float32)
    lib().oracle_widen_f16(u, out, u.size)
    return out


def _rows_arg(rows, S):
    if rows is None:
        return None, S, None
    arr = np.ascontiguousarray(rows, np.int32)
    return arr.ctypes.data, int(arr.size), arr


def attention_rows(Q, K, V, causal, rows=None):
    """Full-softmax attention for the selected rows: [nrows][H_local*d_h] fp32."""
    H_local, S, d_h = Q.shape
    ptr, n, keep = _rows_arg(rows, S)
    O = np.empty((n, H_local * d_h), np.float32)
    lib().oracle_attention_rows(np.ascontiguousarray(Q, np.float32), np.ascontiguousarray(K, np.float32),
                                np.ascontiguousarray(V, np.float32), H_local, S, d_h, int(bool(causal)), ptr, n, O)
    return O


def project_rows(O, W):
    n, d_local = O.shape
    d = W.shape[1]
    out = np.empty((n, d), np.float32)
    lib().oracle_project_rows(np.ascontiguousarray(O, np.float32), np.ascontiguousarray(W, np.float32),
                              n, d_local, d, 0, out)
    return out


def block_rows(per_rank, d, causal, rows=None):
    """Sum over ranks of attention + projection. per_rank: iterable of (Q, K, V, W_O) fp32 arrays."""
    out = None
    for Q, K, V, W in per_rank:
        H_local, S, d_h = Q.shape
        ptr, n, keep = _rows_arg(rows, S)
        if out is None:
            out = np.zeros((n, d), np.float32)
        rc = lib().oracle_block_rows(np.ascontiguousarray(Q, np.float32), np.ascontiguousarray(K, np.float32),
                                     np.ascontiguousarray(V, np.float32), np.ascontiguousarray(W, np.float32),
                                     H_local, S, d_h, d, int(bool(causal)), ptr, n, 1, out)
        if rc:
            raise MemoryError("oracle_block_rows")
    return out


def compare(a, ref):
    """(max_abs, max_ref): the reference's pass metric is max_abs / max_ref (attn_tests.cu:135-137)."""
    a = np.ascontiguousarray(a, np.float32).ravel()
    ref = np.ascontiguousarray(ref, np.float32).ravel()
    ma, mr = C.c_float(), C.c_float()
    lib().oracle_compare(a, ref, a.size, C.byref(ma), C.byref(mr))
    return float(ma.value), float(mr.value)
