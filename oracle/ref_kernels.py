"""ctypes binding of oracle/_ref/libzoph_ref_kernels.so: the reference project's own forward-path kernels
(src/custom_kernels.h compiled unmodified behind oracle/ref_shim.cu), driven with the reference's launch shapes.

TEST INFRASTRUCTURE ONLY: it pins the CPU oracle to the reference's code.  The library is built where the reference's
sources are present (`make -C oracle ref`) and travels with the repository to the GPU machine; nothing here reads the
reference at run time.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(_HERE, "_ref", "libzoph_ref_kernels.so")
_LIB = None

c_int_p = ctypes.POINTER(ctypes.c_int)
c_float_p = ctypes.POINTER(ctypes.c_float)


def build(ref_src="/root/reference/src", force=False):
    """Compile the library if the reference's kernel file is available; returns the path or None."""
    src = os.path.join(ref_src, "custom_kernels.h")
    if not os.path.exists(src):
        return SO if os.path.exists(SO) else None
    shim = os.path.join(_HERE, "ref_shim.cu")
    if force or not os.path.exists(SO) or os.path.getmtime(SO) < os.path.getmtime(shim):
        subprocess.check_call(["make", "-C", _HERE, "-s", "ref", "REF_SRC=" + ref_src])
    return SO


def available():
    return os.path.exists(SO)


def lib():
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(SO)
        L.ref_prep_vocab.argtypes = [c_int_p, ctypes.c_int, c_int_p, c_int_p]
        L.ref_sparse_lookup.argtypes = [c_float_p, ctypes.c_int, ctypes.c_int, c_int_p, ctypes.c_int, c_float_p]
        L.ref_matrix_bias.argtypes = [ctypes.c_int, ctypes.c_int, c_float_p, c_float_p]
        L.ref_lstm_cell.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(c_float_p), c_float_p, c_float_p,
                                    c_float_p, c_float_p, c_int_p, c_float_p, c_float_p]
        L.ref_attention_localp.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(c_float_p), c_float_p,
                                           c_int_p, c_float_p, ctypes.c_int, c_int_p, c_float_p, c_float_p, c_int_p,
                                           c_float_p, c_int_p]
        _LIB = L
    return _LIB


def _f(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


def _i(a):
    return np.ascontiguousarray(a, dtype=np.int32).reshape(-1)


def _fp(a):
    return None if a is None else a.ctypes.data_as(c_float_p)


def _ip(a):
    return a.ctypes.data_as(c_int_p)


def _ok(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what}: CUDA error {rc}")


def prep_vocab(ids):
    ids = _i(ids)
    a, b = np.zeros_like(ids), np.zeros_like(ids)
    _ok(lib().ref_prep_vocab(_ip(ids), ids.size, _ip(a), _ip(b)), "ref_prep_vocab")
    return a, b


def sparse_lookup(W, H, V, ids):
    W, ids = _f(W), _i(ids)
    x = np.zeros(H * ids.size, dtype=np.float32)
    _ok(lib().ref_sparse_lookup(_fp(W), H, V, _ip(ids), ids.size, _fp(x)), "ref_sparse_lookup")
    return x


def matrix_bias(V, N, mat, vec):
    mat = _f(mat).copy()
    vec = _f(vec)
    _ok(lib().ref_matrix_bias(V, N, _fp(mat), _fp(vec)), "ref_matrix_bias")
    return mat


def lstm_cell(H, B, w17, x, h_prev, c_prev, htild, mask):
    keep = [_f(a) for a in w17]
    arr = (c_float_p * 17)(*[_fp(a) for a in keep])
    x, h_prev, c_prev, htild, mask = _f(x), _f(h_prev), _f(c_prev), _f(htild), _i(mask)
    h, c = np.zeros(H * B, np.float32), np.zeros(H * B, np.float32)
    _ok(lib().ref_lstm_cell(H, B, arr, _fp(x), _fp(h_prev), _fp(c_prev), _fp(htild), _ip(mask), _fp(h), _fp(c)),
        "ref_lstm_cell")
    return h, c


def attention_localp(H, B, D, w6, h_t, mask, hs_all, S_max, lens, offs):
    keep = [_f(a) for a in w6]
    arr = (c_float_p * 6)(*[_fp(a) for a in keep])
    h_t, hs_all, mask = _f(h_t), _f(hs_all), _i(mask)
    info = _i(np.concatenate([_i(lens), _i(offs)]))
    W2 = 2 * D + 1
    out = np.zeros(H * B, np.float32)
    al = np.zeros(W2 * B, np.float32)
    idx = np.zeros(W2 * B, np.int32)
    p_t = np.zeros(B, np.float32)
    vit = np.zeros(B, np.int32)
    _ok(lib().ref_attention_localp(H, B, D, arr, _fp(h_t), _ip(mask), _fp(hs_all), S_max, _ip(info), _fp(out), _fp(al),
                                   _ip(idx), _fp(p_t), _ip(vit)), "ref_attention_localp")
    return out, al, idx, p_t, vit
