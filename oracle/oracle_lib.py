"""ctypes binding of the C++ CPU oracle (oracle/zoph_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline /
reference arms of the benchmark.  The product package never imports this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

c_int_p = ctypes.POINTER(ctypes.c_int)
c_float_p = ctypes.POINTER(ctypes.c_float)
c_double_p = ctypes.POINTER(ctypes.c_double)


def build(force=False):
    """Compile liboracle with the committed Makefile (g++ only)."""
    so = os.path.join(_HERE, "libzoph_oracle.so")
    src = os.path.join(_HERE, "zoph_oracle.cpp")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "libzoph_oracle.so")
        if not os.path.exists(so):
            build()
        L = ctypes.CDLL(so)
        L.orc_model_create.restype = ctypes.c_void_p
        L.orc_model_create.argtypes = [c_int_p]
        L.orc_model_destroy.argtypes = [ctypes.c_void_p]
        L.orc_model_num_tensors.argtypes = [ctypes.c_void_p]
        L.orc_model_tensor_shape.argtypes = [ctypes.c_void_p, ctypes.c_int, c_int_p, c_int_p]
        L.orc_model_set_tensor.argtypes = [ctypes.c_void_p, ctypes.c_int, c_float_p, ctypes.c_int]
        L.orc_score_batch.restype = ctypes.c_double
        L.orc_score_batch.argtypes = [ctypes.c_void_p, c_int_p, ctypes.c_int, c_int_p, c_int_p, ctypes.c_int,
                                      ctypes.c_int, c_double_p, c_float_p]
        L.orc_beam_decode.argtypes = [ctypes.c_void_p, c_int_p, c_int_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_float, ctypes.c_float, ctypes.c_float, ctypes.c_int, ctypes.c_int,
                                      c_int_p, c_int_p, c_float_p]
        L.orc_beam_decode_align.argtypes = L.orc_beam_decode.argtypes + [c_int_p]
        L.orc_beam_decode_margins.argtypes = [ctypes.c_void_p, c_int_p, c_int_p, ctypes.c_int, ctypes.c_int, ctypes.c_float,
                                              ctypes.c_float, ctypes.c_float, ctypes.c_int, c_float_p]
        L.orc_attention_viterbi.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                            ctypes.POINTER(c_float_p), c_float_p, c_int_p, c_float_p, ctypes.c_int,
                                            c_int_p, c_int_p, c_float_p, c_int_p]
        L.orc_beam_decode_ensemble.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.POINTER(c_int_p),
                                               ctypes.POINTER(c_int_p), ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                               ctypes.c_float, ctypes.c_float, ctypes.c_float, ctypes.c_int,
                                               ctypes.c_int, c_int_p, c_int_p, c_float_p, c_int_p]
        L.orc_gather.argtypes = [c_float_p, ctypes.c_int, c_int_p, ctypes.c_int, c_float_p]
        L.orc_lstm_cell.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(c_float_p), c_float_p, c_float_p,
                                    c_float_p, c_float_p, c_int_p, c_float_p, c_float_p]
        L.orc_attention.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(c_float_p),
                                    c_float_p, c_int_p, c_float_p, ctypes.c_int, c_int_p, c_int_p, c_float_p,
                                    c_float_p, c_int_p]
        L.orc_softmax_logp.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, c_float_p, c_float_p, c_float_p,
                                       c_int_p, c_double_p, c_double_p]
        L.orc_softmax_dist.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, c_float_p, c_float_p, c_float_p,
                                       c_float_p]
        L.orc_set_acc_float.argtypes = [ctypes.c_int]
        L.orc_num_threads.restype = ctypes.c_int
        _LIB = L
    return _LIB


def _fp(a):
    return a.ctypes.data_as(c_float_p) if a is not None else None


def _ip(a):
    return a.ctypes.data_as(c_int_p) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


CFG_KEYS = ("num_layers", "H", "V_src", "V_tgt", "lm", "attention", "feed_input", "D")


class OracleModel:
    """cfg: dict with CFG_KEYS; tensors: list of float32 arrays (column-major, flat) in weight-file order."""

    def __init__(self, cfg, tensors):
        self.cfg = dict(cfg)
        arr = (ctypes.c_int * 8)(*[int(cfg[k]) for k in CFG_KEYS])
        self._h = lib().orc_model_create(arr)
        n = lib().orc_model_num_tensors(self._h)
        assert n == len(tensors), (n, len(tensors))
        self._keep = []
        for i, t in enumerate(tensors):
            r, c = ctypes.c_int(), ctypes.c_int()
            lib().orc_model_tensor_shape(self._h, i, ctypes.byref(r), ctypes.byref(c))
            t = _f32(t).reshape(-1)
            assert t.size == r.value * c.value, (i, t.size, r.value, c.value)
            self._keep.append(t)
            lib().orc_model_set_tensor(self._h, i, _fp(t), 0)

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:  # module globals may be gone at interpreter shutdown
            lib().orc_model_destroy(self._h)
            self._h = None

    def shapes(self):
        out = []
        for i in range(lib().orc_model_num_tensors(self._h)):
            r, c = ctypes.c_int(), ctypes.c_int()
            lib().orc_model_tensor_shape(self._h, i, ctypes.byref(r), ctypes.byref(c))
            out.append((r.value, c.value))
        return out

    def score_batch(self, src_ids, tgt_in, tgt_out, want_top=False):
        """src_ids [S,B] or None; tgt_in/tgt_out [T,B]. Returns logp [T,B] float64 (and top states [T,B,H])."""
        tgt_in, tgt_out = _i32(tgt_in), _i32(tgt_out)
        T, B = tgt_in.shape
        if src_ids is not None:
            src_ids = _i32(src_ids)
            S = src_ids.shape[0]
        else:
            S = 0
        out = np.zeros((T, B), dtype=np.float64)
        top = np.zeros((T, B, self.cfg["H"]), dtype=np.float32) if want_top else None
        lib().orc_score_batch(self._h, _ip(src_ids), S, _ip(tgt_in), _ip(tgt_out), T, B,
                              out.ctypes.data_as(c_double_p), _fp(top))
        return (out, top) if want_top else out

    def beam_decode(self, sources, beam, k_best=1, min_ratio=0.5, max_ratio=1.5, penalty=0.0, longest_sent=100,
                    want_align=False):
        """sources: list of reversed id lists. Returns (ids [n,k,Lmax], len [n,k], score [n,k]) and, with want_align,
        the viterbi alignment stored with every hypothesis position [n,k,Lmax]."""
        n = len(sources)
        flat = _i32(np.concatenate([np.asarray(s, dtype=np.int32) for s in sources]))
        lens = _i32([len(s) for s in sources])
        Lmax = longest_sent + 4
        ids = np.zeros((n, k_best, Lmax), dtype=np.int32)
        ln = np.zeros((n, k_best), dtype=np.int32)
        sc = np.zeros((n, k_best), dtype=np.float32)
        al = np.zeros((n, k_best, Lmax), dtype=np.int32) if want_align else None
        lib().orc_beam_decode_align(self._h, _ip(flat), _ip(lens), n, beam, k_best, min_ratio, max_ratio, penalty,
                                    longest_sent, Lmax, _ip(ids), _ip(ln), _fp(sc), _ip(al))
        return (ids, ln, sc, al) if want_align else (ids, ln, sc)


def localp_window_positions(model, src_ids, tgt_in, tgt_out):
    """The window positions p_t [T,B] (NaN where masked) the oracle's local-p attention computed while scoring the
    batch.  The window is cut at int(p_t): a test aid for telling a one-position window shift on a near-integer p_t
    from a real disagreement."""
    T, B = np.asarray(tgt_in).shape
    lib().orc_pt_log_start.argtypes = [ctypes.c_int]
    lib().orc_pt_log_read.argtypes = [c_float_p, ctypes.c_int]
    lib().orc_pt_log_read.restype = ctypes.c_int
    lib().orc_pt_log_start(1)
    try:
        model.score_batch(src_ids, tgt_in, tgt_out)
        out = np.full(T * B, np.nan, dtype=np.float32)
        n = lib().orc_pt_log_read(_fp(out), T * B)
    finally:
        lib().orc_pt_log_start(0)
    assert n == T * B, f"expected {T * B} window positions, the oracle logged {n}"
    return out.reshape(T, B)


def localp_clear_tokens(model, src_ids, tgt_in, tgt_out, rtol=1e-5):
    """Boolean [T,B]: True for the tokens whose local-p windows, at this and every earlier step of the sentence, were cut
    at a p_t farther than rtol * p_t from an integer.  From the first near-integer step on, a correct fp32
    implementation may attend a window shifted by one position, and (with feed-input) carries the difference to the
    end of the sentence.  Also returns the smallest distance seen."""
    pt = localp_window_positions(model, src_ids, tgt_in, tgt_out)
    with np.errstate(invalid="ignore"):
        fr = pt - np.floor(pt)
        margin = np.minimum(fr, 1.0 - fr)
        near = margin < rtol * np.maximum(pt, 1.0)
    near = np.where(np.isnan(pt), False, near)
    clear = np.cumsum(near, axis=0) == 0
    return clear, float(np.nanmin(margin))


def beam_decode_margins(model, sources, beam, min_ratio=0.5, max_ratio=1.5, penalty=0.0, longest_sent=100):
    """Per sentence the smallest score difference that decided anything in the oracle's beam search: at every step
    between the last candidate that entered the beam and the best one left behind, and at the end between the best and
    the second-best hypothesis.  A test aid for telling real disagreements from near-ties."""
    n = len(sources)
    flat = _i32(np.concatenate([np.asarray(s, dtype=np.int32) for s in sources]))
    lens = _i32([len(s) for s in sources])
    out = np.zeros(n, dtype=np.float32)
    lib().orc_beam_decode_margins(model._h, _ip(flat), _ip(lens), n, beam, min_ratio, max_ratio, penalty, longest_sent,
                                  _fp(out))
    return out


def beam_decode_ensemble(models, sources_per_model, beam, k_best=1, min_ratio=0.5, max_ratio=1.5, penalty=0.0,
                         longest_sent=100, want_align=False):
    """Ensemble beam search (probability averaging, src/ensemble_factory.hpp:768-795): models = OracleModel list,
    sources_per_model[k] = the k-th model's reversed id lists.  Returns (ids [n,k,Lmax], len [n,k], score [n,k])."""
    K, n = len(models), len(sources_per_model[0])
    flats = [_i32(np.concatenate([np.asarray(s, dtype=np.int32) for s in srcs])) for srcs in sources_per_model]
    lens = [_i32([len(s) for s in srcs]) for srcs in sources_per_model]
    Lmax = longest_sent + 4
    ids = np.zeros((n, k_best, Lmax), dtype=np.int32)
    ln = np.zeros((n, k_best), dtype=np.int32)
    sc = np.zeros((n, k_best), dtype=np.float32)
    hs = (ctypes.c_void_p * K)(*[m._h for m in models])
    fp = (c_int_p * K)(*[_ip(f) for f in flats])
    lp = (c_int_p * K)(*[_ip(l) for l in lens])
    al = np.zeros((n, k_best, Lmax), dtype=np.int32) if want_align else None
    lib().orc_beam_decode_ensemble(hs, K, fp, lp, n, beam, k_best, min_ratio, max_ratio, penalty, longest_sent, Lmax,
                                   _ip(ids), _ip(ln), _fp(sc), _ip(al))
    return (ids, ln, sc, al) if want_align else (ids, ln, sc)


def gather(W, H, ids):
    W, ids = _f32(W).reshape(-1), _i32(ids).reshape(-1)
    x = np.zeros(H * ids.size, dtype=np.float32)
    lib().orc_gather(_fp(W), H, _ip(ids), ids.size, _fp(x))
    return x


def lstm_cell(H, B, w17, x, h_prev, c_prev, htild, mask):
    """w17: list of 17 arrays or None, in file order (index 8 = embedding, unused)."""
    keep = [None if a is None else _f32(a).reshape(-1) for a in w17]
    arr = (c_float_p * 17)(*[_fp(a) if a is not None else None for a in keep])
    x, h_prev, c_prev = _f32(x).reshape(-1), _f32(h_prev).reshape(-1), _f32(c_prev).reshape(-1)
    htild = None if htild is None else _f32(htild).reshape(-1)
    mask = _i32(mask)
    h = np.zeros(H * B, dtype=np.float32)
    c = np.zeros(H * B, dtype=np.float32)
    lib().orc_lstm_cell(H, B, arr, _fp(x), _fp(h_prev), _fp(c_prev), _fp(htild), _ip(mask), _fp(h), _fp(c))
    return h, c


def attention(att_type, H, B, D, w6, h_t, mask, hs_all, S_max, lens, offs):
    keep = [_f32(a).reshape(-1) for a in w6]
    arr = (c_float_p * 6)(*[_fp(a) for a in keep])
    h_t, hs_all = _f32(h_t).reshape(-1), _f32(hs_all).reshape(-1)
    mask, lens, offs = _i32(mask), _i32(lens), _i32(offs)
    out = np.zeros(H * B, dtype=np.float32)
    n_al = (2 * D + 1) * B if att_type == 1 else S_max * B
    al = np.zeros(n_al, dtype=np.float32)
    idx = np.full(n_al, -1, dtype=np.int32)
    lib().orc_attention(att_type, H, B, D, arr, _fp(h_t), _ip(mask), _fp(hs_all), S_max, _ip(lens), _ip(offs),
                        _fp(out), _fp(al), _ip(idx) if att_type == 1 else None)
    return out, al, idx


def attention_viterbi(att_type, H, B, D, w6, h_t, mask, hs_all, S_max, lens, offs):
    """The attention step's viterbi alignment per column (get_viterbi_alignment_kernel)."""
    keep = [_f32(a).reshape(-1) for a in w6]
    arr = (c_float_p * 6)(*[_fp(a) for a in keep])
    h_t, hs_all = _f32(h_t).reshape(-1), _f32(hs_all).reshape(-1)
    mask, lens, offs = _i32(mask), _i32(lens), _i32(offs)
    out = np.zeros(H * B, dtype=np.float32)
    vit = np.zeros(B, dtype=np.int32)
    lib().orc_attention_viterbi(att_type, H, B, D, arr, _fp(h_t), _ip(mask), _fp(hs_all), S_max, _ip(lens), _ip(offs),
                                _fp(out), _ip(vit))
    return out, vit


def softmax_logp(V, H, N, Dm, b_d, h, target, want_all=False):
    Dm, b_d, h, target = _f32(Dm).reshape(-1), _f32(b_d).reshape(-1), _f32(h).reshape(-1), _i32(target)
    lp = np.zeros(N, dtype=np.float64)
    allp = np.zeros(V * N, dtype=np.float64) if want_all else None
    lib().orc_softmax_logp(V, H, N, _fp(Dm), _fp(b_d), _fp(h), _ip(target), lp.ctypes.data_as(c_double_p),
                           allp.ctypes.data_as(c_double_p) if want_all else None)
    return (lp, allp) if want_all else lp


def softmax_dist(V, H, N, Dm, b_d, h):
    Dm, b_d, h = _f32(Dm).reshape(-1), _f32(b_d).reshape(-1), _f32(h).reshape(-1)
    p = np.zeros(V * N, dtype=np.float32)
    lib().orc_softmax_dist(V, H, N, _fp(Dm), _fp(b_d), _fp(h), _fp(p))
    return p


def set_acc_float(on):
    """GEMM accumulation of the oracle: False / 0 = double (the default), True / 1 = float with k ascending (the
    reference's SGEMM arithmetic in its plainest order), 2 = float with k descending, 3 = float in blocks of 32."""
    lib().orc_set_acc_float(int(on))


def fp32_noise_floor(score, want=None):
    """Largest relative deviation of `score()` (a callable returning log-probs) over the float summation orders from
    its double-accumulating result: how far a correct fp32 implementation may sit from the oracle on this input.
    Returns (floor, want)."""
    set_acc_float(0)
    if want is None:
        want = score()
    floor = 0.0
    try:
        for mode in (1, 2, 3):
            set_acc_float(mode)
            got = score()
            nz = np.abs(want) > 0
            floor = max(floor, float((np.abs(got - want)[nz] / np.abs(want)[nz]).max()))
    finally:
        set_acc_float(0)
    return floor, want


def num_threads():
    return lib().orc_num_threads()


def set_num_threads(n):
    """Number of OpenMP threads the oracle's GEMMs use (launchers such as torchrun export OMP_NUM_THREADS=1)."""
    lib().orc_set_num_threads(int(n))
