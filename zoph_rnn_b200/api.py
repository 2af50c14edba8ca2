"""Host-side mirror of the reference's layer API over the C ABI (include/zrnn.h).

Class and method names follow the reference's C++ classes (Input_To_Hidden_Layer,
Hidden_To_Hidden_Layer, attention_layer, softmax_layer, neuralMT_model) so that tests read like
calls into the reference.  PyTorch is used only to own device memory and streams; every bit of
arithmetic happens inside libzrnn.so.
"""
import ctypes

import numpy as np
import torch

from . import _lib
from ._lib import (ATT_GLOBAL_DOT, ATT_LOCAL_P, ATT_NONE, BF16, F32, F32_3XTF32, F32_F16X2, F32_SIMT, TF32,  # noqa: F401
                   ModelConfig,
                   ZrnnError, check, lib)


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


def _host_list(tensors):
    keep = [_f32(t) for t in tensors]
    arr = (_lib.c_float_p * len(keep))(*[k.ctypes.data_as(_lib.c_float_p) for k in keep])
    return keep, arr


def _dev_i32(a):
    return torch.as_tensor(np.ascontiguousarray(a, dtype=np.int32)).cuda()


def prep_vocab_indices(ids_raw):
    """ids with -1 padding (int32 CUDA tensor) -> (ids with -1 replaced by 0, 0/1 mask).
    Mirrors Input_To_Hidden_Layer::prep_GPU_vocab_indices (src/Input_To_Hidden_Layer.hpp:1178-1225)."""
    ids = torch.empty_like(ids_raw)
    mask = torch.empty_like(ids_raw)
    check(lib().zrnn_prep_vocab_indices(_ptr(ids_raw), ids_raw.numel(), _ptr(ids), _ptr(mask), _stream()))
    return ids, mask


def gemm(W, X, n_rows, m_cols, K, mode=0):
    """C = W * X (column-major flat CUDA tensors), the reference's cublas_gemm_wrapper N/N case.
    mode 0 fp32 FMA, 1 bf16 tensor cores, 2 tf32, 3 3xTF32."""
    C = torch.empty(n_rows * m_cols, dtype=torch.float32, device="cuda")
    check(lib().zrnn_gemm(mode, n_rows, m_cols, K, _ptr(W), n_rows, _ptr(X), K, _ptr(C), n_rows, _stream()))
    return C


class _LstmLayer:
    def __init__(self):
        self._h = ctypes.c_void_p()

    def load_weights(self, tensors):
        """tensors in the reference's file order (see zrnn_lstm_load in include/zrnn.h)."""
        keep, arr = _host_list(tensors)
        check(lib().zrnn_lstm_load(self._h, arr, len(keep)))

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                lib().zrnn_lstm_destroy(self._h)
                self._h = None
        except TypeError:  # interpreter shutdown: module globals are already gone
            pass


class Input_To_Hidden_Layer(_LstmLayer):
    """Layer 0: embedding gather + LSTM (src/Input_To_Hidden_Layer.h:146-203)."""

    def __init__(self, LSTM_size, input_vocab_size, feed_input=False, dtype=F32):
        super().__init__()
        self.H, self.V, self.feed_input = LSTM_size, input_vocab_size, bool(feed_input)
        check(lib().zrnn_ih_create(LSTM_size, input_vocab_size, int(feed_input), dtype, ctypes.byref(self._h)))

    def gather(self, ids_nonm1):
        x = torch.empty(ids_nonm1.numel() * self.H, dtype=torch.float32, device="cuda")
        check(lib().zrnn_ih_gather(self._h, _ptr(ids_nonm1), ids_nonm1.numel(), _ptr(x), _stream()))
        return x

    def forward_prop(self, ids_nonm1, mask01, h_prev, c_prev, h_tild_prev=None):
        """LSTM_IH_Node::forward_prop (src/LSTM.hpp:76-421). Tensors are flat column-major H x B."""
        B = ids_nonm1.numel()
        h, c = torch.empty_like(h_prev), torch.empty_like(c_prev)
        check(lib().zrnn_ih_forward(self._h, _ptr(ids_nonm1), _ptr(mask01), _ptr(h_prev), _ptr(c_prev),
                                    _ptr(h_tild_prev), B, _ptr(h), _ptr(c), _stream()))
        return h, c


class Hidden_To_Hidden_Layer(_LstmLayer):
    """Layers >= 1 (src/Hidden_To_Hidden_Layer.h:138-177)."""

    def __init__(self, LSTM_size, dtype=F32):
        super().__init__()
        self.H = LSTM_size
        check(lib().zrnn_hh_create(LSTM_size, dtype, ctypes.byref(self._h)))

    def forward_prop(self, h_below, mask01, h_prev, c_prev):
        """LSTM_HH_Node::forward_prop (src/LSTM_HH.hpp:103-333)."""
        B = h_prev.numel() // self.H
        h, c = torch.empty_like(h_prev), torch.empty_like(c_prev)
        check(lib().zrnn_hh_forward(self._h, _ptr(h_below), _ptr(mask01), _ptr(h_prev), _ptr(c_prev), B, _ptr(h),
                                    _ptr(c), _stream()))
        return h, c


class attention_layer:
    """src/attention_layer.h:28-33; att_type ATT_LOCAL_P (the reference's model) or ATT_GLOBAL_DOT."""

    def __init__(self, LSTM_size, D, att_type=ATT_LOCAL_P, dtype=F32):
        self._h = ctypes.c_void_p()
        self.H, self.D, self.att_type = LSTM_size, D, att_type
        self._keep = None
        check(lib().zrnn_att_create(LSTM_size, D, att_type, dtype, ctypes.byref(self._h)))

    def load_weights(self, tensors):
        keep, arr = _host_list(tensors)
        check(lib().zrnn_att_load(self._h, arr, len(keep)))

    def prep_minibatch_info(self, hs, S_max, B_src, lens, offsets, cols_per_sentence=1):
        """attention_layer::prep_minibatch_info (src/attention_layer.hpp:580-583) + the source-state table."""
        self._keep = (hs, lens, offsets)
        self.S_max = S_max
        check(lib().zrnn_att_set_source(self._h, _ptr(hs), S_max, B_src, _ptr(lens), _ptr(offsets), cols_per_sentence))

    def forward_prop(self, h_t, mask01, want_alignments=False):
        """attention_node::forward_prop (src/attention_node.hpp:73-394)."""
        B = h_t.numel() // self.H
        out = torch.empty_like(h_t)
        al = None
        if want_alignments:
            n = (2 * self.D + 1) * B if self.att_type == ATT_LOCAL_P else self.S_max * B
            al = torch.zeros(n, dtype=torch.float32, device="cuda")
        check(lib().zrnn_att_forward(self._h, _ptr(h_t), _ptr(mask01), B, _ptr(out), _ptr(al), _stream()))
        return (out, al) if want_alignments else out

    def forward_prop_viterbi(self, h_t, mask01):
        """forward_prop plus get_viterbi_alignment_kernel (src/custom_kernels.h:1621-1635): returns
        (h_tilde, viterbi [B] int32)."""
        B = h_t.numel() // self.H
        out = torch.empty_like(h_t)
        vit = torch.zeros(B, dtype=torch.int32, device="cuda")
        check(lib().zrnn_att_forward_viterbi(self._h, _ptr(h_t), _ptr(mask01), B, _ptr(out), _ptr(vit), _stream()))
        return out, vit

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                lib().zrnn_att_destroy(self._h)
                self._h = None
        except TypeError:
            pass


class softmax_layer:
    """src/softmax.hpp; rows [shard_lo, shard_hi) of D for vocabulary sharding."""

    def __init__(self, output_vocab_size, LSTM_size, dtype=F32, shard_lo=0, shard_hi=None, _borrowed=None):
        self.V, self.H = output_vocab_size, LSTM_size
        self.lo, self.hi = shard_lo, output_vocab_size if shard_hi is None else shard_hi
        self._owned = _borrowed is None
        if _borrowed is not None:
            self._h = ctypes.c_void_p(_borrowed)
        else:
            self._h = ctypes.c_void_p()
            check(lib().zrnn_softmax_create(self.V, self.H, dtype, self.lo, self.hi, ctypes.byref(self._h)))

    def load_weights(self, D, b_d):
        D, b_d = _f32(D), _f32(b_d)
        check(lib().zrnn_softmax_load(self._h, D.ctypes.data_as(_lib.c_float_p), b_d.ctypes.data_as(_lib.c_float_p)))

    def compute_loss(self, h, targets, mask01):
        """get_perplexity_GPU + compute_loss_GPU (src/softmax.hpp:636-692, 867-900): ln p(target) per column."""
        N = targets.numel()
        out = torch.empty(N, dtype=torch.float32, device="cuda")
        check(lib().zrnn_softmax_score(self._h, _ptr(h), _ptr(targets), _ptr(mask01), N, _ptr(out), _stream()))
        return out

    def compute_loss_noalloc(self, h, targets, mask01, out):
        """compute_loss for callers that may not allocate: scratch comes from the library's built-in array and
        the result goes into the caller's `out` tensor (see zrnn_softmax_score_noalloc in include/zrnn.h)."""
        check(lib().zrnn_softmax_score_noalloc(self._h, _ptr(h), _ptr(targets), _ptr(mask01), targets.numel(),
                                               _ptr(out), _stream()))
        return out

    def partials(self, h, targets):
        N = targets.numel()
        mx, sm, tg = (torch.empty(N, dtype=torch.float32, device="cuda") for _ in range(3))
        check(lib().zrnn_softmax_partials(self._h, _ptr(h), _ptr(targets), N, _ptr(mx), _ptr(sm), _ptr(tg), _stream()))
        return mx, sm, tg

    @staticmethod
    def combine(mx, sm, tg, mask01):
        """mx/sm/tg: [G, N] shard-major CUDA tensors."""
        G, N = mx.shape
        out = torch.empty(N, dtype=torch.float32, device="cuda")
        check(lib().zrnn_softmax_combine(_ptr(mx.contiguous()), _ptr(sm.contiguous()), _ptr(tg.contiguous()), G, N,
                                         _ptr(mask01), _ptr(out), _stream()))
        return out

    def topk(self, h, k):
        """get_distribution_GPU + per-column pre-selection (src/softmax.hpp:514-632, src/decoder.h:1197-1219)."""
        N = h.numel() // self.H
        val = torch.empty(N * k, dtype=torch.float32, device="cuda")
        idx = torch.empty(N * k, dtype=torch.int32, device="cuda")
        eos = torch.empty(N, dtype=torch.float32, device="cuda")
        check(lib().zrnn_softmax_topk(self._h, _ptr(h), N, k, _ptr(val), _ptr(idx), _ptr(eos), _stream()))
        return val.view(N, k), idx.view(N, k), eos

    def topk_shard(self, h, k):
        """This layer's rows only: (logp [N,k] under the layer's own normaliser, local row ids [N,k], lse [N],
        <EOF> value [N] or -inf)."""
        N = h.numel() // self.H
        val = torch.empty(N * k, dtype=torch.float32, device="cuda")
        idx = torch.empty(N * k, dtype=torch.int32, device="cuda")
        lse = torch.empty(N, dtype=torch.float32, device="cuda")
        eos = torch.empty(N, dtype=torch.float32, device="cuda")
        check(lib().zrnn_softmax_topk_shard(self._h, _ptr(h), N, k, _ptr(val), _ptr(idx), _ptr(lse), _ptr(eos), _stream()))
        return val.view(N, k), idx.view(N, k), lse, eos

    @staticmethod
    def merge_topk(val, idx, lse, eos, shard_lo):
        """val / idx [G,N,k], lse / eos [G,N] CUDA tensors and the shards' first word ids -> what topk() of the whole
        vocabulary returns."""
        G, N, k = val.shape
        lo = torch.as_tensor(np.asarray(shard_lo, dtype=np.int32), device="cuda")
        oval = torch.empty(N * k, dtype=torch.float32, device="cuda")
        oidx = torch.empty(N * k, dtype=torch.int32, device="cuda")
        oeos = torch.empty(N, dtype=torch.float32, device="cuda")
        check(lib().zrnn_topk_merge(_ptr(val.contiguous()), _ptr(idx.contiguous()), _ptr(lse.contiguous()),
                                    _ptr(eos.contiguous()), _ptr(lo), G, N, k, _ptr(oval), _ptr(oidx), _ptr(oeos),
                                    _stream()))
        return oval.view(N, k), oidx.view(N, k), oeos

    def topk_sharded(self, comm, h, k):
        """topk() of the whole vocabulary over the ranks of `comm` (a Communicator); this layer holds the rank's rows."""
        N = h.numel() // self.H
        val = torch.empty(N * k, dtype=torch.float32, device="cuda")
        idx = torch.empty(N * k, dtype=torch.int32, device="cuda")
        eos = torch.empty(N, dtype=torch.float32, device="cuda")
        check(lib().zrnn_softmax_topk_sharded(self._h, comm._h, _ptr(h), N, k, _ptr(val), _ptr(idx), _ptr(eos), _stream()))
        return val.view(N, k), idx.view(N, k), eos

    def __del__(self):
        try:
            if getattr(self, "_h", None) and self._owned:
                lib().zrnn_softmax_destroy(self._h)
            self._h = None
        except TypeError:
            pass


def shard_range(V, world, rank):
    """Rows of the output vocabulary that rank `rank` of `world` holds."""
    lo, hi = ctypes.c_int(), ctypes.c_int()
    check(lib().zrnn_shard_range(V, world, rank, ctypes.byref(lo), ctypes.byref(hi)))
    return lo.value, hi.value


class Communicator:
    """The library's collective layer (NCCL behind the C ABI).  `Communicator.unique_id()` on rank 0, the 128 bytes
    to every rank by any host channel, then `Communicator(id, rank, world)` on every rank; world == 1 needs no id."""

    def __init__(self, unique_id, rank, world):
        self._h = ctypes.c_void_p()
        self.rank, self.world = rank, world
        check(lib().zrnn_comm_create(unique_id, rank, world, ctypes.byref(self._h)))

    @staticmethod
    def unique_id():
        buf = ctypes.create_string_buffer(128)
        check(lib().zrnn_comm_unique_id(buf))
        return buf.raw

    @classmethod
    def from_torch_distributed(cls, group=None):
        """One communicator per rank of an initialised torch.distributed group (the id travels through it)."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [cls.unique_id() if rank == 0 and world > 1 else None]
        if world > 1:
            dist.broadcast_object_list(box, src=0, group=group)
        return cls(box[0], rank, world)

    def all_gather(self, send, recv):
        check(lib().zrnn_comm_all_gather(self._h, _ptr(send), _ptr(recv), send.numel() * send.element_size(), _stream()))
        return recv

    STAGES = ("stack", "gather_states", "vocab_rows", "gather_partials_combine", "d2h")

    def last_stage_ms(self):
        """Device time of the stages of this rank's last sharded scoring call."""
        ms = (ctypes.c_float * 5)()
        check(lib().zrnn_comm_last_stage_ms(self._h, ms))
        return dict(zip(self.STAGES, [float(x) for x in ms]))

    def close(self):
        if getattr(self, "_h", None):
            lib().zrnn_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except TypeError:
            pass


class neuralMT_model:
    """src/model.h: the whole model.  cfg is a dict with keys num_layers, H, V_src, V_tgt, lm, attention,
    feed_input, D (zoph_rnn_b200.synth.make_cfg builds one)."""

    def __init__(self, cfg=None, dtype=F32, _handle=None, shard=None):
        """shard = (lo, hi): keep only those rows of the softmax on this GPU (see shard_range, Communicator)."""
        self._h = ctypes.c_void_p()
        self.shard = shard
        if _handle is not None:
            self._h = _handle
            c = ModelConfig()
            check(lib().zrnn_model_get_config(self._h, ctypes.byref(c)))
            self.cfg = {k: getattr(c, k) for k, _ in ModelConfig._fields_}
        else:
            c = ModelConfig(cfg["num_layers"], cfg["H"], cfg["V_src"], cfg["V_tgt"], cfg["lm"], cfg["attention"],
                            cfg["feed_input"], cfg["D"], dtype)
            if shard is None:
                check(lib().zrnn_model_create(ctypes.byref(c), ctypes.byref(self._h)))
            else:
                check(lib().zrnn_model_create_sharded(ctypes.byref(c), shard[0], shard[1], ctypes.byref(self._h)))
            self.cfg = dict(cfg, dtype=dtype)

    @classmethod
    def from_file(cls, path, att_type=ATT_LOCAL_P, D=10, dtype=F32):
        """neuralMT_model::load_weights (src/model.hpp:2172-2241) from a text model.nn."""
        h = ctypes.c_void_p()
        check(lib().zrnn_model_load_file(str(path).encode(), att_type, D, dtype, ctypes.byref(h)))
        return cls(_handle=h)

    @classmethod
    def from_file_sharded(cls, path, comm, att_type=ATT_LOCAL_P, D=10, dtype=F32):
        """from_file for one rank of a vocabulary-sharded group (comm: a Communicator)."""
        h = ctypes.c_void_p()
        check(lib().zrnn_model_load_file_sharded(str(path).encode(), att_type, D, dtype, comm.world, comm.rank,
                                                 ctypes.byref(h)))
        m = cls(_handle=h)
        m.shard = shard_range(m.cfg["V_tgt"], comm.world, comm.rank)
        return m

    def tensor_spec(self):
        out = []
        for i in range(lib().zrnn_model_num_tensors(self._h)):
            name = ctypes.create_string_buffer(32)
            r, c = ctypes.c_int(), ctypes.c_int()
            check(lib().zrnn_model_tensor_info(self._h, i, name, ctypes.byref(r), ctypes.byref(c)))
            out.append((name.value.decode(), r.value, c.value))
        return out

    def load_weights(self, tensors):
        for i, t in enumerate(tensors):
            t = _f32(t)
            check(lib().zrnn_model_set_tensor(self._h, i, t.ctypes.data_as(_lib.c_float_p)))
        check(lib().zrnn_model_finalize(self._h))

    def get_error(self, src_ids, tgt_in, tgt_out):
        """neuralMT_model::getError (src/model.hpp:1463-1802) through the host-buffer entry point.
        Arrays are [S,B] / [T,B] int32 (NumPy, or pinned CPU torch tensors).  Returns (logp [T,B], total)."""
        def host(a):
            if a is None:
                return None, None
            if isinstance(a, torch.Tensor):
                return a, ctypes.c_void_p(a.data_ptr())
            a = np.ascontiguousarray(a, dtype=np.int32)
            return a, ctypes.c_void_p(a.ctypes.data)
        ks, ps = host(src_ids)
        ki, pi = host(tgt_in)
        ko, po = host(tgt_out)
        T, B = ki.shape
        S = ks.shape[0] if ks is not None else 0
        out = np.empty((T, B), dtype=np.float32)
        tot = ctypes.c_double()
        check(lib().zrnn_score_batch(self._h, ps, S, pi, po, T, B, ctypes.c_void_p(out.ctypes.data), ctypes.byref(tot)))
        return out, tot.value

    def get_error_sharded(self, comm, src_ids, tgt_in, tgt_out):
        """get_error over the ranks of `comm` for a model created with shard=...; every rank passes the same batch
        and receives the whole (logp [T,B], total)."""
        ks = None if src_ids is None else np.ascontiguousarray(src_ids, dtype=np.int32)
        ki = np.ascontiguousarray(tgt_in, dtype=np.int32)
        ko = np.ascontiguousarray(tgt_out, dtype=np.int32)
        T, B = ki.shape
        S = ks.shape[0] if ks is not None else 0
        out = np.empty((T, B), dtype=np.float32)
        tot = ctypes.c_double()
        check(lib().zrnn_score_batch_sharded(self._h, comm._h, None if ks is None else ctypes.c_void_p(ks.ctypes.data), S,
                                             ctypes.c_void_p(ki.ctypes.data), ctypes.c_void_p(ko.ctypes.data), T, B,
                                             ctypes.c_void_p(out.ctypes.data), ctypes.byref(tot)))
        return out, tot.value

    def decode_sharded(self, comm, sources, beam=12, k_best=1, min_ratio=0.5, max_ratio=1.5, penalty=0.0,
                       longest_sent=100):
        """decode() with the softmax's pre-selection sharded over the ranks of `comm`; every rank gets the result."""
        n = len(sources)
        Lmax = longest_sent + 4
        ids = np.empty((n, k_best, Lmax), dtype=np.int32)
        ln = np.empty((n, k_best), dtype=np.int32)
        sc = np.empty((n, k_best), dtype=np.float32)
        if n == 0:
            return ids, ln, sc
        flat = np.ascontiguousarray(np.concatenate([np.asarray(s, dtype=np.int32) for s in sources]), dtype=np.int32)
        lens = np.ascontiguousarray([len(s) for s in sources], dtype=np.int32)
        check(lib().zrnn_beam_decode_batch_sharded(self._h, comm._h, ctypes.c_void_p(flat.ctypes.data),
                                                   ctypes.c_void_p(lens.ctypes.data), n, beam, k_best, min_ratio,
                                                   max_ratio, penalty, longest_sent, ctypes.c_void_p(ids.ctypes.data),
                                                   ctypes.c_void_p(ln.ctypes.data), ctypes.c_void_p(sc.ctypes.data)))
        return ids, ln, sc

    def get_error_device(self, d_src, S, d_tin, d_tout, T, B, d_logp):
        """Device-resident variant: int32 CUDA tensors in, float32 CUDA tensor out, asynchronous."""
        check(lib().zrnn_score_batch_device(self._h, _ptr(d_src), S, _ptr(d_tin), _ptr(d_tout), T, B, _ptr(d_logp),
                                            _stream()))

    def forward_states_device(self, d_src, S, d_tin, T, B, d_top):
        """Recurrent stack only: fills d_top (float32 CUDA tensor, H x (T*B) column-major) and skips the softmax."""
        check(lib().zrnn_forward_states_device(self._h, _ptr(d_src), S, _ptr(d_tin), T, B, _ptr(d_top), _stream()))

    def last_top_states(self):
        """The vectors the last scoring call handed to the softmax, flat column-major H x (T*B)."""
        n = ctypes.c_int()
        check(lib().zrnn_model_copy_top_states(self._h, None, 0, ctypes.byref(n), None))
        out = torch.empty(n.value * self.cfg["H"], dtype=torch.float32, device="cuda")
        check(lib().zrnn_model_copy_top_states(self._h, _ptr(out), n.value, ctypes.byref(n), _stream()))
        return out

    def softmax(self):
        return softmax_layer(self.cfg["V_tgt"], self.cfg["H"], _borrowed=lib().zrnn_model_softmax(self._h))

    def decode(self, sources, beam=12, k_best=1, min_ratio=0.5, max_ratio=1.5, penalty=0.0, longest_sent=100,
               want_align=False):
        """ensemble_factory::decode_file_batch (src/ensemble_factory.hpp:583-765) for a list of reversed source
        id arrays.  Returns (ids [n,k,longest_sent+4], len [n,k], score [n,k]); with want_align also the viterbi
        alignment stored with every hypothesis position [n,k,longest_sent+4] (src/decoder.h:1266-1267)."""
        n = len(sources)
        Lmax = longest_sent + 4
        if n == 0:
            empty = (np.empty((0, k_best, Lmax), np.int32), np.empty((0, k_best), np.int32),
                     np.empty((0, k_best), np.float32))
            return empty + (np.empty((0, k_best, Lmax), np.int32),) if want_align else empty
        flat = np.ascontiguousarray(np.concatenate([np.asarray(s, dtype=np.int32) for s in sources]), dtype=np.int32)
        lens = np.ascontiguousarray([len(s) for s in sources], dtype=np.int32)
        ids = np.empty((n, k_best, Lmax), dtype=np.int32)
        ln = np.empty((n, k_best), dtype=np.int32)
        sc = np.empty((n, k_best), dtype=np.float32)
        if want_align:
            al = np.empty((n, k_best, Lmax), dtype=np.int32)
            check(lib().zrnn_beam_decode_batch_align(self._h, ctypes.c_void_p(flat.ctypes.data),
                                                     ctypes.c_void_p(lens.ctypes.data), n, beam, k_best, min_ratio,
                                                     max_ratio, penalty, longest_sent, ctypes.c_void_p(ids.ctypes.data),
                                                     ctypes.c_void_p(ln.ctypes.data), ctypes.c_void_p(sc.ctypes.data),
                                                     ctypes.c_void_p(al.ctypes.data)))
            return ids, ln, sc, al
        check(lib().zrnn_beam_decode_batch(self._h, ctypes.c_void_p(flat.ctypes.data), ctypes.c_void_p(lens.ctypes.data),
                                           n, beam, k_best, min_ratio, max_ratio, penalty, longest_sent,
                                           ctypes.c_void_p(ids.ctypes.data), ctypes.c_void_p(ln.ctypes.data),
                                           ctypes.c_void_p(sc.ctypes.data)))
        return ids, ln, sc

    def decode_device(self, d_src_padded, src_lens, S_max, beam, k_best, min_ratio, max_ratio, penalty, longest_sent,
                      d_ids, d_len, d_score):
        lens = np.ascontiguousarray(src_lens, dtype=np.int32)
        check(lib().zrnn_beam_decode_batch_device(self._h, _ptr(d_src_padded), ctypes.c_void_p(lens.ctypes.data), S_max,
                                                  len(lens), beam, k_best, min_ratio, max_ratio, penalty, longest_sent,
                                                  _ptr(d_ids), _ptr(d_len), _ptr(d_score), _stream()))

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                lib().zrnn_model_destroy(self._h)
                self._h = None
        except TypeError:
            pass


def decode_ensemble(models, sources_per_model, beam=12, k_best=1, min_ratio=0.5, max_ratio=1.5, penalty=0.0,
                    longest_sent=100, want_align=False):
    """ensemble_factory decoding with several models (src/ensemble_factory.hpp:583-795): sources_per_model[k] is the
    k-th model's list of reversed source id arrays.  Returns (ids [n,k,longest_sent+4], len [n,k], score [n,k])."""
    K, n = len(models), len(sources_per_model[0])
    flats = [np.ascontiguousarray(np.concatenate([np.asarray(s, dtype=np.int32) for s in srcs]), dtype=np.int32)
             for srcs in sources_per_model]
    lens = [np.ascontiguousarray([len(s) for s in srcs], dtype=np.int32) for srcs in sources_per_model]
    Lmax = longest_sent + 4
    ids = np.empty((n, k_best, Lmax), dtype=np.int32)
    ln = np.empty((n, k_best), dtype=np.int32)
    sc = np.empty((n, k_best), dtype=np.float32)
    hs = (ctypes.c_void_p * K)(*[m._h.value if isinstance(m._h, ctypes.c_void_p) else m._h for m in models])
    fp = (ctypes.c_void_p * K)(*[f.ctypes.data for f in flats])
    lp = (ctypes.c_void_p * K)(*[l.ctypes.data for l in lens])
    if want_align:  # alignment voting over the models (src/ensemble_factory.hpp:798-834)
        al = np.empty((n, k_best, Lmax), dtype=np.int32)
        check(lib().zrnn_beam_decode_ensemble_align(hs, K, fp, lp, n, beam, k_best, min_ratio, max_ratio, penalty,
                                                    longest_sent, ctypes.c_void_p(ids.ctypes.data),
                                                    ctypes.c_void_p(ln.ctypes.data), ctypes.c_void_p(sc.ctypes.data),
                                                    ctypes.c_void_p(al.ctypes.data)))
        return ids, ln, sc, al
    check(lib().zrnn_beam_decode_ensemble(hs, K, fp, lp, n, beam, k_best, min_ratio, max_ratio, penalty, longest_sent,
                                          ctypes.c_void_p(ids.ctypes.data), ctypes.c_void_p(ln.ctypes.data),
                                          ctypes.c_void_p(sc.ctypes.data)))
    return ids, ln, sc


def read_model_file_header(path):
    """(header ints [9], how many the file carried, source vocabulary lines, target vocabulary lines) of a
    model.nn, parsed on the host (src/add_model_info.h:7-9)."""
    hdr = (ctypes.c_int * 9)()
    n, ns, nt = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    check(lib().zrnn_model_file_header(str(path).encode(), hdr, ctypes.byref(n), ctypes.byref(ns), ctypes.byref(nt)))
    return list(hdr), n.value, ns.value, nt.value


def read_model_file(path, shapes):
    """Parses the first len(shapes) matrices ((rows, cols) in file order) of a model.nn on the host and returns
    them as flat column-major float32 arrays: read_matrix_GPU without the upload (src/Eigen_Util.h:83-112)."""
    n = len(shapes)
    rows = (ctypes.c_int * n)(*[int(r) for r, _ in shapes])
    cols = (ctypes.c_int * n)(*[int(c) for _, c in shapes])
    outs = [np.empty(int(r) * int(c), dtype=np.float32) for r, c in shapes]
    ptrs = (ctypes.c_void_p * n)(*[o.ctypes.data for o in outs])
    check(lib().zrnn_model_file_read(str(path).encode(), n, rows, cols, ptrs))
    return outs


def launch_count():
    return lib().zrnn_launch_count()


def reset_launch_count():
    lib().zrnn_reset_launch_count()


KERNEL_CLASSES = ("gather", "lstm_cell", "attention", "softmax_gemm", "softmax_reduce", "beam_step", "state_reorder")


def kernel_timing_report():
    """{class name: {"launches": n, "ms": total}} for the classes that ran while zrnn_kernel_timing was on."""
    out = {}
    for i, name in enumerate(KERNEL_CLASSES):
        n, ms = ctypes.c_longlong(), ctypes.c_double()
        check(lib().zrnn_kernel_timing_read(i, ctypes.byref(n), ctypes.byref(ms)))
        if n.value:
            out[name] = dict(launches=n.value, ms=ms.value)
    return out
