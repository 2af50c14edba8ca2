"""ctypes loader for libzrnn.so (the C-ABI library declared in include/zrnn.h).

There is no CPU or PyTorch fallback: if the library is missing the import of any compute
entry point fails loudly.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libzrnn.so")

c_int_p = ctypes.POINTER(ctypes.c_int)
c_float_p = ctypes.POINTER(ctypes.c_float)
c_void_p = ctypes.c_void_p

OK, E_ARG, E_CUDA, E_NCCL, E_TIMEOUT, E_IO, E_STATE = range(7)
F32, BF16, TF32, F32_SIMT, F32_3XTF32, F32_F16X2 = 0, 1, 2, 3, 4, 5
ATT_NONE, ATT_LOCAL_P, ATT_GLOBAL_DOT = 0, 1, 2


class ModelConfig(ctypes.Structure):
    _fields_ = [(k, ctypes.c_int) for k in
                ("num_layers", "H", "V_src", "V_tgt", "lm", "attention", "feed_input", "D", "dtype")]


class ZrnnError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"zrnn status {status}: {message}")
        self.status = status


# name -> (restype, argtypes); every symbol include/zrnn.h and include/zrnn_debug.h declare
SIGNATURES = {
    "zrnn_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "zrnn_last_error": (ctypes.c_char_p, []),
    "zrnn_version": (ctypes.c_int, []),
    "zrnn_built_for_sm": (ctypes.c_int, []),
    "zrnn_debug_tc_profile": (ctypes.c_int, [c_void_p]),
    "zrnn_debug_tc_timeline": (ctypes.c_int, [c_void_p, ctypes.c_int]),
    "zrnn_debug_decoder_timeline": (ctypes.c_int, [c_void_p, ctypes.c_int]),
    "zrnn_debug_bounded_wait": (ctypes.c_int, [ctypes.c_longlong, c_void_p]),
    "zrnn_device_count": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int)]),
    "zrnn_set_device": (ctypes.c_int, [ctypes.c_int]),
    "zrnn_launch_count": (ctypes.c_longlong, []),
    "zrnn_reset_launch_count": (None, []),
    "zrnn_kernel_timing": (ctypes.c_int, [ctypes.c_int]),
    "zrnn_kernel_timing_read": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(ctypes.c_longlong),
                                               ctypes.POINTER(ctypes.c_double)]),
    "zrnn_gemm": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, c_void_p, ctypes.c_int,
                                 c_void_p, ctypes.c_int, c_void_p, ctypes.c_int, c_void_p]),
    "zrnn_tc_error": (ctypes.c_int, []),
    "zrnn_prep_vocab_indices": (ctypes.c_int, [c_void_p, ctypes.c_int, c_void_p, c_void_p, c_void_p]),
    "zrnn_ih_create": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(c_void_p)]),
    "zrnn_hh_create": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.POINTER(c_void_p)]),
    "zrnn_lstm_load": (ctypes.c_int, [c_void_p, ctypes.POINTER(c_float_p), ctypes.c_int]),
    "zrnn_ih_gather": (ctypes.c_int, [c_void_p, c_void_p, ctypes.c_int, c_void_p, c_void_p]),
    "zrnn_ih_forward": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_int,
                                       c_void_p, c_void_p, c_void_p]),
    "zrnn_hh_forward": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_int, c_void_p,
                                       c_void_p, c_void_p]),
    "zrnn_lstm_destroy": (ctypes.c_int, [c_void_p]),
    "zrnn_att_create": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(c_void_p)]),
    "zrnn_att_load": (ctypes.c_int, [c_void_p, ctypes.POINTER(c_float_p), ctypes.c_int]),
    "zrnn_att_set_source": (ctypes.c_int, [c_void_p, c_void_p, ctypes.c_int, ctypes.c_int, c_void_p, c_void_p,
                                           ctypes.c_int]),
    "zrnn_att_forward": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_int, c_void_p, c_void_p, c_void_p]),
    "zrnn_att_forward_viterbi": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_int, c_void_p, c_void_p,
                                                c_void_p]),
    "zrnn_att_destroy": (ctypes.c_int, [c_void_p]),
    "zrnn_softmax_create": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                           ctypes.POINTER(c_void_p)]),
    "zrnn_softmax_load": (ctypes.c_int, [c_void_p, c_float_p, c_float_p]),
    "zrnn_softmax_score": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_int, c_void_p, c_void_p]),
    "zrnn_softmax_score_noalloc": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_int, c_void_p,
                                                  c_void_p]),
    "zrnn_softmax_score_noalloc_max_floats": (ctypes.c_int, []),
    "zrnn_softmax_partials": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_int, c_void_p, c_void_p, c_void_p,
                                             c_void_p]),
    "zrnn_softmax_combine": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_int, ctypes.c_int, c_void_p,
                                            c_void_p, c_void_p]),
    "zrnn_softmax_topk": (ctypes.c_int, [c_void_p, c_void_p, ctypes.c_int, ctypes.c_int, c_void_p, c_void_p, c_void_p,
                                         c_void_p]),
    "zrnn_softmax_destroy": (ctypes.c_int, [c_void_p]),
    "zrnn_comm_unique_id": (ctypes.c_int, [ctypes.c_char_p]),
    "zrnn_comm_create": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(c_void_p)]),
    "zrnn_comm_from_nccl": (ctypes.c_int, [c_void_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(c_void_p)]),
    "zrnn_comm_rank": (ctypes.c_int, [c_void_p, c_int_p, c_int_p]),
    "zrnn_comm_all_gather": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_size_t, c_void_p]),
    "zrnn_comm_last_stage_ms": (ctypes.c_int, [c_void_p, c_float_p]),
    "zrnn_comm_destroy": (ctypes.c_int, [c_void_p]),
    "zrnn_shard_range": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, c_int_p, c_int_p]),
    "zrnn_softmax_topk_shard": (ctypes.c_int, [c_void_p, c_void_p, ctypes.c_int, ctypes.c_int, c_void_p, c_void_p,
                                               c_void_p, c_void_p, c_void_p]),
    "zrnn_topk_merge": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_int, ctypes.c_int,
                                       ctypes.c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "zrnn_softmax_topk_sharded": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_int, ctypes.c_int, c_void_p,
                                                 c_void_p, c_void_p, c_void_p]),
    "zrnn_model_create": (ctypes.c_int, [ctypes.POINTER(ModelConfig), ctypes.POINTER(c_void_p)]),
    "zrnn_model_create_sharded": (ctypes.c_int, [ctypes.POINTER(ModelConfig), ctypes.c_int, ctypes.c_int,
                                                 ctypes.POINTER(c_void_p)]),
    "zrnn_model_num_tensors": (ctypes.c_int, [c_void_p]),
    "zrnn_model_tensor_info": (ctypes.c_int, [c_void_p, ctypes.c_int, ctypes.c_char_p, c_int_p, c_int_p]),
    "zrnn_model_set_tensor": (ctypes.c_int, [c_void_p, ctypes.c_int, c_float_p]),
    "zrnn_model_finalize": (ctypes.c_int, [c_void_p]),
    "zrnn_model_load_file": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                            ctypes.POINTER(c_void_p)]),
    "zrnn_model_load_file_sharded": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                    ctypes.c_int, ctypes.POINTER(c_void_p)]),
    "zrnn_model_file_header": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                              ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]),
    "zrnn_model_file_read": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                            ctypes.POINTER(ctypes.c_int), ctypes.POINTER(c_void_p)]),
    "zrnn_model_get_config": (ctypes.c_int, [c_void_p, ctypes.POINTER(ModelConfig)]),
    "zrnn_score_batch": (ctypes.c_int, [c_void_p, c_void_p, ctypes.c_int, c_void_p, c_void_p, ctypes.c_int,
                                        ctypes.c_int, c_void_p, ctypes.POINTER(ctypes.c_double)]),
    "zrnn_score_batch_device": (ctypes.c_int, [c_void_p, c_void_p, ctypes.c_int, c_void_p, c_void_p, ctypes.c_int,
                                               ctypes.c_int, c_void_p, c_void_p]),
    "zrnn_forward_states_device": (ctypes.c_int, [c_void_p, c_void_p, ctypes.c_int, c_void_p, ctypes.c_int, ctypes.c_int,
                                                  c_void_p, c_void_p]),
    "zrnn_model_copy_top_states": (ctypes.c_int, [c_void_p, c_void_p, ctypes.c_int, c_int_p, c_void_p]),
    "zrnn_model_softmax": (c_void_p, [c_void_p]),
    "zrnn_beam_decode_batch": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                              ctypes.c_float, ctypes.c_float, ctypes.c_float, ctypes.c_int, c_void_p,
                                              c_void_p, c_void_p]),
    "zrnn_beam_decode_batch_device": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_int, ctypes.c_int,
                                                     ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float,
                                                     ctypes.c_float, ctypes.c_int, c_void_p, c_void_p, c_void_p,
                                                     c_void_p]),
    "zrnn_beam_decode_batch_align": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_int, ctypes.c_int,
                                                    ctypes.c_int, ctypes.c_float, ctypes.c_float, ctypes.c_float,
                                                    ctypes.c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "zrnn_beam_decode_batch_align_device": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_int, ctypes.c_int,
                                                           ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float,
                                                           ctypes.c_float, ctypes.c_int, c_void_p, c_void_p, c_void_p,
                                                           c_void_p, c_void_p]),
    "zrnn_beam_decode_ensemble": (ctypes.c_int, [ctypes.POINTER(c_void_p), ctypes.c_int, ctypes.POINTER(c_void_p),
                                                 ctypes.POINTER(c_void_p), ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                 ctypes.c_float, ctypes.c_float, ctypes.c_float, ctypes.c_int, c_void_p,
                                                 c_void_p, c_void_p]),
    "zrnn_beam_decode_ensemble_align": (ctypes.c_int, [ctypes.POINTER(c_void_p), ctypes.c_int, ctypes.POINTER(c_void_p),
                                                       ctypes.POINTER(c_void_p), ctypes.c_int, ctypes.c_int,
                                                       ctypes.c_int, ctypes.c_float, ctypes.c_float, ctypes.c_float,
                                                       ctypes.c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "zrnn_score_batch_sharded": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_int, c_void_p, c_void_p,
                                                ctypes.c_int, ctypes.c_int, c_void_p, ctypes.POINTER(ctypes.c_double)]),
    "zrnn_beam_decode_batch_sharded": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_int, ctypes.c_int,
                                                      ctypes.c_int, ctypes.c_float, ctypes.c_float, ctypes.c_float,
                                                      ctypes.c_int, c_void_p, c_void_p, c_void_p]),
    "zrnn_model_destroy": (ctypes.c_int, [c_void_p]),
}

_LIB = None


def lib():
    """The loaded library; raises if it has not been built (python -m zoph_rnn_b200.build)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m zoph_rnn_b200.build` "
                              "(there is no CPU fallback)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = L
    return _LIB


def check(status):
    if status != OK:
        raise ZrnnError(status, lib().zrnn_last_error().decode("utf-8", "replace"))
