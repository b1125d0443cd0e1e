"""ctypes binding of libqlm_b200.so -- one prototype per declaration in include/qlm_b200.h."""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

# binary layout of qlmb_span == the reference's QSpanD (qlm.cuh:30-38)
SPAN_DTYPE = np.dtype([("pof", "<u8"), ("gof", "<u8"), ("qi0", "<u8"), ("n", "<u8"),
                       ("gi0", "<i4"), ("ngrp", "<i4"), ("sref", "<f4"), ("_pad", "<i4")])

F32, BF16 = 0, 1
KN, NK = 0, 1


class QlmbError(RuntimeError):
    pass


class MoeLayer(C.Structure):
    _fields_ = [("N", C.c_int), ("D", C.c_int), ("F", C.c_int), ("E", C.c_int), ("K", C.c_int),
                ("dtype", C.c_int),
                ("w1_codes", C.c_void_p), ("w3_codes", C.c_void_p), ("w2_codes", C.c_void_p),
                ("w1_scales", C.c_void_p), ("w3_scales", C.c_void_p), ("w2_scales", C.c_void_p),
                ("wr", C.c_void_p), ("bias", C.c_void_p), ("bias_stride", C.c_int), ("aux", C.c_float)]


vp, ci, cf, u64, sz = C.c_void_p, C.c_int, C.c_float, C.c_uint64, C.c_size_t

# name -> (restype, argtypes); the symbol test walks this table against the header
class StateFile(C.Structure):
    _fields_ = [("dmax", C.c_int), ("group", C.c_int), ("adam", C.c_int), ("nspan", C.c_int), ("packed", C.c_int),
                ("iter", C.c_int), ("nq", C.c_ulonglong), ("ngrp", C.c_ulonglong), ("nfloat", C.c_ulonglong),
                ("Mc", C.c_void_p), ("Vc", C.c_void_p), ("d", C.c_void_p), ("r", C.c_void_p), ("m8", C.c_void_p),
                ("v8", C.c_void_p), ("s", C.c_void_p), ("m8s", C.c_void_p), ("v8s", C.c_void_p), ("sref", C.c_void_p),
                ("have_sref", C.c_int), ("prev_gn", C.c_float), ("have_prev_gn", C.c_int)]


class EpPeers(C.Structure):
    _fields_ = [("rank", C.c_int), ("world", C.c_int), ("base", C.c_void_p * 8)]


PROTOTYPES = {
    "qlmb_last_error": (C.c_char_p, []),
    "qlmb_version": (ci, []),
    "qlmb_check_device": (ci, [vp]),
    "qlmb_selftest_wait_expires": (ci, [ci, vp]),
    "qlmb_selftest_stream_read": (ci, [vp, u64, ci, ci, vp]),
    "qlmb_skipped_steps": (ci, [vp, ci, vp]),
    "qlmb_prof_enable": (ci, [ci]),
    "qlmb_side_stream_enable": (ci, [ci]),
    "qlmb_prof_read": (ci, [vp, vp, ci]),
    "qlmb_encode": (ci, [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp]),
    "qlmb_render": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, ci, vp]),
    "qlmb_step": (ci, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, cf, cf, cf, cf, cf, vp, cf, cf,
                       ci, u64, ci, vp, ci, ci, ci, vp]),
    "qlmb_set_v4": (ci, [ci]),
    "qlmb_ngram_key": (ci, [vp, vp, ci, ci, ci, ci, ci, vp]),
    "qlmb_dec_ngkey": (ci, [vp, vp, vp, ci, ci, ci, ci, vp]),
    "qlmb_ngram_gather": (ci, [vp, vp, vp, ci, ci, ci, vp]),
    "qlmb_nggate_fwd": (ci, [vp, vp, vp, vp, ci, vp, vp, vp, ci, ci, vp]),
    "qlmb_nggate_bwd": (ci, [vp, vp, vp, vp, ci, vp, vp, vp, vp, vp, ci, ci, vp]),
    "qlmb_ng_touched": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, vp]),
    "qlmb_ng_scatter_compact": (ci, [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp]),
    "qlmb_eg_key": (ci, [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp]),
    "qlmb_eg_gather": (ci, [vp, vp, vp, ci, ci, ci, vp]),
    "qlmb_eg_scatter_compact": (ci, [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp]),
    "qlmb_ng_step": (ci, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, cf, cf, cf, cf, cf, cf, cf, u64, u64, vp, vp]),
    "qlmb_modelfile_write": (ci, [C.c_char_p, vp, vp, u64, vp, ci]),
    "qlmb_modelfile_read_header": (ci, [C.c_char_p, vp, vp, vp]),
    "qlmb_modelfile_read": (ci, [C.c_char_p, vp, u64, vp, ci, vp]),
    "qlmb_q4n_work_bytes": (u64, [u64, ci]),
    "qlmb_q4n_max_bytes": (u64, [u64, ci]),
    "qlmb_q4n_export": (ci, [vp, u64, vp, vp, u64, ci, vp, vp]),
    "qlmb_q4n_index": (ci, [vp, u64, u64, ci, vp]),
    "qlmb_q4n_decode": (ci, [vp, vp, vp, u64, ci, vp]),
    "qlmb_qfile_write": (ci, [C.c_char_p, vp, ci, ci, vp, u64, vp, ci]),
    "qlmb_qfile_read_header": (ci, [C.c_char_p, vp, vp, vp, vp]),
    "qlmb_qfile_read": (ci, [C.c_char_p, vp, u64]),
    "qlmb_servo": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, cf, cf, ci, vp]),
    "qlmb_gnorm": (ci, [vp, sz, vp, vp, ci, ci, vp, vp]),
    "qlmb_gnorm_noalloc": (ci, [vp, sz, vp, vp, ci, ci, vp, vp]),
    "qlmb_sqsum": (ci, [vp, sz, vp, vp]),
    "qlmb_gnorm_close": (ci, [vp, ci, vp, vp]),
    "qlmb_gemm_nt": (ci, [vp, ci, vp, vp, ci, ci, ci, cf, vp]),
    "qlmb_cast_bf16": (ci, [vp, vp, vp, ci, ci, vp]),
    "qlmb_embed": (ci, [vp, ci, vp, vp, ci, ci, vp]),
    "qlmb_embed_bwd": (ci, [vp, vp, ci, vp, ci, ci, ci, vp]),
    "qlmb_rmsnorm_fwd": (ci, [vp, ci, vp, vp, ci, vp, ci, ci, vp]),
    "qlmb_rmsnorm_bwd": (ci, [vp, ci, ci, vp, vp, vp, ci, vp, vp, vp, ci, ci, ci, vp]),
    "qlmb_rope": (ci, [vp, ci, vp, vp, ci, ci, ci, ci, ci, vp]),
    "qlmb_softmax_ce": (ci, [vp, ci, vp, vp, vp, ci, ci, ci, ci, vp]),
    "qlmb_gemv_decode_stack": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, ci, vp]),
    "qlmb_gemv_decode_norm_stack": (ci, [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp]),
    "qlmb_dec_qkv": (ci, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp]),
    "qlmb_gemv_decode_res_norm": (ci, [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, vp]),
    "qlmb_dec_rope": (ci, [vp, ci, vp, vp, vp, ci, ci, ci, ci, vp]),
    "qlmb_dec_kv": (ci, [vp, vp, vp, vp, vp, ci, ci, ci, vp]),
    "qlmb_dec_attn": (ci, [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp]),
    "qlmb_dec_greedy": (ci, [vp, vp, vp, ci, ci, vp]),
    "qlmb_dec_sample": (ci, [vp, vp, vp, vp, ci, ci, vp]),
    "qlmb_attn_fwd": (ci, [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp]),
    "qlmb_attn_bwd": (ci, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp]),
    "qlmb_adamw": (ci, [vp, vp, vp, vp, sz, cf, cf, cf, cf, cf, cf, vp, vp]),
    "qlmb_linear_fwd": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, vp, ci, vp]),
    "qlmb_linear_dgrad": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, cf, ci, vp]),
    "qlmb_linear_wgrad": (ci, [vp, vp, vp, ci, ci, ci, ci, cf, ci, vp]),
    "qlmb_gemv_decode": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, ci, vp]),
    "qlmb_router_topk": (ci, [vp, vp, vp, ci, vp, vp, ci, vp, vp, vp, ci, ci, ci, ci, vp]),
    "qlmb_router_bias_update": (ci, [vp, vp, ci, ci, ci, ci, cf, ci, vp]),
    "qlmb_perm_build": (ci, [vp, ci, ci, ci, ci, ci, vp, vp, vp, vp, vp, vp]),
    "qlmb_moe_arena_bytes": (sz, [ci, ci, ci, ci, ci]),
    "qlmb_moe_arena_member": (vp, [vp, ci, ci, ci, ci, ci, C.c_char_p]),
    "qlmb_moe_forward": (ci, [C.POINTER(MoeLayer), vp, vp, vp, vp, vp]),
    "qlmb_moe_decode": (ci, [C.POINTER(MoeLayer), vp, vp, vp, vp, vp]),
    "qlmb_moe_forward_routed": (ci, [C.POINTER(MoeLayer), vp, vp, vp, vp, vp, vp]),
    "qlmb_moe_backward": (ci, [C.POINTER(MoeLayer), vp, vp, vp, vp, vp, vp, vp, vp, cf, vp]),
    "qlmb_moe_route": (ci, [C.POINTER(MoeLayer), vp, vp, vp, vp]),
    "qlmb_moe_experts_forward": (ci, [C.POINTER(MoeLayer), vp, vp, vp, vp, ci, vp]),
    "qlmb_moe_combine": (ci, [C.POINTER(MoeLayer), vp, vp, vp, vp, vp]),
    "qlmb_moe_dgate": (ci, [C.POINTER(MoeLayer), vp, vp, vp, vp, vp]),
    "qlmb_moe_experts_backward": (ci, [C.POINTER(MoeLayer), vp, vp, vp, ci, vp, vp, vp, cf, vp]),
    "qlmb_moe_route_backward": (ci, [C.POINTER(MoeLayer), vp, vp, vp, vp, vp, cf, vp]),
    "qlmb_statefile_write": (ci, [C.c_char_p, C.POINTER(StateFile)]),
    "qlmb_statefile_read_header": (ci, [C.c_char_p, C.POINTER(StateFile)]),
    "qlmb_statefile_read": (ci, [C.c_char_p, C.POINTER(StateFile)]),
    "qlmb_peer_alloc": (ci, [C.c_size_t, C.POINTER(vp)]),
    "qlmb_peer_free": (ci, [vp]),
    "qlmb_peer_export": (ci, [vp, vp]),
    "qlmb_peer_open": (ci, [vp, C.POINTER(vp)]),
    "qlmb_peer_close": (ci, [vp]),
    "qlmb_ep_route": (ci, [C.POINTER(MoeLayer), vp, vp, vp]),
    "qlmb_ep_experts_forward": (ci, [C.POINTER(MoeLayer), vp, C.POINTER(EpPeers), vp, vp, ci, ci, ci, vp, vp]),
    "qlmb_ep_combine": (ci, [C.POINTER(MoeLayer), vp, vp, vp, vp, vp]),
    "qlmb_ep_dgate": (ci, [C.POINTER(MoeLayer), vp, vp, vp, vp]),
    "qlmb_ep_experts_backward": (ci, [C.POINTER(MoeLayer), vp, C.POINTER(MoeLayer), vp, C.POINTER(EpPeers), vp, ci, ci,
                                      vp, vp, vp, vp, cf, vp]),
    "qlmb_ep_route_backward": (ci, [C.POINTER(MoeLayer), vp, vp, vp, vp, vp, cf, vp]),
    "qlmb_comm_unique_id": (ci, [vp]),
    "qlmb_comm_init": (ci, [C.POINTER(vp), vp, ci, ci]),
    "qlmb_comm_destroy": (ci, [vp]),
    "qlmb_comm_rank": (ci, [vp]),
    "qlmb_comm_world": (ci, [vp]),
    "qlmb_comm_allreduce_f32": (ci, [vp, vp, u64, ci, vp]),
    "qlmb_comm_allgather": (ci, [vp, vp, vp, u64, vp]),
    "qlmb_comm_barrier": (ci, [vp, vp]),
    "qlmb_dp_grad_sync": (ci, [vp, vp, u64, vp]),
    "qlmb_dp_gnorm_close": (ci, [vp, vp, ci, ci, vp, vp]),
    "qlmb_zero1_step": (ci, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, cf, cf, cf, cf, cf, vp, cf, cf,
                             ci, u64, ci, vp, ci, vp]),
    "qlmb_zero1_gather_scales": (ci, [vp, vp, ci, vp]),
    "qlmb_ep_window_open": (ci, [vp, vp, C.POINTER(EpPeers), vp]),
    "qlmb_ep_window_close": (ci, [vp, C.POINTER(EpPeers), vp]),
    "qlmb_ep_layer_forward": (ci, [vp, C.POINTER(MoeLayer), vp, C.POINTER(MoeLayer), vp, C.POINTER(EpPeers), vp, vp, ci, vp,
                                   vp, vp, vp]),
    "qlmb_ep_layer_backward": (ci, [vp, C.POINTER(MoeLayer), vp, C.POINTER(MoeLayer), vp, C.POINTER(EpPeers), vp, vp, vp, vp,
                                    vp, vp, vp, vp, vp, cf, ci, vp]),
}

_lib = None


def lib_path():
    return os.path.join(HERE, "libqlm_b200.so")


def lib():
    """The loaded library.  Raises if it was not built: there is no fallback path."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise QlmbError("%s is missing: build it with `python -m cudalm_c_b200.build` "
                            "(there is no CPU fallback)" % path)
        L = C.CDLL(path)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(rc):
    if rc != 0:
        raise QlmbError("libqlm_b200 status %d: %s" % (rc, lib().qlmb_last_error().decode()))


def ptr(t):
    """Device (or host) address of a torch tensor / numpy array / None."""
    if t is None:
        return None
    if isinstance(t, np.ndarray):
        return t.ctypes.data
    return t.data_ptr()


def stream_ptr(stream=None):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream
