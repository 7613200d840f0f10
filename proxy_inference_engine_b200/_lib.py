"""ctypes binding of libpie_b200.so (include/pie_b200.h).

The library is the product: there is no Python/CPU fallback.  If it is missing, ``load()`` raises and every
operator of this package fails with it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("PIE_LIB") or os.path.join(_HERE, "libpie_b200.so")  # PIE_LIB: experiment builds
CSRC = os.path.join(_HERE, "csrc")

PIE_OK = 0
STATUS = {1: "EINVAL_SHAPE", 2: "EINVAL_DTYPE", 3: "EUNSUPPORTED", 4: "ECUDA", 5: "ENULL", 6: "EALIGN",
          7: "EWORKSPACE", 8: "ESTATIC_LIMIT"}
EPI_STORE, EPI_RESADD, EPI_SILUMUL = 0, 1, 2
DTYPE_BF16, DTYPE_F32 = 0, 1


class QmvSeg(C.Structure):
    _fields_ = [("wq", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p), ("N", C.c_int)]


class KvLayout(C.Structure):
    _fields_ = [("batch_stride", C.c_longlong), ("head_stride", C.c_longlong), ("tok_stride", C.c_longlong),
                ("page_table", C.c_void_p), ("pt_stride", C.c_int), ("page_size", C.c_int)]


class KvqCache(C.Structure):
    """pie_kvq_cache"""
    _fields_ = [("k_quant", C.c_void_p), ("k_scales", C.c_void_p), ("k_biases", C.c_void_p),
                ("v_quant", C.c_void_p), ("v_scales", C.c_void_p), ("v_biases", C.c_void_p),
                ("capacity", C.c_longlong), ("page_table", C.c_void_p), ("pt_stride", C.c_int), ("page_size", C.c_int),
                ("group_size", C.c_int), ("bits", C.c_int)]


class TpPeers(C.Structure):
    """pie_tp_peers"""
    _fields_ = [("base", C.c_void_p * 8), ("rank", C.c_int), ("world", C.c_int), ("max_elems", C.c_int),
                ("epoch", C.c_void_p)]


class TpFused(C.Structure):
    """pie_tp_fused"""
    _fields_ = [("peers", TpPeers), ("mode", C.c_int), ("h_out", C.c_void_p)]


class StepLayer(C.Structure):
    """pie_step_layer"""
    _fields_ = [("q", QmvSeg), ("k", QmvSeg), ("v", QmvSeg), ("o", QmvSeg), ("gate", QmvSeg), ("up", QmvSeg),
                ("down", QmvSeg), ("input_norm", C.c_void_p), ("post_norm", C.c_void_p), ("kcache", C.c_void_p),
                ("vcache", C.c_void_p), ("kv", KvLayout)]


class StepModel(C.Structure):
    """pie_step_model"""
    _fields_ = [("n_layers", C.c_int), ("hidden", C.c_int), ("ffn", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int),
                ("D", C.c_int), ("vocab", C.c_int), ("bits", C.c_int), ("group_size", C.c_int),
                ("rms_eps", C.c_float), ("attn_scale", C.c_float), ("rope_freqs", C.c_void_p), ("embed", QmvSeg),
                ("head", QmvSeg), ("final_norm", C.c_void_p)]


class StepIO(C.Structure):
    """pie_step_io"""
    _fields_ = [("B", C.c_int), ("tokens", C.c_void_p), ("positions", C.c_void_p), ("seq", C.c_void_p),
                ("seq_ld", C.c_int), ("h", C.c_void_p), ("qkv", C.c_void_p), ("attn", C.c_void_p),
                ("act", C.c_void_p), ("logits", C.c_void_p), ("attn_ws", C.c_void_p), ("attn_ws_bytes", C.c_size_t),
                ("nsplit", C.c_int), ("qmv_ws", C.c_void_p), ("qmv_ws_bytes", C.c_size_t), ("trace", C.c_void_p)]


_vp, _i, _ll, _f, _sz = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_size_t

# name -> (restype, argtypes); must list every symbol include/pie_b200.h declares (tests check this)
SIGNATURES = {
    "pie_abi_version": (_i, []),
    "pie_status_string": (C.c_char_p, [_i]),
    "pie_last_cuda_error": (C.c_char_p, []),
    "pie_launch_count": (C.c_ulonglong, []),
    "pie_quantize": (_i, [_vp, _i, _vp, _vp, _vp, _ll, _i, _i, _i, _vp]),
    "pie_dequantize": (_i, [_vp, _vp, _vp, _vp, _vp, _ll, _ll, _i, _i, _i, _vp]),
    "pie_qmv_workspace_bytes": (_sz, [_i, _ll, _i, _i, _i, _i]),
    "pie_qmv": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "pie_qmv_fused": (_i, [_vp, _i, _vp, _i, _i, _i, C.POINTER(QmvSeg), _i, _i, _i, _vp, _f, _i, _vp, _i, _vp,
                           _sz, _i, _vp]),
    "pie_qmm": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "pie_rms_norm": (_i, [_vp, _vp, _vp, _ll, _i, _f, _vp]),
    "pie_rope": (_i, [_vp, _vp, _ll, _i, _i, _i, _i, _f, _f, _i, _vp, _vp]),
    "pie_rope_kv_append": (_i, [_vp, _vp, _vp, _vp, C.POINTER(KvLayout), _vp, _vp, _i, _i, _i, _i, _vp]),
    "pie_kv_write": (_i, [_vp, _vp, C.POINTER(KvLayout), _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "pie_decode_attn_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "pie_decode_attn_pick_splits": (_i, [_i, _i, _i, _i]),
    "pie_decode_attn": (_i, [_vp, _vp, _vp, _vp, C.POINTER(KvLayout), _vp, _i, _i, _i, _i, _f, _i, _vp, _sz, _vp]),
    "pie_rope_table": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "pie_kvq_append": (_i, [_vp, _vp, C.POINTER(KvqCache), _vp, _vp, _i, _i, _i, _i, _vp]),
    "pie_kvq_write": (_i, [C.POINTER(KvqCache), _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "pie_decode_attn_q8_pick_splits": (_i, [_i, _i, _i, _i]),
    "pie_decode_attn_q8": (_i, [_vp, _vp, C.POINTER(KvqCache), _vp, _i, _i, _i, _i, _f, _i, _vp, _sz, _vp]),
    "pie_decode_attn_static": (_i, [_vp, _vp, _vp, _vp, C.POINTER(KvLayout), _vp, _i, _i, _i, _i, _f, _i, _vp]),
    "pie_decode_attn_fused": (_i, [_vp, _vp, _vp, _vp, C.POINTER(KvLayout), _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _vp,
                                   _sz, _i, _vp]),
    "pie_prefill_attn": (_i, [_vp, _vp, _vp, _vp, C.POINTER(KvLayout), _i, _i, _i, _i, _i, _i, _f, _vp]),
    "pie_silu_mul": (_i, [_vp, _vp, _vp, _ll, _vp]),
    "pie_add": (_i, [_vp, _vp, _vp, _ll, _vp]),
    "pie_argmax": (_i, [_vp, _vp, _i, _i, _vp, _vp, _i, _vp]),
    "pie_qmv_fused_tp": (_i, [_vp, _i, _vp, _i, _i, _i, C.POINTER(QmvSeg), _i, _i, _i, _vp, _f, _i, _vp, _i, _vp,
                              _sz, _i, C.POINTER(TpFused), _vp]),
    "pie_tp_buffer_bytes": (_sz, [_i, _i, _sz]),
    "pie_tp_gather_offset": (_sz, [_i, _i]),
    "pie_tp_allreduce": (_i, [_vp, _vp, _vp, _i, _i, C.POINTER(TpPeers), _vp]),
    "pie_tp_allgather": (_i, [_vp, _i, _i, C.POINTER(TpPeers), _vp]),
    "pie_page_allocator_create": (_vp, [_sz, _i, _i]),
    "pie_page_allocator_destroy": (None, [_vp]),
    "pie_page_allocate": (_ll, [_vp]),
    "pie_page_free": (_i, [_vp, C.c_uint32]),
    "pie_page_add_ref": (_i, [_vp, C.c_uint32]),
    "pie_page_ref_count": (_ll, [_vp, C.c_uint32]),
    "pie_page_num_tokens": (_ll, [_vp, C.c_uint32]),
    "pie_page_set_num_tokens": (_i, [_vp, C.c_uint32, C.c_uint32]),
    "pie_page_allocator_size": (_sz, [_vp]),
    "pie_page_allocator_num_free": (_sz, [_vp]),
    "pie_page_allocate_n": (_i, [_vp, _vp, _i]),
    "pie_page_free_n": (_i, [_vp, _vp, _i]),
    "pie_page_add_ref_n": (_i, [_vp, _vp, _i]),
    "pie_page_allocator_bench_refcount": (C.c_double, [_vp, _i]),
    "pie_page_allocator_stress": (_ll, [_vp, _i, _i]),
    "pie_debug_stamps": (_i, [_vp, _sz]),
    "pie_sample": (_i, [_vp, _vp, _i, _i, _i, _f, _f, _f, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "pie_decode_step_plan_bytes": (_sz, [_i]),
    "pie_decode_step_pick_splits": (_i, [_i, _i, _i, _i]),
    "pie_decode_step_attn_ws_bytes": (_sz, [_i, _i, _i, _i]),
    "pie_decode_step_plan": (_i, [C.POINTER(StepModel), C.POINTER(StepLayer), C.POINTER(StepIO), _vp, _sz]),
    "pie_decode_step": (_i, [_vp, _vp, _sz, _vp, _vp]),
}


class HybBatch(C.Structure):
    """pieh_batch"""
    _fields_ = [("T", C.c_int), ("n_seq", C.c_int), ("tok_seq", C.c_void_p), ("tok_pos", C.c_void_p),
                ("seq_start", C.c_void_p), ("seq_len", C.c_void_p), ("seq_ctx", C.c_void_p), ("seq_slot", C.c_void_p),
                ("block_table", C.c_void_p), ("bt_stride", C.c_int), ("n_tiles", C.c_int), ("tile_seq", C.c_void_p),
                ("tile_row", C.c_void_p)]


class HybDelta(C.Structure):
    """pieh_delta"""
    _fields_ = [("H", C.c_int), ("G", C.c_int), ("dk", C.c_int), ("dv", C.c_int), ("taps", C.c_int),
                ("conv_w", C.c_void_p), ("A_log", C.c_void_p), ("dt_bias", C.c_void_p), ("out_norm", C.c_void_p),
                ("eps", C.c_float), ("conv_state", C.c_void_p), ("state", C.c_void_p)]


class HybAttn(C.Structure):
    """pieh_attn"""
    _fields_ = [("H", C.c_int), ("G", C.c_int), ("d", C.c_int), ("dv", C.c_int), ("rot_dims", C.c_int),
                ("rot_freqs", C.c_void_p), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p), ("eps", C.c_float),
                ("scale", C.c_float), ("softcap", C.c_float), ("window", C.c_int), ("lam", C.c_float),
                ("out_scale", C.c_float), ("k_pages", C.c_void_p), ("v_pages", C.c_void_p), ("kv_dtype", C.c_int)]


class HybBiasAttn(C.Structure):
    """pieh_bias_attn"""
    _fields_ = [("H", C.c_int), ("G", C.c_int), ("d", C.c_int), ("dv", C.c_int), ("k_off", C.c_longlong),
                ("v_off", C.c_longlong), ("g_off", C.c_longlong), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p),
                ("eps", C.c_float), ("scale", C.c_float), ("temp_coef", C.c_float), ("temp_every", C.c_double),
                ("slopes", C.c_void_p), ("sink", C.c_int), ("window", C.c_int), ("k_pages", C.c_void_p),
                ("v_pages", C.c_void_p), ("kv_dtype", C.c_int),
                # optional pieces, zero / NULL = off
                ("sinks", C.c_void_p), ("gate_heads", C.c_int), ("rot_dims", C.c_int), ("rot_cs", C.c_void_p),
                ("v_mix", C.c_void_p), ("v_keep", C.c_void_p), ("sigmoid", C.c_int), ("score_bias", C.c_void_p)]


class HybMixSum(C.Structure):
    """pieh_mix_sum"""
    _fields_ = [("parts", C.c_void_p), ("part_row", C.c_void_p), ("part_w", C.c_void_p), ("top", C.c_int),
                ("shared", C.c_void_p), ("shared_gate", C.c_void_p), ("gate_ld", C.c_longlong)]


class HybMoePlan(C.Structure):
    """pieh_moe_plan"""
    _fields_ = [("E", C.c_int), ("top", C.c_int), ("n_groups", C.c_int), ("keep_groups", C.c_int), ("scale", C.c_float),
                ("slot_row", C.c_void_p), ("slot_expert", C.c_void_p), ("pair_slot", C.c_void_p), ("pair_w", C.c_void_p),
                ("tiles64", C.c_void_p), ("tiles128", C.c_void_p), ("counters", C.c_void_p), ("softmax_top", C.c_int)]


class HybCanon(C.Structure):
    """pieh_canon"""
    _fields_ = [("taps", C.c_int), ("n_out", C.c_int), ("w", C.c_void_p * 4), ("out", C.c_void_p * 4),
                ("state", C.c_void_p)]


class HybGdelta(C.Structure):
    """pieh_gdelta"""
    _fields_ = [("H", C.c_int), ("dk", C.c_int), ("dv", C.c_int), ("r_off", C.c_longlong), ("k_off", C.c_longlong),
                ("v_off", C.c_longlong), ("a_off", C.c_longlong), ("a_bias", C.c_void_p), ("decay_scale", C.c_float),
                ("key_eps", C.c_float), ("state", C.c_void_p)]


class HybSsd(C.Structure):
    """pieh_ssd"""
    _fields_ = [("H", C.c_int), ("P", C.c_int), ("N", C.c_int), ("G", C.c_int), ("taps", C.c_int), ("xbc_off", C.c_longlong),
                ("dt_off", C.c_longlong), ("conv_w", C.c_void_p), ("conv_b", C.c_void_p), ("dt_bias", C.c_void_p),
                ("A_log", C.c_void_p), ("D", C.c_void_p), ("conv_state", C.c_void_p), ("state", C.c_void_p)]


_PB, _PD, _PA = C.POINTER(HybBatch), C.POINTER(HybDelta), C.POINTER(HybAttn)
_PBA, _PMS, _PMP = C.POINTER(HybBiasAttn), C.POINTER(HybMixSum), C.POINTER(HybMoePlan)
_PCN = C.POINTER(HybCanon)
_PGD, _PSS = C.POINTER(HybGdelta), C.POINTER(HybSsd)
# libpie_b200_hybrid.so: every symbol include/pie_b200_hybrid.h declares (tests check this), + the page allocator
HYBRID_SIGNATURES = {
    "pieh_abi_version": (_i, []),
    "pieh_last_cuda_error": (C.c_char_p, []),
    "pieh_launch_count": (C.c_ulonglong, []),
    "pieh_pipeline_error": (C.c_uint, []),
    "pieh_set_pdl": (None, [_i]),
    "pieh_linear": (_i, [_vp, _i, _ll, _vp, _i, _ll, _vp, _i, _vp, _i, _i, _i, _i, _f, _vp, _vp, _i, _vp]),
    "pieh_embed_streams": (_i, [_vp, _vp, _i, _vp, _i, _i, _i, _i, _vp]),
    "pieh_stream_norm": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _f, _f, _i, _i, _i, _vp]),
    "pieh_stream_update": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "pieh_delta_prepare": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _ll, _PD, _PB, _vp]),
    "pieh_delta_scan": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _PD, _PB, _vp]),
    "pieh_delta_gate": (_i, [_vp, _i, _vp, _vp, _ll, _ll, _PD, _i, _vp]),
    "pieh_attn_prepare": (_i, [_vp, _vp, _ll, _PA, _PB, _vp]),
    "pieh_attn_run": (_i, [_vp, _i, _vp, _PA, _PB, _vp]),
    "pieh_linear_glu": (_i, [_vp, _i, _ll, _vp, _i, _ll, _vp, _i, _i, _i, _i, _f, _f, _f, _vp]),
    "pieh_embed_positions": (_i, [_vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    "pieh_postnorm_add": (_i, [_vp, _vp, _i, _vp, _PMS, _vp, _f, _i, _i, _vp]),
    "pieh_bias_attn_prepare": (_i, [_vp, _vp, _ll, _PBA, _PB, _vp]),
    "pieh_bias_attn_run": (_i, [_vp, _i, _vp, _vp, _ll, _PBA, _PB, _vp]),
    "pieh_linear_batched": (_i, [_vp, _i, _ll, _ll, _vp, _i, _ll, _ll, _vp, _i, _ll, _i, _i, _i, _i, _i, _vp, _ll, _ll, _vp]),
    "pieh_rot_table": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "pieh_embed_scaled": (_i, [_vp, _vp, _i, _vp, _f, _i, _i, _i, _vp]),
    "pieh_residual_norm": (_i, [_vp, _vp, _PMS, _vp, _vp, _f, _i, _i, _vp]),
    "pieh_canon_conv": (_i, [_PCN, _i, _vp, _i, _PB, _vp]),
    "pieh_mingru_scan": (_i, [_vp, _i, _vp, _ll, _i, _vp, _vp, _PB, _vp]),
    "pieh_latent_prepare": (_i, [_vp, _i, _vp, _ll, _i, _ll, _i, _vp, _vp, _f, _vp, _i, _PB, _vp]),
    "pieh_linear_act": (_i, [_vp, _i, _ll, _vp, _i, _ll, _vp, _i, _vp, _i, _i, _i, _i, _f, _f, _vp]),
    "pieh_sandwich_add": (_i, [_vp, _vp, _PMS, _vp, _f, _vp, _vp, _vp, _i, _vp, _f, _i, _i, _vp]),
    "pieh_gated_group_norm": (_i, [_vp, _i, _vp, _ll, _vp, _ll, _vp, _i, _i, _f, _i, _i, _i, _vp]),
    "pieh_gdelta_prepare": (_i, [_vp, _vp, _vp, _vp, _ll, _vp, _ll, _PGD, _i, _vp]),
    "pieh_gdelta_scan": (_i, [_vp, _vp, _ll, _vp, _vp, _vp, _PGD, _PB, _vp]),
    "pieh_ssd_prepare": (_i, [_vp, _vp, _vp, _ll, _PSS, _PB, _vp]),
    "pieh_ssd_scan": (_i, [_vp, _vp, _vp, _PSS, _PB, _vp]),
    "pieh_moe_route": (_i, [_vp, _ll, _PMP, _i, _vp]),
    "pieh_moe_linear": (_i, [_vp, _i, _ll, _vp, _i, _ll, _vp, _i, _ll, _i, _i, _i, _i, _i, _f, _f, _f, _PMP, _vp]),
}
HYBRID_LIB_PATH = os.environ.get("PIE_HYBRID_LIB") or os.path.join(_HERE, "libpie_b200_hybrid.so")
EPI_NONE, EPI_RELU2, EPI_SOFTCAP, EPI_STREAMS, EPI_GLU, EPI_SIGMUL, EPI_TANH, EPI_XIELU = 0, 1, 2, 3, 4, 5, 6, 7

_lib = None
_hyb = None


def build(verbose: bool = False, target: str = "all") -> str:
    """Compile csrc/ for sm_100a into libpie_b200.so and libpie_b200_hybrid.so (nvcc cross-compiles without a GPU);
    target="hybrid" compiles the second one only.  Concurrent callers serialise on a lock file beside the sources."""
    import fcntl

    out = None if verbose else subprocess.DEVNULL
    with open(os.path.join(CSRC, ".build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        subprocess.check_call(["make", "-s", "-j8", "-C", CSRC, target], stdout=out)
    return LIB_PATH


def load_hybrid(build_if_missing: bool = False):
    """libpie_b200_hybrid.so.  build_if_missing: run `make hybrid` first -- compiles on first use and after a source
    change, a no-op otherwise (the servers' and the trace runner's choice; a plain import stays free of side effects)."""
    global _hyb
    if _hyb is None:
        if build_if_missing and not os.environ.get("PIE_HYBRID_LIB"):
            try:                       # incremental: nothing happens when the library is newer than its sources
                build(target="hybrid")
            except (OSError, subprocess.CalledProcessError):
                if not os.path.exists(HYBRID_LIB_PATH):
                    raise              # a read-only checkout or a box without nvcc still runs a library that is there
        if not os.path.exists(HYBRID_LIB_PATH):
            raise RuntimeError(f"{HYBRID_LIB_PATH} is missing: build it with `make -C {CSRC} hybrid`. "
                               "proxy_inference_engine_b200 has no CPU fallback.")
        L = C.CDLL(HYBRID_LIB_PATH)
        for name, (res, args) in list(HYBRID_SIGNATURES.items()) + [(k, v) for k, v in SIGNATURES.items()
                                                                      if k.startswith("pie_page_")]:
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _hyb = L
    return _hyb


def check_hybrid(status: int, what: str) -> None:
    if status == PIE_OK:
        return
    msg = f"[{what}] {STATUS.get(status, status)}"
    if status == 4:
        raise RuntimeError(msg + ": " + load_hybrid().pieh_last_cuda_error().decode())
    raise ValueError(msg)


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `make -C {CSRC}` (or __graft_entry__.build()). "
                "proxy_inference_engine_b200 has no CPU fallback.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(status: int, what: str) -> None:
    """Map a pie_status to the exception the reference raises for the same condition (ops.cpp:82-134)."""
    if status == PIE_OK:
        return
    L = load()
    msg = f"[{what}] {L.pie_status_string(status).decode()} ({STATUS.get(status, status)})"
    if status == 4:
        raise RuntimeError(msg + ": " + L.pie_last_cuda_error().decode())
    raise ValueError(msg)
