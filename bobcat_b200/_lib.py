"""ctypes binding of ``libbobcat_cuda.so`` (declared in ``include/bobcat_cuda.h``).

The library is the product; this module only declares its signatures. There is no fallback: if the
shared library is missing, importing anything that needs it raises with the build command.
"""

from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libbobcat_cuda.so")

vp, u32, i32, u64, sz, f32 = C.c_void_p, C.c_uint32, C.c_int32, C.c_uint64, C.c_size_t, C.c_float


class Hparams(C.Structure):
    _fields_ = [(n, i32 if n == "architecture" else u32) for n in (
        "architecture", "n_layers", "n_attention_layers", "n_conv_layers", "n_delta_layers", "n_embd", "n_ff", "n_vocab",
        "n_heads", "n_kv_heads", "head_dim", "n_rot", "conv_kernel", "n_experts", "n_experts_used", "n_ff_expert",
        "n_k_heads", "n_v_heads", "k_head_dim", "v_head_dim")] + [("rope_theta", f32), ("norm_eps", f32)]


class Sampling(C.Structure):
    _fields_ = [("temperature", f32), ("top_k", u32), ("top_p", f32), ("min_p", f32), ("repeat_penalty", f32)]


class Trace(C.Structure):
    _fields_ = [("embedding", C.POINTER(f32)), ("layers", C.POINTER(f32)), ("final_norm", C.POINTER(f32)), ("n_tokens", u32)]


class ProfileEntry(C.Structure):
    _fields_ = [("name", C.c_char_p), ("n_rows", u32), ("n_cols", u32), ("calls", u64), ("seconds", C.c_double), ("bytes", u64)]


EMIT_FN = C.CFUNCTYPE(i32, u32, vp)

# name -> (restype, argtypes). `None` restype means void; the default restype is the status code.
_VIEW = [vp, sz]
SIGNATURES = {
    "bc_last_error": (C.c_char_p, []),
    "bc_version": (C.c_char_p, []),
    "bc_backend_open": (i32, [i32, vp, C.POINTER(vp)]),
    "bc_backend_close": (None, [vp]),
    "bc_backend_stream": (vp, [vp]),
    "bc_buffer_new": (i32, [vp, sz, C.POINTER(vp)]),
    "bc_buffer_free": (None, [vp]),
    "bc_buffer_len": (sz, [vp]),
    "bc_buffer_device_ptr": (vp, [vp]),
    "bc_buffer_write": (i32, [vp, sz, vp, sz]),
    "bc_buffer_read": (i32, [vp, sz, vp, sz]),
    "bc_matrix_upload": (i32, [vp, i32, vp, u32, u32, C.POINTER(vp)]),
    "bc_begin": (i32, [vp]),
    "bc_barrier": (i32, [vp]),
    "bc_commit": (i32, [vp, C.POINTER(u64)]),
    "bc_wait": (i32, [vp, u64, C.POINTER(C.c_double)]),
    "bc_end": (i32, [vp, C.POINTER(C.c_double)]),
    "bc_discard": (None, [vp]),
    "bc_set_profiling": (i32, [vp, i32]),
    "bc_profile": (i32, [vp, C.POINTER(ProfileEntry), sz, C.POINTER(sz)]),
    "bc_op_matvec": (i32, [vp, i32] + _VIEW + [u32, u32] + _VIEW + _VIEW + _VIEW + [f32, i32]),
    "bc_op_matvec_swiglu": (i32, [vp, i32] + _VIEW + _VIEW + [u32, u32] + _VIEW + _VIEW + [f32] + _VIEW),
    "bc_op_matvec_conv": (i32, [vp, i32] + _VIEW + [u32] + _VIEW + _VIEW + [f32] + _VIEW + _VIEW + _VIEW + [u32, u32]),
    "bc_op_short_conv": (i32, [vp] + _VIEW + _VIEW + _VIEW + _VIEW + [u32, u32, u32]),
    "bc_op_matmul": (i32, [vp, i32] + _VIEW + [u32, u32] + _VIEW + _VIEW + [u32, i32]),
    "bc_op_expand": (i32, [vp, i32] + _VIEW + _VIEW + [u32, u32, i32]),
    "bc_op_embed": (i32, [vp, i32] + _VIEW + [u32] + _VIEW + _VIEW + [u32, u32]),
    "bc_op_rms_norm": (i32, [vp] + _VIEW + _VIEW + _VIEW + [u32, u32, f32]),
    "bc_op_norm_rope": (i32, [vp] + _VIEW + _VIEW + [i32] + _VIEW + [u32] * 8 + [f32, f32]),
    "bc_op_convert_half": (i32, [vp] + _VIEW + _VIEW + [u32]),
    "bc_op_copy": (i32, [vp] + _VIEW + _VIEW + [u32]),
    "bc_op_attention": (i32, [vp] + _VIEW + _VIEW + _VIEW + [i32] + _VIEW + _VIEW + [u32] * 6),
    "bc_attention_scratch_floats": (sz, [u32, u32, u32, u32]),
    "bc_attention_static": (i32, [vp, vp, vp, vp, i32, vp] + [u32] * 6),
    "bc_op_argmax": (i32, [vp] + _VIEW + _VIEW + [u32]),
    "bc_op_sample": (i32, [vp] + _VIEW + [u32] + _VIEW + [u32, C.POINTER(Sampling), f32] + _VIEW),
    "bc_seq_sample": (i32, [vp, C.POINTER(Sampling), f32, vp, sz, C.POINTER(u32)]),
    "bc_readback_new": (i32, [vp, sz, C.POINTER(vp)]),
    "bc_readback_free": (None, [vp]),
    "bc_op_argmax_readback": (i32, [vp] + _VIEW + _VIEW + [vp, sz, u32]),
    "bc_read_readback": (i32, [vp, vp, sz, C.POINTER(u32)]),
    "bc_op_silu_mul": (i32, [vp] + _VIEW + _VIEW + [u32]),
    "bc_op_gdn_conv": (i32, [vp] + _VIEW + _VIEW + _VIEW + _VIEW + [u32] * 3),
    "bc_op_gdn_gates": (i32, [vp] + _VIEW + _VIEW + _VIEW + _VIEW + [u32] * 2),
    "bc_op_gdn_recurrence": (i32, [vp] + _VIEW + _VIEW + _VIEW + _VIEW + _VIEW + [u32] * 5 + [i32]),
    "bc_op_gdn_gated_norm": (i32, [vp] + _VIEW + _VIEW + _VIEW + [u32, u32, f32]),
    "bc_op_attention_gate": (i32, [vp] + _VIEW + _VIEW + [u32] * 3),
    "bc_route_bytes": (sz, [u32, u32]),
    "bc_op_moe_route": (i32, [vp] + _VIEW + _VIEW + [f32] + _VIEW + _VIEW + _VIEW + _VIEW + [u32] * 4),
    "bc_op_moe_group": (i32, [vp] + _VIEW + _VIEW + _VIEW + [u32] * 3),
    "bc_op_matvec_experts_swiglu": (i32, [vp, i32] + _VIEW + _VIEW + [u32] * 3 + _VIEW + _VIEW + [u32] + _VIEW + [u32]),
    "bc_op_matvec_experts_down": (i32, [vp, i32] + _VIEW + [u32] * 3 + _VIEW + _VIEW + [u32] + _VIEW + [u32]),
    "bc_op_matmul_experts": (i32, [vp, i32] + _VIEW + _VIEW + [u32] * 3 + _VIEW + [i32] + _VIEW + _VIEW + [u32] + _VIEW + [u32]),
    "bc_op_moe_combine": (i32, [vp] + _VIEW + _VIEW + _VIEW + [u32] * 3),
    "bc_model_load": (i32, [C.c_char_p, C.POINTER(vp)]),
    "bc_model_free": (None, [vp]),
    "bc_model_hparams": (i32, [vp, C.POINTER(Hparams)]),
    "bc_model_attention_layers": (i32, [vp, vp, sz]),
    "bc_model_decode_bytes": (u64, [vp]),
    "bc_seq_new": (i32, [vp, vp, u32, i32, C.POINTER(vp)]),
    "bc_seq_new_tensor_parallel": (i32, [vp, vp, vp, u32, i32, C.POINTER(vp)]),
    "bc_seq_new_paged": (i32, [vp, vp, u32, i32, C.POINTER(vp)]),
    "bc_kv_page_locate": (i32, [u32] * 8 + [C.POINTER(u64), C.POINTER(u32), C.POINTER(u64)]),
    "bc_seq_kv_pages": (i32, [vp, C.POINTER(u32), C.POINTER(u32), C.POINTER(u32)]),
    "bc_seq_prefix_save": (i32, [vp, C.POINTER(vp)]),
    "bc_seq_prefix_load": (i32, [vp, vp]),
    "bc_prefix_free": (None, [vp]),
    "bc_prefix_n_past": (u32, [vp]),
    "bc_seq_free": (None, [vp]),
    "bc_seq_n_past": (u32, [vp]),
    "bc_seq_step": (i32, [vp, u32, vp, sz, C.POINTER(Trace)]),
    "bc_seq_prefill": (i32, [vp, vp, sz, vp, sz, vp, sz, C.POINTER(Trace)]),
    "bc_seq_greedy_token": (i32, [vp, C.POINTER(u32)]),
    "bc_seq_generate": (i32, [vp, vp, sz]),
    "bc_seq_generate_next": (i32, [vp, vp, sz]),
    "bc_seq_generate_stream": (i32, [vp, u32, EMIT_FN, vp, vp, sz, C.POINTER(sz)]),
    "bc_seq_reset": (i32, [vp]),
    "bc_seq_checkpoint": (i32, [vp, C.POINTER(vp)]),
    "bc_seq_restore": (i32, [vp, vp]),
    "bc_checkpoint_free": (None, [vp]),
    "bc_seq_timings": (i32, [vp, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "bc_seq_read_state": (i32, [vp, i32, u32, vp, sz, C.POINTER(sz)]),
    "bc_batch_new": (i32, [vp, vp, u32, u32, i32, C.POINTER(vp)]),
    "bc_batch_free": (None, [vp]),
    "bc_batch_n_seqs": (u32, [vp]),
    "bc_batch_seq": (i32, [vp, u32, C.POINTER(vp)]),
    "bc_batch_generate": (i32, [vp, vp, sz]),
    "bc_batch_set_exact": (i32, [vp, i32]),
    "bc_batch_timings": (i32, [vp, C.POINTER(C.c_double), C.POINTER(u64)]),
    "bc_comm_unique_id": (i32, [vp, sz]),
    "bc_comm_init": (i32, [vp, vp, sz, i32, i32, C.POINTER(vp)]),
    "bc_comm_free": (None, [vp]),
    "bc_comm_rank": (i32, [vp]),
    "bc_comm_world": (i32, [vp]),
    "bc_comm_collectives": (u64, [vp]),
    "bc_comm_peer_reduces": (u64, [vp]),
    "bc_batch_new_expert_parallel": (i32, [vp, vp, vp, u32, u32, i32, C.POINTER(vp)]),
    "bc_seq_step_on_device": (i32, [vp, u32]),
    "bc_engine_new": (i32, [vp, vp, u32, i32, u64, C.POINTER(vp)]),
    "bc_engine_free": (None, [vp]),
    "bc_engine_generate": (i32, [vp, vp, sz, C.c_int64, u32, C.POINTER(Sampling), EMIT_FN, vp, vp, sz, C.POINTER(sz), C.POINTER(u32)]),
    "bc_engine_score": (i32, [vp, vp, vp, sz, vp, vp, vp]),
    "bc_engine_consumed": (u32, [vp]),
    "bc_seq_launches": (u64, [vp]),
    "bc_seq_set_skip": (i32, [vp, C.c_char_p, u32, u32]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library, declaring every signature. Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "bobcat_b200: %s is missing. Build it with `python -m bobcat_b200.build` "
            "(nvcc, sm_100a). There is no CPU fallback." % LIB_PATH)
    L = C.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(L, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = L
    return L
