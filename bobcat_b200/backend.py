"""``Cuda``: the op backend, with the method names and argument order of the reference's ``Metal``
(crates/bobcat-metal/src/backend.rs:1027-2698). Every method is a thin call into the C ABI; the
kernels live in ``libbobcat_cuda.so``."""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib, errors

F32, F16, Q4_0, Q8_0, Q6_K = 0, 1, 2, 8, 14
OVERWRITE, ACCUMULATE, SWIGLU = 0, 1, 2


class Buffer:
    """Device memory owned by one backend (``bobcat_metal::Buffer``, backend.rs:302-327)."""

    def __init__(self, cuda: "Cuda", handle):
        self.cuda = cuda
        self._h = handle

    def __len__(self) -> int:
        return int(self.cuda._L.bc_buffer_len(self._h))

    def at(self, offset: int) -> "View":
        return View(self, offset)

    def floats(self, index: int) -> "View":
        return View(self, index * 4)

    @property
    def device_ptr(self) -> int:
        return int(self.cuda._L.bc_buffer_device_ptr(self._h) or 0)

    def free(self) -> None:
        if self._h:
            self.cuda._L.bc_buffer_free(self._h)
            self._h = None

    def __del__(self):
        try:
            if self._h and self.cuda._h:
                self.free()
        except Exception:
            pass


@dataclass
class View:
    buffer: Buffer
    offset: int = 0


@dataclass
class Norm:
    """RMS normalisation fused into a multiply (backend.rs:344-350)."""
    weight: View
    eps: float


def _v(view):
    if view is None:
        return None, 0
    if isinstance(view, Buffer):
        return view._h, 0
    return view.buffer._h, view.offset


class Readback:
    """Token slots the CPU reads while later recordings still run (``Readback``, backend.rs:324-333)."""

    def __init__(self, cuda: "Cuda", handle):
        self.cuda, self._h = cuda, handle

    def close(self) -> None:
        if self._h:
            self.cuda._L.bc_readback_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Cuda:
    """One CUDA device, one stream, the buffers allocated on it, and the op launches."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self._L = _lib.load()
        h = C.c_void_p()
        errors.check(self._L.bc_backend_open(device, stream, C.byref(h)), self._L)
        self._h = h
        self.device = device

    @classmethod
    def open(cls, device: int = 0, stream: int | None = None) -> "Cuda":
        return cls(device, stream)

    def close(self) -> None:
        if self._h:
            self._L.bc_backend_close(self._h)
            self._h = None

    @property
    def stream(self) -> int:
        return int(self._L.bc_backend_stream(self._h) or 0)

    def _check(self, status: int) -> None:
        errors.check(status, self._L)

    # ---- buffers
    def new_buffer(self, n_bytes: int) -> Buffer:
        h = C.c_void_p()
        self._check(self._L.bc_buffer_new(self._h, n_bytes, C.byref(h)))
        return Buffer(self, h)

    def upload_matrix(self, fmt: int, raw: np.ndarray, n_rows: int, n_cols: int) -> Buffer:
        raw = np.ascontiguousarray(raw).view(np.uint8)
        h = C.c_void_p()
        self._check(self._L.bc_matrix_upload(self._h, fmt, raw.ctypes.data_as(C.c_void_p), n_rows, n_cols, C.byref(h)))
        return Buffer(self, h)

    def write(self, view, data: np.ndarray) -> None:
        b, off = _v(view)
        data = np.ascontiguousarray(data)
        self._check(self._L.bc_buffer_write(b, off, data.ctypes.data_as(C.c_void_p), data.nbytes))

    def read(self, view, out: np.ndarray) -> np.ndarray:
        b, off = _v(view)
        assert out.flags["C_CONTIGUOUS"]
        self._check(self._L.bc_buffer_read(b, off, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def buffer_from(self, data: np.ndarray) -> Buffer:
        data = np.ascontiguousarray(data)
        buf = self.new_buffer(max(data.nbytes, 4))
        if data.nbytes:
            self.write(buf, data)
        return buf

    # ---- submission
    def begin(self) -> None:
        self._check(self._L.bc_begin(self._h))

    def barrier(self) -> None:
        self._check(self._L.bc_barrier(self._h))

    def commit(self) -> int:
        t = C.c_uint64()
        self._check(self._L.bc_commit(self._h, C.byref(t)))
        return int(t.value)

    def wait(self, ticket: int) -> float:
        s = C.c_double()
        self._check(self._L.bc_wait(self._h, ticket, C.byref(s)))
        return float(s.value)

    def end(self) -> float:
        s = C.c_double()
        self._check(self._L.bc_end(self._h, C.byref(s)))
        return float(s.value)

    def discard(self) -> None:
        self._L.bc_discard(self._h)

    def set_profiling(self, enabled: bool) -> None:
        self._check(self._L.bc_set_profiling(self._h, int(enabled)))

    def profile(self) -> list[dict]:
        n = C.c_size_t()
        self._check(self._L.bc_profile(self._h, None, 0, C.byref(n)))
        arr = (_lib.ProfileEntry * max(1, n.value))()
        self._check(self._L.bc_profile(self._h, arr, n.value, C.byref(n)))
        return [dict(name=arr[i].name.decode(), n_rows=arr[i].n_rows, n_cols=arr[i].n_cols, calls=arr[i].calls,
                     seconds=arr[i].seconds, bytes=arr[i].bytes) for i in range(n.value)]

    # ---- ops (argument order follows the reference's methods)
    def matvec(self, fmt, weights, n_rows, n_cols, x, y, norm: Norm | None = None, accumulate: bool = False) -> None:
        nb, no = _v(norm.weight) if norm else (None, 0)
        self._check(self._L.bc_op_matvec(self._h, fmt, *_v(weights), n_rows, n_cols, *_v(x), *_v(y), nb, no,
                                         norm.eps if norm else 0.0, int(accumulate)))

    def matvec_swiglu(self, fmt, gate, up, n_rows, n_cols, x, norm: Norm, y) -> None:
        self._check(self._L.bc_op_matvec_swiglu(self._h, fmt, *_v(gate), *_v(up), n_rows, n_cols, *_v(x), *_v(norm.weight), norm.eps, *_v(y)))

    def matvec_conv(self, fmt, in_proj, n_cols, x, norm: Norm | None, taps, history, out, n_embd, kernel) -> None:
        nb, no = _v(norm.weight) if norm else (None, 0)
        self._check(self._L.bc_op_matvec_conv(self._h, fmt, *_v(in_proj), n_cols, *_v(x), nb, no, norm.eps if norm else 0.0,
                                              *_v(taps), *_v(history), *_v(out), n_embd, kernel))

    def short_conv(self, bcx, taps, history, out, n_embd, kernel, n_tokens) -> None:
        self._check(self._L.bc_op_short_conv(self._h, *_v(bcx), *_v(taps), *_v(history), *_v(out), n_embd, kernel, n_tokens))

    short_conv_batch = short_conv

    def matmul(self, fmt, weights, n_rows, n_cols, x, y, n_tokens, store) -> None:
        self._check(self._L.bc_op_matmul(self._h, fmt, *_v(weights), n_rows, n_cols, *_v(x), *_v(y), n_tokens, store))

    def expand(self, fmt, weights, out, n_rows, n_cols, out_half: bool = True) -> None:
        self._check(self._L.bc_op_expand(self._h, fmt, *_v(weights), *_v(out), n_rows, n_cols, int(out_half)))

    def embed(self, fmt, weights, n_vocab, tokens, out, n_embd, n_tokens) -> None:
        self._check(self._L.bc_op_embed(self._h, fmt, *_v(weights), n_vocab, *_v(tokens), *_v(out), n_embd, n_tokens))

    def rms_norm(self, x, weight, out, n_cols, n_rows, eps) -> None:
        self._check(self._L.bc_op_rms_norm(self._h, *_v(x), *_v(weight), *_v(out), n_cols, n_rows, eps))

    def norm_rope(self, src, dst, dst_half, weight, n_heads, head_dim, head_stride, n_rot, first_pos, n_tokens, src_stride,
                  dst_stride, theta, eps) -> None:
        self._check(self._L.bc_op_norm_rope(self._h, *_v(src), *_v(dst), int(dst_half), *_v(weight), n_heads, head_dim, head_stride,
                                            n_rot, first_pos, n_tokens, src_stride, dst_stride, theta, eps))

    def convert_half(self, src, dst, n) -> None:
        self._check(self._L.bc_op_convert_half(self._h, *_v(src), *_v(dst), n))

    def copy(self, src, dst, n) -> None:
        self._check(self._L.bc_op_copy(self._h, *_v(src), *_v(dst), n))

    def attention(self, q, k_cache, v_cache, kv_half, scratch, out, n_heads, n_kv_heads, head_dim, first_pos, n_queries, n_ctx) -> None:
        self._check(self._L.bc_op_attention(self._h, *_v(q), *_v(k_cache), *_v(v_cache), int(kv_half), *_v(scratch), *_v(out),
                                            n_heads, n_kv_heads, head_dim, first_pos, n_queries, n_ctx))

    def attention_scratch_floats(self, n_heads, head_dim, n_ctx, n_queries) -> int:
        return int(self._L.bc_attention_scratch_floats(n_heads, head_dim, n_ctx, n_queries))

    def argmax(self, x, out, n) -> None:
        self._check(self._L.bc_op_argmax(self._h, *_v(x), *_v(out), n))

    def sample(self, logits, n, recent, n_recent, settings: "_lib.Sampling", uniform: float, out) -> None:
        rb, ro = _v(recent) if recent is not None else (None, 0)
        self._check(self._L.bc_op_sample(self._h, *_v(logits), n, rb, ro, n_recent, C.byref(settings), uniform, *_v(out)))

    def new_readback(self, slots: int) -> "Readback":
        h = C.c_void_p()
        self._check(self._L.bc_readback_new(self._h, slots, C.byref(h)))
        return Readback(self, h)

    def argmax_readback(self, x, out, readback: "Readback", slot: int, n: int) -> None:
        self._check(self._L.bc_op_argmax_readback(self._h, *_v(x), *_v(out), readback._h, slot, n))

    def read_readback(self, readback: "Readback", slot: int) -> int:
        tok = C.c_uint32()
        self._check(self._L.bc_read_readback(self._h, readback._h, slot, C.byref(tok)))
        return int(tok.value)

    # ---- mixture of experts (argument order of backend.rs:1428-1737)
    def route_bytes(self, n_used, n_tokens) -> int:
        return int(self._L.bc_route_bytes(n_used, n_tokens))

    def moe_route(self, x, norm, router, bias, route, n_cols, n_experts, n_used, n_tokens) -> None:
        """``norm`` is None or ``(Norm, normed_view)``."""
        if norm is None:
            nb, no, eps, ob, oo = None, 0, 0.0, None, 0
        else:
            (nb, no), eps, (ob, oo) = _v(norm[0].weight), norm[0].eps, _v(norm[1])
        self._check(self._L.bc_op_moe_route(self._h, *_v(x), nb, no, eps, ob, oo, *_v(router), *_v(bias), *_v(route), n_cols, n_experts,
                                            n_used, n_tokens))

    def moe_group(self, route, offsets, entries, n_experts, n_used, n_tokens) -> None:
        self._check(self._L.bc_op_moe_group(self._h, *_v(route), *_v(offsets), *_v(entries), n_experts, n_used, n_tokens))

    def matvec_experts_swiglu(self, fmt, gate, up, n_rows, n_cols, n_experts, x, route, n_used, y, n_tokens) -> None:
        self._check(self._L.bc_op_matvec_experts_swiglu(self._h, fmt, *_v(gate), *_v(up), n_rows, n_cols, n_experts, *_v(x), *_v(route), n_used,
                                                        *_v(y), n_tokens))

    def matvec_experts_down(self, fmt, down, n_rows, n_cols, n_experts, x, route, n_used, y, n_tokens) -> None:
        self._check(self._L.bc_op_matvec_experts_down(self._h, fmt, *_v(down), n_rows, n_cols, n_experts, *_v(x), *_v(route), n_used, *_v(y),
                                                      n_tokens))

    def matmul_experts(self, fmt, weights, up, n_rows, n_cols, n_experts, x, gather, offsets, entries, n_used, y, n_tokens) -> None:
        ub, uo = _v(up)
        self._check(self._L.bc_op_matmul_experts(self._h, fmt, *_v(weights), ub, uo, n_rows, n_cols, n_experts, *_v(x), int(gather), *_v(offsets),
                                                 *_v(entries), n_used, *_v(y), n_tokens))

    def moe_combine(self, expert_out, route, y, n_embd, n_used, n_tokens) -> None:
        self._check(self._L.bc_op_moe_combine(self._h, *_v(expert_out), *_v(route), *_v(y), n_embd, n_used, n_tokens))

    # ---- Qwen3.5 (argument order of backend.rs:1739-2032)
    def gdn_conv(self, x, taps, history, out, conv_dim, kernel, n_tokens) -> None:
        self._check(self._L.bc_op_gdn_conv(self._h, *_v(x), *_v(taps), *_v(history), *_v(out), conv_dim, kernel, n_tokens))

    def gdn_gates(self, beta, alpha, a, dt_bias, n_v_heads, n_tokens) -> None:
        self._check(self._L.bc_op_gdn_gates(self._h, *_v(beta), *_v(alpha), *_v(a), *_v(dt_bias), n_v_heads, n_tokens))

    def gdn_recurrence(self, qkv, beta, decay, state, out, n_k_heads, n_v_heads, k_dim, v_dim, n_tokens, normalize=True) -> None:
        self._check(self._L.bc_op_gdn_recurrence(self._h, *_v(qkv), *_v(beta), *_v(decay), *_v(state), *_v(out), n_k_heads, n_v_heads, k_dim,
                                                 v_dim, n_tokens, int(normalize)))

    def gdn_gated_norm(self, x, z, weight, v_dim, n_rows, eps) -> None:
        self._check(self._L.bc_op_gdn_gated_norm(self._h, *_v(x), *_v(z), *_v(weight), v_dim, n_rows, eps))

    def attention_gate(self, out, q_gate, n_heads, head_dim, n_tokens) -> None:
        self._check(self._L.bc_op_attention_gate(self._h, *_v(out), *_v(q_gate), n_heads, head_dim, n_tokens))

    def silu_mul(self, x, gate, n) -> None:
        self._check(self._L.bc_op_silu_mul(self._h, *_v(x), *_v(gate), n))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
