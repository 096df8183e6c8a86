"""ctypes binding of the CPU parity checker (test infrastructure, not product code).

Only the tests, the smoke check and the benchmark's CPU-baseline leg import this module. The GGUF
file is parsed here with the third-party ``gguf`` package (the version the reference's tooling
pins), independently of the product's own C++ GGUF reader, and the tensors are handed to the C++
restatement by name.
"""

from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    path = _build.build()
    L = C.CDLL(path)
    vp, u32, u64, f32p = C.c_void_p, C.c_uint32, C.c_uint64, C.POINTER(C.c_float)
    L.orc_model_new.restype = vp
    L.orc_model_new.argtypes = [C.c_char_p]
    L.orc_model_free.argtypes = [vp]
    L.orc_model_set_u32.argtypes = [vp, C.c_char_p, u32]
    L.orc_model_set_f32.argtypes = [vp, C.c_char_p, C.c_float]
    L.orc_model_set_array.argtypes = [vp, C.c_char_p, C.POINTER(u32), u64]
    L.orc_model_add_tensor.argtypes = [vp, C.c_char_p, u32, vp, C.POINTER(u64), u32]
    L.orc_model_set_threads.argtypes = [vp, C.c_int]
    L.orc_model_finish.argtypes = [vp]
    L.orc_model_finish.restype = C.c_int
    L.orc_model_error.argtypes = [vp]
    L.orc_model_error.restype = C.c_char_p
    L.orc_model_shape.argtypes = [vp, C.POINTER(u32)]
    L.orc_state_new.restype = vp
    L.orc_state_new.argtypes = [vp, u32]
    L.orc_state_free.argtypes = [vp]
    L.orc_state_n_past.argtypes = [vp]
    L.orc_state_n_past.restype = u32
    L.orc_step.argtypes = [vp, u32, vp, vp, vp, vp, vp]
    L.orc_step.restype = C.c_int
    for name in ("orc_state_conv", "orc_state_delta"):
        fn = getattr(L, name)
        fn.argtypes = [vp, u32, vp]
        fn.restype = u64
    L.orc_state_kv.argtypes = [vp, u32, C.c_int, vp]
    L.orc_state_kv.restype = u64
    L.orc_dequantize.argtypes = [u32, vp, u64, vp]
    L.orc_matvec.argtypes = [u32, vp, vp, u64, vp, u64, C.c_int]
    L.orc_rms_norm.argtypes = [vp, vp, u64, C.c_float, vp]
    L.orc_rope_neox.argtypes = [vp, u64, u32, C.c_float]
    L.orc_softmax.argtypes = [vp, u64]
    L.orc_silu.argtypes = [C.c_float]
    L.orc_silu.restype = C.c_float
    L.orc_dot.argtypes = [vp, vp, u64]
    L.orc_dot.restype = C.c_float
    L.orc_lfm2_route.argtypes = [vp, vp, u64, u64, vp]
    L.orc_f16_to_f32.argtypes = [C.c_uint16]
    L.orc_f16_to_f32.restype = C.c_float
    _lib = L
    return L


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def default_threads() -> int:
    return max(1, len(os.sched_getaffinity(0)))


# ---------------------------------------------------------------------------------------------
# scalar ops
# ---------------------------------------------------------------------------------------------

TYPE_IDS = {"F32": 0, "F16": 1, "Q4_0": 2, "Q8_0": 8, "Q6_K": 14, "BF16": 30}


def dequantize(type_id: int, raw: np.ndarray, n: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw).view(np.uint8)
    out = np.empty(n, dtype=np.float32)
    lib().orc_dequantize(type_id, _ptr(raw), n, _ptr(out))
    return out


def matvec(type_id: int, raw: np.ndarray, x: np.ndarray, n_rows: int, threads: int | None = None) -> np.ndarray:
    raw = np.ascontiguousarray(raw).view(np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(n_rows, dtype=np.float32)
    lib().orc_matvec(type_id, _ptr(raw), _ptr(x), x.size, _ptr(y), n_rows, threads or default_threads())
    return y


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty_like(x)
    lib().orc_rms_norm(_ptr(x), _ptr(w), x.size, eps, _ptr(out))
    return out


def rope_neox(vec: np.ndarray, pos: int, theta: float) -> np.ndarray:
    out = np.ascontiguousarray(vec, dtype=np.float32).copy()
    lib().orc_rope_neox(_ptr(out), out.size, pos, theta)
    return out


def softmax(x: np.ndarray) -> np.ndarray:
    out = np.ascontiguousarray(x, dtype=np.float32).copy()
    lib().orc_softmax(_ptr(out), out.size)
    return out


def silu(x: float) -> float:
    return float(lib().orc_silu(x))


def lfm2_route(logits: np.ndarray, bias: np.ndarray, n_used: int):
    """Return (ids of every expert, picked first; scores with picked entries turned into weights)."""
    scores = np.ascontiguousarray(logits, dtype=np.float32).copy()
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    experts = np.empty(scores.size, dtype=np.uint32)
    lib().orc_lfm2_route(_ptr(scores), _ptr(bias), scores.size, n_used, _ptr(experts))
    return experts, scores


# ---------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------


class Model:
    """A GGUF model held by the CPU checker. ``step`` mirrors the reference's ``Model::step``."""

    def __init__(self, path: str, threads: int | None = None):
        import gguf

        L = lib()
        self._reader = gguf.GGUFReader(path)  # keeps the memory map (and so the tensor bytes) alive
        fields = self._reader.fields
        arch = fields["general.architecture"].contents()
        self.architecture = arch
        self._h = L.orc_model_new(arch.encode())
        for key, field in fields.items():
            if not key.startswith(arch + "."):
                continue
            value = field.contents()
            k = key.encode()
            if isinstance(value, bool):
                continue
            if isinstance(value, int):
                L.orc_model_set_u32(self._h, k, value)
            elif isinstance(value, float):
                L.orc_model_set_f32(self._h, k, value)
            elif isinstance(value, list) and value and all(isinstance(v, int) for v in value):
                arr = (C.c_uint32 * len(value))(*value)
                L.orc_model_set_array(self._h, k, arr, len(value))
        self._keep = []
        for t in self._reader.tensors:
            shape = [int(d) for d in t.shape]
            arr = (C.c_uint64 * len(shape))(*shape)
            data = np.ascontiguousarray(t.data)
            self._keep.append(data)
            L.orc_model_add_tensor(self._h, t.name.encode(), int(t.tensor_type), _ptr(data), arr, len(shape))
        L.orc_model_set_threads(self._h, threads or default_threads())
        if L.orc_model_finish(self._h) != 0:
            raise ValueError("oracle could not load %s: %s" % (path, L.orc_model_error(self._h).decode()))
        shape = (C.c_uint32 * 11)()
        L.orc_model_shape(self._h, shape)
        (self.n_layers, self.n_embd, self.n_vocab, self.n_attention_layers, self.n_other_layers, self.n_heads,
         self.n_kv_heads, self.head_dim, self.n_ff, self.n_experts, self.n_experts_used) = [int(v) for v in shape]

    def set_threads(self, threads: int) -> None:
        lib().orc_model_set_threads(self._h, threads)

    def state(self, n_ctx: int) -> "State":
        return State(self, n_ctx)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_model_free(self._h)
            self._h = None


class State:
    def __init__(self, model: Model, n_ctx: int):
        self.model = model
        self.n_ctx = n_ctx
        self._h = lib().orc_state_new(model._h, n_ctx)
        if not self._h:
            raise ValueError("the context must hold a token")

    @property
    def n_past(self) -> int:
        return int(lib().orc_state_n_past(self._h))

    def step(self, token: int, want_logits: bool = True, want_trace: bool = False, want_experts: bool = False):
        """Run one token. Returns a dict with the requested outputs."""
        m = self.model
        out = {}
        logits = np.empty(m.n_vocab, dtype=np.float32) if want_logits else None
        emb = np.empty(m.n_embd, dtype=np.float32) if want_trace else None
        layers = np.empty((m.n_layers, m.n_embd), dtype=np.float32) if want_trace else None
        final = np.empty(m.n_embd, dtype=np.float32) if want_trace else None
        experts = None
        if want_experts and m.n_experts_used:
            experts = np.full((m.n_layers, m.n_experts_used), -1, dtype=np.int32)
        p = lambda a: _ptr(a) if a is not None else None
        rc = lib().orc_step(self._h, token, p(logits), p(emb), p(layers), p(final), p(experts))
        if rc == 1:
            raise IndexError("context full")
        if rc == 2:
            raise ValueError("token outside the vocabulary")
        if want_logits:
            out["logits"] = logits
        if want_trace:
            out.update(embedding=emb, layers=layers, final_norm=final)
        if experts is not None:
            out["experts"] = experts
        return out

    def _read(self, fn, *args):
        n = int(fn(self._h, *args, None))
        out = np.empty(n, dtype=np.float32)
        fn(self._h, *args, _ptr(out))
        return out

    def conv_state(self, index: int = 0) -> np.ndarray:
        return self._read(lib().orc_state_conv, index)

    def delta_state(self, index: int) -> np.ndarray:
        return self._read(lib().orc_state_delta, index)

    def kv(self, index: int, which: int) -> np.ndarray:
        return self._read(lib().orc_state_kv, index, which)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_state_free(self._h)
            self._h = None


def greedy(model: Model, prompt, n_decode: int, n_ctx: int | None = None):
    """Prompt then greedy decode, as the reference's tests do (first maximum wins).
    Returns (generated tokens, logits after the last prompt token)."""
    st = model.state(n_ctx or (len(prompt) + n_decode + 1))
    logits = None
    for i, tok in enumerate(prompt):
        logits = st.step(int(tok), want_logits=(i == len(prompt) - 1)).get("logits")
    prompt_logits = logits
    out = []
    for _ in range(n_decode):
        tok = int(np.argmax(logits))
        out.append(tok)
        logits = st.step(tok)["logits"]
    return out, prompt_logits
