"""``Model``, ``Lfm2Cuda`` and ``Qwen35Cuda``: the sequence API, with the method names of the
reference's ``lfm2::Model`` / ``Lfm2Metal`` (crates/bobcat/src/lfm2.rs:186, lfm2_metal.rs:103-762)
and ``Qwen35Metal`` (crates/bobcat/src/qwen35_metal.rs:112-676). All work happens in the C ABI."""

from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib, errors
from .backend import Cuda


class Trace:
    """Activations of a run of tokens (``lfm2::Trace``, lfm2.rs:630-675)."""

    def __init__(self, n_embd: int, n_layers: int, n_tokens: int):
        self.embedding = np.zeros((n_tokens, n_embd), dtype=np.float32)
        self.layers = np.zeros((n_layers, n_tokens, n_embd), dtype=np.float32)
        self.final_norm = np.zeros((n_tokens, n_embd), dtype=np.float32)
        self.n_tokens = n_tokens

    def _c(self) -> _lib.Trace:
        fp = C.POINTER(C.c_float)
        return _lib.Trace(self.embedding.ctypes.data_as(fp), self.layers.ctypes.data_as(fp), self.final_norm.ctypes.data_as(fp), self.n_tokens)


class Model:
    """A GGUF model on the host (``Model::load``)."""

    def __init__(self, path: str):
        self._L = _lib.load()
        h = C.c_void_p()
        errors.check(self._L.bc_model_load(str(path).encode(), C.byref(h)), self._L)
        self._h = h
        hp = _lib.Hparams()
        errors.check(self._L.bc_model_hparams(self._h, C.byref(hp)), self._L)
        self.hp = hp

    @classmethod
    def load(cls, path: str) -> "Model":
        return cls(path)

    def hyperparameters(self) -> _lib.Hparams:
        return self.hp

    def attention_layers(self) -> list[bool]:
        out = np.zeros(self.hp.n_layers, dtype=np.uint8)
        errors.check(self._L.bc_model_attention_layers(self._h, out.ctypes.data_as(C.c_void_p), out.size), self._L)
        return [bool(v) for v in out]

    def decode_bytes(self) -> int:
        return int(self._L.bc_model_decode_bytes(self._h))

    def trace(self, n_tokens: int) -> Trace:
        return Trace(self.hp.n_embd, self.hp.n_layers, n_tokens)

    def close(self) -> None:
        if self._h:
            self._L.bc_model_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Checkpoint:
    def __init__(self, lib, handle):
        self._L, self._h = lib, handle

    def __del__(self):
        try:
            if self._h:
                self._L.bc_checkpoint_free(self._h)
                self._h = None
        except Exception:
            pass


class Prefix:
    """A cached prefix on the device (``bc_prefix``)."""

    def __init__(self, lib, handle):
        self._L, self._h = lib, handle

    def n_past(self) -> int:
        return int(self._L.bc_prefix_n_past(self._h))

    def close(self) -> None:
        if self._h:
            self._L.bc_prefix_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class SeqCuda:
    """The device state of one decode. ``Lfm2Cuda`` and ``Qwen35Cuda`` are this class."""

    def __init__(self, model: Model, cuda: Cuda, n_ctx: int, kv_half: bool, _borrowed=None, comm=None, paged: bool = False):
        """With ``comm`` (a ``sharding.Comm``) the sequence is tensor-parallel over the
        communicator's ranks: every rank creates one and calls the same methods. With ``paged``
        the KV caches are made of pages that cached prefixes can share."""
        self._L = _lib.load()
        self.model, self.cuda, self.comm = model, cuda, comm
        self._owned = _borrowed is None
        if _borrowed is None and paged:
            h = C.c_void_p()
            errors.check(self._L.bc_seq_new_paged(model._h, cuda._h, n_ctx, int(kv_half), C.byref(h)), self._L)
        elif _borrowed is None and comm is not None:
            h = C.c_void_p()
            errors.check(self._L.bc_seq_new_tensor_parallel(model._h, cuda._h, comm._h, n_ctx, int(kv_half), C.byref(h)), self._L)
        elif _borrowed is None:
            h = C.c_void_p()
            errors.check(self._L.bc_seq_new(model._h, cuda._h, n_ctx, int(kv_half), C.byref(h)), self._L)
        else:
            h = _borrowed
        self._h = h
        self.n_ctx = n_ctx

    def _check(self, status: int) -> None:
        errors.check(status, self._L)

    def n_past(self) -> int:
        return int(self._L.bc_seq_n_past(self._h))

    def launches(self) -> int:
        return int(self._L.bc_seq_launches(self._h))

    def step(self, token: int, logits: np.ndarray | None = None, trace: Trace | None = None) -> None:
        t = trace._c() if trace is not None else None
        self._check(self._L.bc_seq_step(self._h, token, logits.ctypes.data_as(C.c_void_p) if logits is not None else None,
                                        logits.size if logits is not None else 0, C.byref(t) if t is not None else None))

    def prefill(self, tokens, logits: np.ndarray | None = None, final_norm: np.ndarray | None = None, trace: Trace | None = None) -> None:
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        t = trace._c() if trace is not None else None
        p = lambda a: a.ctypes.data_as(C.c_void_p) if a is not None else None
        n = lambda a: a.size if a is not None else 0
        self._check(self._L.bc_seq_prefill(self._h, p(tokens), tokens.size, p(logits), n(logits), p(final_norm), n(final_norm),
                                           C.byref(t) if t is not None else None))

    def greedy_token(self) -> int:
        tok = C.c_uint32()
        self._check(self._L.bc_seq_greedy_token(self._h, C.byref(tok)))
        return int(tok.value)

    def generate(self, n: int) -> np.ndarray:
        out = np.zeros(n, dtype=np.uint32)
        self._check(self._L.bc_seq_generate(self._h, out.ctypes.data_as(C.c_void_p), n))
        return out

    def sample(self, settings: "_lib.Sampling", uniform: float, recent=()) -> int:
        """The next token from the current logits by the reference sampler's rules, on the device."""
        recent = np.ascontiguousarray(recent, dtype=np.uint32)
        tok = C.c_uint32()
        self._check(self._L.bc_seq_sample(self._h, C.byref(settings), uniform, recent.ctypes.data_as(C.c_void_p) if recent.size else None,
                                          recent.size, C.byref(tok)))
        return int(tok.value)

    def generate_next(self, n: int) -> np.ndarray:
        out = np.zeros(n, dtype=np.uint32)
        self._check(self._L.bc_seq_generate_next(self._h, out.ctypes.data_as(C.c_void_p), n))
        return out

    def generate_stream(self, max_tokens: int, emit) -> np.ndarray:
        """``emit(token) -> bool``; returns the tokens the sequence gained."""
        failure = []

        def trampoline(token, _user):
            try:
                return 1 if emit(int(token)) else 0
            except Exception as e:  # an exception must not cross the C boundary
                failure.append(e)
                return 0

        cb = _lib.EMIT_FN(trampoline)
        gained = np.zeros(max(1, max_tokens), dtype=np.uint32)
        n = C.c_size_t()
        self._check(self._L.bc_seq_generate_stream(self._h, max_tokens, cb, None, gained.ctypes.data_as(C.c_void_p), gained.size, C.byref(n)))
        if failure:
            raise failure[0]
        return gained[: n.value].copy()

    def reset(self) -> None:
        self._check(self._L.bc_seq_reset(self._h))

    def checkpoint(self) -> Checkpoint:
        h = C.c_void_p()
        self._check(self._L.bc_seq_checkpoint(self._h, C.byref(h)))
        return Checkpoint(self._L, h)

    def restore(self, checkpoint: Checkpoint) -> None:
        self._check(self._L.bc_seq_restore(self._h, checkpoint._h))

    def save_prefix(self) -> "Prefix":
        h = C.c_void_p()
        self._check(self._L.bc_seq_prefix_save(self._h, C.byref(h)))
        return Prefix(self._L, h)

    def load_prefix(self, prefix: "Prefix") -> None:
        self._check(self._L.bc_seq_prefix_load(self._h, prefix._h))

    def kv_pages(self) -> tuple[int, int, int]:
        """(positions per page, pages mapped, pages shared); zeros with contiguous caches."""
        a, b, c = C.c_uint32(), C.c_uint32(), C.c_uint32()
        self._check(self._L.bc_seq_kv_pages(self._h, C.byref(a), C.byref(b), C.byref(c)))
        return int(a.value), int(b.value), int(c.value)

    def timings(self) -> tuple[float, float]:
        e, g = C.c_double(), C.c_double()
        self._check(self._L.bc_seq_timings(self._h, C.byref(e), C.byref(g)))
        return float(e.value), float(g.value)

    def last_encode_seconds(self) -> float:
        return self.timings()[0]

    def last_gpu_seconds(self) -> float:
        return self.timings()[1]

    def read_state(self, which: int, layer: int = 0) -> np.ndarray:
        n = C.c_size_t()
        self._check(self._L.bc_seq_read_state(self._h, which, layer, None, 0, C.byref(n)))
        out = np.zeros(n.value, dtype=np.float32)
        if n.value:
            self._check(self._L.bc_seq_read_state(self._h, which, layer, out.ctypes.data_as(C.c_void_p), out.size, C.byref(n)))
        return out

    def set_skip(self, name: str | None, n_rows: int = 0, n_cols: int = 0) -> None:
        """Timing diagnostics: leave one kind of launch out of the forward passes (None restores)."""
        self._check(self._L.bc_seq_set_skip(self._h, name.encode() if name else None, n_rows, n_cols))

    def traced_routes(self) -> np.ndarray:
        """Expert ids the last traced pass picked: [layer][trace row][n_used] (rows of layers
        without experts are zero)."""
        hp = self.model.hp
        words = self.read_state(4).view(np.uint32)
        return words.reshape(hp.n_layers, -1, 2 * hp.n_experts_used)[:, :, : hp.n_experts_used].copy()

    def close(self) -> None:
        if self._h:
            if self._owned:
                self._L.bc_seq_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


Lfm2Cuda = SeqCuda
Qwen35Cuda = SeqCuda


class BatchCuda:
    """Several sequences of one model that decode together, one token each per pass (the C ABI's
    ``bc_batch``): ``seq(i)`` is sequence i with the single-sequence methods (prefill, reset, ...),
    ``generate(n)`` gives every sequence n greedy tokens and returns them as [n_seqs][n]."""

    def __init__(self, model: Model, cuda: Cuda, n_seqs: int, n_ctx: int, kv_half: bool, comm=None):
        """With ``comm`` (a ``sharding.Comm``) the experts of a mixture-of-experts model are sharded
        over the communicator's ranks and ``n_seqs`` counts this rank's own sequences."""
        self._L = _lib.load()
        self.model, self.cuda, self.n_seqs, self.n_ctx, self.comm = model, cuda, n_seqs, n_ctx, comm
        h = C.c_void_p()
        if comm is None:
            errors.check(self._L.bc_batch_new(model._h, cuda._h, n_seqs, n_ctx, int(kv_half), C.byref(h)), self._L)
        else:
            errors.check(self._L.bc_batch_new_expert_parallel(model._h, cuda._h, comm._h, n_seqs, n_ctx, int(kv_half), C.byref(h)), self._L)
        self._h = h
        self._seqs = []
        for i in range(n_seqs):
            sh = C.c_void_p()
            errors.check(self._L.bc_batch_seq(self._h, i, C.byref(sh)), self._L)
            self._seqs.append(SeqCuda(model, cuda, n_ctx, kv_half, _borrowed=sh))

    def seq(self, index: int) -> SeqCuda:
        return self._seqs[index]

    def set_exact(self, exact: bool) -> None:
        """f32 operands on the f32 tile kernels (True) or half-precision operands on the tensor
        cores (False, the default) for the batched pass."""
        errors.check(self._L.bc_batch_set_exact(self._h, int(exact)), self._L)

    def generate(self, n: int) -> np.ndarray:
        out = np.zeros((self.n_seqs, n), dtype=np.uint32)
        errors.check(self._L.bc_batch_generate(self._h, out.ctypes.data_as(C.c_void_p), n), self._L)
        return out

    def last_gpu_seconds(self) -> float:
        g = C.c_double()
        errors.check(self._L.bc_batch_timings(self._h, C.byref(g), None), self._L)
        return float(g.value)

    def launches(self) -> int:
        n = C.c_uint64()
        errors.check(self._L.bc_batch_timings(self._h, None, C.byref(n)), self._L)
        return int(n.value)

    def close(self) -> None:
        if self._h:
            for s in self._seqs:
                s.close()
            self._L.bc_batch_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass



class Engine:
    """The token-level half of the reference's ``Engine`` (crates/bobcat-cli/src/engine.rs): a
    sequence that reuses what earlier requests left on the device, and ``score``."""

    def __init__(self, model: Model, cuda: Cuda, n_ctx: int, kv_half: bool = True, seed: int = 0):
        self._L = _lib.load()
        self.model, self.cuda = model, cuda
        h = C.c_void_p()
        errors.check(self._L.bc_engine_new(model._h, cuda._h, n_ctx, int(kv_half), seed, C.byref(h)), self._L)
        self._h = h

    def generate(self, tokens, max_tokens: int, turn: int = -1, sampling=None, emit=None) -> tuple[list[int], int]:
        """Returns (generated tokens, prompt tokens that were already on the device)."""
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        out = np.zeros(max(1, max_tokens), dtype=np.uint32)
        n, cached = C.c_size_t(), C.c_uint32()
        failure = []

        def trampoline(token, _user):
            try:
                return 1 if emit(int(token)) else 0
            except Exception as e:
                failure.append(e)
                return 0

        cb = _lib.EMIT_FN(trampoline) if emit else C.cast(None, _lib.EMIT_FN)
        errors.check(self._L.bc_engine_generate(self._h, tokens.ctypes.data_as(C.c_void_p), tokens.size, turn, max_tokens,
                                                C.byref(sampling) if sampling is not None else None, cb, None,
                                                out.ctypes.data_as(C.c_void_p), out.size, C.byref(n), C.byref(cached)), self._L)
        if failure:
            raise failure[0]
        return out[: n.value].tolist(), int(cached.value)

    def score(self, prompts, labels) -> list[list[float]]:
        flat_p = np.concatenate([np.asarray(p, dtype=np.uint32) for p in prompts]) if prompts else np.zeros(0, dtype=np.uint32)
        flat_l = np.concatenate([np.asarray(l, dtype=np.uint32) for l in labels] + [np.zeros(0, dtype=np.uint32)])
        off_p = np.cumsum([0] + [len(p) for p in prompts]).astype(np.uint64)
        off_l = np.cumsum([0] + [len(l) for l in labels]).astype(np.uint64)
        scores = np.zeros(max(1, flat_l.size), dtype=np.float64)
        ptr = lambda a: a.ctypes.data_as(C.c_void_p)
        errors.check(self._L.bc_engine_score(self._h, ptr(flat_p), ptr(off_p), len(prompts), ptr(flat_l), ptr(off_l), ptr(scores)), self._L)
        return [scores[int(off_l[i]):int(off_l[i + 1])].tolist() for i in range(len(prompts))]

    def consumed(self) -> int:
        return int(self._L.bc_engine_consumed(self._h))

    def close(self) -> None:
        if self._h:
            self._L.bc_engine_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
