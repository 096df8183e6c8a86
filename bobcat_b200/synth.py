"""Synthetic model files: random-init GGUF models with the shapes, metadata keys and tensor names
the reference's loaders demand (crates/bobcat/src/lfm2.rs:737-1004, crates/bobcat/src/qwen35.rs:
629-752). They stand in for the downloaded checkpoints the reference benchmarks on.

Recipe (fixed; the tensor order below is part of it because each tensor's random stream is keyed
by its position): every linear is N(0, 0.02) quantised to Q4_0; embeddings, conv taps, routers,
biases and DeltaNet vectors are N(0, 0.02) in F32; every norm weight is 1.0; ``ssm_a`` is
-exp(N(0, 0.02)) so the DeltaNet state decays. Values are drawn by ``libbobcat_synth.so`` (plain
C++, built from ``synthlib/`` with g++; not part of the product library) with a counter-based
generator, so a file depends only on (config, seed), not on thread count.
"""

from __future__ import annotations

import ctypes as C
import os
import subprocess

F32, Q4_0, Q8_0 = 0, 2, 8
NORMAL, CONSTANT, NEG_EXP_NORMAL = 0, 1, 2
STD = 0.02

HERE = os.path.dirname(os.path.abspath(__file__))
SYNTH_SOURCES = [os.path.join(HERE, "synthlib", "gguf_writer.cpp"), os.path.join(HERE, "synthlib", "synth_writer.h")]
SYNTH_LIB = os.path.join(HERE, "libbobcat_synth.so")
_synth = None


def build_writer(force: bool = False) -> str:
    """Compile the writer library in-tree when it is missing or older than its sources."""
    stale = force or not os.path.exists(SYNTH_LIB) or any(os.path.getmtime(f) > os.path.getmtime(SYNTH_LIB) for f in SYNTH_SOURCES)
    if stale:
        subprocess.run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-o", SYNTH_LIB, SYNTH_SOURCES[0], "-lpthread"], check=True)
    return SYNTH_LIB


def _writer_lib() -> C.CDLL:
    global _synth
    if _synth is None:
        L = C.CDLL(build_writer())
        vp, u32, u64, i32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32
        L.bcs_last_error.restype = C.c_char_p
        L.bcs_writer_new.argtypes = [C.c_char_p, u64, C.POINTER(vp)]
        L.bcs_writer_kv_u32.argtypes = [vp, C.c_char_p, u32]
        L.bcs_writer_kv_f32.argtypes = [vp, C.c_char_p, C.c_float]
        L.bcs_writer_kv_str.argtypes = [vp, C.c_char_p, C.c_char_p]
        L.bcs_writer_kv_u32_array.argtypes = [vp, C.c_char_p, C.POINTER(u32), u64]
        L.bcs_writer_tensor.argtypes = [vp, C.c_char_p, i32, C.POINTER(u64), u32, i32, C.c_float]
        L.bcs_writer_finish.argtypes = [vp]
        _synth = L
    return _synth


def _check(status: int, L) -> None:
    if status != 0:
        raise OSError("synthetic model writer: %s" % L.bcs_last_error().decode())


def _even_attention(n_layers: int, n_attention: int) -> list[int]:
    return [(i + 1) * n_layers // n_attention - 1 for i in range(n_attention)]


# The five benchmark shapes, then small shapes of the same families for tests.
CONFIGS: dict[str, dict] = {
    "lfm2-350m": dict(arch="lfm2", vocab=65536, hidden=1024, layers=16, attention=[2, 5, 8, 10, 12, 14], heads=16, kv_heads=8,
                      ff=4608, conv_kernel=3, theta=1e6, eps=1e-5),
    "lfm2-2.6b": dict(arch="lfm2", vocab=65536, hidden=2048, layers=30, attention=_even_attention(30, 8), heads=32, kv_heads=8,
                      ff=10752, conv_kernel=3, theta=1e6, eps=1e-5),
    "qwen35-2b": dict(arch="qwen35", vocab=151936, hidden=2048, layers=24, heads=8, kv_heads=2, head_dim=256, n_rot=64, ff=6144,
                      k_heads=16, v_heads=32, k_dim=128, v_dim=128, conv_kernel=4, theta=1e7, eps=1e-6),
    "lfm2moe-8b-a1b": dict(arch="lfm2moe", vocab=65536, hidden=2048, layers=24, attention=_even_attention(24, 6), heads=32, kv_heads=8,
                           ff=7168, conv_kernel=3, theta=1e6, eps=1e-5, experts=32, experts_used=4, ff_expert=1792, dense_layers=2),
    "qwen35-9b": dict(arch="qwen35", vocab=151936, hidden=4096, layers=32, heads=16, kv_heads=4, head_dim=256, n_rot=64, ff=12288,
                      k_heads=16, v_heads=32, k_dim=128, v_dim=128, conv_kernel=4, theta=1e7, eps=1e-6),
    "lfm2-tiny": dict(arch="lfm2", vocab=512, hidden=128, layers=4, attention=[1, 3], heads=4, kv_heads=2, ff=256, conv_kernel=3,
                      theta=1e6, eps=1e-5),
    "lfm2-small": dict(arch="lfm2", vocab=2048, hidden=256, layers=6, attention=[2, 5], heads=8, kv_heads=2, ff=704, conv_kernel=3,
                       theta=1e6, eps=1e-5),
    # Wide enough that every pipeline of the prefill kernels wraps its stages many times (16 chunks of 64 columns
    # in the projections, 44 in the down projection) and heads of 64 elements take the tensor-core attention.
    "lfm2-medium": dict(arch="lfm2", vocab=4096, hidden=1024, layers=4, attention=[1, 3], heads=16, kv_heads=4, ff=2816, conv_kernel=3,
                        theta=1e6, eps=1e-5),
    # The embedding (and tied output) matrix in Q8_0, as quantised checkpoints keep it in a quantised type.
    "lfm2-tiny-q8": dict(arch="lfm2", vocab=512, hidden=128, layers=4, attention=[1, 3], heads=4, kv_heads=2, ff=256, conv_kernel=3,
                         theta=1e6, eps=1e-5, embd_type=Q8_0),
    "lfm2moe-tiny": dict(arch="lfm2moe", vocab=512, hidden=128, layers=4, attention=[1, 3], heads=4, kv_heads=2, ff=256, conv_kernel=3,
                         theta=1e6, eps=1e-5, experts=8, experts_used=2, ff_expert=96, dense_layers=1),
    "qwen35-tiny": dict(arch="qwen35", vocab=512, hidden=128, layers=4, heads=2, kv_heads=1, head_dim=64, n_rot=32, ff=256, k_heads=2,
                        v_heads=4, k_dim=32, v_dim=32, conv_kernel=4, theta=1e7, eps=1e-6),
}


class _Writer:
    def __init__(self, path: str, seed: int):
        self.L = _writer_lib()
        h = C.c_void_p()
        _check(self.L.bcs_writer_new(path.encode(), seed, C.byref(h)), self.L)
        self.h = h

    def u32(self, key, value):
        _check(self.L.bcs_writer_kv_u32(self.h, key.encode(), value), self.L)

    def f32(self, key, value):
        _check(self.L.bcs_writer_kv_f32(self.h, key.encode(), value), self.L)

    def string(self, key, value):
        _check(self.L.bcs_writer_kv_str(self.h, key.encode(), value.encode()), self.L)

    def array(self, key, values):
        arr = (C.c_uint32 * len(values))(*values)
        _check(self.L.bcs_writer_kv_u32_array(self.h, key.encode(), arr, len(values)), self.L)

    def tensor(self, name, ttype, dims, init=NORMAL, value=STD):
        arr = (C.c_uint64 * len(dims))(*dims)
        _check(self.L.bcs_writer_tensor(self.h, name.encode(), ttype, arr, len(dims), init, value), self.L)

    def ones(self, name, dims):
        self.tensor(name, F32, dims, CONSTANT, 1.0)

    def finish(self):
        h, self.h = self.h, None
        _check(self.L.bcs_writer_finish(h), self.L)


def _write_lfm2(w: _Writer, c: dict) -> None:
    arch = c["arch"]
    hidden, layers = c["hidden"], c["layers"]
    attention = set(c["attention"])
    head_dim = hidden // c["heads"]
    w.string("general.architecture", arch)
    w.u32(f"{arch}.block_count", layers)
    w.u32(f"{arch}.embedding_length", hidden)
    w.u32(f"{arch}.feed_forward_length", c["ff"])
    w.u32(f"{arch}.attention.head_count", c["heads"])
    w.array(f"{arch}.attention.head_count_kv", [c["kv_heads"] if il in attention else 0 for il in range(layers)])
    w.u32(f"{arch}.shortconv.l_cache", c["conv_kernel"])
    w.f32(f"{arch}.rope.freq_base", c["theta"])
    w.f32(f"{arch}.attention.layer_norm_rms_epsilon", c["eps"])
    moe = arch == "lfm2moe"
    if moe:
        w.u32(f"{arch}.expert_count", c["experts"])
        w.u32(f"{arch}.expert_used_count", c["experts_used"])
        w.u32(f"{arch}.expert_feed_forward_length", c["ff_expert"])
        w.u32(f"{arch}.expert_gating_func", 2)
        w.u32(f"{arch}.leading_dense_block_count", c["dense_layers"])
    w.tensor("token_embd.weight", c.get("embd_type", F32), [hidden, c["vocab"]])
    w.ones("token_embd_norm.weight", [hidden])
    for il in range(layers):
        p = f"blk.{il}."
        w.ones(p + "attn_norm.weight", [hidden])
        w.ones(p + "ffn_norm.weight", [hidden])
        if il in attention:
            w.tensor(p + "attn_q.weight", Q4_0, [hidden, c["heads"] * head_dim])
            w.tensor(p + "attn_k.weight", Q4_0, [hidden, c["kv_heads"] * head_dim])
            w.tensor(p + "attn_v.weight", Q4_0, [hidden, c["kv_heads"] * head_dim])
            w.tensor(p + "attn_output.weight", Q4_0, [c["heads"] * head_dim, hidden])
            w.ones(p + "attn_q_norm.weight", [head_dim])
            w.ones(p + "attn_k_norm.weight", [head_dim])
        else:
            w.tensor(p + "shortconv.conv.weight", F32, [c["conv_kernel"], hidden])
            w.tensor(p + "shortconv.in_proj.weight", Q4_0, [hidden, 3 * hidden])
            w.tensor(p + "shortconv.out_proj.weight", Q4_0, [hidden, hidden])
        if moe and il >= c["dense_layers"]:
            w.tensor(p + "ffn_gate_inp.weight", F32, [hidden, c["experts"]])
            w.tensor(p + "exp_probs_b.bias", F32, [c["experts"]])
            w.tensor(p + "ffn_gate_exps.weight", Q4_0, [hidden, c["ff_expert"], c["experts"]])
            w.tensor(p + "ffn_up_exps.weight", Q4_0, [hidden, c["ff_expert"], c["experts"]])
            w.tensor(p + "ffn_down_exps.weight", Q4_0, [c["ff_expert"], hidden, c["experts"]])
        else:
            w.tensor(p + "ffn_gate.weight", Q4_0, [hidden, c["ff"]])
            w.tensor(p + "ffn_up.weight", Q4_0, [hidden, c["ff"]])
            w.tensor(p + "ffn_down.weight", Q4_0, [c["ff"], hidden])


def _write_qwen35(w: _Writer, c: dict) -> None:
    hidden, layers, hd = c["hidden"], c["layers"], c["head_dim"]
    key_dim, value_dim = c["k_heads"] * c["k_dim"], c["v_heads"] * c["v_dim"]
    conv_dim = 2 * key_dim + value_dim
    a = "qwen35"
    w.string("general.architecture", a)
    w.u32(f"{a}.block_count", layers)
    w.u32(f"{a}.nextn_predict_layers", 0)
    w.u32(f"{a}.embedding_length", hidden)
    w.u32(f"{a}.feed_forward_length", c["ff"])
    w.u32(f"{a}.attention.head_count", c["heads"])
    w.u32(f"{a}.attention.head_count_kv", c["kv_heads"])
    w.u32(f"{a}.attention.key_length", hd)
    w.u32(f"{a}.attention.value_length", hd)
    w.u32(f"{a}.rope.dimension_count", c["n_rot"])
    w.f32(f"{a}.rope.freq_base", c["theta"])
    w.f32(f"{a}.attention.layer_norm_rms_epsilon", c["eps"])
    w.u32(f"{a}.ssm.conv_kernel", c["conv_kernel"])
    w.u32(f"{a}.ssm.group_count", c["k_heads"])
    w.u32(f"{a}.ssm.time_step_rank", c["v_heads"])
    w.u32(f"{a}.ssm.inner_size", value_dim)
    w.u32(f"{a}.ssm.state_size", c["k_dim"])
    w.tensor("token_embd.weight", F32, [hidden, c["vocab"]])
    w.ones("output_norm.weight", [hidden])
    for il in range(layers):
        p = f"blk.{il}."
        w.ones(p + "attn_norm.weight", [hidden])
        w.ones(p + "post_attention_norm.weight", [hidden])
        if il % 4 == 3:
            w.tensor(p + "attn_q.weight", Q4_0, [hidden, 2 * c["heads"] * hd])
            w.tensor(p + "attn_k.weight", Q4_0, [hidden, c["kv_heads"] * hd])
            w.tensor(p + "attn_v.weight", Q4_0, [hidden, c["kv_heads"] * hd])
            w.tensor(p + "attn_output.weight", Q4_0, [c["heads"] * hd, hidden])
            w.ones(p + "attn_q_norm.weight", [hd])
            w.ones(p + "attn_k_norm.weight", [hd])
        else:
            w.tensor(p + "attn_qkv.weight", Q4_0, [hidden, conv_dim])
            w.tensor(p + "attn_gate.weight", Q4_0, [hidden, value_dim])
            w.tensor(p + "ssm_beta.weight", Q4_0, [hidden, c["v_heads"]])
            w.tensor(p + "ssm_alpha.weight", Q4_0, [hidden, c["v_heads"]])
            w.tensor(p + "ssm_conv1d.weight", F32, [c["conv_kernel"], conv_dim])
            w.tensor(p + "ssm_dt.bias", F32, [c["v_heads"]])
            w.tensor(p + "ssm_a", F32, [c["v_heads"]], NEG_EXP_NORMAL, STD)
            w.ones(p + "ssm_norm.weight", [c["v_dim"]])
            w.tensor(p + "ssm_out.weight", Q4_0, [value_dim, hidden])
        w.tensor(p + "ffn_gate.weight", Q4_0, [hidden, c["ff"]])
        w.tensor(p + "ffn_up.weight", Q4_0, [hidden, c["ff"]])
        w.tensor(p + "ffn_down.weight", Q4_0, [c["ff"], hidden])


def write_model(path: str, config: str | dict, seed: int = 0) -> str:
    """Write the synthetic model ``config`` (a name in CONFIGS or a dict of the same keys)."""
    c = CONFIGS[config] if isinstance(config, str) else config
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    w = _Writer(path, seed)
    if c["arch"] in ("lfm2", "lfm2moe"):
        _write_lfm2(w, c)
    elif c["arch"] == "qwen35":
        _write_qwen35(w, c)
    else:
        raise ValueError("unknown architecture %r" % c["arch"])
    w.finish()
    return path


def cached_model(config: str, seed: int = 0, directory: str | None = None) -> str:
    """Write ``config`` under a scratch directory unless that file already exists there."""
    directory = directory or os.environ.get("BOBCAT_SYNTH_DIR", "/tmp/bobcat_synth")
    path = os.path.join(directory, "%s-seed%d.gguf" % (config, seed))
    if not os.path.exists(path):
        tmp = path + ".tmp.%d" % os.getpid()
        write_model(tmp, config, seed)
        os.replace(tmp, path)
    return path
