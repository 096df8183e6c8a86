"""Host-side checks that need no GPU: the C ABI library loads and exports every declared symbol;
the synthetic GGUF writer produces files the `gguf` package and the library's own reader agree
on; the reader rejects malformed files as the reference's parser does
(crates/bobcat-gguf/tests/malformed.rs)."""

import ctypes as C
import os
import re

import numpy as np
import pytest

from bobcat_b200 import Model, _lib, errors, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = "".join(open(os.path.join(ROOT, "include", name)).read() for name in sorted(os.listdir(os.path.join(ROOT, "include"))) if name.endswith(".h"))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bc_[a-z0-9_]+)\s*\(", text)) - {"bc_emit_fn"})


def test_library_exports_every_declared_symbol(lib):
    names = declared_symbols()
    assert len(names) > 50
    for name in names:
        assert hasattr(lib, name), name
        assert name in _lib.SIGNATURES, "no ctypes signature for " + name
    assert sorted(_lib.SIGNATURES) == names


def test_no_device_is_an_error_not_a_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    h = C.c_void_p()
    assert lib.bc_backend_open(0, None, C.byref(h)) == errors.NoDevice.status
    assert b"CUDA" in lib.bc_last_error()


@pytest.mark.parametrize("config", ["lfm2-tiny", "lfm2moe-tiny", "qwen35-tiny"])
def test_written_file_parses_and_loads(config, model_path):
    import gguf
    path = model_path(config)
    reader = gguf.GGUFReader(path)
    c = synth.CONFIGS[config]
    assert reader.fields["general.architecture"].contents() == c["arch"]
    m = Model.load(path)
    hp = m.hyperparameters()
    assert (hp.n_layers, hp.n_embd, hp.n_vocab, hp.n_ff) == (c["layers"], c["hidden"], c["vocab"], c["ff"])
    if c["arch"] == "qwen35":
        assert hp.n_attention_layers + hp.n_delta_layers == hp.n_layers and hp.n_rot == c["n_rot"]
        assert (hp.n_k_heads, hp.n_v_heads, hp.k_head_dim, hp.v_head_dim) == (c["k_heads"], c["v_heads"], c["k_dim"], c["v_dim"])
    else:
        assert m.attention_layers() == [il in c["attention"] for il in range(c["layers"])]
        assert hp.head_dim == c["hidden"] // c["heads"] and hp.n_kv_heads == c["kv_heads"]
    assert m.decode_bytes() > 0
    for t in reader.tensors:
        if t.name.endswith("norm.weight"):
            assert np.all(t.data == 1.0), t.name
        if t.name.endswith("ssm_a"):
            assert np.all(t.data < 0)


def test_writer_quantises_like_ggml(tmp_path, lib):
    """Draw the same normal values as F32 and as Q4_0 and check the quantised bytes against the
    `gguf` package's reference quantiser."""
    import gguf

    def write(ttype, path):
        w = synth._Writer(str(path), 11)
        w.string("general.architecture", "test")
        w.tensor("t", ttype, [256, 40])
        w.finish()
        return gguf.GGUFReader(str(path)).tensors[0]

    f = write(synth.F32, tmp_path / "f.gguf")
    q = write(synth.Q4_0, tmp_path / "q.gguf")
    values = np.array(f.data, dtype=np.float32).reshape(40, 256)
    assert abs(values.std() - 0.02) < 1e-3 and abs(values.mean()) < 1e-3
    want = gguf.quants.quantize(values, gguf.GGMLQuantizationType.Q4_0)
    assert np.array_equal(np.array(q.data).reshape(want.shape), want)


def test_writer_is_deterministic(tmp_path):
    a = synth.write_model(str(tmp_path / "a.gguf"), "lfm2-tiny", 3)
    b = synth.write_model(str(tmp_path / "b.gguf"), "lfm2-tiny", 3)
    c = synth.write_model(str(tmp_path / "c.gguf"), "lfm2-tiny", 4)
    assert open(a, "rb").read() == open(b, "rb").read()
    assert open(a, "rb").read() != open(c, "rb").read()


def test_every_truncation_fails(model_path, tmp_path):
    data = open(model_path("lfm2-tiny"), "rb").read()
    header_end = data.index(b"blk.3.ffn_down.weight") + 64
    cut = tmp_path / "cut.gguf"
    # Every prefix of the header, then sparse prefixes of the data section.
    lengths = list(range(1, header_end, 7)) + list(range(header_end, len(data), len(data) // 50))
    for n in lengths:
        cut.write_bytes(data[:n])
        with pytest.raises((errors.Gguf, errors.MissingTensor, errors.Metadata)):
            Model.load(str(cut))


def test_corrupt_headers_fail(model_path, tmp_path):
    data = bytearray(open(model_path("lfm2-tiny"), "rb").read())
    bad = tmp_path / "bad.gguf"

    def expect_failure(mutated: bytes):
        bad.write_bytes(mutated)
        with pytest.raises(errors.BobcatError):
            Model.load(str(bad))

    m = bytearray(data); m[0:4] = b"GGML"; expect_failure(m)               # magic
    m = bytearray(data); m[4:8] = (1).to_bytes(4, "little"); expect_failure(m)  # version
    m = bytearray(data); m[8:16] = (2 ** 60).to_bytes(8, "little"); expect_failure(m)   # tensor count
    m = bytearray(data); m[16:24] = (2 ** 60).to_bytes(8, "little"); expect_failure(m)  # metadata count
    # general.alignment is the first entry: key length 17, key, type u32, value.
    at = 24 + 8 + 17 + 4
    m = bytearray(data); m[at:at + 4] = (24).to_bytes(4, "little"); expect_failure(m)   # not a power of two
    # An architecture the loaders do not know.
    m = bytes(data).replace(b"\x04\x00\x00\x00\x00\x00\x00\x00lfm2", b"\x04\x00\x00\x00\x00\x00\x00\x00lfm9", 1)
    bad.write_bytes(m)
    with pytest.raises(errors.Architecture):
        Model.load(str(bad))
    with pytest.raises(errors.Io):
        Model.load(str(tmp_path / "missing.gguf"))


def test_missing_tensor_and_shape_errors(tmp_path):
    c = dict(synth.CONFIGS["lfm2-tiny"])
    path = str(tmp_path / "m.gguf")
    w = synth._Writer(path, 0)
    synth._write_lfm2(w, c)
    w.finish()
    data = open(path, "rb").read()
    (tmp_path / "renamed.gguf").write_bytes(data.replace(b"blk.2.ffn_up.weight", b"blk.2.ffn_uq.weight", 1))
    with pytest.raises(errors.MissingTensor):
        Model.load(str(tmp_path / "renamed.gguf"))
    c["ff"] = 320  # tensors of another width than the metadata says
    w = synth._Writer(path, 0)
    synth._write_lfm2(w, c)
    w.finish()
    data = open(path, "rb").read()
    key = b"lfm2.feed_forward_length"
    at = data.index(key) + len(key) + 4
    (tmp_path / "shape.gguf").write_bytes(data[:at] + (256).to_bytes(4, "little") + data[at + 4:])
    with pytest.raises(errors.TensorShape):
        Model.load(str(tmp_path / "shape.gguf"))
