"""Generate the golden activations that pin the CPU parity checker (``oracle/``).

Method (the one the reference's ``tools/ref_dump.py`` uses on downloaded checkpoints, applied here
to randomly initialised models because no checkpoint can be downloaded): write a small synthetic
GGUF model, dequantise its tensors with the ``gguf`` package, load them into the matching
``transformers`` model class built from an explicit config, run float32 on the CPU, and record the
token embeddings, every layer's output, the final norm, the logits and a greedy continuation.

Run from the repository root, in an environment with ``transformers``, ``torch`` and ``gguf``:

    python tests/golden/make_transformers_golden.py

It writes ``tests/golden/<config>.npz``. The tests regenerate the same GGUF file (the writer is
deterministic), run the C++ restatement on it, and compare with these arrays.
"""

from __future__ import annotations

import hashlib
import os
import re
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import gguf  # noqa: E402
import torch  # noqa: E402
import transformers  # noqa: E402

from bobcat_b200 import synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
CONFIGS = ["lfm2-tiny", "lfm2moe-tiny", "qwen35-tiny"]
N_PROMPT, N_GENERATE, PROMPT_SEED = 12, 8, 1
LAYER = re.compile(r"blk\.(\d+)\.(.+)")

LFM2_NAMES = {
    "attn_norm.weight": "operator_norm.weight", "ffn_norm.weight": "ffn_norm.weight",
    "attn_q.weight": "self_attn.q_proj.weight", "attn_k.weight": "self_attn.k_proj.weight",
    "attn_v.weight": "self_attn.v_proj.weight", "attn_output.weight": "self_attn.out_proj.weight",
    "attn_q_norm.weight": "self_attn.q_layernorm.weight", "attn_k_norm.weight": "self_attn.k_layernorm.weight",
    "shortconv.conv.weight": "conv.conv.weight", "shortconv.in_proj.weight": "conv.in_proj.weight",
    "shortconv.out_proj.weight": "conv.out_proj.weight", "ffn_gate.weight": "feed_forward.w1.weight",
    "ffn_up.weight": "feed_forward.w3.weight", "ffn_down.weight": "feed_forward.w2.weight",
    "ffn_gate_inp.weight": "feed_forward.gate.weight", "exp_probs_b.bias": "feed_forward.expert_bias",
    "ffn_down_exps.weight": "feed_forward.experts.down_proj",
}
QWEN_NAMES = {
    "attn_norm.weight": "input_layernorm.weight", "post_attention_norm.weight": "post_attention_layernorm.weight",
    "ffn_gate.weight": "mlp.gate_proj.weight", "ffn_up.weight": "mlp.up_proj.weight", "ffn_down.weight": "mlp.down_proj.weight",
    "attn_q.weight": "self_attn.q_proj.weight", "attn_k.weight": "self_attn.k_proj.weight", "attn_v.weight": "self_attn.v_proj.weight",
    "attn_output.weight": "self_attn.o_proj.weight", "attn_q_norm.weight": "self_attn.q_norm.weight",
    "attn_k_norm.weight": "self_attn.k_norm.weight", "attn_qkv.weight": "linear_attn.in_proj_qkv.weight",
    "attn_gate.weight": "linear_attn.in_proj_z.weight", "ssm_beta.weight": "linear_attn.in_proj_b.weight",
    "ssm_alpha.weight": "linear_attn.in_proj_a.weight", "ssm_conv1d.weight": "linear_attn.conv1d.weight",
    "ssm_dt.bias": "linear_attn.dt_bias", "ssm_a": "linear_attn.A_log", "ssm_norm.weight": "linear_attn.norm.weight",
    "ssm_out.weight": "linear_attn.out_proj.weight",
}
QWEN_CENTERED = {"attn_norm.weight", "post_attention_norm.weight", "attn_q_norm.weight", "attn_k_norm.weight"}


def dequantized(t) -> torch.Tensor:
    values = gguf.quants.dequantize(t.data, t.tensor_type)
    return torch.from_numpy(np.ascontiguousarray(values, dtype=np.float32))


def build_lfm2(c: dict, tensors: dict):
    layer_types = ["full_attention" if il in set(c["attention"]) else "conv" for il in range(c["layers"])]
    common = dict(vocab_size=c["vocab"], hidden_size=c["hidden"], num_hidden_layers=c["layers"], num_attention_heads=c["heads"],
                  num_key_value_heads=c["kv_heads"], norm_eps=c["eps"], conv_L_cache=c["conv_kernel"], layer_types=layer_types,
                  rope_parameters={"rope_type": "default", "rope_theta": c["theta"]}, tie_word_embeddings=True,
                  max_position_embeddings=4096)
    moe = c["arch"] == "lfm2moe"
    if moe:
        config = transformers.Lfm2MoeConfig(intermediate_size=c["ff"], moe_intermediate_size=c["ff_expert"], num_dense_layers=c["dense_layers"],
                                            num_experts_per_tok=c["experts_used"], num_experts=c["experts"], use_expert_bias=True,
                                            norm_topk_prob=True, routed_scaling_factor=1.0, **common)
        model = transformers.Lfm2MoeForCausalLM(config)
    else:
        config = transformers.Lfm2Config(intermediate_size=c["ff"], block_auto_adjust_ff_dim=False, **common)
        model = transformers.Lfm2ForCausalLM(config)
    state = {"model.embed_tokens.weight": dequantized(tensors.pop("token_embd.weight")),
             "model.embedding_norm.weight": dequantized(tensors.pop("token_embd_norm.weight"))}
    halves: dict[int, dict] = {}
    for name, t in tensors.items():
        layer, suffix = LAYER.fullmatch(name).groups()
        layer = int(layer)
        values = dequantized(t)
        if suffix in ("ffn_gate_exps.weight", "ffn_up_exps.weight"):
            halves.setdefault(layer, {})[suffix] = values
            if len(halves[layer]) == 2:
                # transformers stacks each expert's gate and up matrices into one tensor, gate first.
                state[f"model.layers.{layer}.feed_forward.experts.gate_up_proj"] = torch.cat(
                    [halves[layer]["ffn_gate_exps.weight"], halves[layer]["ffn_up_exps.weight"]], dim=1)
            continue
        if suffix == "shortconv.conv.weight":
            values = values.unsqueeze(1)  # [hidden, taps] -> [hidden, 1, taps]
        state[f"model.layers.{layer}.{LFM2_NAMES[suffix]}"] = values
    missing, unexpected = model.load_state_dict(state, strict=False)
    missing = [m for m in missing if "lm_head" not in m]
    assert not missing and not unexpected, (missing, unexpected)
    model.tie_weights()
    return model


def build_qwen35(c: dict, tensors: dict):
    layer_types = ["full_attention" if il % 4 == 3 else "linear_attention" for il in range(c["layers"])]
    config = transformers.models.qwen3_5.configuration_qwen3_5.Qwen3_5TextConfig(
        vocab_size=c["vocab"], hidden_size=c["hidden"], intermediate_size=c["ff"], num_hidden_layers=c["layers"],
        num_attention_heads=c["heads"], num_key_value_heads=c["kv_heads"], rms_norm_eps=c["eps"], tie_word_embeddings=True,
        rope_parameters={"rope_type": "default", "rope_theta": c["theta"], "partial_rotary_factor": c["n_rot"] / c["head_dim"]},
        head_dim=c["head_dim"], linear_conv_kernel_dim=c["conv_kernel"], linear_key_head_dim=c["k_dim"], linear_value_head_dim=c["v_dim"],
        linear_num_key_heads=c["k_heads"], linear_num_value_heads=c["v_heads"], layer_types=layer_types, max_position_embeddings=4096)
    model = transformers.Qwen3_5ForCausalLM(config)
    n_k, n_v, kd, vd = c["k_heads"], c["v_heads"], c["k_dim"], c["v_dim"]
    ratio = n_v // n_k
    # GGUF value head j reads key head j % n_k (llama.cpp's converter order); transformers' value
    # head h reads key head h // ratio. GGUF head j = g * n_k + k is transformers' head k * ratio + g.
    hf_of_gguf = np.array([(j % n_k) * ratio + j // n_k for j in range(n_v)])
    gguf_of_hf = np.argsort(hf_of_gguf)

    def heads_to_hf(values: torch.Tensor, per_head: int, dim: int = 0) -> torch.Tensor:
        shape = list(values.shape)
        shape[dim:dim + 1] = [n_v, per_head]
        v = values.reshape(shape).index_select(dim, torch.from_numpy(gguf_of_hf))
        return v.reshape(values.shape)

    state = {"model.embed_tokens.weight": dequantized(tensors.pop("token_embd.weight")),
             "model.norm.weight": dequantized(tensors.pop("output_norm.weight")) - 1}
    key_dim = n_k * kd
    for name, t in tensors.items():
        layer, suffix = LAYER.fullmatch(name).groups()
        values = dequantized(t)
        if suffix in QWEN_CENTERED:
            values = values - 1
        elif suffix == "ssm_a":
            values = heads_to_hf(torch.log(-values), 1)
        elif suffix == "ssm_dt.bias":
            values = heads_to_hf(values, 1)
        elif suffix in ("ssm_beta.weight", "ssm_alpha.weight"):
            values = heads_to_hf(values, 1, 0)
        elif suffix == "attn_gate.weight":
            values = heads_to_hf(values, vd, 0)
        elif suffix == "attn_qkv.weight":
            values = torch.cat([values[: 2 * key_dim], heads_to_hf(values[2 * key_dim:], vd, 0)], dim=0)
        elif suffix == "ssm_conv1d.weight":
            values = torch.cat([values[: 2 * key_dim], heads_to_hf(values[2 * key_dim:], vd, 0)], dim=0).unsqueeze(1)
        elif suffix == "ssm_out.weight":
            values = heads_to_hf(values, vd, 1)
        state[f"model.layers.{layer}.{QWEN_NAMES[suffix]}"] = values
    missing, unexpected = model.load_state_dict(state, strict=False)
    missing = [m for m in missing if "lm_head" not in m]
    assert not missing and not unexpected, (missing, unexpected)
    model.tie_weights()
    return model


def dump(config_name: str) -> None:
    c = synth.CONFIGS[config_name]
    path = os.path.join("/tmp/bobcat_synth", "golden-%s.gguf" % config_name)
    synth.write_model(path, config_name, seed=0)
    digest = hashlib.sha256(open(path, "rb").read()).hexdigest()
    reader = gguf.GGUFReader(path)
    tensors = {t.name: t for t in reader.tensors}
    torch.manual_seed(0)
    model = build_qwen35(c, tensors) if c["arch"] == "qwen35" else build_lfm2(c, tensors)
    model.eval()
    tokens = np.random.default_rng(PROMPT_SEED).integers(0, c["vocab"], size=N_PROMPT).astype(np.int64)
    input_ids = torch.from_numpy(tokens)[None]
    captured: dict[str, torch.Tensor] = {}

    def capture(name):
        def hook(_m, _i, output):
            captured[name] = (output[0] if isinstance(output, tuple) else output).detach()
        return hook

    decoder = model.model
    final_norm = getattr(decoder, "embedding_norm", None) or decoder.norm
    handles = [decoder.embed_tokens.register_forward_hook(capture("embedding")), final_norm.register_forward_hook(capture("final_norm"))]
    for index, layer in enumerate(decoder.layers):
        handles.append(layer.register_forward_hook(capture("layer_%02d" % index)))
    with torch.no_grad():
        logits = model(input_ids).logits
    for h in handles:
        h.remove()
    with torch.no_grad():
        out = model.generate(input_ids, do_sample=False, max_new_tokens=N_GENERATE, min_new_tokens=N_GENERATE)
    generated = out[0, N_PROMPT:].numpy().astype(np.int32)
    layers = np.stack([captured["layer_%02d" % i][0].numpy() for i in range(c["layers"])])
    np.savez_compressed(
        os.path.join(HERE, config_name + ".npz"), tokens=tokens.astype(np.int32), generated=generated,
        embedding=captured["embedding"][0].numpy().astype(np.float32), layers=layers.astype(np.float32),
        final_norm=captured["final_norm"][0].numpy().astype(np.float32), logits=logits[0].numpy().astype(np.float32),
        gguf_sha256=np.array(digest), versions=np.array("torch %s transformers %s gguf" % (torch.__version__, transformers.__version__)))
    print(config_name, "tokens", tokens.tolist(), "generated", generated.tolist(), "sha", digest[:12])


if __name__ == "__main__":
    for name in (sys.argv[1:] or CONFIGS):
        dump(name)
