"""Generates tests/golden/hf_forward_golden.npz: logits of seeded Llama, Qwen2 and GPT-2 networks computed by an
implementation that shares no code with this repository (Hugging Face `transformers`, float64, eager attention).

The CPU oracle's transformer forwards (restated from wgml's models/llama2/cpu.rs and models/gpt2/cpu.rs) and the CUDA
models are checked against these logits in tests/test_oracle_hf.py and tests/test_gpu_hf.py: wgml's own tests hold no
numeric vectors for the forward pass, so this is the independent anchor of the architecture reading -- RoPE pairing
and frequencies, grouped-query head mapping, attention scaling, SwiGLU, biases, GPT-2's fused qkv, learned positions,
tanh GELU and tied head.  It does not pin wgml's summation order (nothing available offline does).

The weights are not stored: `draw_llama` / `draw_gpt2` (numpy only) draw them from a seed under their GGUF names and
in GGUF conventions, here and in the tests; the fixture holds token ids, logits and a checksum of the drawn weights,
so that a change of numpy's random stream shows up as a checksum mismatch and not as a parity failure.  The shapes are
those of the small networks the GPU parity tests already use (head sizes 48 and 64, grouped queries).

Conventions.  A GGUF Llama file holds attn_q / attn_k with the rows of every head permuted so that RoPE pairs
elements (2i, 2i+1) (wgml's RoPEVariant::Original); transformers pairs (i, i + head/2).  The generator un-permutes
the GGUF-convention matrices for the Hugging Face model.  Qwen2 files keep the (i, i + head/2) pairing
(RoPEVariant::Neox), so the matrices are shared as they are.  GPT-2's Conv1D weights are the transposes of the GGUF
matrices.

Run from the repository root:  python tests/golden/make_hf_golden.py
"""
import os

import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
T = 12   # positions per network


SEEDS = {"llama": 101, "qwen2": 102, "gpt2": 103}
LLAMA_CFGS = {
    # tiny-llama widths (head 48) with grouped queries, two layers, a small vocabulary
    "llama": dict(dim=288, hidden_dim=768, n_layers=2, n_q_heads=6, n_kv_heads=3, vocab_size=256, seq_len=32,
                  rope_base_freq=10000.0, rms_norm_eps=1e-5),
    # head 64, four query heads per KV head, biases, Qwen2's theta and epsilon
    "qwen2": dict(dim=512, hidden_dim=1024, n_layers=2, n_q_heads=8, n_kv_heads=2, vocab_size=256, seq_len=32,
                  rope_base_freq=1000000.0, rms_norm_eps=1e-6),
}
GPT2_CFG = dict(n_vocab=200, n_seq=32, n_embd=256, n_head=4, n_layer=2, ff_len=1024)


def _f(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def draw_llama(kind: str):
    """(config, {GGUF tensor name: f32 array}, token ids) of the seeded Llama-family network `kind`."""
    cfg = dict(LLAMA_CFGS[kind])
    rng = np.random.default_rng(SEEDS[kind])
    dim, hid, L = cfg["dim"], cfg["hidden_dim"], cfg["n_layers"]
    kv = cfg["n_kv_heads"] * (dim // cfg["n_q_heads"])

    def mat(r, c):
        return _f(rng.standard_normal((r, c)) / np.sqrt(c))

    t = {"token_embd.weight": _f(rng.standard_normal((cfg["vocab_size"], dim)) * 0.5),
         "output.weight": mat(cfg["vocab_size"], dim),
         "output_norm.weight": _f(1.0 + 0.1 * rng.standard_normal(dim))}
    for l in range(L):
        p = f"blk.{l}."
        t[p + "attn_q.weight"], t[p + "attn_k.weight"], t[p + "attn_v.weight"] = mat(dim, dim), mat(kv, dim), mat(kv, dim)
        t[p + "attn_output.weight"] = mat(dim, dim)
        t[p + "ffn_gate.weight"], t[p + "ffn_up.weight"], t[p + "ffn_down.weight"] = mat(hid, dim), mat(hid, dim), mat(dim, hid)
        t[p + "attn_norm.weight"] = _f(1.0 + 0.1 * rng.standard_normal(dim))
        t[p + "ffn_norm.weight"] = _f(1.0 + 0.1 * rng.standard_normal(dim))
        if kind == "qwen2":
            for n, sz in (("attn_q.bias", dim), ("attn_k.bias", kv), ("attn_v.bias", kv)):
                t[p + n] = _f(0.2 * rng.standard_normal(sz))
    tokens = rng.integers(0, cfg["vocab_size"], T).astype(np.uint32)
    return cfg, t, tokens


def draw_gpt2():
    """(config, {GGUF tensor name: f32 array}, token ids) of the seeded GPT-2 network."""
    cfg = dict(GPT2_CFG)
    rng = np.random.default_rng(SEEDS["gpt2"])
    n, ff, L = cfg["n_embd"], cfg["ff_len"], cfg["n_layer"]

    def mat(r, c):
        return _f(rng.standard_normal((r, c)) / np.sqrt(c))

    def vec(sz, mean=0.0, sd=0.1):
        return _f(mean + sd * rng.standard_normal(sz))

    t = {"token_embd.weight": _f(rng.standard_normal((cfg["n_vocab"], n)) * 0.5),
         "position_embd.weight": _f(rng.standard_normal((cfg["n_seq"], n)) * 0.2),
         "output_norm.weight": vec(n, 1.0), "output_norm.bias": vec(n)}
    for l in range(L):
        p = f"blk.{l}."
        t[p + "attn_qkv.weight"], t[p + "attn_output.weight"] = mat(3 * n, n), mat(n, n)
        t[p + "ffn_up.weight"], t[p + "ffn_down.weight"] = mat(ff, n), mat(n, ff)
        t[p + "attn_qkv.bias"], t[p + "attn_output.bias"], t[p + "ffn_up.bias"], t[p + "ffn_down.bias"] = vec(3 * n), vec(n), vec(ff), vec(n)
        t[p + "attn_norm.weight"], t[p + "attn_norm.bias"] = vec(n, 1.0), vec(n)
        t[p + "ffn_norm.weight"], t[p + "ffn_norm.bias"] = vec(n, 1.0), vec(n)
    tokens = rng.integers(0, cfg["n_vocab"], T).astype(np.uint32)
    return cfg, t, tokens


def checksum(tensors: dict) -> int:
    """CRC-32 over the bytes of all tensors in name order."""
    c = 0
    for k in sorted(tensors):
        c = zlib.crc32(np.ascontiguousarray(tensors[k]).tobytes(), zlib.crc32(k.encode(), c))
    return c


def _unpermute_rope_rows(w: np.ndarray, n_heads: int) -> np.ndarray:
    """GGUF row 2i / 2i+1 of a head -> Hugging Face row i / i + head/2."""
    rows = w.shape[0]
    head = rows // n_heads
    out = np.empty_like(w)
    for h in range(n_heads):
        blk = w[h * head:(h + 1) * head]
        out[h * head:h * head + head // 2] = blk[0::2]
        out[h * head + head // 2:(h + 1) * head] = blk[1::2]
    return out


def _load(model, sd, may_miss):
    import torch
    missing, unexpected = model.load_state_dict({k: torch.from_numpy(np.ascontiguousarray(v, dtype=np.float64)) for k, v in sd.items()},
                                                strict=False)
    assert not unexpected and all(any(s in m for s in may_miss) for m in missing), (missing, unexpected)


def hf_llama_logits(kind: str, cfg: dict, t: dict, tokens: np.ndarray) -> np.ndarray:
    import torch
    from transformers import LlamaConfig, LlamaForCausalLM, Qwen2Config, Qwen2ForCausalLM
    common = dict(vocab_size=cfg["vocab_size"], hidden_size=cfg["dim"], intermediate_size=cfg["hidden_dim"],
                  num_hidden_layers=cfg["n_layers"], num_attention_heads=cfg["n_q_heads"], num_key_value_heads=cfg["n_kv_heads"],
                  hidden_act="silu", max_position_embeddings=cfg["seq_len"], rms_norm_eps=cfg["rms_norm_eps"],
                  rope_theta=cfg["rope_base_freq"], tie_word_embeddings=False, attn_implementation="eager")
    if kind == "llama":
        model = LlamaForCausalLM(LlamaConfig(attention_bias=False, mlp_bias=False, **common))
    else:
        model = Qwen2ForCausalLM(Qwen2Config(use_sliding_window=False, **common))
    model = model.double().eval()
    fix = _unpermute_rope_rows if kind == "llama" else (lambda w, n: w)
    sd = {"model.embed_tokens.weight": t["token_embd.weight"], "lm_head.weight": t["output.weight"],
          "model.norm.weight": t["output_norm.weight"]}
    for l in range(cfg["n_layers"]):
        p, h = f"blk.{l}.", f"model.layers.{l}."
        sd[h + "self_attn.q_proj.weight"] = fix(t[p + "attn_q.weight"], cfg["n_q_heads"])
        sd[h + "self_attn.k_proj.weight"] = fix(t[p + "attn_k.weight"], cfg["n_kv_heads"])
        sd[h + "self_attn.v_proj.weight"] = t[p + "attn_v.weight"]
        sd[h + "self_attn.o_proj.weight"] = t[p + "attn_output.weight"]
        sd[h + "mlp.gate_proj.weight"] = t[p + "ffn_gate.weight"]
        sd[h + "mlp.up_proj.weight"] = t[p + "ffn_up.weight"]
        sd[h + "mlp.down_proj.weight"] = t[p + "ffn_down.weight"]
        sd[h + "input_layernorm.weight"] = t[p + "attn_norm.weight"]
        sd[h + "post_attention_layernorm.weight"] = t[p + "ffn_norm.weight"]
        if kind == "qwen2":
            sd[h + "self_attn.q_proj.bias"] = t[p + "attn_q.bias"]
            sd[h + "self_attn.k_proj.bias"] = t[p + "attn_k.bias"]
            sd[h + "self_attn.v_proj.bias"] = t[p + "attn_v.bias"]
    _load(model, sd, ("rotary", "inv_freq"))
    with torch.no_grad():
        return model(torch.from_numpy(tokens.astype(np.int64))[None]).logits[0].numpy()


def hf_gpt2_logits(cfg: dict, t: dict, tokens: np.ndarray) -> np.ndarray:
    import torch
    from transformers import GPT2Config, GPT2LMHeadModel
    model = GPT2LMHeadModel(GPT2Config(vocab_size=cfg["n_vocab"], n_positions=cfg["n_seq"], n_embd=cfg["n_embd"], n_layer=cfg["n_layer"],
                                       n_head=cfg["n_head"], n_inner=cfg["ff_len"], activation_function="gelu_new", resid_pdrop=0.0,
                                       embd_pdrop=0.0, attn_pdrop=0.0, layer_norm_epsilon=1e-5, attn_implementation="eager")).double().eval()
    sd = {"transformer.wte.weight": t["token_embd.weight"], "transformer.wpe.weight": t["position_embd.weight"],
          "transformer.ln_f.weight": t["output_norm.weight"], "transformer.ln_f.bias": t["output_norm.bias"],
          "lm_head.weight": t["token_embd.weight"]}
    for l in range(cfg["n_layer"]):
        p, h = f"blk.{l}.", f"transformer.h.{l}."
        sd[h + "attn.c_attn.weight"], sd[h + "attn.c_attn.bias"] = t[p + "attn_qkv.weight"].T, t[p + "attn_qkv.bias"]
        sd[h + "attn.c_proj.weight"], sd[h + "attn.c_proj.bias"] = t[p + "attn_output.weight"].T, t[p + "attn_output.bias"]
        sd[h + "mlp.c_fc.weight"], sd[h + "mlp.c_fc.bias"] = t[p + "ffn_up.weight"].T, t[p + "ffn_up.bias"]
        sd[h + "mlp.c_proj.weight"], sd[h + "mlp.c_proj.bias"] = t[p + "ffn_down.weight"].T, t[p + "ffn_down.bias"]
        sd[h + "ln_1.weight"], sd[h + "ln_1.bias"] = t[p + "attn_norm.weight"], t[p + "attn_norm.bias"]
        sd[h + "ln_2.weight"], sd[h + "ln_2.bias"] = t[p + "ffn_norm.weight"], t[p + "ffn_norm.bias"]
    _load(model, sd, (".attn.bias", "masked_bias"))
    with torch.no_grad():
        return model(torch.from_numpy(tokens.astype(np.int64))[None]).logits[0].numpy()


def main():
    out = {}
    for name in ("llama", "qwen2", "gpt2"):
        if name == "gpt2":
            cfg, t, tokens = draw_gpt2()
            logits = hf_gpt2_logits(cfg, t, tokens)
        else:
            cfg, t, tokens = draw_llama(name)
            logits = hf_llama_logits(name, cfg, t, tokens)
        out[f"{name}/tokens"] = tokens
        out[f"{name}/logits"] = logits.astype(np.float64)
        out[f"{name}/weights_crc32"] = np.uint32(checksum(t))
        print(name, "logits", logits.shape, "max |logit|", float(np.abs(logits).max()), "crc", checksum(t))
    path = os.path.join(HERE, "hf_forward_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
