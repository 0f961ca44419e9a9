"""Shared builders for the model parity tests: the same seeded tensors go to the oracle and to the GPU."""
import numpy as np

import oracle
from wgml_b200 import synth
from wgml_b200.models import Gpt2, Gpt2Params, Llama2, Llama2Config, LlamaModelType

SMALL_LLAMA = dict(arch="llama", dim=512, hidden_dim=1024, n_layers=2, n_q_heads=8, n_kv_heads=8, vocab_size=1000,
                   seq_len=96, rope_base_freq=10000.0, rms_norm_eps=1e-5, default_qtype=synth.Q4_K)
SMALL_GPT2 = dict(arch="gpt2", n_vocab=1001, n_seq=128, n_embd=256, n_head=4, n_layer=2, ff_len=1024, default_qtype=synth.Q8_0)


def llama_pair(cfg: dict, seed=0, biases=False, qwen=False, scale=0.01, fused=True, tensors=None):
    t = tensors if tensors is not None else synth.llama_tensors(cfg, seed, biases=biases, scale=scale)
    c = Llama2Config(cfg["dim"], cfg["hidden_dim"], cfg["n_layers"], cfg["n_q_heads"], cfg["n_kv_heads"], cfg["vocab_size"],
                     cfg["seq_len"], cfg["rope_base_freq"], cfg["rms_norm_eps"])
    gpu = Llama2(c, LlamaModelType.Qwen2 if qwen else LlamaModelType.Llama)
    gpu.load_tensors(t)
    gpu.set_fused(fused)
    cpu = oracle.Llama2Oracle(cfg, t, rope_variant=1 if qwen else 0)
    return gpu, cpu, t


def gpt2_pair(cfg: dict, seed=0, fused=True, scale=0.01):
    t = synth.gpt2_tensors(cfg, seed, scale=scale)
    p = Gpt2Params(cfg["n_vocab"], cfg["n_seq"], cfg["n_embd"], cfg["n_head"], cfg["n_layer"], cfg["ff_len"], 3 * cfg["n_embd"], 7)
    gpu = Gpt2(p)
    gpu.load_tensors(t)
    gpu.set_fused(fused)
    cpu = oracle.Gpt2Oracle(cfg, t)
    return gpu, cpu, t


def rel_err(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))
