"""Batched prompt prefill: the tensor-core product for up to eight input vectors against the oracle, and the
token loop with the prompt sent through passes of eight positions against the position-by-position loop and
against the oracle (cache rows, logits after the prompt, greedy tokens)."""
import numpy as np
import pytest
import torch

import oracle
from conftest import ATOL, RTOL, assert_close
from helpers import SMALL_GPT2, SMALL_LLAMA, gpt2_pair, llama_pair
from wgml_b200 import _lib, ops, synth

pytestmark = pytest.mark.gpu


def make(nrows, ncols, seed, n_vec):
    qt, arr = synth.matrix(ops.Q4_K, nrows, ncols, seed, "pf")
    x = np.random.default_rng(seed + 1).standard_normal((n_vec, ncols)).astype(np.float32)
    return np.ascontiguousarray(arr).view(np.uint8), x


@pytest.mark.parametrize("shape", [(128, 256, 8), (256, 512, 3), (384, 768, 8), (4096, 4096, 8), (1408, 11008, 5),
                                   (148 * 128 + 256, 1024, 1), (11008, 4096, 8)])
def test_batched_product_vs_oracle(shape):
    """Every vector of the batch against the f64 product of the same bit-exact weights (1e-3 relative / 1e-4 of
    the output RMS, the tolerance of the matrix-vector kernels)."""
    nrows, ncols, n_vec = shape
    raw, x = make(nrows, ncols, 7, n_vec)
    # vectors of very different magnitudes share a pass: exponents are per vector and group
    x *= (10.0 ** np.arange(-3, -3 + n_vec))[:, None].astype(np.float32)
    t = ops.Q4KTiles(raw, nrows, ncols)
    out = torch.full((n_vec, nrows), float("nan"), device="cuda")
    t.gemm(out, torch.from_numpy(x).cuda())
    ops.device_status()
    got = out.cpu().numpy()
    for i in range(n_vec):
        _, o64 = oracle.gemv_quant(ops.Q4_K, raw, nrows, ncols, x[i], want_f64=True)
        atol = ATOL * float(np.sqrt(np.mean(o64 ** 2)))
        assert_close(got[i], o64, RTOL, atol, f"batched product {nrows}x{ncols}, vector {i} of {n_vec}")


@pytest.mark.parametrize("shape", [(128, 256, 8), (256, 512, 3), (384, 768, 8), (4096, 4096, 8), (1408, 11008, 5), (4096, 11008, 8)])
def test_batched_q6k_product_vs_oracle(shape):
    """The Q6_K kernel (scales folded into a two-plane operand, one exponent per vector and super-block)."""
    nrows, ncols, n_vec = shape
    qt, arr = synth.matrix(ops.Q6_K, nrows, ncols, 9, "pf6")
    raw = np.ascontiguousarray(arr).view(np.uint8)
    x = np.random.default_rng(3).standard_normal((n_vec, ncols)).astype(np.float32)
    x *= (10.0 ** np.arange(-3, -3 + n_vec))[:, None].astype(np.float32)
    t = ops.Q6KTiles(raw, nrows, ncols)
    out = torch.full((n_vec, nrows), float("nan"), device="cuda")
    t.gemm(out, torch.from_numpy(x).cuda())
    ops.device_status()
    got = out.cpu().numpy()
    for i in range(n_vec):
        _, o64 = oracle.gemv_quant(ops.Q6_K, raw, nrows, ncols, x[i], want_f64=True)
        atol = ATOL * float(np.sqrt(np.mean(o64 ** 2)))
        assert_close(got[i], o64, RTOL, atol, f"batched Q6_K product {nrows}x{ncols}, vector {i} of {n_vec}")


@pytest.mark.parametrize("shape", [(128, 256, 8), (256, 512, 3), (768, 768, 8), (3072, 768, 8), (768, 3072, 5), (4096, 4096, 8)])
def test_batched_q80_product_vs_oracle(shape):
    """The Q8_0 kernel (codes as the operand, read from the ring stage the copy landed them in)."""
    nrows, ncols, n_vec = shape
    qt, arr = synth.matrix(ops.Q8_0, nrows, ncols, 13, "pf8")
    raw = np.ascontiguousarray(arr).view(np.uint8).reshape(-1).copy()
    blocks = raw.reshape(-1, 34)
    blocks[::7, 2:] = 0x80      # whole blocks of -128, the code the operand format must keep signed
    blocks[3::11, 2:] = 0x7F
    x = np.random.default_rng(5).standard_normal((n_vec, ncols)).astype(np.float32)
    x *= (10.0 ** np.arange(-3, -3 + n_vec))[:, None].astype(np.float32)
    t = ops.Q80Tiles(raw, nrows, ncols)
    out = torch.full((n_vec, nrows), float("nan"), device="cuda")
    t.gemm(out, torch.from_numpy(x).cuda())
    ops.device_status()
    got = out.cpu().numpy()
    for i in range(n_vec):
        _, o64 = oracle.gemv_quant(ops.Q8_0, raw, nrows, ncols, x[i], want_f64=True)
        atol = ATOL * float(np.sqrt(np.mean(o64 ** 2)))
        assert_close(got[i], o64, RTOL, atol, f"batched Q8_0 product {nrows}x{ncols}, vector {i} of {n_vec}")


def test_batched_q6k_product_extreme_scales_and_codes():
    """All-0x00 / all-0xFF code bytes and scales of -128 / 127: the largest magnitudes of the folded operand."""
    nrows, ncols = 128, 512
    rng = np.random.default_rng(4)
    blocks = np.zeros((nrows * ncols // 256, 210), np.uint8)
    blocks[:, :192] = rng.choice(np.array([0x00, 0xFF], np.uint8), size=(blocks.shape[0], 192))
    blocks[:, 192:208] = rng.choice(np.array([0x80, 0x7F, 0x01, 0xFF], np.uint8), size=(blocks.shape[0], 16))
    blocks[:, 208:210] = np.frombuffer(np.float16(0.01).tobytes(), np.uint8)
    raw = blocks.reshape(-1)
    x = rng.standard_normal((8, ncols)).astype(np.float32)
    t = ops.Q6KTiles(raw, nrows, ncols)
    out = torch.zeros(8, nrows, device="cuda")
    t.gemm(out, torch.from_numpy(x).cuda())
    ops.device_status()
    for i in range(8):
        _, o64 = oracle.gemv_quant(ops.Q6_K, raw, nrows, ncols, x[i], want_f64=True)
        assert_close(out[i].cpu().numpy(), o64, RTOL, ATOL * float(np.sqrt(np.mean(o64 ** 2))), f"extreme Q6_K blocks, vector {i}")


def test_batched_product_matches_the_single_vector_kernels():
    nrows, ncols = 4096, 4096
    raw, x = make(nrows, ncols, 11, 8)
    x[3, 64:96] = 0.0          # an all-zero group
    x[5] = 0.0                 # an all-zero vector
    xd = torch.from_numpy(x).cuda()
    t = ops.Q4KTiles(raw, nrows, ncols)
    m = ops.GpuQuantMatrix(ops.Q4_K, raw, nrows, ncols)
    out = torch.zeros(8, nrows, device="cuda")
    t.gemm(out, xd)
    ref = torch.zeros(8, nrows, device="cuda")
    gq = ops.GemvQuant.from_device()
    for i in range(8):
        gq.dispatch(ref[i], m, xd[i])
    ops.device_status()
    assert torch.all(out[5] == 0)
    scale = float(ref.pow(2).mean().sqrt())
    assert_close(out.cpu().numpy(), ref.cpu().numpy().astype(np.float64), RTOL, ATOL * scale, "batched vs matrix-vector kernel")


def test_batched_product_refuses_bad_batches():
    raw, x = make(128, 256, 1, 8)
    t = ops.Q4KTiles(raw, 128, 256)
    with pytest.raises(_lib.WgbError):
        t.gemm(torch.zeros(9, 128, device="cuda"), torch.zeros(9, 256, device="cuda"))
    with pytest.raises(_lib.WgbError):
        t.gemm(torch.zeros(8, 128, device="cuda"), torch.zeros(8, 512, device="cuda"))


def _caches(gpu, n):
    return [(gpu.key_cache(l)[:n].cpu().numpy(), gpu.value_cache(l)[:n].cpu().numpy()) for l in range(gpu.config.n_layers)]


@pytest.mark.parametrize("case", [
    dict(n_prompt=45, n_kv_heads=8, qwen=False, mixed=False),     # five full passes and a remainder of four (a short pass)
    dict(n_prompt=20, n_kv_heads=2, qwen=True, mixed=False),      # grouped-query heads, biases, Neox RoPE; remainder 3 stays sequential
    dict(n_prompt=34, n_kv_heads=8, qwen=False, mixed=True),      # a Q6_K and a Q8_0 matrix among the Q4_K ones
    # a context of several 256-row chunks: the prompt attention of a (head, pair of positions) is shared by blocks
    dict(n_prompt=700, n_kv_heads=4, qwen=False, mixed=False, seq_len=720, n_layers=2, n_gen=6),
    # eight chunks and more: eight positions per attention block
    dict(n_prompt=1900, n_kv_heads=8, qwen=False, mixed=False, seq_len=1920, n_layers=1, n_gen=4),
])
def test_prefill_matches_sequential_loop_and_oracle(case):
    cfg = dict(SMALL_LLAMA, n_layers=case.get("n_layers", 3), n_kv_heads=case["n_kv_heads"], seq_len=case.get("seq_len", SMALL_LLAMA["seq_len"]))
    tensors = synth.llama_tensors(cfg, 21, biases=case["qwen"], scale=0.002)
    if case["mixed"]:
        tensors["blk.0.attn_v.weight"] = synth.matrix(synth.Q6_K, 512, 512, 3, "v6", 0.002)
        tensors["blk.1.ffn_down.weight"] = synth.matrix(synth.Q6_K, 512, 1024, 3, "d6", 0.002)
        tensors["blk.2.ffn_up.weight"] = synth.matrix(synth.Q8_0, 1024, 512, 3, "up8", 0.002)
        tensors["blk.1.attn_q.weight"] = synth.matrix(synth.Q5_K, 512, 512, 3, "q5", 0.002)   # no tensor-core path: position by position
    seq, cpu, _ = llama_pair(cfg, biases=case["qwen"], qwen=case["qwen"], tensors=tensors)
    bat, _, _ = llama_pair(cfg, biases=case["qwen"], qwen=case["qwen"], tensors=tensors)
    bat.set_prefill(True)
    n_prompt, n_gen = case["n_prompt"], case.get("n_gen", 12)
    prompt = synth.prompt(n_prompt, cfg["vocab_size"], seed=5)
    tok_seq = seq.decode(prompt, n_gen)
    tok_bat = bat.decode(prompt, n_gen)
    rem = (n_prompt - 1) % 8
    assert bat.prefill_positions() == n_prompt - 1 - (rem if rem < 4 else 0)
    assert seq.prefill_positions() == 0
    exp_tokens, margin = cpu.decode(prompt, n_gen)
    assert np.array_equal(tok_bat[: n_prompt - 1], prompt[1:])
    assert np.array_equal(tok_bat, tok_seq), "greedy tokens differ between batched and sequential prefill"
    assert np.array_equal(tok_bat, exp_tokens), "greedy tokens differ from the oracle"
    # cache rows of the prompt (written by the passes) and of the generated positions (written after them)
    n = n_prompt - 1 + n_gen
    kc, vc = cpu.caches()
    for l, ((kb, vb), (ks, vs)) in enumerate(zip(_caches(bat, n), _caches(seq, n))):
        sk = max(1.0, float(np.abs(kc[l, :n]).max()))
        sv = max(1.0, float(np.abs(vc[l, :n]).max()))
        assert_close(kb, kc[l, :n], RTOL, ATOL * sk, f"key cache {l} vs oracle")
        assert_close(vb, vc[l, :n], RTOL, ATOL * sv, f"value cache {l} vs oracle")
        assert_close(kb, ks.astype(np.float64), RTOL, ATOL * sk, f"key cache {l} vs sequential")
        assert_close(vb, vs.astype(np.float64), RTOL, ATOL * sv, f"value cache {l} vs sequential")
    # logits of the last step
    lb, ls_ = bat.logits().cpu().numpy(), seq.logits().cpu().numpy()
    assert_close(lb, ls_.astype(np.float64), RTOL, ATOL * max(1.0, float(np.abs(ls_).max())), "final logits vs sequential")


def test_prefill_resumes_at_a_later_position_and_can_be_switched_off():
    cfg = dict(SMALL_LLAMA, n_layers=2)
    a, cpu, t = llama_pair(cfg, seed=8, scale=0.002)
    b, _, _ = llama_pair(cfg, tensors=t)
    b.set_prefill(True)
    p1 = synth.prompt(18, cfg["vocab_size"], seed=1)
    p2 = synth.prompt(27, cfg["vocab_size"], seed=2)
    ta = np.concatenate([a.decode(p1, 3), a.decode(p2, 5, start_pos=18 - 1 + 3)])
    tb = np.concatenate([b.decode(p1, 3), b.decode(p2, 5, start_pos=18 - 1 + 3)])
    assert np.array_equal(ta, tb)
    assert b.prefill_positions() == 16 + 24
    b.set_prefill(False)
    assert b.prefill_positions() == 0
    assert np.array_equal(b.decode(p1, 3), ta[: 17 + 3])


def test_prefill_with_the_sampler_and_up_to_the_last_cache_row():
    """Sampled generation after a batched prompt equals sampled generation after a position-by-position prompt (same
    seed: the coin depends on the position only), and a sequence may end on the last row of the cache."""
    cfg = dict(SMALL_LLAMA, n_layers=2, seq_len=64)
    a, _, t = llama_pair(cfg, seed=12, scale=0.002)
    b, _, _ = llama_pair(cfg, tensors=t)
    b.set_prefill(True)
    for m in (a, b):
        m.set_sampler(0.9, 0.95, seed=77)
    prompt = synth.prompt(41, cfg["vocab_size"], seed=3)
    n_gen = cfg["seq_len"] - 40          # positions 0 .. 63: the last step writes cache row 63
    ta, tb = a.decode(prompt, n_gen), b.decode(prompt, n_gen)
    assert b.prefill_positions() == 40
    assert np.array_equal(ta, tb)
    with pytest.raises(_lib.WgbError):   # one step more would leave the cache
        b.decode(prompt, n_gen + 1)


@pytest.mark.parametrize("case", [
    dict(cfg=dict(SMALL_GPT2), n_prompt=45, qtype=synth.Q8_0),                                   # five passes and a short one
    dict(cfg=dict(SMALL_GPT2), n_prompt=19, qtype=synth.Q5_1),                                   # no tensor-core copy: per position
    dict(cfg=dict(synth.CONFIGS["gpt2-124m"], n_layer=2), n_prompt=300, qtype=synth.Q8_0),       # 124M widths, two chunks of context
])
def test_gpt2_prefill_matches_sequential_loop_and_oracle(case):
    cfg = dict(case["cfg"], default_qtype=case["qtype"])
    seq, cpu, _ = gpt2_pair(cfg, seed=31, scale=0.002)
    bat, _, _ = gpt2_pair(cfg, seed=31, scale=0.002)
    bat.set_prefill(True)
    n_prompt, n_gen = case["n_prompt"], 10
    prompt = synth.prompt(n_prompt, cfg["n_vocab"], seed=7)
    tok_seq = seq.decode(prompt, n_gen)
    tok_bat = bat.decode(prompt, n_gen)
    rem = (n_prompt - 1) % 8
    assert bat.prefill_positions() == n_prompt - 1 - (rem if rem < 4 else 0)
    exp = cpu.decode(prompt, n_gen)
    assert np.array_equal(tok_bat[: n_prompt - 1], prompt[1:])
    assert np.array_equal(tok_bat, tok_seq), "greedy tokens differ between batched and sequential prefill"
    assert np.array_equal(tok_bat, exp), "greedy tokens differ from the oracle"
    n = n_prompt - 1 + n_gen
    kc, vc = cpu.caches()
    for l in range(bat.params.n_layer):
        sk = max(1.0, float(np.abs(kc[l, :n]).max()))
        sv = max(1.0, float(np.abs(vc[l, :n]).max()))
        assert_close(bat.key_cache(l)[:n].cpu().numpy(), kc[l, :n], RTOL, ATOL * sk, f"key cache {l} vs oracle")
        assert_close(bat.value_cache(l)[:n].cpu().numpy(), vc[l, :n], RTOL, ATOL * sv, f"value cache {l} vs oracle")
    lb, ls_ = bat.logits().cpu().numpy(), seq.logits().cpu().numpy()
    assert_close(lb, ls_.astype(np.float64), RTOL, ATOL * max(1.0, float(np.abs(ls_).max())), "final logits vs sequential")
    bat.set_prefill(False)
    assert np.array_equal(bat.decode(prompt, n_gen), tok_seq)


def test_prefill_of_a_tensor_parallel_rank_wants_its_communicator():
    from wgml_b200.models import Llama2, Llama2Config
    cfg = SMALL_LLAMA
    c = Llama2Config(cfg["dim"], cfg["hidden_dim"], cfg["n_layers"], cfg["n_q_heads"], cfg["n_kv_heads"], cfg["vocab_size"],
                     cfg["seq_len"], cfg["rope_base_freq"], cfg["rms_norm_eps"])
    m = Llama2(c, tp_rank=0, tp_size=2)
    m.load_tensors(synth.llama_tensors(cfg, 1, scale=0.002))
    with pytest.raises(_lib.WgbError) as e:
        m.set_prefill(True)
    assert e.value.status == _lib.ERR_UNSUPPORTED and "communicator" in e.value.message
