"""Failure detection on the device without a fault: a tensor-parallel rank whose peer never delivers.

A two-rank model is built on ONE GPU as rank 0, with both ranks' mailboxes and flags mapped to local buffers
(wgb_llama2_set_exchange_buffers).  Nothing ever raises rank 1's flags, so the first kernel that gathers the
partial products waits until the configured limit, leaves code 6 in the status word and carries on; every later
wait is skipped, the decode call notices within two batches of 64 steps and returns WGB_ERR_TIMEOUT.  The
context stays usable: the next call on another model succeeds."""
import time

import numpy as np
import pytest
import torch

from helpers import SMALL_LLAMA, llama_pair
from wgml_b200 import _lib, synth, tp
from wgml_b200.models import Llama2, Llama2Config

pytestmark = pytest.mark.gpu


def test_missing_peer_times_out_and_the_context_survives():
    cfg = dict(SMALL_LLAMA, seq_len=400)
    t = synth.llama_tensors(cfg, seed=3, scale=0.002)
    c = Llama2Config(cfg["dim"], cfg["hidden_dim"], cfg["n_layers"], cfg["n_q_heads"], cfg["n_kv_heads"], cfg["vocab_size"],
                     cfg["seq_len"], cfg["rope_base_freq"], cfg["rms_norm_eps"])
    lib = _lib.load()
    old = lib.wgb_get_wait_limit_ms()
    m = Llama2(c, tp_rank=0, tp_size=2)
    try:
        m.load_tensors(t)
        mail_bytes, flag_bytes = m.exchange_bytes()
        bufs = [torch.zeros(mail_bytes // 4, dtype=torch.float32, device="cuda") for _ in range(2)]
        flags = [torch.zeros(flag_bytes // 4, dtype=torch.int32, device="cuda") for _ in range(2)]
        m.set_exchange_buffers([b.data_ptr() for b in bufs], [f.data_ptr() for f in flags])
        tp.set_wait_limit_ms(50)
        torch.cuda.synchronize()
        t0 = time.monotonic()
        with pytest.raises(_lib.WgbError) as e:
            m.decode(synth.prompt(4, cfg["vocab_size"], 3), 300)
        dt = time.monotonic() - t0
        assert e.value.status == _lib.ERR_TIMEOUT, e.value
        assert "code 6" in str(e.value)
        assert dt < 3.0, f"the call took {dt:.2f} s: the waits did not fail fast"
        # the status word was cleared by the report, and the device answers
        assert lib.wgb_device_status() == _lib.OK
    finally:
        tp.set_wait_limit_ms(old)
        m.close()
    gpu, cpu, _ = llama_pair(SMALL_LLAMA, seed=3, scale=0.002)
    prompt = synth.prompt(4, SMALL_LLAMA["vocab_size"], 3)
    exp, _ = cpu.decode(prompt, 8)
    assert np.array_equal(gpu.decode(prompt, 8), exp)
    assert lib.wgb_device_status() == _lib.OK
    gpu.close()


def test_wait_limit_is_validated():
    lib = _lib.load()
    old = lib.wgb_get_wait_limit_ms()
    assert lib.wgb_set_wait_limit_ms(0) == _lib.ERR_INVALID
    assert lib.wgb_set_wait_limit_ms(700000) == _lib.ERR_INVALID
    assert lib.wgb_get_wait_limit_ms() == old
