"""One rank of the tensor-parallel GPU parity test (launched by test_gpu_tp.py through torch.distributed.run).

Every rank builds its shard of the same seeded model and decodes the same prompt; rank 0 also runs the
unsharded model on its GPU and writes both results for the test to compare."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from wgml_b200 import _lib, synth, tp  # noqa: E402
from wgml_b200.models import Llama2, Llama2Config  # noqa: E402

CASES = {
    # grouped-query attention, Q4_K, uneven split of the FFN blocks over 2 ranks (3 blocks)
    "gqa_q4k": dict(arch="llama", dim=512, hidden_dim=768, n_layers=3, n_q_heads=8, n_kv_heads=4, vocab_size=1000,
                    seq_len=96, rope_base_freq=10000.0, rms_norm_eps=1e-5, default_qtype=synth.Q4_K),
    # dense f32 (the tiny reference-runnable configuration, shortened)
    "tiny_f32": dict(synth.CONFIGS["tiny-llama"], n_layers=2, seq_len=64),
}


def main():
    out = sys.argv[1]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = tp.init_from_torch_distributed()
    res = {}
    for name, cfg in CASES.items():
        t = synth.llama_tensors(cfg, seed=5, scale=0.002 if cfg["default_qtype"] != synth.F32 else 0.02)
        c = Llama2Config(cfg["dim"], cfg["hidden_dim"], cfg["n_layers"], cfg["n_q_heads"], cfg["n_kv_heads"], cfg["vocab_size"],
                         cfg["seq_len"], cfg["rope_base_freq"], cfg["rms_norm_eps"])
        prompt = synth.prompt(8, cfg["vocab_size"], seed=5)
        # (fused schedule, direct exchange through peer memory): direct needs the fused schedule
        for fused, direct in ((True, True), (True, False), (False, False)):
            m = Llama2(c, tp_rank=rank, tp_size=world)
            m.load_tensors(t)
            m.set_fused(fused)
            tp.attach(m, comm, direct=direct)
            toks = m.decode(prompt, 24)
            if fused:
                # the per-launch timing path replays the step with time stamps (direct exchange) or events (NCCL);
                # it must leave the exchange counters intact: decode the same sequence again afterwards
                prof = m.profile_step(int(toks[-1]), len(toks))
                assert len(prof) >= 5 * cfg["n_layers"] + 1, len(prof)
                again = m.decode(prompt, 24)
                assert np.array_equal(again, toks), (name, fused, direct, again, toks)
                assert _lib.load().wgb_device_status() == _lib.OK
            m.dispatch(int(toks[-1]), len(toks))      # one eager step after the graph replays
            logits = m.logits().cpu().numpy()
            x = m.x().cpu().numpy()
            torch.cuda.synchronize()
            dist.barrier()
            if rank == 0:
                key = f"{name}/{int(fused)}{int(direct)}"
                res[key + "/tp_tokens"] = toks
                res[key + "/tp_logits"] = logits
                res[key + "/tp_x"] = x
            m.close()
        # vocabulary-sharded head: every rank computes half of the logits, an all-gather completes them; the tokens and the
        # full logits must be those of the replicated head
        for fused, direct in ((True, True), (False, False)):
            m = Llama2(c, tp_rank=rank, tp_size=world)
            m.load_tensors(t)
            m.set_fused(fused)
            tp.attach(m, comm, direct=direct, vocab_shard=True)
            toks = m.decode(prompt, 24)
            if fused:
                prof = m.profile_step(int(toks[-1]), len(toks))
                assert len(prof) >= 5 * cfg["n_layers"] + 1, len(prof)
                assert np.array_equal(m.decode(prompt, 24), toks), (name, "vocab shard: decode after the profiled step")
            m.dispatch(int(toks[-1]), len(toks))
            logits = m.logits().cpu().numpy()
            assert _lib.load().wgb_device_status() == _lib.OK
            torch.cuda.synchronize()
            dist.barrier()
            if rank == 0:
                res[f"{name}/vs{int(fused)}{int(direct)}/tp_tokens"] = toks
                res[f"{name}/vs{int(fused)}{int(direct)}/tp_logits"] = logits
            m.close()
        if name == "gqa_q4k":
            # batched prompt passes on the sharded model (partial products summed over the group by an all-reduce),
            # for both exchanges of the token loop that follows them
            long_prompt = synth.prompt(30, cfg["vocab_size"], seed=6)
            for direct in (True, False):
                m = Llama2(c, tp_rank=rank, tp_size=world)
                m.load_tensors(t)
                tp.attach(m, comm, direct=direct)
                m.set_prefill(True)
                toks = m.decode(long_prompt, 16)
                assert m.prefill_positions() == 29, m.prefill_positions()   # 3 full passes and one of five positions
                assert _lib.load().wgb_device_status() == _lib.OK
                logits = m.logits().cpu().numpy()
                torch.cuda.synchronize()
                dist.barrier()
                if rank == 0:
                    res[f"{name}/prefill{int(direct)}/tp_tokens"] = toks
                    res[f"{name}/prefill{int(direct)}/tp_logits"] = logits
                m.close()
            if rank == 0:
                m = Llama2(c)
                m.load_tensors(t)
                res[f"{name}/prefill/ref_tokens"] = m.decode(long_prompt, 16)
                res[f"{name}/prefill/ref_logits"] = m.logits().cpu().numpy()
                m.close()
        if rank == 0:
            m = Llama2(c)
            m.load_tensors(t)
            toks = m.decode(prompt, 24)
            m.dispatch(int(toks[-1]), len(toks))
            res[f"{name}/ref_tokens"] = toks
            res[f"{name}/ref_logits"] = m.logits().cpu().numpy()
            res[f"{name}/ref_x"] = m.x().cpu().numpy()
            m.close()
        dist.barrier()
    if rank == 0:
        np.savez(out, **res)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
