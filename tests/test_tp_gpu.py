"""Tensor-parallel decode on 2 GPUs against the single-GPU runtime and the CPU oracle (needs >= 2 CUDA devices)."""
import os
import types

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _cfg():
    return types.SimpleNamespace(hidden_size=1024, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
                                 intermediate_size=2048, vocab_size=3000, rms_norm_eps=1e-5, rope_theta=10000.0,
                                 head_dim=128)


def _rank_main(rank, world, port, out):
    import torch.distributed as dist
    from llm_decode_kernels_b200.model import DecodeConfig, Model
    from llm_decode_kernels_b200.shapes import random_llama_state
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    try:
        c = _cfg()
        sd = {k: (v * 3 if v.dim() == 2 else v) for k, v in random_llama_state(c, "cpu", 3).items()}
        m = Model(sd, c, DecodeConfig(max_ctx=96, seed=4, device=f"cuda:{rank}", tp_rank=rank, tp_world=world))
        assert not m.persistent and m.n_q == 8 // world and m.V == 3000 // world
        g = torch.Generator().manual_seed(1)
        prompt = torch.randint(0, 3000, (20,), generator=g).tolist()
        res = {}
        for use_graph in (False, True):
            m.kv.zero_()
            m.prepare(96, use_graph=use_graph, part_size=32)
            m.reset(0)
            res[use_graph] = m.teacher_force(prompt, use_graph=use_graph, collect_logits=True).float().cpu()
        toks = m.generate(prompt, 12)
        if rank == 0:
            torch.save({"eager": res[False], "graph": res[True], "tokens": toks, "prompt": prompt}, out)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_tp2_matches_single_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from llm_decode_kernels_b200.model import DecodeConfig, Model
    from llm_decode_kernels_b200.shapes import random_llama_state
    out = str(tmp_path / "tp2.pt")
    mp.spawn(_rank_main, args=(2, 29900 + os.getpid() % 1000, out), nprocs=2, join=True)
    got = torch.load(out)
    c = _cfg()
    sd = {k: (v * 3 if v.dim() == 2 else v) for k, v in random_llama_state(c, "cpu", 3).items()}
    m = Model(sd, c, DecodeConfig(max_ctx=96, seed=4, step_kernel="multi"))
    m.prepare(96, use_graph=False, part_size=32)
    m.reset(0)
    ref = m.teacher_force(got["prompt"], use_graph=False, collect_logits=True).float().cpu()
    scale = ref.abs().max().item()
    for key in ("eager", "graph"):
        assert (got[key] - ref).abs().max().item() <= 1e-2 * scale, key    # only the summation order differs
    assert (got["eager"] - got["graph"]).abs().max().item() <= 2e-3 * scale
    assert got["tokens"][0] == int(ref[-1].argmax())
