"""Tensor-parallel decode on 2 GPUs against the CPU oracle and the single-GPU runtime (needs >= 2 CUDA devices)."""
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


def _rank_main(rank, world, port, out, modes, tp_comm, fuse):
    import datetime
    import torch.distributed as dist
    from llm_decode_kernels_b200.model import DecodeConfig, Model
    from llm_decode_kernels_b200.shapes import random_llama_state
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"),
                            timeout=datetime.timedelta(seconds=60))   # a stuck collective ends with an error
    try:
        c = _cfg()
        sd = {k: (v * 3 if v.dim() == 2 else v) for k, v in random_llama_state(c, "cpu", 3).items()}
        m = Model(sd, c, DecodeConfig(max_ctx=96, seed=4, device=f"cuda:{rank}", tp_rank=rank, tp_world=world,
                                      tp_comm=tp_comm, tp_allreduce=fuse if isinstance(fuse, str) else ("gemv" if fuse else "kernel")))
        assert m.norm_in_gemv == (fuse is True and tp_comm == "p2p")
        assert not m.persistent and m.n_q == 8 // world and m.V == 3000 // world
        assert (m.comm is not None) == (tp_comm == "p2p")
        g = torch.Generator().manual_seed(1)
        prompt = torch.randint(0, 3000, (20,), generator=g).tolist()
        res = {}
        for use_graph in modes:
            m.kv.zero_()
            m.prepare(96, use_graph=use_graph, part_size=32)
            m.reset(0)
            assert (m.graph is not None) == (use_graph and tp_comm == "p2p")
            res[use_graph] = m.teacher_force(prompt, use_graph=use_graph, collect_logits=True).float().cpu()
        toks = m.generate(prompt, 12, use_graph=modes[-1])
        assert m.step_error() == 0
        if len(modes) == 2:   # the captured graph replays exactly what the eager launches compute
            assert torch.equal(res[modes[0]], res[modes[1]])
        if rank == 0:
            torch.save({"logits": res[modes[-1]], "tokens": toks, "prompt": prompt, "bt": m.bt.cpu()}, out)
        dist.barrier()
        if m.comm is not None:
            m.comm.close()
    finally:
        dist.destroy_process_group()


def _spawn(world, out, modes, tp_comm, fuse, limit_s=150):
    """Child processes with a deadline: a rank that never returns is killed and the test fails, it does not hang."""
    ctx = mp.get_context("spawn")
    port = 29900 + (os.getpid() + len(modes) + len(tp_comm)) % 1000
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, out, modes, tp_comm, fuse)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(limit_s)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:
        p.kill()
    assert not stuck, "a rank did not finish in time"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]


@pytest.mark.parametrize("tp_comm,modes,fuse", [
    ("nccl", (False,), True),          # NCCL collectives: launched eagerly
    ("p2p", (False, True), True),      # all-reduce inside the row-split GEMVs: eager, then one graph
    ("p2p", (False, True), False),     # exchange kernels of their own, fused with add + RMSNorm
    ("p2p", (False, True), "push")])   # GEMVs that push tagged words, consumed by the add + RMSNorm kernel
def test_tp2_matches_single_gpu(tmp_path, tp_comm, modes, fuse):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from llm_decode_kernels_b200.model import DecodeConfig, Model
    from llm_decode_kernels_b200.shapes import random_llama_state
    out = str(tmp_path / "tp2.pt")
    _spawn(2, out, modes, tp_comm, fuse)
    got = torch.load(out)
    c = _cfg()
    sd = {k: (v * 3 if v.dim() == 2 else v) for k, v in random_llama_state(c, "cpu", 3).items()}
    m = Model(sd, c, DecodeConfig(max_ctx=96, seed=4, step_kernel="multi"))
    m.prepare(96, use_graph=False, part_size=32)
    m.reset(0)
    ref = m.teacher_force(got["prompt"], use_graph=False, collect_logits=True).float().cpu()
    scale = ref.abs().max().item()
    assert (got["logits"] - ref).abs().max().item() <= 1e-2 * scale    # only the summation order differs
    assert got["tokens"][0] == int(got["logits"][-1].argmax())
    # the CPU oracle on the unsharded model: RTN quantization works group by group along K and row by row, so
    # quantizing a shard gives the bits of the same rows / column groups of the quantized whole matrix
    from oracle import model_oracle as MO
    ocfg = types.SimpleNamespace(group=128, quant="rtn", qparams=None, max_ctx=96, page=16, shuffle_pages=True)
    o = MO.OracleModel(sd, c, ocfg, block_table=got["bt"])
    want = o.teacher_force(got["prompt"], collect_logits=True).float()
    assert (got["logits"] - want).abs().max().item() <= 1.5e-2 * want.abs().max().item()
