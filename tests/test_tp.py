"""Tensor-parallel shard arithmetic (llm_decode_kernels_b200/tp.py), on CPU.

The kernels need a GPU; what decides whether a sharded step is right is host logic: which rows and columns a rank
keeps and what has to be summed or gathered. Here every rank computes its part with the CPU oracle's operators, the
parts are combined with real collectives over a 2-rank gloo group, and the result must equal the unsharded oracle
(bit-equal where no summation order changes, to tolerance where partial sums are added)."""
import os
import types

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llm_decode_kernels_b200 import quant as PQ
from llm_decode_kernels_b200 import tp as TP
from oracle import ops_oracle as R

N_Q, N_KV, D, I, V, H, G = 8, 4, 64, 512, 1000, 512, 128
DIMS = (N_Q, N_KV, D, I, V)


def weights(seed=0):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: (torch.randn(*s, generator=g) * 0.05).half()
    return {"qkv": rn((N_Q + 2 * N_KV) * D, H), "o": rn(H, N_Q * D), "gu": rn(2 * I, H), "down": rn(H, I),
            "lm_head": rn(V, H)}


def test_partition_and_checks():
    assert TP.part(8, 1, 4) == (2, 4)
    with pytest.raises(ValueError):
        TP.part(10, 0, 4)
    TP.check(64, 8, 128, 28672, 128256, 128, 8)             # Llama-3-70B shape on 8 ranks
    with pytest.raises(ValueError):
        TP.check(32, 4, 64, 5632, 32000, 128, 8)            # TinyLlama has 4 KV heads: 8 ranks do not divide them
    with pytest.raises(ValueError):
        TP.check(8, 4, 64, 320, 1000, 128, 2)               # 160 columns per rank would cut a 128-wide group


@pytest.mark.parametrize("world", [2, 4])
def test_rows_cover_the_matrix_once(world):
    qkv = torch.cat([TP.qkv_rows(N_Q, N_KV, D, r, world) for r in range(world)])
    assert sorted(qkv.tolist()) == list(range((N_Q + 2 * N_KV) * D))
    gu = torch.cat([TP.gate_up_rows(I, r, world) for r in range(world)])
    assert sorted(gu.tolist()) == list(range(2 * I))
    # a rank's qkv rows are [its q heads; its k heads; its v heads], each a whole number of heads
    r1 = TP.qkv_rows(N_Q, N_KV, D, 1, world)
    nq, nk = N_Q // world * D, N_KV // world * D
    assert r1[0] == nq and r1[nq] == N_Q * D + nk and r1[nq + nk] == (N_Q + N_KV) * D + nk


@pytest.mark.parametrize("kind", ["qkv", "o", "gu", "down", "lm_head"])
def test_shard_then_quantize_equals_quantize_then_shard(kind):
    """RTN works per row and per group, and slices keep rows and groups whole."""
    w = weights()[kind]
    full = PQ.quantize(w, G)
    for rank in range(2):
        a = PQ.quantize(TP.shard_weight(kind, w, DIMS, rank, 2), G)
        b = TP.shard_qsz(kind, full, DIMS, G, rank, 2)
        assert all(torch.equal(x, y) for x, y in zip(a, b)), (kind, rank)


def _rank_main(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = weights()
        deq = lambda kind: PQ.QuantLinear(TP.shard_weight(kind, w[kind], DIMS, rank, world), G).w_ref
        g = torch.Generator().manual_seed(7)
        x = torch.randn(H, generator=g).half()
        # attention block: local heads only, then o_proj partial sums are all-reduced
        qkv = R.gemv_ref(deq("qkv"), x)
        nq, nk = N_Q // world, N_KV // world
        attn_in = qkv[: nq * D]                                     # (stand-in for attention output: q itself)
        o = R.gemv_ref(deq("o"), attn_in).float()
        dist.all_reduce(o)
        # MLP: gate|up local rows, SwiGLU local, down partial sums all-reduced
        act = R.swiglu_ref(R.gemv_ref(deq("gu"), x))
        down = R.gemv_ref(deq("down"), act).float()
        dist.all_reduce(down)
        # LM head: vocabulary shards gathered
        lg = R.gemv_ref(deq("lm_head"), x)
        parts = [torch.empty_like(lg) for _ in range(world)]
        dist.all_gather(parts, lg)
        qkv_parts = [torch.empty_like(qkv) for _ in range(world)]
        dist.all_gather(qkv_parts, qkv)
        if rank == 0:
            torch.save({"o": o, "down": down, "logits": torch.cat(parts), "qkv_parts": qkv_parts}, out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_sharded_step_pieces_equal_unsharded(tmp_path, world):
    out = str(tmp_path / "r0.pt")
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank_main, args=(world, port, out), nprocs=world, join=True)
    got = torch.load(out)
    w = weights()
    deq = {k: PQ.QuantLinear(v, G).w_ref for k, v in w.items()}
    g = torch.Generator().manual_seed(7)
    x = torch.randn(H, generator=g).half()
    qkv = R.gemv_ref(deq["qkv"], x)
    # gathered shards, put back in head order, are the unsharded qkv exactly (row slicing changes no arithmetic)
    rebuilt = torch.empty_like(qkv)
    for r in range(world):
        rebuilt[TP.qkv_rows(N_Q, N_KV, D, r, world)] = got["qkv_parts"][r]
    assert torch.equal(rebuilt, qkv)
    assert torch.equal(got["logits"], R.gemv_ref(deq["lm_head"], x))
    o_ref = deq["o"].float() @ qkv[: N_Q * D].float()
    # each rank fed its own q heads, in rank order = the first N_Q * D entries of qkv
    assert torch.allclose(got["o"], o_ref, rtol=0, atol=2e-3 * o_ref.abs().max().item())
    act = R.swiglu_ref(R.gemv_ref(deq["gu"], x))
    d_ref = deq["down"].float() @ act.float()
    assert torch.allclose(got["down"], d_ref, rtol=0, atol=2e-3 * d_ref.abs().max().item())


def test_rank_failure_is_reported_not_hung():
    """A rank that dies before the collective: the survivor's all_reduce must end with an error within the group's
    timeout instead of hanging (host-side failure, CPU ranks)."""
    ctx = mp.get_context("spawn")
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_failure_main, args=(r, port)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    assert procs[0].exitcode == 17 and procs[1].exitcode == 0


def _failure_main(rank, port):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2, timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        os._exit(0)                      # leaves between steps, nothing in flight
    t = torch.ones(4)
    try:
        dist.all_reduce(t)
    except Exception:
        os._exit(17)                     # reported
    os._exit(1)                          # a silent success would be wrong
