"""Small, self-ending workloads to run under `ncu` (the reference has bench/ncu_probe.py for the same purpose).

    python -m llm_decode_kernels_b200.ncu_probe gemv  [--n 32000 --k 2048 --copies 8 --iters 3 --tiled | --rows 16]
    python -m llm_decode_kernels_b200.ncu_probe attn  [--ctx 8192 --batch 8 --part 256 --version 0 --iters 3]
    python -m llm_decode_kernels_b200.ncu_probe step  [--layers 4 --tokens 4]

gemv: `copies` distinct quantized matrices (together larger than the 126 MB L2) are multiplied in turn, so every
      launch streams its weights from HBM. attn: batched paged attention over a KV pool larger than L2.
step: a TinyLlama-shape decoder cut to `layers` layers decodes a few tokens eagerly (no graph), so every kernel of
      the decode step shows up as its own launch (--step-kernel persistent: one decode_step_kernel launch per token). Everything is a few hundred MB on the device and ends in seconds.
"""
import argparse

import torch

from . import ext
from .quant import QuantLinear


def probe_gemv(a):
    K = ext.load()
    torch.manual_seed(0)
    mats = [QuantLinear((torch.randn(a.n, a.k, device="cuda") * 0.02).half(), 128, keep_ref=False)
            for _ in range(a.copies)]
    x = torch.randn(a.k, device="cuda").half()
    y = torch.empty(a.n, dtype=torch.half, device="cuda")
    tiled = [K.gemv_tile_repack(m.packed, m.sz, 128) for m in mats] if a.tiled else None
    for _ in range(a.iters):
        for i, m in enumerate(mats):
            if a.tiled:
                K.gemv_w4a16_tiled(tiled[i], x, y, a.n, a.k)
            else:
                K.gemv_w4a16(2, a.rows, 0, 0, m.packed, m.sz, x, y, 128)
    torch.cuda.synchronize()
    print("gemv bytes per launch:", mats[0].nbytes() + 2 * a.k + 2 * a.n)


def probe_attn(a):
    K = ext.load()
    torch.manual_seed(0)
    n_q, n_kv, D, page, PS = 32, 4, 64, 16, a.part
    pages_per_seq = (a.ctx + page - 1) // page
    pool = pages_per_seq * a.batch + 3
    kc = torch.randn(pool, n_kv, page, D, device="cuda").half()
    vc = torch.randn(pool, n_kv, page, D, device="cuda").half()
    bt = torch.randperm(pool, device="cuda")[: pages_per_seq * a.batch].int().view(a.batch, pages_per_seq).contiguous()
    q = torch.randn(a.batch, n_q, D, device="cuda").half()
    pos = torch.full((a.batch,), a.ctx - 1, dtype=torch.int32, device="cuda")
    S = (a.ctx + PS - 1) // PS
    o_part = torch.empty(a.batch, n_q, S, D, device="cuda")
    m_part, l_part = torch.empty(a.batch, n_q, S, device="cuda"), torch.empty(a.batch, n_q, S, device="cuda")
    out = torch.empty(a.batch, n_q, D, dtype=torch.half, device="cuda")
    for _ in range(a.iters):
        K.paged_attention_batched(q, kc, vc, bt, pos, PS, o_part, m_part, l_part, out, version=a.version)
    torch.cuda.synchronize()
    print("attention bytes per launch:", 2 * a.ctx * n_kv * D * 2 * a.batch)


def probe_step(a):
    from .model import DecodeConfig, Model
    from .shapes import TINYLLAMA, config, random_llama_state
    c = config(TINYLLAMA, num_hidden_layers=a.layers)
    m = Model(random_llama_state(c, "cuda", 0), c, DecodeConfig(max_ctx=256, seed=0, step_kernel=a.step_kernel))
    m.prepare(256, use_graph=False)
    m.reset(0)
    m.teacher_force(list(range(1, a.tokens + 1)), use_graph=False)
    torch.cuda.synchronize()
    print("tokens decoded:", a.tokens, "last token", int(m.tok))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemv", "attn", "step"])
    ap.add_argument("--n", type=int, default=32000)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--copies", type=int, default=8)
    ap.add_argument("--tiled", action="store_true", help="gemv: tensor-core kernel from the tile-layout copy")
    ap.add_argument("--rows", type=int, default=0, help="gemv: R of b200_gemv_w4a16 (0 library's choice, 16 segmented)")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--part", type=int, default=256)
    ap.add_argument("--version", type=int, default=0, help="attention kernel: 0 library's choice, 1..3")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=4)
    ap.add_argument("--step-kernel", default="multi", choices=["multi", "persistent"])
    a = ap.parse_args()
    {"gemv": probe_gemv, "attn": probe_attn, "step": probe_step}[a.op](a)
