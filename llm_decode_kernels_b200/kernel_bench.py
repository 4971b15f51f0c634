"""Kernel micro-benchmarks (the reference's bench/kernel_bench.py, re-done for a B200).

    python -m llm_decode_kernels_b200.kernel_bench [bandwidth] [gemv] [attention] [--out FILE.json]

bandwidth : achievable HBM read bandwidth, register loads (b200_bw_read) and bulk-copy ring (b200_bw_read_bulk)
gemv      : the single-GEMV configuration (5632 x 2048, g128) and every TinyLlama / Llama-3-70B GEMV shape, all GEMV
            kernels of the library, cold weights (enough distinct copies to exceed the L2 rotate inside one graph)
attention : paged split-K attention, 32 query / 4 KV heads, head_dim 64, page 16, batch 1 at contexts 128..8192 and
            batch 8 with contexts drawn from [128, 8192]; KV pools larger than the L2 where the case allows

Timing: CUDA events around a CUDA graph that holds `reps` launches, 3 warm-up replays, median of 5. Every case is
checked against a plain fp32 torch evaluation of the same op on the device before it is timed (the reference's rule:
no speed number before the accuracy gate).
Prints one JSON object; --out also writes it to a file.
"""
import argparse
import json
import statistics
from pathlib import Path

import torch

from . import ext
from .quant import QuantLinear

L2_BYTES = 126 << 20


def graph_time_us(fn, reps_in_graph, replays=5):
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    for _ in range(3):
        g.replay()
    ts = []
    for _ in range(replays):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / reps_in_graph)
    return statistics.median(ts)


def bench_bandwidth(K):
    buf = torch.ones(2 << 30, dtype=torch.uint8, device="cuda")
    sink = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = {}
    for blocks, threads, unroll in ((148 * 8, 512, 4), (148 * 4, 1024, 8), (148 * 16, 256, 8)):
        us = graph_time_us(lambda: K.bw_read(buf, sink, blocks, threads, unroll), 1)
        out[f"bw_read blocks={blocks} threads={threads} unroll={unroll}"] = round(buf.numel() / us / 1e3, 1)
    for stage, stages in ((16384, 12), (32768, 6), (8192, 24), (4096, 32)):
        us = graph_time_us(lambda: K.bw_read_bulk(buf, sink, 148, stage, stages), 1)
        out[f"bw_read_bulk stage={stage} stages={stages}"] = round(buf.numel() / us / 1e3, 1)
    assert int(sink) == 0
    return {"unit": "GB/s", "bytes": buf.numel(), "results": out, "achievable_read_gbps": max(out.values())}


GEMV_SHAPES = {"config1 5632x2048": (5632, 2048), "qkv 2560x2048": (2560, 2048), "o 2048x2048": (2048, 2048),
               "gate_up 11264x2048": (11264, 2048), "down 2048x5632": (2048, 5632), "lm_head 32000x2048": (32000, 2048),
               "70b qkv 10240x8192": (10240, 8192), "70b gate_up 57344x8192": (57344, 8192),
               "70b down 8192x28672": (8192, 28672), "70b tp8 o 8192x1024": (8192, 1024)}
GEMV_KERNELS = {"tensor-core (default)": (2, 0, 0, 0), "segmented": (2, 16, 0, 0), "rows R=2 warps=8": (2, 2, 8, 0),
                "rows R=4 warps=8": (2, 4, 8, 0), "plain": (0, 1, 4, 0)}


def bench_gemv(K):
    rows = {}
    for name, (N, Kd) in GEMV_SHAPES.items():
        nbytes = N * Kd // 2 + 4 * N * Kd // 128 + 2 * Kd + 2 * N
        copies = max(2, -(-2 * L2_BYTES // nbytes))
        torch.manual_seed(0)
        mats = [QuantLinear((torch.randn(N, Kd, device="cuda") * 0.02).half(), 128, keep_ref=(i == 0))
                for i in range(copies)]
        x = torch.randn(Kd, device="cuda").half()
        y = torch.empty(N, dtype=torch.half, device="cuda")
        ref = mats[0].w_ref.float() @ x.float()
        row = {"bytes": nbytes, "copies": copies, "floor_us_at_8TBs": round(nbytes / 8e6, 3)}
        for label, cfg in GEMV_KERNELS.items():
            if label == "plain" and N * Kd > 5e7:
                continue
            K.gemv_w4a16(*cfg, mats[0].packed, mats[0].sz, x, y, 128)
            err = (y.float() - ref).abs().max().item() / ref.abs().max().item()
            assert err <= 5e-3, (name, label, err)

            def run():
                for m in mats:
                    K.gemv_w4a16(*cfg, m.packed, m.sz, x, y, 128)
            us = graph_time_us(run, copies)
            row[label] = {"us": round(us, 2), "gbps": round(nbytes / us / 1e3, 1), "max_rel_err": float(f"{err:.2e}")}
        tiled = [K.gemv_tile_repack(m.packed, m.sz, 128) for m in mats]
        K.gemv_w4a16_tiled(tiled[0], x, y, N, Kd)
        err = (y.float() - ref).abs().max().item() / ref.abs().max().item()
        assert err <= 5e-3, (name, "tiled", err)

        def run_tiled():
            for tw in tiled:
                K.gemv_w4a16_tiled(tw, x, y, N, Kd)
        us = graph_time_us(run_tiled, copies)
        row["tensor-core, tile layout"] = {"us": round(us, 2), "gbps": round(nbytes / us / 1e3, 1),
                                           "max_rel_err": float(f"{err:.2e}")}
        del tiled
        rows[name] = row
        del mats
    return rows


def attention_fp32(q, kc, vc, bt, ctxs, page):
    """Plain fp32 attention over the gathered pages of every sequence: q [B, n_q, D] -> [B, n_q, D]."""
    B, n_q, D = q.shape
    n_kv = kc.shape[1]
    out = torch.empty(B, n_q, D, device=q.device)
    for b, ctx in enumerate(ctxs):
        pages = bt[b, :(ctx + page - 1) // page].long()
        k = kc[pages].permute(1, 0, 2, 3).reshape(n_kv, -1, D)[:, :ctx].float()      # [n_kv, ctx, D]
        v = vc[pages].permute(1, 0, 2, 3).reshape(n_kv, -1, D)[:, :ctx].float()
        qg = q[b].float().view(n_kv, n_q // n_kv, D)
        p = torch.softmax(qg @ k.transpose(1, 2) / D ** 0.5, dim=-1)
        out[b] = (p @ v).view(n_q, D)
    return out


def bench_attention(K):
    n_q, n_kv, D, page = 32, 4, 64, 16
    out = {}
    g = torch.Generator().manual_seed(0)
    cases = [(1, [c]) for c in (128, 512, 2048, 8192)] + [(8, torch.randint(128, 8193, (8,), generator=g).tolist())]
    for B, ctxs in cases:
        pages_per_seq = [(c + page - 1) // page for c in ctxs]
        seq_bytes = sum(2 * c * n_kv * D * 2 for c in ctxs)
        sets = max(2, min(64, -(-2 * L2_BYTES // seq_bytes)))      # distinct KV sets rotated inside the graph
        pool = sum(pages_per_seq) * sets + 3
        torch.manual_seed(1)
        kc = torch.randn(pool, n_kv, page, D, device="cuda").half()
        vc = torch.randn(pool, n_kv, page, D, device="cuda").half()
        perm = torch.randperm(pool)
        bts, o = [], 0
        for _ in range(sets):
            bt = torch.zeros(B, max(pages_per_seq), dtype=torch.int32)
            for b, n in enumerate(pages_per_seq):
                bt[b, :n] = perm[o:o + n]
                o += n
            bts.append(bt.cuda())
        q = torch.randn(B, n_q, D, device="cuda").half()
        pos = torch.tensor([c - 1 for c in ctxs], dtype=torch.int32, device="cuda")
        ref = attention_fp32(q, kc, vc, bts[0], ctxs, page)
        row = {}
        for ver, label in ((1, "v1 register loads"), (2, "v2 ring, fp32 pipes"), (3, "v3 ring, tensor cores")):
            best = None
            for PS in (64, 128, 256, 512, 1024):
                if PS > max(ctxs) and PS != 64:
                    continue
                S = (max(ctxs) + PS - 1) // PS
                o_part = torch.empty(B, n_q, S, D, device="cuda")
                m_part, l_part = torch.empty(B, n_q, S, device="cuda"), torch.empty(B, n_q, S, device="cuda")
                res = torch.empty(B, n_q, D, dtype=torch.half, device="cuda")
                K.paged_attention_batched(q, kc, vc, bts[0], pos, PS, o_part, m_part, l_part, res, version=ver)
                err = (res.float() - ref).abs().max().item() / ref.abs().max().item()
                assert err <= 2e-3, (B, ctxs, PS, ver, err)

                def run():
                    for bt in bts:
                        K.paged_attention_batched(q, kc, vc, bt, pos, PS, o_part, m_part, l_part, res, version=ver)
                us = graph_time_us(run, sets)
                if best is None or us < best["us"]:
                    best = {"part_size": PS, "us": round(us, 2), "gbps": round(seq_bytes / us / 1e3, 1),
                            "max_rel_err": float(f"{err:.2e}")}
            row[label] = best
        key = f"batch {B} ctx {ctxs[0] if B == 1 else 'U[128,8192] sum ' + str(sum(ctxs))}"
        out[key] = dict(row, bytes=seq_bytes, kv_sets=sets, floor_us_at_8TBs=round(seq_bytes / 8e6, 3))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("sections", nargs="*", default=["bandwidth", "gemv", "attention"])
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    K = ext.load()
    res = {"gpu": torch.cuda.get_device_name(0)}
    for s in a.sections:
        res[s] = {"bandwidth": bench_bandwidth, "gemv": bench_gemv, "attention": bench_attention}[s](K)
    txt = json.dumps(res, indent=1)
    print(txt)
    if a.out:
        Path(a.out).write_text(txt)


if __name__ == "__main__":
    main()
