"""Kernel micro-benchmarks (the reference's bench/kernel_bench.py, re-done for a B200).

    python -m llm_decode_kernels_b200.kernel_bench [bandwidth] [gemv] [attention] [gemm] [--out FILE.json]

bandwidth : achievable HBM read bandwidth, register loads (b200_bw_read) and bulk-copy ring (b200_bw_read_bulk)
gemv      : the single-GEMV configuration (5632 x 2048, g128) and every TinyLlama / Llama-3-70B GEMV shape, all GEMV
            kernels of the library, cold weights (enough distinct copies to exceed the L2 rotate inside one graph)
gemm      : the prompt's batched GEMM on the tcgen05 tensor cores, TinyLlama shapes at 16 / 64 / 256 tokens (on request)
attention : paged split-K attention, 32 query / 4 KV heads, head_dim 64, page 16, batch 1 at contexts 128..8192 and
            batch 8 with contexts drawn from [128, 8192]; KV pools larger than the L2 where the case allows

Timing (the discipline of the reference's bench/timing.py:119-138): CUDA events around every replay of a CUDA graph
that holds `reps` launches, 5 warm-up replays, then 30 timed ones; reported are the median, the inter-quartile range
and the SM clock read through NVML right after the timed replays. Every case is checked against a plain fp32 torch
evaluation of the same op on the device before it is timed (the reference's rule: no speed number before the
accuracy gate).

`attention` also rewrites configs/attn_policy.json - the best split size per context, batch 1 - which Model reads
(DecodeConfig.attn_policy_path); the reference grows the same file from the same sweep (bench/kernel_bench.py:182-202).
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


def sm_clock_mhz(index=0):
    """Current SM clock through NVML (None when NVML is not there)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        return pynvml.nvmlDeviceGetClockInfo(pynvml.nvmlDeviceGetHandleByIndex(index), pynvml.NVML_CLOCK_SM)
    except Exception:
        return None


def graph_stats(fn, reps_in_graph, replays=30, warm=5):
    """fn() issues `reps_in_graph` launches; they are captured in one graph. Returns microseconds per launch:
    {"us": median, "iqr_us": q3 - q1, "sm_mhz": clock after the timed replays}."""
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    for _ in range(warm):
        g.replay()
    ts = []
    for _ in range(replays):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / reps_in_graph)
    q = statistics.quantiles(ts, n=4)
    return {"us": round(statistics.median(ts), 3), "iqr_us": round(q[2] - q[0], 3), "sm_mhz": sm_clock_mhz()}


def graph_time_us(fn, reps_in_graph, replays=30):
    return graph_stats(fn, reps_in_graph, replays)["us"]


def isolated_stats(fns, replays=3):
    """Every fn of `fns` is one launch on cold data; each gets a graph of its own and is timed alone (events around a
    single replay, the graphs taken in turn so that no launch finds its data in the L2)."""
    graphs = []
    for fn in fns:
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        graphs.append(g)
    for g in graphs:
        g.replay()
    ts = []
    for _ in range(replays):
        for g in graphs:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
    q = statistics.quantiles(ts, n=4)
    return {"us": round(statistics.median(ts), 3), "iqr_us": round(q[2] - q[0], 3), "sm_mhz": sm_clock_mhz()}


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
TINY_SHAPES = ("config1 5632x2048", "qkv 2560x2048", "o 2048x2048", "gate_up 11264x2048", "down 2048x5632",
               "lm_head 32000x2048")
GEMV_KERNELS = {"tensor-core (default)": (2, 0, 0, 0), "segmented": (2, 16, 0, 0), "rows R=2 warps=8": (2, 2, 8, 0),
                "rows R=4 warps=8": (2, 4, 8, 0), "plain": (0, 1, 4, 0)}
POLICY_PATH = Path(__file__).resolve().parent / "configs" / "attn_policy.json"


def gemv_bytes(N, Kd, group=128):
    """Algorithmic bytes of one GEMV: packed weights + (scale, zero) + x + y (reference bench/kernel_bench.py:74)."""
    return N * Kd // 2 + 4 * N * Kd // group + 2 * Kd + 2 * N


def gemv_case(K, N, Kd, kernels=True, isolated=False):
    """One GEMV shape on cold weights: enough distinct matrices to exceed twice the L2, multiplied in turn inside one
    graph (dependent launches chained, as in a decode step). Returns the row of the report."""
    nbytes = gemv_bytes(N, Kd)
    copies = max(2, -(-2 * L2_BYTES // nbytes))
    torch.manual_seed(0)
    mats = [QuantLinear((torch.randn(N, Kd, device="cuda") * 0.02).half(), 128, keep_ref=(i == 0))
            for i in range(copies)]
    x = torch.randn(Kd, device="cuda").half()
    y = torch.empty(N, dtype=torch.half, device="cuda")
    ref = mats[0].w_ref.float() @ x.float()
    row = {"bytes": nbytes, "copies": copies, "floor_us_at_8TBs": round(nbytes / 8e6, 3)}

    def record(label, one, err):
        assert err <= 5e-3, (N, Kd, label, err)
        st = graph_stats(lambda: [one(i) for i in range(copies)], copies)
        st.update(gbps=round(nbytes / st["us"] / 1e3, 1), max_rel_err=float(f"{err:.2e}"))
        if isolated:
            iso = isolated_stats([(lambda i=i: one(i)) for i in range(copies)])
            st["isolated"] = dict(iso, gbps=round(nbytes / iso["us"] / 1e3, 1))
        row[label] = st

    if kernels:
        for label, cfg in GEMV_KERNELS.items():
            if label == "plain" and N * Kd > 5e7:
                continue
            K.gemv_w4a16(*cfg, mats[0].packed, mats[0].sz, x, y, 128)
            err = (y.float() - ref).abs().max().item() / ref.abs().max().item()
            record(label, lambda i, cfg=cfg: K.gemv_w4a16(*cfg, mats[i].packed, mats[i].sz, x, y, 128), err)
    tiled = [K.gemv_tile_repack(m.packed, m.sz, 128) for m in mats]
    K.gemv_w4a16_tiled(tiled[0], x, y, N, Kd)
    err = (y.float() - ref).abs().max().item() / ref.abs().max().item()
    record("tensor-core, tile layout", lambda i: K.gemv_w4a16_tiled(tiled[i], x, y, N, Kd), err)
    return row


def bench_gemv(K):
    return {name: gemv_case(K, N, Kd, isolated=name in TINY_SHAPES) for name, (N, Kd) in GEMV_SHAPES.items()}


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


ATTN_VERSIONS = ((1, "v1 register loads"), (2, "v2 ring, fp32 pipes"), (3, "v3 ring, tensor cores"))
ATTN_CONTEXTS = (128, 512, 2048, 8192)


def attention_case(K, B, ctxs, versions=ATTN_VERSIONS, part_sizes=(64, 128, 256, 512, 1024)):
    """Paged split-K attention, 32 query / 4 KV heads, head_dim 64, pages of 16 tokens, block table a random
    permutation; every kernel version at every split size, the best split size kept per version."""
    n_q, n_kv, D, page = 32, 4, 64, 16
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
    for ver, label in versions:
        best = None
        for PS in part_sizes:
            if PS > max(ctxs) and PS != part_sizes[0]:
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
            st = graph_stats(run, sets)
            if best is None or st["us"] < best["us"]:
                best = dict(st, part_size=PS, gbps=round(seq_bytes / st["us"] / 1e3, 1),
                            max_rel_err=float(f"{err:.2e}"))
        row[label] = best
    return dict(row, bytes=seq_bytes, kv_sets=sets, floor_us_at_8TBs=round(seq_bytes / 8e6, 3))


def write_attn_policy(rows, path=POLICY_PATH):
    """rows: {context: best part_size} at batch 1 -> the policy file Model reads. One entry per tuned context
    ("contexts up to max_ctx use part_size"), plus a catch-all for anything longer."""
    ctxs = sorted(rows)
    policy = [{"max_ctx": c, "part_size": int(rows[c])} for c in ctxs]
    policy.append({"max_ctx": 1 << 30, "part_size": int(rows[ctxs[-1]])})
    path.parent.mkdir(exist_ok=True)
    path.write_text(json.dumps({"gpu": torch.cuda.get_device_name(0), "heads": "32q/4kv x64", "page": 16,
                                "kernel": "v3 ring, tensor cores", "policy": policy}, indent=1) + "\n")


def bench_attention(K, write_policy=True):
    out = {}
    g = torch.Generator().manual_seed(0)
    best_ps = {}
    for c in ATTN_CONTEXTS:
        row = attention_case(K, 1, [c])
        out[f"batch 1 ctx {c}"] = row
        best_ps[c] = row["v3 ring, tensor cores"]["part_size"]
    ctxs = torch.randint(128, 8193, (8,), generator=g).tolist()
    out[f"batch 8 ctx U[128,8192] sum {sum(ctxs)}"] = attention_case(K, 8, ctxs)
    if write_policy:
        write_attn_policy(best_ps)
        out["policy_written"] = str(POLICY_PATH)
    return out


def headline_kernels(K, peak_gbs):
    """The single-kernel configurations of the benchmark suite in the short form bench.py records: the 5632 x 2048
    GEMV (tile layout; isolated launches and the dependent-launch chain over cold matrices) and paged attention with
    the library's default kernel at batch 1, contexts 128 .. 8192, and batch 8 with contexts from [128, 8192]."""
    N, Kd = GEMV_SHAPES["config1 5632x2048"]
    row = gemv_case(K, N, Kd, kernels=False, isolated=True)["tensor-core, tile layout"]
    res = {"gemv_config1": {"shape": f"{N}x{Kd} g128", "bytes": gemv_bytes(N, Kd), "us_chained": row["us"],
                            "iqr_us_chained": row["iqr_us"], "gbps_chained": row["gbps"],
                            "frac_chained": round(row["gbps"] / peak_gbs, 4), "us_isolated": row["isolated"]["us"],
                            "iqr_us_isolated": row["isolated"]["iqr_us"], "gbps_isolated": row["isolated"]["gbps"],
                            "frac_isolated": round(row["isolated"]["gbps"] / peak_gbs, 4), "sm_mhz": row["sm_mhz"],
                            "max_rel_err": row["max_rel_err"],
                            "how": "cold weights (distinct matrices > 2 x L2 taken in turn); chained = one graph of "
                                   "dependent launches, isolated = one launch per graph replay; median of 30 / IQR"}}
    att = {}
    g = torch.Generator().manual_seed(0)
    cases = [(1, [c]) for c in ATTN_CONTEXTS] + [(8, torch.randint(128, 8193, (8,), generator=g).tolist())]
    for B, ctxs in cases:
        r = attention_case(K, B, ctxs, versions=((3, "v3"),), part_sizes=(64, 256, 1024))
        key = f"b{B}_ctx{ctxs[0]}" if B == 1 else "b8_ctx_u128_8192"
        att[key] = {"us": r["v3"]["us"], "iqr_us": r["v3"]["iqr_us"], "part_size": r["v3"]["part_size"],
                    "bytes": r["bytes"], "gbps": r["v3"]["gbps"], "frac": round(r["v3"]["gbps"] / peak_gbs, 4),
                    "max_rel_err": r["v3"]["max_rel_err"], "sm_mhz": r["v3"]["sm_mhz"]}
    res["attention_config2"] = att
    return res


def bench_gemm(K, shapes=None, tokens=(16, 64, 256)):
    """The prompt's batched W4A16 GEMM (b200_gemm_w4a16) on the TinyLlama matrix shapes at 16 / 64 / 256 tokens:
    microseconds, dense TFLOP/s (2 T N K), the rate at which the packed weights stream, and the time the same work
    takes as T GEMV launches (tile layout). Checked against an fp32 product with the dequantized matrix first."""
    out = {}
    for name in shapes or ("qkv 2560x2048", "o 2048x2048", "gate_up 11264x2048", "down 2048x5632",
                           "lm_head 32000x2048"):
        N, Kd = GEMV_SHAPES[name]
        torch.manual_seed(0)
        ql = QuantLinear((torch.randn(N, Kd, device="cuda") * 0.02).half(), 128, keep_ref=True)
        tiled = K.gemv_tile_repack(ql.packed, ql.sz, 128)
        x1, y1 = torch.randn(Kd, device="cuda").half(), torch.empty(N, dtype=torch.half, device="cuda")
        gemv_us = graph_time_us(lambda: [K.gemv_w4a16_tiled(tiled, x1, y1, N, Kd) for _ in range(20)], 20)
        row = {"gemv_us": gemv_us}
        for T in tokens:
            x = torch.randn(T, Kd, device="cuda").half()
            y = torch.empty(T, N, dtype=torch.half, device="cuda")
            K.gemm_w4a16(ql.packed, ql.sz, x, y, 128)
            ref = x.float() @ ql.w_ref.float().t()
            err = ((y.float() - ref).abs().max() / ref.abs().max()).item()
            assert err <= 2e-3, (name, T, err)
            st = graph_stats(lambda: [K.gemm_w4a16(ql.packed, ql.sz, x, y, 128) for _ in range(10)], 10)
            row[f"T{T}"] = {"us": st["us"], "iqr_us": st["iqr_us"], "tflops": round(2 * T * N * Kd / st["us"] / 1e6, 1),
                            "weight_gbps": round(gemv_bytes(N, Kd) / st["us"] / 1e3, 1),
                            "vs_T_gemvs": round(T * gemv_us / st["us"], 1), "max_rel_err": round(err, 6),
                            "sm_mhz": st["sm_mhz"]}
        out[name] = row
    out["status"] = K.gemm_status()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("sections", nargs="*", default=["bandwidth", "gemv", "attention"])
    ap.add_argument("--out", default=None)
    ap.add_argument("--gemm-shape", action="append", default=None, help="gemm: only this shape (a key of GEMV_SHAPES)")
    ap.add_argument("--gemm-tokens", type=int, action="append", default=None, help="gemm: only this many tokens")
    a = ap.parse_args()
    K = ext.load()
    res = {"gpu": torch.cuda.get_device_name(0)}
    run = {"bandwidth": bench_bandwidth, "gemv": bench_gemv, "attention": bench_attention,
           "gemm": lambda k: bench_gemm(k, a.gemm_shape, tuple(a.gemm_tokens or (16, 64, 256)))}
    for s in a.sections:
        res[s] = run[s](K)
    txt = json.dumps(res, indent=1)
    print(txt)
    if a.out:
        Path(a.out).write_text(txt)


if __name__ == "__main__":
    main()
