"""Launch shapes of the tensor-core GEMV, found by measurement (the reference's scripts/autotune.py:1-58 for a B200).

    python -m llm_decode_kernels_b200.autotune [--shapes tinyllama|70b|all] [--out configs/autotune.json]

For every matrix shape of the benchmark models - as the tile-layout GEMV sees it: layout 1, and layout 2 (paired
gate|up, N = outputs) - every (ksplit, blocks) the kernel accepts is timed on cold weights (distinct matrices larger
than twice the L2, multiplied in turn inside one graph of dependent launches, median of 30 replays) after its result
has been checked against fp32; the fastest goes into the table, next to what the built-in heuristic reaches. Model
registers the table at construction (DecodeConfig.autotune_path -> b200_gemv_w4a16_tune).
"""
import argparse
import json
from pathlib import Path

import torch

from . import ext
from .kernel_bench import L2_BYTES, gemv_bytes, graph_stats
from .quant import QuantLinear

OUT = Path(__file__).resolve().parent / "configs" / "autotune.json"
SMS = 148
# (name, layout, rows of the matrix, K); layout 2: rows = 2 x outputs
TINYLLAMA = [("config1", 1, 5632, 2048), ("qkv", 1, 2560, 2048), ("o", 1, 2048, 2048), ("gate_up", 2, 11264, 2048),
             ("down", 1, 2048, 5632), ("lm_head", 1, 32000, 2048)]
LLAMA70B = [("70b tp8 qkv", 1, 1280, 8192), ("70b tp8 o", 1, 8192, 1024), ("70b tp8 gate_up", 2, 7168, 8192),
            ("70b tp8 down", 1, 8192, 3584), ("70b tp8 lm_head", 1, 16032, 8192),
            ("70b tp4 qkv", 1, 2560, 8192), ("70b tp4 o", 1, 8192, 2048), ("70b tp4 gate_up", 2, 14336, 8192),
            ("70b tp4 down", 1, 8192, 7168), ("70b tp2 qkv", 1, 5120, 8192), ("70b tp2 o", 1, 8192, 4096),
            ("70b tp2 gate_up", 2, 28672, 8192), ("70b tp2 down", 1, 8192, 14336)]


def tune_shape(K, name, layout, rows, Kd):
    N = rows // 2 if layout == 2 else rows                 # outputs
    nbytes = gemv_bytes(rows, Kd) - (2 * N if layout == 2 else 0)
    copies = max(2, -(-2 * L2_BYTES // nbytes))
    torch.manual_seed(0)
    mats = [QuantLinear((torch.randn(rows, Kd, device="cuda") * 0.02).half(), 128, keep_ref=(i == 0))
            for i in range(copies)]
    tiled = [K.gemv_tile_repack(m.packed, m.sz, 128, gate_up=layout == 2) for m in mats]
    x = torch.randn(Kd, device="cuda").half()
    y = torch.empty(N, dtype=torch.half, device="cuda")
    full = mats[0].w_ref.float() @ x.float()
    if layout == 2:
        g, u = full[:N].half().float(), full[N:].half().float()
        ref = (torch.nn.functional.silu(g).half() * u.half()).float()
    else:
        ref = full
    del mats

    def run():
        for t in tiled:
            K.gemv_w4a16_tiled(t, x, y, N, Kd, swiglu=layout == 2)

    def measure():
        K.gemv_w4a16_tiled(tiled[0], x, y, N, Kd, swiglu=layout == 2)
        err = (y.float() - ref).abs().max().item() / ref.abs().max().item()
        assert err <= 5e-3, (name, err)
        return graph_stats(run, copies)["us"]

    K.gemv_tune(layout, N, Kd, 0, 0)
    base = measure()
    tiles = (N + 7) // 8 if layout == 2 else (N + 15) // 16
    best = None
    for ksplit in (1, 2, 4, 8):
        if ksplit > Kd // 128:
            continue
        groups = -(-tiles // (8 // ksplit))
        for blocks in sorted({min(groups, b) for b in (SMS, 2 * SMS, groups, -(-groups // 2), -(-groups // 3))}):
            K.gemv_tune(layout, N, Kd, ksplit, blocks)
            us = measure()
            if best is None or us < best["us"]:
                best = {"ksplit": ksplit, "blocks": blocks, "us": us}
    K.gemv_tune(layout, N, Kd, 0, 0)
    return {"name": name, "layout": layout, "N": N, "K": Kd, "ksplit": best["ksplit"], "blocks": best["blocks"],
            "us": round(best["us"], 3), "gbps": round(nbytes / best["us"] / 1e3, 1), "heuristic_us": round(base, 3)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="tinyllama", choices=["tinyllama", "70b", "all"])
    ap.add_argument("--out", default=str(OUT))
    a = ap.parse_args()
    K = ext.load()
    shapes = {"tinyllama": TINYLLAMA, "70b": LLAMA70B, "all": TINYLLAMA + LLAMA70B}[a.shapes]
    rows = []
    for spec in shapes:
        rows.append(tune_shape(K, *spec))
        print(rows[-1], flush=True)
    out = Path(a.out)
    old = json.load(open(out)).get("gemv", []) if out.is_file() else []
    keep = [r for r in old if (r["layout"], r["N"], r["K"]) not in {(n["layout"], n["N"], n["K"]) for n in rows}]
    out.parent.mkdir(exist_ok=True)
    # only entries that beat the heuristic by more than the noise go into the table
    table = keep + [r for r in rows if r["us"] < 0.97 * r["heuristic_us"]]
    out.write_text(json.dumps({"gpu": torch.cuda.get_device_name(0), "gemv": table, "measured": rows}, indent=1) + "\n")
    print(f"wrote {out}: {len(table)} entries")


if __name__ == "__main__":
    main()
