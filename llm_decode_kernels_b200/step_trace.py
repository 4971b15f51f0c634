"""Where the time of the persistent step kernel goes, phase by phase (per-CTA `globaltimer` stamps).

    python -m llm_decode_kernels_b200.step_trace [--layers 22] [--ctx 256] [--reps 5] [--out FILE.json]

Builds libb200decode_trace.so - the same sources compiled with -DB200_STEP_TRACE, in which thread 0 of every CTA
stores the nanosecond timer at fixed points of every phase - loads it instead of the normal library, decodes `ctx`
tokens of a TinyLlama-shape model to fill the cache, then traces `reps` steps. Prints, for each of the four matrices
of a layer, the time spent up to each stamp since the one before, averaged over layers and steps, as the median over
the CTAs and the slowest CTA:
    stage         x of the phase is staged (this includes waiting for the CTAs that produce it)
    wait_weights  time warp 0 spent waiting for the matrix's ring stages to land in shared memory (all stages)
    mma           this warp's tile-units are multiplied (the interval up to the stamp, without those waits)
    barrier       all warps of the CTA have left their partial sums
    emit          the partial sums are added and the outputs stored
and the attention phase on the CTAs that own a head (the others go straight on and wait in the next staging).
The normal build carries none of this; numbers printed here are for finding the slow phase, not benchmark values.
"""
import argparse
import json
from pathlib import Path

import numpy as np
import torch

from . import build as B
from . import ext

HEAD, PER_PHASE, N_ATT, MATS = 8, 5, 5, ("qkv", "o", "gate_up", "down")
PER_LAYER = 4 * PER_PHASE + N_ATT
ATT_STAMPS = ("q k v polled and rotated", "cached tokens folded", "merged and stored", "left",
              "of which waiting for K/V stages")
STAMPS = ("stage", "wait_weights", "mma", "barrier", "emit")     # what ends at each of a phase's five stamps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=22)
    ap.add_argument("--ctx", type=int, default=256)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--out", default=None)
    ap.add_argument("--define", action="append", default=[],
                    help="further macros of the build under trace, e.g. B200_STEP_MAX_SLICES=1 (one CTA per query head)")
    a = ap.parse_args()
    tag = "".join("_" + d.split("=")[-1] for d in a.define)
    lib = B.build(defines=("B200_STEP_TRACE", *a.define), lib=B.PKG / f"libb200decode_trace{tag}.so")
    ext.load_library(path=lib)
    from .model import DecodeConfig, Model
    from .shapes import TINYLLAMA, config, random_llama_state
    c = config(TINYLLAMA, num_hidden_layers=a.layers)
    m = Model(random_llama_state(c, "cuda", 0), c, DecodeConfig(max_ctx=a.ctx + 64, seed=0, step_kernel="persistent"))
    m.prepare(a.ctx + 64, use_graph=False)
    grid, L = m._step_static["grid"], a.layers
    width = HEAD + PER_LAYER * (L + 1)
    trace = torch.zeros(grid, width, dtype=torch.int64, device="cuda")
    m._step_desc.trace = trace.data_ptr()
    m.reset(0)
    g = torch.Generator().manual_seed(0)
    m.teacher_force(torch.randint(0, c.vocab_size, (a.ctx,), generator=g), use_graph=False)
    torch.cuda.synchronize()
    n_att = m.n_q                                   # CTAs 0 .. n_q-1 run attention
    acc, totals = [], []
    for _ in range(a.reps):
        trace.zero_()
        m.run_step(False)
        torch.cuda.synchronize()
        t = trace.cpu().numpy().astype(np.float64)
        lay = t[:, HEAD:HEAD + PER_LAYER * L].reshape(grid, L, PER_LAYER)
        G = 4 * PER_PHASE                            # first attention slot; the last one is "attention left"
        d = np.zeros((grid, L, PER_LAYER))
        # a layer's first stamp follows the kernel start or the last emit of the layer before
        prev = np.concatenate([t[:, :1], lay[:, :-1, G - 1]], axis=1)
        waits = {}
        for i in range(G):
            if i % PER_PHASE == 1:                  # a duration, not a time: what warp 0 waited for ring stages
                waits[i] = lay[:, :, i]
                continue
            if i == PER_PHASE:                      # o.stage follows attention where there is one, else the qkv emit
                left = lay[:, :, PER_LAYER - 2]
                prev = np.where(left > 0, left, prev)
            cur = np.where(lay[:, :, i] > 0, lay[:, :, i], prev)   # a CTA without tiles of a matrix never waits for it
            d[:, :, i] = cur - prev
            prev = cur
        for i, w in waits.items():                  # the wait is part of the interval that ends at the "mma" stamp
            d[:, :, i] = w
            d[:, :, i + 1] -= w
        prev = lay[:, :, PER_PHASE - 1]             # attention follows the qkv emit
        for i in range(G, PER_LAYER - 1):
            d[:, :, i] = np.where(lay[:, :, i] > 0, lay[:, :, i] - prev, 0.0)
            prev = lay[:, :, i]
        d[:, :, PER_LAYER - 1] = lay[:, :, PER_LAYER - 1]   # a duration
        acc.append(d)
        totals.append((t[0, 2] - t[:, 0].min()) / 1e3)
    assert m.step_error() == 0, m.step_error()
    d = np.mean(np.stack(acc), axis=0).mean(axis=1) / 1e3       # [grid, PER_LAYER] us, mean over steps and layers
    res = {"layers": L, "context": a.ctx, "us_per_step": round(float(np.mean(totals)), 2), "phases_us": {}}
    for k, name in enumerate(MATS):
        for j, what in enumerate(STAMPS):
            col = d[:, PER_PHASE * k + j]
            res["phases_us"][f"{name}.{what}"] = {"median_cta": round(float(np.median(col)), 3),
                                                  "slowest_cta": round(float(col.max()), 3)}
    for j, what in enumerate(ATT_STAMPS):
        col = d[:n_att, 4 * PER_PHASE + j]
        res["phases_us"][f"attention.{what}"] = {"median_cta": round(float(np.median(col)), 3),
                                                 "slowest_cta": round(float(col.max()), 3)}
    res["layer_us_median_cta"] = round(float(np.median(d[:, :4 * PER_PHASE].sum(axis=1))), 3)
    txt = json.dumps(res, indent=1)
    print(txt)
    if a.out:
        Path(a.out).write_text(txt)


if __name__ == "__main__":
    main()
