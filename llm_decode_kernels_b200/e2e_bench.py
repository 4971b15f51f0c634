"""End-to-end decode benchmarks beside the headline one (the reference's bench/e2e.py, for the two configurations
that bench.py does not time).

    python -m llm_decode_kernels_b200.e2e_bench ctx [--quant gptq|rtn] [--tokens 64] [--out FILE.json]
        TinyLlama shape, tokens/s at KV contexts 512 .. 8192 (cache pre-filled with N(0,1), as the reference does), and
        at context 2048 with each fusion switched off in turn (DecodeConfig.ablate). --quant gptq calibrates on 128
        synthetic sequences of 512 uniform random ids with clipping (the stand-in for the WikiText-2 calibration set).

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m llm_decode_kernels_b200.e2e_bench tp
             [--layers 80] [--ctx 4096] [--tokens 128] [--tp-comm p2p|nccl]
        Llama-3-70B shape, random N(0, 0.02) weights, W4A16 g128, batch-1 greedy decode of `tokens` tokens from a
        pre-filled context, tensor-parallel over the N ranks (N = 1 without torchrun). Prints one JSON line on rank 0:
        tokens/s, microseconds per token, bytes each GPU streams per token and the fraction of the measured HBM
        bandwidth that is.

Timing: CUDA events around the decode steps on the launching stream, after 8 warm-up steps, max over ranks.
"""
import argparse
import json
import os
import time
from pathlib import Path

import torch

from .model import DecodeConfig, Model
from .shapes import LLAMA3_70B, TINYLLAMA, LazyRandomState, config, random_llama_state

ROOT = Path(__file__).resolve().parents[1]


def peak_hbm_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def time_decode(m, ctx, tokens, warm=8, dist=None):
    """Decode `tokens` tokens starting at context `ctx` (cache contents as they are); returns microseconds per token."""
    m.reset(ctx - warm)
    for _ in range(warm):
        m.run_step()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(tokens):
        m.run_step()
    e1.record()
    e1.synchronize()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device=m.tok.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
    return ms * 1e3 / tokens


def run_ctx(a):
    c = config(TINYLLAMA)
    qparams, quant = None, "rtn"
    if a.quant == "gptq":
        # calibration works on a HF module (as the reference's driver does): a random-init LlamaForCausalLM of the shape
        from transformers import LlamaConfig, LlamaForCausalLM
        from . import gptq
        torch.manual_seed(0)
        hf = LlamaForCausalLM(LlamaConfig(**TINYLLAMA, max_position_embeddings=2048, initializer_range=0.02))
        hf = hf.half().cuda().eval()
        tok = type("Tok", (), {"bos_token_id": 1, "vocab_size": c.vocab_size})()
        t0 = time.time()
        qparams = gptq.calibrate(hf, tok, 128, clip=True, n=128, L=512, lm_head=True, log=lambda *x: None)
        quant = "pre"
        sd = {k: v.detach() for k, v in hf.state_dict().items()}
        print(f"calibrated in {time.time() - t0:.1f} s", flush=True)
    else:
        sd = random_llama_state(c, "cuda", 0)
    peak, kind = peak_hbm_gbs()
    res = {"gpu": torch.cuda.get_device_name(0), "quant": a.quant, "tokens_timed": a.tokens, "contexts": {},
           "ablations_at_2048": {}}
    max_ctx = 8192 + a.tokens + 16

    def build(**kw):
        return Model(sd, c, DecodeConfig(group=128, quant=quant, qparams=qparams, max_ctx=max_ctx, seed=0,
                                         fuse_rope_attention=a.fuse_rope, **kw))

    m = build(**({"step_kernel": a.step_kernel} if a.step_kernel != "auto" else {}))
    m.kv.normal_()
    for ctx in a.contexts or (512, 1024, 2048, 4096, 8192):
        m.prepare(ctx + a.tokens + 8)
        us = time_decode(m, ctx, a.tokens)
        nbytes = m.bytes_per_token(ctx + a.tokens // 2)
        res["contexts"][ctx] = {"us_per_token": round(us, 1), "tok_s": round(1e6 / us, 1), "bytes_per_token": nbytes,
                                "frac_of_hbm": round(nbytes / us / 1e3 / peak, 4),
                                "step_kernel": "persistent" if m.persistent else "multi", "part_size": m.part_size}
        print(ctx, res["contexts"][ctx], flush=True)
    del m
    for name, kw in () if a.no_ablations else (("all fused, one launch per operator", dict(step_kernel="multi")),
                     ("dequant-in-GEMV off", dict(ablate=("dequant",))),
                     ("residual+RMSNorm off", dict(ablate=("norm",))),
                     ("SwiGLU off", dict(ablate=("swiglu",))),
                     ("RoPE+KV-append off", dict(ablate=("rope",)))):
        m = build(**kw)
        m.kv.normal_()
        m.prepare(2048 + a.tokens + 8)
        us = time_decode(m, 2048, a.tokens)
        res["ablations_at_2048"][name] = {"us_per_token": round(us, 1), "tok_s": round(1e6 / us, 1)}
        print(name, res["ablations_at_2048"][name], flush=True)
        del m
        torch.cuda.empty_cache()
    res["peak_hbm_gbs"], res["peak_source"] = peak, kind
    txt = json.dumps(res, indent=1)
    print(txt)
    if a.out:
        Path(a.out).write_text(txt)


def tp_record(rank, world, local, dist, layers=80, ctx=4096, tokens=128, tp_comm="p2p", gemv="tiled",
              allreduce="auto"):
    """Build this rank's shard of the 70B-shape model, decode `tokens` tokens from a pre-filled context `ctx` and
    return the record (a dict; identical on every rank up to the rank-local fields). `dist` is the initialised
    torch.distributed module, or None for one GPU."""
    dev = f"cuda:{local}"
    c = config(LLAMA3_70B, num_hidden_layers=layers)
    t0 = time.time()
    cfg = DecodeConfig(group=128, max_ctx=ctx + tokens + 16, page=16, device=dev, seed=0, tp_rank=rank,
                       tp_world=world, tp_comm=tp_comm, step_kernel="multi", tile_weights=gemv == "tiled",
                       keep_packed=False, gemv_stage=(2, 16, 0, 0) if gemv == "segmented" else None,
                       tp_allreduce=allreduce)
    m = Model(LazyRandomState(c, dev, 0), c, cfg)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    build_s = time.time() - t0
    m.kv.normal_()
    m.prepare(ctx + tokens + 8)
    if dist is not None:
        dist.barrier()
    us = time_decode(m, ctx, tokens, dist=dist)
    err = m.step_error()
    nbytes = m.bytes_per_token(ctx + tokens // 2)      # what THIS rank streams per token
    peak, kind = peak_hbm_gbs()
    rec = {"metric": "batch-1 decode tok/s (W4A16), tensor-parallel", "value": round(1e6 / us, 2), "unit": "tok/s",
           "n_gpus": world, "us_per_token": round(us, 1), "ms_per_token": round(us / 1e3, 3),
           "us_per_layer": round(us / layers, 2),
           "config": {"workload": f"llama-3-70b-shape W4A16 g128 RTN, {layers} layers, batch 1, context {ctx}, "
                                  f"{tokens} greedy tokens", "tp": world, "comm": tp_comm if world > 1 else None,
                      "gemv": gemv, "graph": m.graph is not None,
                      "allreduce": m.tp_allreduce if world > 1 and tp_comm == "p2p" else None},
           "bytes_per_token_per_gpu": nbytes, "floor_us_at_peak": round(nbytes / peak / 1e3, 1),
           "frac_of_hbm_per_gpu": round(nbytes / us / 1e3 / peak, 4), "peak_hbm_gbs": peak, "peak_source": kind,
           "exchanges_per_token": 2 * layers + 1 if world > 1 else 0, "build_s": round(build_s, 1),
           "step_error": err, "scaling": "strong", "data": "synthetic"}
    if m.comm is not None:
        dist.barrier()
        m.comm.close()
    del m
    torch.cuda.empty_cache()
    return rec


def run_tp(a):
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import datetime
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"),
                                timeout=datetime.timedelta(seconds=600))
    line = tp_record(rank, world, local, dist, a.layers, a.ctx, a.tokens, a.tp_comm, a.gemv, a.allreduce)
    if rank == 0:
        print(json.dumps(line), flush=True)
        if a.out:
            Path(a.out).write_text(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_prefill(a):
    """Prompt processing at the TinyLlama shape: Model.prefill (batched GEMM on the tensor cores, every matrix read
    once per 256 tokens) against stepping through the prompt (one graph replay per token, what the reference does).
    Device time by CUDA events around the whole prompt, median of 5; both leave the same next token (checked)."""
    c = config(TINYLLAMA)
    sd = random_llama_state(c, "cuda", 0)
    m = Model(sd, c, DecodeConfig(group=128, max_ctx=4096 + 16, seed=0))
    res = {"gpu": torch.cuda.get_device_name(0), "prompts": {}}
    g = torch.Generator().manual_seed(0)

    def timed(fn, reps=5):
        ts = []
        for _ in range(reps):
            m.reset(0)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2]

    for n in (128, 512, 2048, 4096):
        prompt = torch.randint(0, c.vocab_size, (n,), generator=g).cuda()
        m.prepare(n + 8)
        m.reset(0)
        m.prefill(prompt)
        tok_prefill = int(m.tok)
        m.reset(0)
        m.teacher_force(prompt)
        tok_steps = int(m.tok)
        ms_p = timed(lambda: m.prefill(prompt))
        ms_s = timed(lambda: m.teacher_force(prompt), reps=3)
        res["prompts"][n] = {"prefill_ms": round(ms_p, 3), "prefill_tok_s": round(n / ms_p * 1e3, 1),
                             "stepping_ms": round(ms_s, 3), "stepping_tok_s": round(n / ms_s * 1e3, 1),
                             "speedup": round(ms_s / ms_p, 2), "same_next_token": tok_prefill == tok_steps,
                             "step_kernel": "persistent" if m.persistent else "multi"}
        print(n, res["prompts"][n], flush=True)
    res["status"] = {"gemm": m.K.gemm_status(), "step": m.step_error()}
    txt = json.dumps(res, indent=1)
    print(txt)
    if a.out:
        Path(a.out).write_text(txt)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["ctx", "tp", "prefill"])
    ap.add_argument("--quant", default="rtn", choices=["rtn", "gptq"])
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--layers", type=int, default=80)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--tp-comm", default="p2p", choices=["p2p", "nccl"])
    ap.add_argument("--gemv", default="tiled", choices=["tiled", "rowmajor", "segmented"],
                    help="tp: tensor-core GEMV from the tile layout (default) / from the row-major tensors / the "
                         "segmented CUDA-core GEMV")
    ap.add_argument("--allreduce", default="auto", choices=["auto", "kernel", "gemv", "push"],
                    help="tp: how the row-split projections are summed over the ranks (DecodeConfig.tp_allreduce)")
    ap.add_argument("--fuse-rope", action="store_true", help="ctx: RoPE + KV-append inside the attention kernel")
    ap.add_argument("--step-kernel", default="auto", choices=["auto", "persistent", "multi"],
                    help="ctx: force the step kernel of the sweep (default: the model's own choice per context)")
    ap.add_argument("--contexts", type=int, nargs="*", default=None, help="ctx: the contexts of the sweep")
    ap.add_argument("--no-ablations", action="store_true", help="ctx: skip the ablation runs")
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    if a.tokens is None:
        a.tokens = 128 if a.what == "tp" else 64
    {"ctx": run_ctx, "tp": run_tp, "prefill": run_prefill}[a.what](a)


if __name__ == "__main__":
    main()
