"""Headline benchmark: batch-1 W4A16 greedy decode, tokens per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--step-kernel auto|persistent|multi]

Workload: TinyLlama-1.1B-shape decoder (22 layers, hidden 2048, intermediate 5632, 32 query /
4 KV heads, head_dim 64, vocab 32000), random init N(0, 0.02), every linear and the LM head W4A16 RTN g128; a
128-token prompt of uniform random ids is teacher-forced through the decode step, then 256 tokens are decoded
greedily with the whole step replayed as one CUDA graph. Synthetic weights and ids stand in for the TinyLlama
checkpoint and its tokenizer, which are not available offline.

One benchmark "step" = one pass of that workload. What is timed:
  value : the 256 free-running graph replays of each pass, CUDA events on the launching stream, KV cache of the
          prompt already resident (the prompt is processed before the events, untimed); tokens = 256 per pass.
  e2e   : Model.generate(prompt, 256) as a user calls it - prompt ids start in pinned host memory and are copied
          to the device, every one of the 128 + 256 decode steps is a graph replay, and each generated token is
          read back to the host as it is produced. Every decode step counts as a token: 384 per pass.
With --gpus N > 1 every rank decodes its own sequence on its own copy of the model (no collective on the data
path: weak scaling); the time is the max over ranks and `value` the sum of all ranks' tokens over it.

Before anything is timed, the step kernel that will be timed decodes 40 tokens of a 2-layer model of the same widths
and its logits are compared with the CPU oracle on identical weights; if they differ beyond the tolerance no line is
printed ("parity_checked" in the line says what was compared).

The line also carries, beside the headline:
  kernels : the single-kernel configurations - the 5632 x 2048 W4A16 GEMV and paged attention at batch 1, contexts
            128 .. 8192, and batch 8 - timed on cold data (llm_decode_kernels_b200/kernel_bench.py: headline_kernels)
  tp      : the Llama-3-70B-shape model, context 4096, 128 tokens, tensor-parallel over the N ranks of this run
            (N = 1: one GPU holds the whole model): tok/s, ms per token, bytes and HBM fraction per GPU; strong
            scaling, collectives on the data path (llm_decode_kernels_b200/e2e_bench.py: tp_record)
The context sweep and the fusion ablations have their own driver: llm_decode_kernels_b200/e2e_bench.py ctx.

`--impl reference` times the CPU restatement of the reference's own CPU path (its Model with backend="ref") on
this host's cores, on a bounded sample of the same workload.
"""
import argparse
import json
import os
import sys
import threading
import time
import types
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from llm_decode_kernels_b200.shapes import TINYLLAMA, random_llama_state  # noqa: E402

PROMPT_LEN, NEW_TOKENS, GROUP = 128, 256, 128


# ---------------------------------------------------------------------------------------------- clocks
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML every 100 ms while the timed region runs."""
    REASONS = {0x2: "sw_power_cap", 0x4: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.stop_flag, self.mhz, self.reasons, self.max_mhz, self.err = index, False, [], set(), None, None

    def run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            while not self.stop_flag:
                self.mhz.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                r = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                self.reasons |= {n for b, n in self.REASONS.items() if r & b}
                time.sleep(0.1)
        except Exception as e:  # NVML missing: report it, do not fail the benchmark
            self.err = repr(e)

    def summary(self):
        if not self.mhz:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "error": self.err}
        s = sorted(self.mhz)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def physical_gpu_index(local):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except (ValueError, IndexError):
            return local
    return local


# ---------------------------------------------------------------------------------------------- CPU leg
def cpu_reference_leg(budget_s, threads, layers_sample=None, log=lambda *a: None):
    """Times the oracle's CPU decode step (the reference's backend='ref' path restated) on a TinyLlama-shape model.

    layers_sample: build only that many of the 22 layers and extrapolate the per-token time linearly in the number
    of layers (every layer has the same shapes); None builds all 22. Returns a dict with tokens/s and what was run."""
    from oracle import model_oracle as MO
    torch.set_num_threads(threads)
    c = types.SimpleNamespace(**TINYLLAMA)
    L = c.num_hidden_layers
    built = L if layers_sample is None else layers_sample
    t0 = time.time()
    sd = random_llama_state(c, "cpu", 0, layers=built)
    cs = types.SimpleNamespace(**{**TINYLLAMA, "num_hidden_layers": built})
    ocfg = types.SimpleNamespace(group=GROUP, quant="rtn", qparams=None, max_ctx=PROMPT_LEN + NEW_TOKENS, page=16,
                                 shuffle_pages=True)
    m = MO.OracleModel(sd, cs, ocfg)
    del sd
    log(f"cpu oracle model ({built} layers) built in {time.time() - t0:.1f}s")
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, c.vocab_size, (PROMPT_LEN,), generator=g).tolist()
    m.reset(0)
    m.tok = prompt[0]
    m.step()                                   # warm-up token (allocations, thread pool)
    t1 = time.time()
    n = 0
    while n < 4 or (time.time() - t1 < budget_s and n < PROMPT_LEN + NEW_TOKENS - 2):
        m.tok = prompt[(n + 1) % PROMPT_LEN]
        m.step()
        n += 1
    dt = (time.time() - t1) / n
    per_token = dt
    how = f"{n} decode steps at ctx 2..{n + 1}, all {L} layers"
    if built != L:
        # time the LM head alone to separate it from the per-layer cost before scaling
        from oracle import ops_oracle as R
        x = torch.randn(c.hidden_size).half()
        th = time.time()
        for _ in range(3):
            R.gemv_ref(m.lm_head.w_ref, x)
        t_head = (time.time() - th) / 3
        per_token = (dt - t_head) * (L / built) + t_head
        how = (f"{n} decode steps at ctx 2..{n + 1} on {built} of {L} layers + LM head, per-layer time scaled "
               f"x{L / built:.0f}")
    return {"value": 1.0 / per_token, "unit": "tok/s", "cores": threads, "kind": "port", "sample": how,
            "s_per_token": per_token, "ops_us": cpu_op_times()}


def cpu_op_times():
    """The single-operator configurations on the host's cores, with the oracle's functions (the reference's ref_ops
    restated): the 5632 x 2048 GEMV from its dequantized fp16 matrix, and paged attention for one sequence (32 query /
    4 kv heads x 64, pages of 16) at contexts 2048 and 8192. Microseconds, best of 3 after a warm-up call."""
    from oracle import ops_oracle as R
    g = torch.Generator().manual_seed(2)

    def best(fn):
        fn()
        ts = []
        for _ in range(3):
            t0 = time.time()
            fn()
            ts.append(time.time() - t0)
        return round(min(ts) * 1e6, 1)
    w = (torch.randn(5632, 2048, generator=g) * 0.02).half()
    x = torch.randn(2048, generator=g).half()
    out = {"gemv_config1_5632x2048": best(lambda: R.gemv_ref(w, x))}
    q = torch.randn(32, 64, generator=g).half()
    for ctx in (2048, 8192):
        pages = ctx // 16 + 2
        kc = torch.randn(pages, 4, 16, 64, generator=g).half()
        vc = torch.randn(pages, 4, 16, 64, generator=g).half()
        bt = torch.randperm(pages, generator=g).int()
        out[f"attention_b1_ctx{ctx}"] = best(lambda: R.paged_attention_ref(q, kc, vc, bt, ctx, 16))
    return out


def run_reference_arm(args, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    budget = 150.0 / max(1, args.steps + args.warmup) * args.steps   # whole run within a few minutes
    r = cpu_reference_leg(min(budget, 90.0), threads, layers_sample=None if args.cpu_full else 2)
    line = {"impl": "reference", "metric": "batch-1 decode tok/s (W4A16)", "value": round(r["value"], 4),
            "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(r["s_per_token"] * 1e3 * (PROMPT_LEN + NEW_TOKENS), 2), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 storage, f32 accumulate", "data": "synthetic",
            "config": workload_config(),
            "cpu_baseline": {"value": round(r["value"], 4), "unit": "tok/s", "cores": threads, "kind": "port",
                             "sample": r["sample"], "ops_us": r["ops_us"]},
            "e2e": {"value": round(r["value"], 4), "unit": "tok/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config():
    return {"workload": "tinyllama-1.1b-shape W4A16 g128 RTN, batch 1, 128-token prompt + 256 greedy tokens, "
                        "one CUDA graph per step", "layers": 22, "hidden": 2048, "intermediate": 5632,
            "heads": "32q/4kv x64", "vocab": 32000, "page": 16,
            "l2": "weights streamed per token (553 MB) exceed the 126 MB L2; no flush needed"}


# ---------------------------------------------------------------------------------------------- GPU arm
def peak_hbm_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# Measured with ncu on the same kernel, TinyLlama shape cut to 6 layers (profiles/decode_step_kernel_tinyllama_6layers.md):
# dram__bytes_read.sum + dram__bytes_write.sum of one launch (175,887,616 + 4,746,752) over the algorithmic bytes of
# that launch (6 layers + LM head + embedding row + KV at context 40: 175,499,264). Traffic grows with the layers in
# proportion to the bytes, so the 22-layer figure is this ratio times the step's bytes.
STEP_TRAFFIC_OVER_ALGORITHMIC = 180634368 / 175499264


def prompt_record(m, n):
    """A prompt of n tokens through Model.prefill (W4A16 GEMM on the tcgen05 tensor cores, every matrix read once per
    256 tokens) against stepping through it one graph replay per token, which is what the reference does: device time
    around the whole prompt, median of 3, and whether both leave the same next token."""
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, m.V_full, (n,), generator=g).to(m.tok.device)
    m.prepare(n + 8)

    def timed(fn):
        ts = []
        for _ in range(3):
            m.reset(0)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[1], int(m.tok)
    m.reset(0)
    m.prefill(prompt)            # warm-up: scratch buffers, launch attributes
    ms_p, tok_p = timed(lambda: m.prefill(prompt))
    ms_s, tok_s = timed(lambda: m.teacher_force(prompt))
    return {"tokens": n, "prefill_ms": round(ms_p, 3), "prefill_tok_s": round(n / ms_p * 1e3, 1),
            "stepping_ms": round(ms_s, 3), "stepping_tok_s": round(n / ms_s * 1e3, 1),
            "same_next_token": tok_p == tok_s, "gemm_status": m.K.gemm_status()}


def parity_gate(dev, step_kernel, n_tokens=40):
    """The accuracy gate in front of the speed numbers: a 2-layer model of the benchmark's widths (hidden 2048,
    intermediate 5632, 32/4 heads x 64, vocabulary 32000) through the step kernel that is about to be timed, against
    the CPU oracle on the same packed weights and block table. Raises if the logits differ by more than 1.5 % of the
    largest logit or a greedy token differs outside the oracle's own near-tie margin."""
    from llm_decode_kernels_b200.model import DecodeConfig, Model
    from oracle import model_oracle as MO
    c = types.SimpleNamespace(**{**TINYLLAMA, "num_hidden_layers": 2})
    sd = random_llama_state(c, "cpu", 3)
    m = Model(sd, c, DecodeConfig(group=GROUP, max_ctx=64, page=16, device=dev, seed=5, step_kernel=step_kernel))
    packed = {f"layers.{i}.{k}": (lw[k].packed.cpu(), lw[k].sz.cpu()) for i, lw in enumerate(m.layers)
              for k in ("qkv", "o", "gu", "down")}
    packed["lm_head"] = (m.lm_head.packed.cpu(), m.lm_head.sz.cpu())
    ocfg = types.SimpleNamespace(group=GROUP, quant="rtn", qparams=None, max_ctx=64, page=16, shuffle_pages=True)
    o = MO.OracleModel(sd, c, ocfg, packed=packed, block_table=m.bt.cpu())
    g = torch.Generator().manual_seed(11)
    stream = torch.randint(0, c.vocab_size, (n_tokens,), generator=g).tolist()
    ref = o.teacher_force(stream, collect_logits=True).float()
    m.prepare(64, use_graph=True)
    m.reset(0)
    got = m.teacher_force(stream, collect_logits=True).float().cpu()
    assert m.step_error() == 0, "a bounded wait inside the step gave up during the parity check"
    scale = ref.abs().max().item()
    err = (got - ref).abs().max().item() / scale
    flips = 0
    for t in range(n_tokens):
        a, b = int(got[t].argmax()), int(ref[t].argmax())
        if a != b:
            flips += 1
            if ref[t, b] - ref[t, a] > 2e-2 * scale:
                raise SystemExit(f"parity check failed: token {t} differs from the oracle outside the noise floor")
    if not err <= 1.5e-2:
        raise SystemExit(f"parity check failed: logits differ from the oracle by {err:.3e} of the largest logit")
    return {"against": "CPU oracle, identical packed weights and block table", "layers": 2, "widths": "benchmark's own",
            "tokens": n_tokens, "step_kernel": "persistent" if m.persistent else "multi",
            "max_logit_err_rel": float(f"{err:.3e}"), "tolerance": 1.5e-2, "near_tie_flips": flips}


def run_b200_arm(args, rank, world, local_rank):
    from llm_decode_kernels_b200 import ext
    from llm_decode_kernels_b200.model import DecodeConfig, Model
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(dev))
    parity = parity_gate(dev, args.step_kernel) if rank == 0 else None
    c = types.SimpleNamespace(**TINYLLAMA)
    sd = random_llama_state(c, dev, 0)
    cfg = DecodeConfig(group=GROUP, max_ctx=PROMPT_LEN + NEW_TOKENS, page=16, device=dev, seed=0,
                       step_kernel=args.step_kernel)
    m = Model(sd, c, cfg)
    del sd
    torch.cuda.empty_cache()
    K = ext.load()
    m.prepare(PROMPT_LEN + NEW_TOKENS, use_graph=True)
    g = torch.Generator().manual_seed(1 + rank)
    prompt = torch.randint(0, c.vocab_size, (PROMPT_LEN,), generator=g).pin_memory()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def one_pass(timed):
        """Prompt (untimed), then 256 graph replays between two events. Returns the milliseconds."""
        m.reset(0)
        m.teacher_force(prompt)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(NEW_TOKENS):
            m.run_step()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1)

    for _ in range(args.warmup):
        one_pass(False)
    sampler = ClockSampler(physical_gpu_index(local_rank))
    barrier()
    sampler.start()
    t_wall = time.time()
    ms = [one_pass(True) for _ in range(args.steps)]
    barrier()
    t_wall = time.time() - t_wall
    dev_ms = sum(ms)
    if dist is not None:
        t = torch.tensor([dev_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms = float(t)
    value = world * args.steps * NEW_TOKENS / (dev_ms * 1e-3)

    # ---- end to end through Model.generate(): pinned-host prompt in, every token read back
    barrier()
    e2e_t = []
    for i in range(args.warmup + args.steps):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        toks = m.generate(prompt, NEW_TOKENS)
        torch.cuda.synchronize()
        if i >= args.warmup:
            e2e_t.append(time.perf_counter() - t0)
    e2e_s = sum(e2e_t)
    if dist is not None:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t)
    sampler.stop_flag = True
    sampler.join(timeout=2)
    e2e_value = world * args.steps * (PROMPT_LEN + NEW_TOKENS) / e2e_s

    # ---- roofline of the dominant kernel: the W4A16 GEMV, timed live over its real per-token launch mix
    lins = [lw[k] for lw in m.layers for k in ("qkv", "o", "gu", "down")] + [m.lm_head]
    bufs = {(l.N, l.K): (torch.randn(l.K, device=dev).half(), torch.empty(l.N, dtype=torch.half, device=dev))
            for l in lins}
    gemv_bytes = sum(l.nbytes + 2 * l.K + 2 * l.N for l in lins)

    def gemv_mix():   # every GEMV of one token, the way Model.linear() issues it in the multi-kernel step
        for l in lins:
            x, y = bufs[(l.N, l.K)]
            if l.tiled is None:
                K.gemv_w4a16(2, 0, 0, 0, l.packed, l.sz, x, y, GROUP)
            elif l.paired:
                K.gemv_w4a16_tiled(l.tiled, x, y[: l.N // 2], l.N // 2, l.K, swiglu=True)
            else:
                K.gemv_w4a16_tiled(l.tiled, x, y, l.N, l.K)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        gemv_mix()
    torch.cuda.current_stream().wait_stream(s)
    gg = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gg):
        gemv_mix()
    for _ in range(3):
        gg.replay()
    reps = 50
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        gg.replay()
    e1.record()
    e1.synchronize()
    gemv_ms = e0.elapsed_time(e1) / reps
    peak, peak_kind = peak_hbm_gbs()
    achieved = gemv_bytes / (gemv_ms * 1e-3) / 1e9
    if m.persistent:
        launches_per_token = 1                       # decode_step_kernel
    else:
        # embed; per layer: (2 norms unless fused into the GEMVs) + 4 GEMVs + rope/append + attention (+ combine)
        # (+ SwiGLU unless it is the gate|up GEMV's epilogue); final norm (unless fused), LM head, argmax
        norms = 0 if m.norm_in_gemv else 1
        swiglu = 0 if m.layers[0]["gu"].paired else 1
        launches_per_token = (1 + m.L * (2 * norms + 4 + 1 + 1 + (1 if m.max_splits > 1 else 0) + swiglu)
                              + norms + 2)
    assert m.step_error() == 0, "a bounded wait inside the step kernel gave up: the numbers would be meaningless"

    ctx_mid = PROMPT_LEN + NEW_TOKENS // 2
    step_bytes = m.bytes_per_token(ctx_mid)
    us_per_token = dev_ms * 1e3 / (args.steps * NEW_TOKENS)
    gemv_roofline = {"kernel": "gemv_w4a16_mma_kernel", "achieved": round(achieved, 1), "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "launches": len(lins), "bytes_per_launch_mix": gemv_bytes,
                     "how": "the 89 GEMVs of one token (tile-layout copies, gate|up with its SwiGLU epilogue) replayed as one "
                            "graph, CUDA events, 50 replays"}
    if m.persistent:
        # the dominant kernel IS the step: algorithmic bytes of one token / the kernel's average duration in the timed
        # region (one launch per graph replay, so the event-timed replay is the launch)
        step_achieved = step_bytes / (us_per_token * 1e-6) / 1e9
        roofline = {"bound": "hbm", "kernel": "decode_step_kernel", "achieved": round(step_achieved, 1), "peak": peak,
                    "peak_source": f"{peak_kind} copy bandwidth", "unit": "GB/s", "frac": round(step_achieved / peak, 4),
                    "traffic": (round(STEP_TRAFFIC_OVER_ALGORITHMIC * step_bytes)
                                if STEP_TRAFFIC_OVER_ALGORITHMIC else None),
                    "bytes_per_launch": step_bytes,
                    "how": "weights + KV bytes of one token at context 256 / CUDA-event time per graph replay; traffic "
                           "= ncu dram bytes of a 6-layer launch scaled by the bytes"}
    else:
        roofline = dict(gemv_roofline, bound="hbm", peak=peak, peak_source=f"{peak_kind} copy bandwidth", traffic=None)
    if m.persistent and parity is not None:
        assert parity["step_kernel"] == "persistent"
    # ---- the single-kernel configurations and the tensor-parallel 70B shape, recorded beside the headline
    kernels = None
    if rank == 0 and not args.no_kernels:
        from llm_decode_kernels_b200.kernel_bench import headline_kernels
        kernels = headline_kernels(K, peak)
        kernels["prompt_256"] = prompt_record(m, 256)
    persistent = m.persistent
    del m, gg, bufs, lins
    torch.cuda.empty_cache()
    tp = None
    if not args.no_tp:
        from llm_decode_kernels_b200.e2e_bench import tp_record
        barrier()
        tp = tp_record(rank, world, local_rank, dist)
    if rank == 0:
        line = {"metric": "batch-1 decode tok/s (W4A16)", "value": round(value, 2), "unit": "tok/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_ms / args.steps, 4),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f16 storage, f32 accumulate (int4 weights)", "data": "synthetic",
                "config": workload_config(),
                "us_per_token": round(us_per_token, 3), "step_kernel": "persistent" if persistent else "multi",
                "step_roofline": {"bytes_per_token": step_bytes,
                                  "floor_us_at_peak": round(step_bytes / (peak * 1e9) * 1e6, 2),
                                  "frac_of_peak": round(step_bytes / (dev_ms * 1e-3 / (args.steps * NEW_TOKENS))
                                                        / 1e9 / peak, 4),
                                  "frac_of_8TBs": round(step_bytes / (dev_ms * 1e-3 / (args.steps * NEW_TOKENS))
                                                        / 8e12, 4)},
                "roofline": roofline, "gemv_roofline": gemv_roofline,
                "e2e": {"value": round(e2e_value, 2), "unit": "tok/s", "h2d_bytes_per_step": PROMPT_LEN * 8,
                        "d2h_bytes_per_step": NEW_TOKENS * 8, "tokens_per_step": PROMPT_LEN + NEW_TOKENS,
                        "ms_per_step": round(e2e_s / args.steps * 1e3, 3)},
                "gpu_launches": launches_per_token * NEW_TOKENS * args.steps,
                "clocks": sampler.summary(), "wall_s_timed_region": round(t_wall, 3),
                "sample_tokens": toks[:8], "parity_checked": parity, "kernels": kernels, "tp": tp}
        if world == 1 and not args.no_cpu:
            r = cpu_reference_leg(args.cpu_seconds, os.cpu_count() or 1, layers_sample=2)
            line["cpu_baseline"] = {k: (round(v, 4) if isinstance(v, float) else v) for k, v in r.items()
                                    if k != "s_per_token"}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="time budget of the cpu_baseline leg")
    ap.add_argument("--cpu-full", action="store_true", help="reference arm: build all 22 layers on the CPU")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-kernels", action="store_true", help="skip the single-kernel configurations")
    ap.add_argument("--no-tp", action="store_true", help="skip the tensor-parallel 70B-shape record")
    ap.add_argument("--step-kernel", default="auto", choices=["auto", "persistent", "multi"],
                    help="how Model runs a decode step (see DecodeConfig.step_kernel)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if world != args.gpus:
        if args.gpus > 1:
            sys.exit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    run_b200_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
