"""Batch-1 decode runtime for Llama-family models on the B200 kernels.

Keeps the public surface of the reference's runtime/model.py: `DecodeConfig` (same fields and defaults,
runtime/model.py:32-50) and `Model(hf_state, hf_config, cfg)` with prepare / capture / run_step / reset /
teacher_force / generate / weight_bytes / kv_bytes_per_token (runtime/model.py:75-297). One decode step is

    embed -> per layer [ add+RMSNorm -> qkv GEMV -> RoPE + paged-KV append -> paged attention (+combine) -> o GEMV
                         -> add+RMSNorm -> gate|up GEMV -> SwiGLU -> down GEMV ]
          -> add+RMSNorm -> LM-head GEMV -> argmax (written to the device token slot) -> pos += 1

with the residual add of `down` deferred into the next layer's first norm, exactly as the reference orders it
(runtime/model.py:216-233). Token id and position live in device memory and every kernel reads them through
pointers, so the step is captured once as a CUDA graph and replayed for every token. Prefill is the same step,
teacher-forced.

This runtime has one backend: the CUDA kernels of libb200decode.so, all weights W4A16. `backend="ref"`,
`weights="fp16"` and CPU devices are refused; the CPU restatement used for checking lives outside the package.
"""
import json
import math
from dataclasses import dataclass, field
from pathlib import Path

import torch

from . import ext, tp as TP
from .quant import QuantLinear

ROOT = Path(__file__).resolve().parent


@dataclass
class DecodeConfig:
    weights: str = "int4"        # only "int4" (W4A16) exists in this runtime
    group: int = 128
    quant: str = "rtn"           # "rtn" | "clip" (RTN + per-group range clipping) | "pre" (use `qparams`, e.g. GPTQ)
                                 # | "packed" (`qparams` holds matrices already in kernel format, see checkpoint.py)
    qparams: dict = field(default=None, repr=False)  # "layers.{i}.{qkv,o,gu,down}" / "lm_head" -> (q, scale, zero);
                                 # with quant="packed": -> (packed int32 [N, K/8], sz fp16 [N, K/group, 2])
    lm_head: str = "auto"        # "auto" / "int4": INT4 head (the only kind here)
    fused: bool = True           # False: residual add, RMSNorm and SwiGLU run as separate torch ops (ablation)
    backend: str = "cuda"        # only "cuda"
    max_ctx: int = 2048
    page: int = 16
    part_size: int = 0           # attention split size; 0 -> policy table, else a size that fills the SMs
    attn_version: int = 0        # accepted for compatibility; the library has one attention kernel
    gemv_stage: tuple = None     # (stage, R, warps, pf) forced everywhere; None -> the library's shape-based choice
    fuse_rope_attention: bool = True   # RoPE + KV-append inside the attention kernel (b200_rope_paged_attention): one
                                       # launch less per layer
    fuse_norm_gemv: bool = True  # residual add + RMSNorm inside the GEMV that consumes them (b200_gemv_w4a16_tiled_norm):
                                 # two launches less per layer; needs tile_weights, one GPU, no ablation switch
    tile_weights: bool = True    # hold every matrix in the tile layout of the tensor-core GEMV and of the persistent
                                 # step (b200_gemv_w4a16_tile_repack) and multiply from it
    keep_packed: bool = True     # False: once a matrix has its tile-layout copy, drop the quantizer's row-major
                                 # packed / scale-zero tensors, which no kernel reads any more (halves the weight
                                 # memory; Linear.packed and Linear.sz are then None)
    autotune_path: str = str(ROOT / "configs" / "autotune.json")
    attn_policy_path: str = str(ROOT / "configs" / "attn_policy.json")
    shuffle_pages: bool = True
    device: str = "cuda"
    # ---- additions (defaults keep the reference behaviour) ----
    seed: int = None             # seed of the page-table shuffle (None: torch's global generator)
    tp_rank: int = 0             # tensor parallelism: this process's rank ...
    tp_world: int = 1            # ... of this many (one process per GPU, torch.distributed initialised by the caller)
    tp_group: object = field(default=None, repr=False)   # process group of the TP ranks (None: the default group)
    tp_comm: str = "p2p"         # collectives of a tensor-parallel step: "p2p" = the library's one-shot exchange over
                                 # NVLink peer memory, fused with the residual add + RMSNorm that follows (all GPUs in
                                 # one node; the step is captured in a CUDA graph); "nccl" = torch.distributed
                                 # all_reduce / all_gather, launched eagerly
    tp_allreduce: str = "auto"   # tp_comm="p2p": how the partial rows of o_proj / down_proj are summed over the ranks.
                                 # "kernel": the GEMV writes its rows locally; one exchange kernel does a flag round,
                                 # loads the peers' rows, sums, residual add + RMSNorm (b200_tp_allreduce_add_rmsnorm).
                                 # "push": the GEMV pushes tagged words into every rank's region and returns; the
                                 # consumer kernel polls its own memory, sums, add + RMSNorm
                                 # (b200_gemv_w4a16_tiled_push + b200_tp_pushed_add_rmsnorm) - no flag round, no
                                 # fence. "gemv": the same push, and the GEMV's blocks collect and sum their own
                                 # rows (b200_gemv_w4a16_tiled_allreduce), the norm inside the next GEMV - two
                                 # launches less per layer. "auto": what measured fastest for the number of ranks
    ablate: tuple = ()           # fusions switched off for ablation runs, any of "dequant" (dequantize the matrix to
                                 # an fp16 buffer, then an fp16 matrix-vector product), "norm", "swiglu" (the two
                                 # that fused=False switches off together) and "rope" (rotation and cache append as
                                 # separate device ops); any entry implies one launch per operator
    step_kernel: str = "auto"    # "persistent": the whole step is one kernel (b200_decode_step); "multi": one launch
                                 # per operator, as the reference does; "auto": persistent when fused and the
                                 # prepared context cap is within PERSISTENT_MAX_CTX


PERSISTENT_MAX_CTX = 10240   # beyond this the one-launch-per-operator step, whose attention uses every SM, is faster
                             # (measured us per token at 2048 / 8192: persistent 468 / 697, multi-kernel 652 / 755)


class Linear:
    """One W4A16 projection in kernel format (reference runtime/model.py:56-72)."""

    def __init__(self, w, cfg: DecodeConfig, key: str = None, keep_ref: bool = False, pre=None, packed=None):
        self.quant = True
        self.tiled = None            # tile-layout copy, made by Model when DecodeConfig.tile_weights is set
        self.paired = False          # the copy pairs gate row i with up row i (GEMV with SwiGLU epilogue)
        if packed is not None:       # already in kernel format: nothing to quantize
            pk, sz = packed
            if pk.dtype != torch.int32 or sz.dtype != torch.float16 or sz.dim() != 3 or sz.shape[2] != 2:
                raise ValueError(f"{key}: packed weights must be int32 [N, K/8] with fp16 (scale, zero) [N, K/group, 2]")
            self.N, self.K = pk.shape[0], pk.shape[1] * 8
            if sz.shape[0] != self.N or sz.shape[1] * cfg.group != self.K:
                raise ValueError(f"{key}: scale/zero shape {tuple(sz.shape)} does not match {self.N} x {self.K}, "
                                 f"group {cfg.group}")
            self.packed, self.sz = pk.to(cfg.device).contiguous(), sz.to(cfg.device).contiguous()
            self.w_ref = None
            self.nbytes = self.packed.numel() * 4 + self.sz.numel() * 2
            return
        self.N, self.K = w.shape
        if cfg.quant == "pre" and pre is None:
            pre = (cfg.qparams or {}).get(key)
            assert pre is not None, f"no precomputed weights for {key}"
        ql = QuantLinear(w.to(cfg.device), cfg.group, keep_ref=keep_ref, clip=cfg.quant == "clip", qsz=pre)
        self.packed, self.sz = ql.packed.to(cfg.device), ql.sz.to(cfg.device)
        self.w_ref = ql.w_ref
        self.nbytes = ql.nbytes()

    def drop_packed(self):
        """Free the row-major tensors once the tile-layout copy exists (DecodeConfig.keep_packed=False)."""
        if self.tiled is not None:
            self.packed = self.sz = None


def _rope_theta(c):
    if getattr(c, "rope_theta", None) is not None:
        return float(c.rope_theta)
    rp = getattr(c, "rope_parameters", None)          # newer transformers keep it here
    if isinstance(rp, dict) and "rope_theta" in rp:
        return float(rp["rope_theta"])
    return 10000.0


class Model:
    def __init__(self, hf_state: dict, hf_config, cfg: DecodeConfig):
        if cfg.backend != "cuda":
            raise ValueError("this runtime has only the CUDA backend; the CPU reference path is not part of it")
        if cfg.weights != "int4" or cfg.lm_head not in ("auto", "int4"):
            raise ValueError("this runtime is W4A16 only (weights='int4', INT4 LM head)")
        if not str(cfg.device).startswith("cuda") or not torch.cuda.is_available():
            raise RuntimeError("a CUDA device is required: there is no CPU fallback")
        self.cfg = cfg
        c = hf_config
        self.H, self.L = c.hidden_size, c.num_hidden_layers
        self.n_q, self.n_kv = c.num_attention_heads, c.num_key_value_heads
        self.D = getattr(c, "head_dim", None) or self.H // self.n_q
        self.I, self.V = c.intermediate_size, c.vocab_size
        self.eps = c.rms_norm_eps
        if self.D not in (64, 128):
            raise ValueError(f"head_dim {self.D}: kernels exist for 64 and 128")
        # tensor parallelism: from here on n_q, n_kv, I and V are THIS RANK's share; the *_full values are the model's
        self.tp, self.tp_rank = cfg.tp_world, cfg.tp_rank
        full = (self.n_q, self.n_kv, self.D, self.I, self.V)
        self.V_full = self.V
        if self.tp > 1:
            TP.check(self.n_q, self.n_kv, self.D, self.I, self.V, cfg.group, self.tp)
            self.n_q, self.n_kv, self.I, self.V = (v // self.tp for v in (self.n_q, self.n_kv, self.I, self.V))
        shard = lambda kind, w: TP.shard_weight(kind, w, full, self.tp_rank, self.tp)
        pre = lambda kind, key: (TP.shard_qsz(kind, (cfg.qparams or {}).get(key), full, cfg.group, self.tp_rank, self.tp)
                                 if cfg.quant == "pre" else None)
        dev = cfg.device
        self.K = ext.load()
        self.K.load_gemv_tunes(cfg.autotune_path)   # measured launch shapes of the GEMVs, if the table exists
        sd = hf_state
        g = lambda k: sd[k].to(dev).half()
        self.emb = g("model.embed_tokens.weight").contiguous()
        if not cfg.keep_packed and "dequant" in cfg.ablate:
            raise ValueError("the 'dequant' ablation reads the row-major tensors: keep_packed must stay True")
        tile = cfg.tile_weights and cfg.gemv_stage is None
        # gate|up is stored with gate row i next to up row i, so its GEMV can finish with SwiGLU (one launch less per
        # layer) - unless that fusion, or the fused dequantization, is switched off for an ablation run
        pair_gu = cfg.fused and not ({"swiglu", "dequant"} & set(cfg.ablate))

        def finish(lin, gate_up=False):
            """Tile-layout copy of a freshly quantized matrix (made layer by layer, so that with keep_packed=False
            the row-major tensors of only one layer are alive at a time)."""
            if tile:
                lin.tiled = self.K.gemv_tile_repack(lin.packed, lin.sz, cfg.group, gate_up=gate_up and pair_gu)
                lin.paired = gate_up and pair_gu and lin.tiled is not None
                if not cfg.keep_packed:
                    lin.drop_packed()
            return lin

        have_packed = cfg.quant == "packed"
        if have_packed and not cfg.qparams:
            raise ValueError("quant='packed' needs qparams = {name: (packed, sz)} (checkpoint.load_quantized)")

        def lin(kind, key, weights, gate_up=False):
            """One projection: from its kernel-format tensors when the configuration brings them (the fp16 weights
            are then never asked for), else quantized from weights()."""
            if have_packed:
                return finish(Linear(None, cfg, key, packed=TP.shard_packed(kind, cfg.qparams[key], full, cfg.group,
                                                                            self.tp_rank, self.tp)), gate_up)
            return finish(Linear(shard(kind, weights()), cfg, key, pre=pre(kind, key)), gate_up)

        self.layers = []
        for i in range(self.L):
            p = f"model.layers.{i}."
            self.layers.append({
                "ln1": g(p + "input_layernorm.weight").contiguous(),
                "ln2": g(p + "post_attention_layernorm.weight").contiguous(),
                "qkv": lin("qkv", f"layers.{i}.qkv", lambda: torch.cat([g(p + "self_attn.q_proj.weight"),
                                                                        g(p + "self_attn.k_proj.weight"),
                                                                        g(p + "self_attn.v_proj.weight")], 0)),
                "o": lin("o", f"layers.{i}.o", lambda: g(p + "self_attn.o_proj.weight")),
                "gu": lin("gu", f"layers.{i}.gu", lambda: torch.cat([g(p + "mlp.gate_proj.weight"),
                                                                     g(p + "mlp.up_proj.weight")], 0), True),
                "down": lin("down", f"layers.{i}.down", lambda: g(p + "mlp.down_proj.weight"))})
        self.norm_f = g("model.norm.weight").contiguous()
        head_key = "lm_head.weight" if "lm_head.weight" in sd else "model.embed_tokens.weight"
        self.lm_head = lin("lm_head", "lm_head", lambda: sd[head_key].to(dev).half())

        # paged KV cache [L, 2, pages, n_kv, P, D]; one block table shared by all layers (one sequence)
        self.n_pages = (cfg.max_ctx + cfg.page - 1) // cfg.page + 1
        self.kv = torch.zeros(self.L, 2, self.n_pages, self.n_kv, cfg.page, self.D, dtype=torch.half, device=dev)
        if cfg.shuffle_pages:
            gen = torch.Generator().manual_seed(cfg.seed) if cfg.seed is not None else None
            self.bt = torch.randperm(self.n_pages, generator=gen).int().to(dev)
        else:
            self.bt = torch.arange(self.n_pages).int().to(dev)
        self.rope_theta = _rope_theta(c)
        self.cos, self.sin = (t.to(dev) for t in rope_tables(cfg.max_ctx + 1, self.D, self.rope_theta))

        # device-resident decode state and static activation buffers
        h16 = dict(dtype=torch.half, device=dev)
        self.tok = torch.zeros(1, dtype=torch.long, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=dev)
        self.history = torch.zeros(cfg.max_ctx + 2, dtype=torch.long, device=dev)  # token chosen at each position
        self.x = torch.empty(self.H, **h16)
        self.x_alt = torch.empty(self.H, **h16)    # second residual buffer of the norm-fused GEMVs (they ping-pong)
        self.normed = torch.empty(self.H, **h16)
        self.qkv = torch.empty((self.n_q + 2 * self.n_kv) * self.D, **h16)
        self.attn = torch.empty(self.n_q, self.D, **h16)
        self.o = torch.empty(self.H, **h16)
        self.gu = torch.empty(2 * self.I, **h16)
        self.act = torch.empty(self.I, **h16)
        self.down = torch.empty(self.H, **h16)
        self.logits = torch.empty(self.V_full, **h16)   # full vocabulary on every rank
        self.logits_local = self.logits if self.tp == 1 else torch.empty(self.V, **h16)
        self.graph = None
        self.host_pos = 0
        bad = set(cfg.ablate) - {"dequant", "norm", "swiglu", "rope"}
        if bad:
            raise ValueError(f"unknown ablation switch {sorted(bad)}")
        self.off = set(cfg.ablate) | (set() if cfg.fused else {"norm", "swiglu"})
        if "dequant" in self.off:   # one fp16 buffer large enough for the biggest matrix
            mats = [lw[n] for lw in self.layers for n in ("qkv", "o", "gu", "down")] + [self.lm_head]
            self.w_fp16 = torch.empty(max(m.N * m.K for m in mats), **h16)
        if "rope" in self.off:
            self.kv_heads = torch.arange(self.n_kv, device=dev)
        self.comm = None
        # measured on the 70B shape (tok/s at 2 / 4 / 8 ranks): push 133 / 151 / 183, gemv 131 / - / 189, kernel 121 /
        # 134 / 141. Push and gemv need the tile-layout copies (their GEMV is the tiled one).
        self.tp_allreduce = cfg.tp_allreduce
        if self.tp_allreduce == "auto":
            tiled = cfg.tile_weights and cfg.gemv_stage is None
            self.tp_allreduce = ("gemv" if self.tp >= 8 and cfg.fuse_norm_gemv else "push") if tiled else "kernel"
        if self.tp > 1:
            if cfg.tp_comm not in ("p2p", "nccl"):
                raise ValueError(f"tp_comm must be 'p2p' or 'nccl', got {cfg.tp_comm!r}")
            if cfg.tp_allreduce not in ("auto", "kernel", "gemv", "push"):
                raise ValueError(f"tp_allreduce must be 'auto', 'kernel', 'gemv' or 'push', got {cfg.tp_allreduce!r}")
            if cfg.tp_comm == "p2p":
                if self.off & {"norm"}:
                    raise ValueError("tp_comm='p2p' fuses the all-reduce with residual add + RMSNorm; it cannot run "
                                     "with that fusion switched off (use tp_comm='nccl')")
                # exchange block: two regions for the all-reduce inside the o_proj / down_proj GEMVs (they alternate),
                # the logit shard, and - for tp_allreduce="kernel", where the exchange is a kernel of its own fused with
                # add + RMSNorm - two plain slots the row-split projections write their partials into
                gslot = self.K.tp_gemv_slot_bytes(self.H, self.tp)
                self.comm = TP.PeerComm(self.K, self.tp_rank, self.tp, [gslot, gslot, 2 * self.V, 2 * self.H, 2 * self.H],
                                        dev, cfg.tp_group)
                self.logits_local = self.comm.slot(2)
        every = [lw[n] for lw in self.layers for n in ("qkv", "o", "gu", "down")] + [self.lm_head]
        self.norm_in_gemv = (cfg.fuse_norm_gemv and not self.off and all(lin.tiled is not None for lin in every)
                             and (self.tp == 1 or (self.comm is not None and self.tp_allreduce == "gemv")))
        tiled_rows = all(lw[n].tiled is not None for lw in self.layers for n in ("o", "down"))
        if self.comm is not None and self.tp_allreduce == "push" and not tiled_rows:
            raise ValueError("tp_allreduce='push' needs the tile-layout copies of o_proj / down_proj (tile_weights)")
        self.tp_push = self.comm is not None and self.tp_allreduce == "push"
        if self.comm is not None and not self.norm_in_gemv and not self.tp_push:
            self.o, self.down = self.comm.slot(3), self.comm.slot(4)
        self.set_attention_partition(cfg.max_ctx)

    @classmethod
    def from_quantized(cls, path, cfg: DecodeConfig = None, **overrides):
        """Build the runtime from a directory written by checkpoint.save_quantized: no quantizer runs, the packed
        tensors go to the device as they are (each rank of a tensor-parallel group cuts its own shard)."""
        import dataclasses
        from . import checkpoint
        c, group, state, qparams = checkpoint.load_quantized(path)
        cfg = dataclasses.replace(cfg or DecodeConfig(), group=group, quant="packed", qparams=qparams, **overrides)
        return cls(state, c, cfg)

    # ------------------------------------------------------------------ attention partitioning
    def _policy_table(self):
        """Rows of the attention policy file (DecodeConfig.attn_policy_path): [{"max_ctx": c, "part_size": p}, ...]
        sorted by context, as kernel_bench writes them; empty when there is no file."""
        path = Path(self.cfg.attn_policy_path)
        if not path.is_file():
            return []
        with open(path) as f:
            rows = json.load(f).get("policy", [])
        return sorted((r for r in rows if r["max_ctx"] < (1 << 30)), key=lambda r: r["max_ctx"])

    def _policy_part_size(self, ctx_cap):
        """Split size for contexts up to ctx_cap: the row of the policy table tuned at the largest context that does
        not exceed ctx_cap (the first row for shorter contexts), which is how the reference picks it
        (runtime/model.py:164-172). Without a table: the smallest multiple of 32 tokens, at least 64, for which
        n_kv x splits still covers every SM about twice."""
        rows = self._policy_table()
        if rows:
            fitting = [r for r in rows if r["max_ctx"] <= ctx_cap]
            return int((fitting[-1] if fitting else rows[0])["part_size"])
        sms = torch.cuda.get_device_properties(self.cfg.device).multi_processor_count
        splits_wanted = max(1, (2 * sms) // self.n_kv)
        return max(64, 32 * math.ceil(ctx_cap / splits_wanted / 32))

    def set_attention_partition(self, ctx_cap, part_size=None):
        """Fix the split-K geometry of attention for contexts up to ctx_cap. The launch grid always has
        ceil(ctx_cap / part_size) splits (a captured graph cannot change it; splits beyond the live context exit at
        once), so the split scratch is sized for that many and the usable context is rounded up to whole splits."""
        size = part_size or self.cfg.part_size or self._policy_part_size(ctx_cap)
        n_splits = max(1, -(-ctx_cap // size))
        self.part_size, self.max_splits, self.ctx_cap = size, n_splits, n_splits * size
        dev = self.cfg.device
        self.o_part = torch.empty(self.n_q, n_splits, self.D, dtype=torch.float32, device=dev)
        self.m_part = torch.empty(self.n_q, n_splits, dtype=torch.float32, device=dev)
        self.l_part = torch.empty_like(self.m_part)
        # arrival counts of the split blocks per kv head: the last one to finish merges the splits (no combine launch)
        self.attn_arrive = torch.zeros(self.n_kv, dtype=torch.int32, device=dev)
        self.graph = None               # a captured graph holds the old geometry
        self._setup_persistent_step()

    def _setup_persistent_step(self):
        """Describe the step for b200_decode_step: device array of per-layer pointers, exchange and control memory.
        The kernel streams the tile-layout copies of the matrices (gate|up in its paired form), the same copies the
        per-operator GEMVs read."""
        mode = self.cfg.step_kernel
        G = self.cfg.group
        mats = [lw[n] for lw in self.layers for n in ("qkv", "o", "gu", "down")] + [self.lm_head]
        fits = (all(k % 128 == 0 and k % G == 0 for k in (self.H, self.n_q * self.D, self.I)) and G % 128 == 0
                and self.cfg.page <= 64 and all(m.tiled is not None for m in mats)
                and all(lw["gu"].paired for lw in self.layers))
        if mode == "persistent" and self.tp > 1:
            raise ValueError("step_kernel='persistent' is single-GPU; tensor-parallel steps use one launch per operator")
        if mode == "persistent" and self.off:
            raise ValueError("step_kernel='persistent' computes the fused operators; it cannot run with fused=False or "
                             "an ablation switch")
        if mode == "persistent" and not fits:
            raise ValueError("step_kernel='persistent' needs tile_weights, hidden, heads*head_dim and intermediate sizes "
                             "that are multiples of 128, a group size that is a multiple of 128 and pages of at most 64 "
                             "tokens; use step_kernel='multi' for this model")
        self.persistent = mode == "persistent" or (mode == "auto" and not self.off and fits and self.tp == 1
                                                   and self.ctx_cap <= PERSISTENT_MAX_CTX)
        if not self.persistent:
            return
        dev = self.cfg.device
        if getattr(self, "_step_static", None) is None:
            grid = torch.cuda.get_device_properties(dev).multi_processor_count
            arr = (ext.StepLayer * self.L)()
            for i, lw in enumerate(self.layers):
                for k, name in enumerate(("qkv", "o", "gu", "down")):
                    arr[i].w[k] = lw[name].tiled.data_ptr()
                    arr[i].sz[k] = 0
                arr[i].ln1, arr[i].ln2 = lw["ln1"].data_ptr(), lw["ln2"].data_ptr()
                arr[i].kc, arr[i].vc = self.kv[i, 0].data_ptr(), self.kv[i, 1].data_ptr()
            host = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8)
            nbytes = self.K.decode_step_xchg_bytes(self.L, self.H, self.I, self.n_q, self.n_kv, self.D, grid)
            self._step_static = {"layers": host.to(dev), "xchg": torch.zeros(nbytes, dtype=torch.uint8, device=dev),
                                 "ctrl": torch.zeros(4, dtype=torch.int32, device=dev), "grid": grid}
        st = self._step_static
        d = ext.StepDesc()
        d.layers = st["layers"].data_ptr()
        d.L, d.H, d.I, d.n_q, d.n_kv, d.D, d.V = self.L, self.H, self.I, self.n_q, self.n_kv, self.D, self.V
        d.log2G, d.log2P, d.eps = self.cfg.group.bit_length() - 1, self.cfg.page.bit_length() - 1, self.eps
        d.emb, d.norm_f = self.emb.data_ptr(), self.norm_f.data_ptr()
        d.w_head, d.sz_head = self.lm_head.tiled.data_ptr(), 0
        d.cos_t, d.sin_t, d.bt = self.cos.data_ptr(), self.sin.data_ptr(), self.bt.data_ptr()
        d.tok, d.pos, d.history = self.tok.data_ptr(), self.pos.data_ptr(), self.history.data_ptr()
        d.logits, d.xchg, d.ctrl = self.logits.data_ptr(), st["xchg"].data_ptr(), st["ctrl"].data_ptr()
        d.ctx_cap, d.grid = min(self.ctx_cap, self.cfg.max_ctx + 1), st["grid"]
        self._step_desc = d

    def step_error(self):
        """Non-zero if a bounded wait inside a kernel of the step gave up (the step's outputs are then invalid): the
        persistent kernel's code (4 = a token id outside the vocabulary was replaced by 0), the peer exchange's, or
        the attention ring's. Synchronises."""
        code = 0
        if getattr(self, "comm", None) is not None:
            code = self.comm.error()
        if getattr(self, "persistent", False):
            code = code or int(self._step_static["ctrl"][1])
        else:
            code = code or self.K.paged_attention_status()
        return code

    def prepare(self, ctx_cap, use_graph=True, part_size=None):
        """Get ready to decode up to context ctx_cap: attention geometry, then (optionally) the CUDA graph."""
        if ctx_cap > self.cfg.max_ctx:
            raise ValueError(f"ctx_cap {ctx_cap} exceeds max_ctx {self.cfg.max_ctx} the caches were sized for")
        self.set_attention_partition(ctx_cap, part_size)
        if use_graph:
            self.capture()

    # ------------------------------------------------------------------ operators
    def gemv_cfg(self, lin):
        return self.cfg.gemv_stage if self.cfg.gemv_stage is not None else (2, 0, 0, 0)

    def linear(self, lin: Linear, x, y):
        if "dequant" in self.off:   # ablation: weights go through an fp16 copy in HBM (4.5x the bytes)
            w16 = self.w_fp16[: lin.N * lin.K].view(lin.N, lin.K)
            self.K.dequant_w4a16(lin.packed, lin.sz, w16, self.cfg.group)
            torch.mv(w16, x, out=y)
            return
        if lin.tiled is not None:
            self.K.gemv_w4a16_tiled(lin.tiled, x, y, lin.N, lin.K)
            return
        s, r, w, pf = self.gemv_cfg(lin)
        self.K.gemv_w4a16(s, r, w, pf, lin.packed, lin.sz, x, y, self.cfg.group)

    def all_reduce(self, t):
        """Sum the partial outputs of a column-split projection over the TP ranks (NCCL, in stream, capturable)."""
        if self.tp > 1:
            torch.distributed.all_reduce(t, group=self.cfg.tp_group)

    def add_norm(self, delta, w, slot=None):
        """x <- x + delta, normed <- RMSNorm(x) * w. With tensor parallelism `delta` is this rank's partial of a
        row-split projection, held in exchange slot `slot`: the sum over the ranks happens here, inside the same
        kernel (tp_comm='p2p') or by an NCCL all-reduce in front of it."""
        if self.tp > 1 and delta is not None:
            if self.tp_push:   # the rows were pushed, as tagged words, into GEMV region `slot` of every rank
                self.K.tp_pushed_add_rmsnorm(self.comm.peers, self.tp_rank, self.comm.offsets[slot], self.x, w,
                                             self.normed, self.eps)
                return
            if self.comm is not None:
                self.K.tp_allreduce_add_rmsnorm(self.comm.peers, self.tp_rank, self.comm.offsets[3 + slot], self.x, w,
                                                self.normed, self.eps)
                return
            self.all_reduce(delta)
        if "norm" not in self.off:
            self.K.add_rmsnorm(self.x, delta, w, self.normed, self.eps)
        else:  # the unfused op sequence, on the device (ablation)
            if delta is not None:
                self.x.add_(delta)
            xf = self.x.float()
            self.normed.copy_(w * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).half())

    def swiglu(self):
        if "swiglu" not in self.off:
            self.K.swiglu(self.gu, self.act)
        else:
            s = torch.nn.functional.silu(self.gu[: self.I].float()).half()
            torch.mul(s, self.gu[self.I:], out=self.act)

    def rope_append_unfused(self, kc, vc):
        """Ablation: rotate q and k and append k, v to the cache as separate device ops (same arithmetic as the fused
        kernel: fp32 rotation of pairs (i, i + D/2), fp16 result; everything indexed by the device-resident pos)."""
        nq, nkv, D = self.n_q, self.n_kv, self.D
        c, s = self.cos.index_select(0, self.pos), self.sin.index_select(0, self.pos)       # [1, D/2]
        qk = self.qkv[: (nq + nkv) * D].view(nq + nkv, D)
        a, b = qk[:, : D // 2].float(), qk[:, D // 2:].float()
        qk.copy_(torch.cat([a * c - b * s, b * c + a * s], dim=-1).half())
        page = self.bt.index_select(0, self.pos // self.cfg.page).long().expand(nkv)
        slot = (self.pos % self.cfg.page).long().expand(nkv)
        kc.index_put_((page, self.kv_heads, slot), qk[nq:])
        vc.index_put_((page, self.kv_heads, slot), self.qkv[(nq + nkv) * D:].view(nkv, D))

    def attention(self, li):
        kc, vc = self.kv[li, 0], self.kv[li, 1]
        if "rope" in self.off:
            self.rope_append_unfused(kc, vc)
            self.K.paged_attention_batched(self.qkv[: self.n_q * self.D].view(1, self.n_q, self.D), kc, vc,
                                           self.bt.view(1, -1), self.pos, self.part_size, self.o_part.unsqueeze(0),
                                           self.m_part.unsqueeze(0), self.l_part.unsqueeze(0),
                                           self.attn.view(1, self.n_q, self.D))
        elif self.cfg.fuse_rope_attention:   # RoPE, cache append and attention in one partial-kernel launch
            self.K.rope_paged_attention(self.qkv, self.cos, self.sin, self.pos, self.bt, kc, vc, self.n_q, self.n_kv,
                                        self.part_size, self.o_part, self.m_part, self.l_part, self.attn,
                                        self.attn_arrive)
        elif self.D == 64:
            self.K.rope_append(self.qkv, self.cos, self.sin, self.pos, self.bt, kc, vc, self.n_q, self.n_kv)
            self.K.paged_attention(self.qkv[: self.n_q * self.D], kc, vc, self.bt, self.pos, self.part_size,
                                   self.o_part, self.m_part, self.l_part, self.attn, 3)
        else:
            self.K.rope_append_batched(self.qkv.view(1, -1), self.cos, self.sin, self.pos, self.bt.view(1, -1), kc, vc,
                                       self.n_q, self.n_kv)
            self.K.paged_attention_batched(self.qkv[: self.n_q * self.D].view(1, self.n_q, self.D), kc, vc,
                                           self.bt.view(1, -1), self.pos, self.part_size, self.o_part.unsqueeze(0),
                                           self.m_part.unsqueeze(0), self.l_part.unsqueeze(0),
                                           self.attn.view(1, self.n_q, self.D))

    # ------------------------------------------------------------------ decode step
    def step(self):
        """One token: reads self.tok / self.pos, writes self.logits, self.tok <- argmax, self.pos += 1."""
        if self.persistent:
            self.K.decode_step(self._step_desc)
            return
        self.K.embed_row(self.emb, self.tok, self.x)
        if self.norm_in_gemv:
            self.step_norm_in_gemv()
            return
        delta = None
        for li, lw in enumerate(self.layers):
            self.add_norm(delta, lw["ln1"], 1)
            self.linear(lw["qkv"], self.normed, self.qkv)
            self.attention(li)
            self.row_split_partial(lw["o"], self.attn.view(-1), self.o, 0)
            self.add_norm(self.o, lw["ln2"], 0)
            if lw["gu"].paired:   # act = SwiGLU(Wgate x, Wup x) in one launch
                self.K.gemv_w4a16_tiled(lw["gu"].tiled, self.normed, self.act, self.I, lw["gu"].K, swiglu=True)
            else:
                self.linear(lw["gu"], self.normed, self.gu)
                self.swiglu()
            self.row_split_partial(lw["down"], self.act, self.down, 1)
            delta = self.down
        self.add_norm(delta, self.norm_f, 1)
        self.linear(self.lm_head, self.normed, self.logits_local)
        if self.comm is not None:   # every rank gathers the whole vocabulary and takes the same argmax: no broadcast
            self.K.tp_allgather(self.comm.peers, self.tp_rank, self.comm.offsets[2], self.logits, self.V)
        elif self.tp > 1:
            torch.distributed.all_gather_into_tensor(self.logits, self.logits_local, group=self.cfg.tp_group)
        self.K.argmax(self.logits, self.tok, self.pos, self.history)

    def step_norm_in_gemv(self):
        """The layers with residual add + RMSNorm done inside the qkv / gate|up / LM-head GEMVs: 6 launches per layer
        (qkv, rope + attention, combine, o, gate|up + SwiGLU, down) instead of 10. The residual stream alternates
        between self.x and self.x_alt: a fused GEMV reads one and writes the other. Tensor parallel (tp_comm="p2p"):
        the same launches - the all-reduce of o_proj and down_proj happens inside those two GEMVs."""
        K, cur, nxt, delta = self.K, self.x, self.x_alt, None
        for li, lw in enumerate(self.layers):
            K.gemv_w4a16_tiled_norm(lw["qkv"].tiled, cur, delta, lw["ln1"], self.eps, nxt, self.qkv, lw["qkv"].N,
                                    lw["qkv"].K)
            cur, nxt = nxt, cur
            self.attention(li)
            self.row_split_linear(lw["o"], self.attn.view(-1), self.o, 0)
            gu = lw["gu"]
            if gu.paired:
                K.gemv_w4a16_tiled_norm(gu.tiled, cur, self.o, lw["ln2"], self.eps, nxt, self.act, self.I, gu.K,
                                        swiglu=True)
            else:
                K.gemv_w4a16_tiled_norm(gu.tiled, cur, self.o, lw["ln2"], self.eps, nxt, self.gu, gu.N, gu.K)
                self.swiglu()
            cur, nxt = nxt, cur
            self.row_split_linear(lw["down"], self.act, self.down, 1)
            delta = self.down
        K.gemv_w4a16_tiled_norm(self.lm_head.tiled, cur, delta, self.norm_f, self.eps, nxt, self.logits_local,
                                self.lm_head.N, self.lm_head.K)
        if self.comm is not None:   # every rank gathers the whole vocabulary and takes the same argmax: no broadcast
            K.tp_allgather(self.comm.peers, self.tp_rank, self.comm.offsets[2], self.logits, self.V)
        K.argmax(self.logits, self.tok, self.pos, self.history)

    def row_split_partial(self, lin, x, y, slot):
        """o_proj / down_proj of the step whose norm is a kernel of its own: this rank's partial rows go to y (one
        GPU: the result; tensor parallel: a slot of the exchange block) or, with tp_allreduce="push", as tagged words
        into GEMV region `slot` of every rank's block."""
        if self.tp_push:
            self.K.gemv_tiled_push(lin.tiled, x, lin.N, lin.K, self.comm.peers, self.tp_rank, self.comm.offsets[slot])
        else:
            self.linear(lin, x, y)

    def row_split_linear(self, lin, x, y, slot):
        """o_proj / down_proj. Tensor parallel: this rank's column shard times its x, summed over the ranks inside the
        same kernel (b200_gemv_w4a16_tiled_allreduce through exchange region `slot`); y is the sum on every rank."""
        if self.comm is None:
            self.linear(lin, x, y)
        else:
            self.K.gemv_tiled_allreduce(lin.tiled, x, y, lin.N, lin.K, self.comm.peers, self.tp_rank,
                                        self.comm.offsets[slot])

    def capture(self):
        """Record step() as one CUDA graph. torch wants the work run once or twice on a side stream before it
        records, and a step has side effects (token, position, history, one KV row per layer), so everything the
        warm-up and the recording touch is saved first and restored afterwards: capturing in mid-sequence loses
        nothing. The warm-up runs at positions 0 and 1, the recording at 0, all inside the page bt[0]."""
        if self.tp > 1 and self.comm is None:
            # tp_comm="nccl": the step is launched eagerly (a capture that contains NCCL collectives is not attempted;
            # the peer-memory exchange, made of this library's own kernels, is captured like everything else)
            self.graph = None
            return
        first_page = int(self.bt[0])
        keep = {"tok": self.tok.clone(), "pos": self.pos.clone(), "hist": self.history[:2].clone(),
                "kv": self.kv[:, :, first_page].clone()}
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        self.pos.zero_()
        with torch.cuda.stream(side):
            self.step()
            self.step()
        torch.cuda.current_stream().wait_stream(side)
        self.pos.zero_()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.step()
        self.graph = graph
        self.tok.copy_(keep["tok"])
        self.pos.copy_(keep["pos"])
        self.history[:2].copy_(keep["hist"])
        self.kv[:, :, first_page].copy_(keep["kv"])
        torch.cuda.synchronize()

    def run_step(self, use_graph=True):
        """One decode step at the next position (graph replay when a graph exists). The host mirrors the position
        only to refuse a step the attention geometry or the caches cannot hold."""
        limit = min(self.ctx_cap, self.cfg.max_ctx)
        if self.host_pos + 1 > limit:
            raise RuntimeError(f"context {self.host_pos + 1} exceeds the prepared attention cap {limit}; call prepare()")
        self.host_pos += 1
        if use_graph and self.graph is not None:
            self.graph.replay()
        else:
            self.step()

    # ------------------------------------------------------------------ high level
    def reset(self, pos=0):
        """Continue from position `pos` (0 = a new sequence; the cache rows below pos are kept)."""
        self.host_pos = pos
        self.pos.fill_(pos)

    def teacher_force(self, tokens, use_graph=True, collect_logits=False):
        """Run one step per given token, feeding tokens[i] at the i-th next position (this is also how a prompt is
        processed). Returns the logits of every step, fp16 [len, V], when collect_logits is set."""
        ids = torch.as_tensor(tokens).long().reshape(-1)
        n = ids.numel()
        if n and (int(ids.min()) < 0 or int(ids.max()) >= self.V_full):
            raise ValueError(f"token ids must lie in [0, {self.V_full})")
        dev = self.tok.device
        if ids.device.type != "cuda":
            ids = (ids.pin_memory() if n else ids).to(dev, non_blocking=True)
        logits = torch.empty(n, self.V_full, dtype=torch.half, device=dev) if collect_logits else None
        for i in range(n):
            self.tok.copy_(ids[i:i + 1])
            self.run_step(use_graph)
            if collect_logits:
                logits[i].copy_(self.logits)
        return logits

    def _prefill_state(self, T):
        """Static buffers of a prompt chunk of T tokens (kept per T and attention geometry, so that a recorded graph
        stays valid)."""
        key = (T, self.part_size, self.max_splits)
        cache = self.__dict__.setdefault("_prefill_cache", {})
        if key not in cache:
            if len(cache) >= 4:   # a few chunk sizes at most: the scratch of a chunk is tens of MB
                cache.pop(next(iter(cache)))
            dev, nq, nkv, D, S = self.tok.device, self.n_q, self.n_kv, self.D, self.max_splits
            h16 = dict(dtype=torch.half, device=dev)
            f32 = dict(dtype=torch.float32, device=dev)
            cache[key] = {
                "T": T, "graph": None, "ids": torch.zeros(T, dtype=torch.long, device=dev),
                "arange": torch.arange(T, dtype=torch.int32, device=dev), "pos": torch.zeros(T, dtype=torch.int32, device=dev),
                "bt": self.bt.view(1, -1).expand(T, -1).contiguous(),
                "x": torch.empty(T, self.H, **h16), "normed": torch.empty(T, self.H, **h16),
                "qkv": torch.empty(T, (nq + 2 * nkv) * D, **h16), "q": torch.empty(T, nq, D, **h16),
                "attn": torch.empty(T, nq, D, **h16), "o": torch.empty(T, self.H, **h16),
                "gu": torch.empty(T, 2 * self.I, **h16), "act": torch.empty(T, self.I, **h16),
                "down": torch.empty(T, self.H, **h16), "o_part": torch.empty(T, nq, S, D, **f32),
                "m_part": torch.empty(T, nq, S, **f32), "l_part": torch.empty(T, nq, S, **f32)}
        st = cache[key]
        st["bt"].copy_(self.bt.view(1, -1).expand(T, -1))   # the block table may have been replaced since
        return st

    def _prefill_chunk(self, st):
        """The launches of one prompt chunk: reads st["ids"] / st["pos"], leaves the final-norm output in st["normed"]."""
        K, G, T, nq, nkv, D = self.K, self.cfg.group, st["T"], self.n_q, self.n_kv, self.D
        x, normed, qkv, q, attn = st["x"], st["normed"], st["qkv"], st["q"], st["attn"]
        torch.index_select(self.emb, 0, st["ids"], out=x)
        delta = None
        for li, lw in enumerate(self.layers):
            K.add_rmsnorm_batched(x, delta, lw["ln1"], normed, self.eps)
            K.gemm_w4a16(lw["qkv"].packed, lw["qkv"].sz, normed, qkv, G)
            K.rope_append_batched(qkv, self.cos, self.sin, st["pos"], st["bt"], self.kv[li, 0], self.kv[li, 1], nq, nkv)
            q.copy_(qkv[:, : nq * D].view(T, nq, D))
            K.paged_attention_batched(q, self.kv[li, 0], self.kv[li, 1], st["bt"], st["pos"], self.part_size,
                                      st["o_part"], st["m_part"], st["l_part"], attn)
            K.gemm_w4a16(lw["o"].packed, lw["o"].sz, attn.view(T, nq * D), st["o"], G)
            K.add_rmsnorm_batched(x, st["o"], lw["ln2"], normed, self.eps)
            K.gemm_w4a16(lw["gu"].packed, lw["gu"].sz, normed, st["gu"], G)
            K.swiglu_batched(st["gu"], st["act"])
            K.gemm_w4a16(lw["down"].packed, lw["down"].sz, st["act"], st["down"], G)
            delta = st["down"]
        K.add_rmsnorm_batched(x, delta, self.norm_f, normed, self.eps)

    def prefill(self, tokens, collect_logits=False, use_graph=True):
        """Process a prompt T tokens at a time instead of one step per token: every weight matrix is read once per
        chunk of up to gemm_max_tokens() tokens (b200_gemm_w4a16, tcgen05 tensor cores), the small operators run in
        their batched forms, and attention runs as a batch of T queries over the same block table, query t seeing
        the cache up to its own position. The reference has no such path (it steps through the prompt,
        runtime/model.py:267-276). Leaves the runtime exactly where teacher_force(tokens) would: K/V rows of the
        prompt in the cache, self.logits / self.tok from the last prompt token, the position behind the prompt.
        The history entries of the prompt positions before the last are not written. Returns the logits of every
        prompt position, fp16 [len, V], when collect_logits is set. With use_graph a long prompt replays one CUDA graph
        per whole chunk from its second chunk on. One GPU, row-major packed weights kept (keep_packed=True)."""
        if self.tp != 1:
            raise ValueError("prefill() is single-GPU; tensor-parallel ranks step through the prompt")
        if self.off:
            raise ValueError("prefill() computes the fused operators; it cannot run with an ablation switch")
        mats = [lw[n] for lw in self.layers for n in ("qkv", "o", "gu", "down")] + [self.lm_head]
        if any(mt.packed is None for mt in mats):
            raise ValueError("prefill() reads the row-major packed tensors: build the model with keep_packed=True")
        if self.cfg.group % 64 or any(mt.K % 64 for mt in mats):
            raise ValueError("prefill() needs a group size and row lengths that are multiples of 64")
        ids = torch.as_tensor(tokens).long().reshape(-1)
        n = ids.numel()
        if n == 0:
            return torch.empty(0, self.V_full, dtype=torch.half, device=self.tok.device) if collect_logits else None
        if int(ids.min()) < 0 or int(ids.max()) >= self.V_full:
            raise ValueError(f"token ids must lie in [0, {self.V_full})")
        limit = min(self.ctx_cap, self.cfg.max_ctx)
        if self.host_pos + n > limit:
            raise RuntimeError(f"context {self.host_pos + n} exceeds the prepared attention cap {limit}; call prepare()")
        dev, K, G = self.tok.device, self.K, self.cfg.group
        if ids.device.type != "cuda":
            ids = ids.pin_memory().to(dev, non_blocking=True)
        h16 = dict(dtype=torch.half, device=dev)
        # tokens per chunk: the GEMM's limit, and split scratch of at most 256 MB
        chunk = max(1, min(K.gemm_max_tokens(), (256 << 20) // (self.n_q * self.max_splits * self.D * 4)))
        all_logits = torch.empty(n, self.V_full, **h16) if collect_logits else None
        for c0 in range(0, n, chunk):
            T = min(chunk, n - c0)
            st = self._prefill_state(T)
            st["ids"].copy_(ids[c0:c0 + T])
            torch.add(st["arange"], self.host_pos + c0, out=st["pos"])
            if st["graph"] is not None:
                st["graph"].replay()
            else:
                self._prefill_chunk(st)
                if use_graph and T == chunk and n - c0 > 2 * chunk:
                    # more whole chunks follow: record the launches (recording runs nothing) and replay them from here on
                    torch.cuda.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        self._prefill_chunk(st)
                    st["graph"] = graph
            if collect_logits:
                K.gemm_w4a16(self.lm_head.packed, self.lm_head.sz, st["normed"], all_logits[c0:c0 + T], G)
        normed = st["normed"]
        if collect_logits:
            self.logits.copy_(all_logits[n - 1])
        else:   # only the last position's logits are needed to go on: one GEMV
            self.linear(self.lm_head, normed[T - 1], self.logits)
        self.host_pos += n
        self.pos.fill_(self.host_pos - 1)
        K.argmax(self.logits, self.tok, self.pos, self.history)   # token after the prompt; pos -> host_pos
        return all_logits

    def generate(self, prompt, n_new, use_graph=True, prefill=False):
        """Greedy decoding of n_new tokens after `prompt`, each token read back to the host as soon as its step has
        run (what the reference's generate does, runtime/model.py:278-286). prefill=True processes the prompt with
        prefill() instead of one step per token. Returns a list of ints."""
        self.reset(0)
        if prefill:
            self.prefill(prompt)
        else:
            self.teacher_force(prompt, use_graph)
        out = []
        while True:
            out.append(int(self.tok))      # device -> host read of the token the last step chose
            if len(out) == n_new:
                return out
            self.run_step(use_graph)

    def generate_on_device(self, prompt, n_new, use_graph=True):
        """Same token stream as generate(), without a host read per token: the steps are queued back to back and
        the tokens come from the device-side history afterwards. Returns an int64 CPU tensor [n_new]."""
        self.reset(0)
        self.teacher_force(prompt, use_graph)
        for _ in range(n_new - 1):
            self.run_step(use_graph)
        first = len(prompt) - 1
        return self.history[first:first + n_new].cpu()

    # ------------------------------------------------------------------ byte accounting (for the roofline)
    def weight_bytes(self):
        """Bytes of weights one token reads, by part: the quantized matrices and norm vectors of the layers, the LM
        head, and one embedding row (the accounting of the reference, runtime/model.py:289-293)."""
        body = 0
        for lw in self.layers:
            body += sum(lw[name].nbytes for name in ("qkv", "o", "gu", "down"))
            body += 2 * (lw["ln1"].numel() + lw["ln2"].numel())
        return {"body": body, "lm_head": self.lm_head.nbytes, "embedding_row": 2 * self.H}

    def kv_bytes_per_token(self, ctx):
        """Cache bytes one token moves at context ctx: K and V rows of ctx tokens read, one of each written, in every
        layer (reference runtime/model.py:295-297)."""
        kv_row = 2 * self.n_kv * self.D             # fp16 row of all kv heads
        return self.L * 2 * kv_row * (ctx + 1)

    def bytes_per_token(self, ctx):
        wb = self.weight_bytes()
        return wb["body"] + wb["lm_head"] + wb["embedding_row"] + self.kv_bytes_per_token(ctx)


def rope_tables(max_pos: int, head_dim: int = 64, theta: float = 10000.0, device="cpu"):
    """cos / sin tables fp32 [max_pos, head_dim/2], angles computed in float64 (reference
    reference/ref_ops.py:30-33); the layout rope_append reads."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64, device=device) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float64, device=device)[:, None] * inv[None]
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()
