"""CPU oracle for the whole batch-1 decode step (torch fp32 math on dequantized weights). TEST INFRASTRUCTURE ONLY.

Restates what the reference's runtime/model.py does when it is built with
DecodeConfig(backend="ref", device="cpu"): the same operator sequence per token, the same deferred
residual add, the same paged KV cache with a shuffled block table, teacher-forced prompt, greedy
free-run with lowest-index argmax. It is the token-stream and logits oracle for the CUDA runtime
and the timed CPU baseline of the benchmark; the product never imports it.

Parity status: PINNED. tests/golden/make_golden.py builds the reference's own Model on a small
random Llama-shaped state dict and stores its logits and greedy tokens; tests/test_oracle_golden.py
requires this class to reproduce them exactly.

Operator order per token (reference runtime/model.py:216-233):
    x = embedding[tok]
    per layer: add_norm(delta, ln1) -> qkv -> rope+append -> attention -> o
               -> add_norm(o, ln2) -> gate|up -> swiglu -> down ; delta = down
    add_norm(delta, final norm) -> lm_head -> tok = argmax ; pos += 1
"""
import numpy as np
import torch

from . import ops_oracle as R
from . import quant_oracle as Q


class OracleLinear:
    """fp16 dequantized weight of one projection. Built either by quantizing `w` with the oracle's
    own quantizer (reference runtime/model.py:56-72) or from tensors already in kernel format."""

    ROWS = 512  # rows are independent: work in row blocks so numpy temporaries stay cache-sized

    def __init__(self, w=None, group=128, clip=False, qsz=None, packed=None, sz=None):
        n = (packed if packed is not None else qsz[0] if qsz is not None else w).shape[0]
        out, n_sz = [], 0
        for r0 in range(0, n, self.ROWS):
            r = slice(r0, r0 + self.ROWS)
            if packed is not None:
                q = Q.unpack(np.ascontiguousarray(packed[r]))
                szn = np.asarray(sz[r])
                s, z = szn[..., 0], szn[..., 1]
            elif qsz is not None:
                q, s, z = (np.asarray(t[r]) for t in qsz)
            else:
                q, s, z = Q.quantize(np.asarray(w[r]), group, clip)
            out.append(Q.dequantize(q, s, z, group))
            n_sz += s.size
        self.w_ref = torch.from_numpy(np.concatenate(out, axis=0))
        self.N, self.K = self.w_ref.shape
        self.nbytes = (self.K // 8) * self.N * 4 + n_sz * 4


class OracleModel:
    """hf_state: dict of HF-Llama-named tensors; hf_config: object with hidden_size,
    num_hidden_layers, num_attention_heads, num_key_value_heads, intermediate_size, vocab_size,
    rms_norm_eps (and optionally rope_theta); cfg: any object with the DecodeConfig fields group,
    quant, qparams, max_ctx, page, shuffle_pages.

    `packed`: optional {"layers.{i}.{qkv,o,gu,down}" | "lm_head": (packed int32, sz fp16)} of weights
    already in kernel format (numpy or CPU tensors); when given they are used instead of
    re-quantizing, so the oracle and the CUDA runtime compute on identical weights.
    `block_table`: optional int32 page permutation to share with the runtime under test."""

    def __init__(self, hf_state, hf_config, cfg, packed=None, block_table=None):
        c = hf_config
        self.cfg = cfg
        self.H, self.L = c.hidden_size, c.num_hidden_layers
        self.n_q, self.n_kv = c.num_attention_heads, c.num_key_value_heads
        # the reference derives head_dim as hidden / heads (runtime/model.py:81); an explicit head_dim attribute,
        # which it does not know, is honoured here for the head_dim-128 shapes
        self.D = getattr(c, "head_dim", None) or self.H // self.n_q
        self.I, self.V = c.intermediate_size, c.vocab_size
        self.eps = c.rms_norm_eps
        sd = hf_state
        h = lambda k: sd[k].to(torch.float16).cpu()
        clip = cfg.quant == "clip"

        def lin(key, w_fn):
            if packed is not None:
                p, sz = packed[key]
                return OracleLinear(group=cfg.group, packed=_np(p), sz=_np(sz))
            if cfg.quant == "pre":
                return OracleLinear(group=cfg.group, qsz=tuple(_np(t) for t in cfg.qparams[key]))
            return OracleLinear(w_fn().numpy(), cfg.group, clip)

        self.emb = h("model.embed_tokens.weight")
        self.layers = []
        for i in range(self.L):
            p = f"model.layers.{i}."
            self.layers.append({
                "ln1": h(p + "input_layernorm.weight"), "ln2": h(p + "post_attention_layernorm.weight"),
                "qkv": lin(f"layers.{i}.qkv", lambda: torch.cat([h(p + "self_attn.q_proj.weight"),
                                                                 h(p + "self_attn.k_proj.weight"),
                                                                 h(p + "self_attn.v_proj.weight")], 0)),
                "o": lin(f"layers.{i}.o", lambda: h(p + "self_attn.o_proj.weight")),
                "gu": lin(f"layers.{i}.gu", lambda: torch.cat([h(p + "mlp.gate_proj.weight"),
                                                               h(p + "mlp.up_proj.weight")], 0)),
                "down": lin(f"layers.{i}.down", lambda: h(p + "mlp.down_proj.weight"))})
        self.norm_f = h("model.norm.weight")
        head_key = "lm_head.weight" if "lm_head.weight" in sd else "model.embed_tokens.weight"
        self.lm_head = lin("lm_head", lambda: h(head_key))

        self.n_pages = (cfg.max_ctx + cfg.page - 1) // cfg.page + 1
        self.kv = torch.zeros(self.L, 2, self.n_pages, self.n_kv, cfg.page, self.D, dtype=torch.float16)
        if block_table is not None:
            self.bt = torch.as_tensor(block_table).to(torch.int32).cpu()
        elif getattr(cfg, "shuffle_pages", True):
            self.bt = torch.randperm(self.n_pages).to(torch.int32)
        else:
            self.bt = torch.arange(self.n_pages, dtype=torch.int32)
        theta = getattr(c, "rope_theta", 10000.0)
        self.cos, self.sin = R.rope_tables(cfg.max_ctx + 1, self.D, theta)
        self.tok, self.pos = 0, 0
        self.logits = None

    def step(self):
        """One token at self.pos from self.tok: fills self.logits, sets self.tok to the argmax and
        advances self.pos."""
        x = self.emb[self.tok].clone()
        delta = None
        for li, lw in enumerate(self.layers):
            x, normed = R.add_rmsnorm_ref(x, delta, lw["ln1"], self.eps)
            qkv = R.gemv_ref(lw["qkv"].w_ref, normed)
            kc, vc = self.kv[li, 0], self.kv[li, 1]
            q = R.rope_append_ref(qkv, self.cos, self.sin, self.pos, kc, vc, self.bt, self.n_q, self.n_kv,
                                  self.D, self.cfg.page)
            attn = R.paged_attention_ref(q, kc, vc, self.bt, self.pos + 1, self.cfg.page)
            o = R.gemv_ref(lw["o"].w_ref, attn.reshape(-1))
            x, normed = R.add_rmsnorm_ref(x, o, lw["ln2"], self.eps)
            gu = R.gemv_ref(lw["gu"].w_ref, normed)
            act = R.swiglu_ref(gu)
            delta = R.gemv_ref(lw["down"].w_ref, act)
        x, normed = R.add_rmsnorm_ref(x, delta, self.norm_f, self.eps)
        self.logits = R.gemv_ref(self.lm_head.w_ref, normed)
        self.tok = R.argmax_ref(self.logits)
        self.pos += 1

    def reset(self, pos=0):
        self.pos = pos

    def teacher_force(self, tokens, collect_logits=False):
        """Feed tokens at positions pos, pos+1, ...; optionally return logits [len, V] fp16."""
        out = []
        for t in tokens:
            self.tok = int(t)
            self.step()
            if collect_logits:
                out.append(self.logits.clone())
        return torch.stack(out) if collect_logits else None

    def generate(self, prompt, n_new):
        """Greedy: teacher-force the prompt, then free-run. Returns n_new token ids (the first is
        the prediction after the last prompt token). reference runtime/model.py:278-286."""
        self.reset(0)
        self.teacher_force(prompt)
        new = [self.tok]
        for _ in range(n_new - 1):
            self.step()
            new.append(self.tok)
        return new


def _np(t):
    return t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else np.asarray(t)
