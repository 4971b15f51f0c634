"""CPU oracle for every operator of the batch-1 decode step (torch, fp32 math). TEST INFRASTRUCTURE ONLY.

Each function restates one operator of the reference's reference/ref_ops.py with the same name,
argument order and rounding points, so the CUDA kernels can be compared with it on identical inputs.
Imported by tests, by the smoke check and by the benchmark's CPU-baseline leg; never by the
product path.

Parity status: PINNED. tests/golden/make_golden.py imports the reference's own ref_ops.py and
stores its outputs; tests/test_oracle_golden.py requires these functions to reproduce them with
zero difference, plus the reference's own known answers (token 37 -> logical page 2, slot 5;
split-combine equals plain softmax to 2e-3).

Rounding points (reference/ref_ops.py:10-96): fp32 accumulation everywhere; fp16 rounding after the
GEMV, after the residual add, after the normalisation (before the fp16 multiply by the weight),
after silu (before the fp16 multiply by `up`), after each rotated component, after attention.
Batched helpers at the bottom (one sequence per loop iteration) are additions with no counterpart
in the reference; they only loop over the single-sequence functions.
"""
import math

import torch


def gemv_ref(w_ref, x):
    """fp16 dequantized weight [N, K] times fp16 x [K]; fp32 accumulate, fp16 out.
    reference/ref_ops.py:10-12."""
    return torch.mv(w_ref.to(torch.float32), x.to(torch.float32)).to(torch.float16)


def add_rmsnorm_ref(x, delta, w, eps):
    """Residual add in fp16, then LlamaRMSNorm. Returns (x + delta, w * normalised).
    reference/ref_ops.py:15-20."""
    summed = x if delta is None else x + delta
    f = summed.to(torch.float32)
    inv = torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + eps)
    return summed, w * (f * inv).to(torch.float16)


def swiglu_ref(gu):
    """gu = gate followed by up. silu(gate) rounded to fp16, times up, rounded to fp16.
    reference/ref_ops.py:23-27."""
    half = gu.shape[-1] // 2
    gate, up = gu[..., :half], gu[..., half:]
    act = torch.nn.functional.silu(gate.to(torch.float32)).to(torch.float16)
    return (act.to(torch.float32) * up.to(torch.float32)).to(torch.float16)


def rope_tables(max_pos, head_dim=64, theta=10000.0, device="cpu"):
    """cos and sin tables [max_pos, head_dim/2] in fp32, computed in float64.
    reference/ref_ops.py:30-33."""
    expo = torch.arange(0, head_dim, 2, dtype=torch.float64, device=device) / head_dim
    inv_freq = 1.0 / (theta ** expo)
    ang = torch.arange(max_pos, dtype=torch.float64, device=device)[:, None] * inv_freq[None, :]
    return ang.cos().to(torch.float32).contiguous(), ang.sin().to(torch.float32).contiguous()


def rope_ref(x, cos, sin, pos):
    """Rotate-half RoPE on x [heads, D]: component i pairs with i + D/2. fp32 math, fp16 out.
    reference/ref_ops.py:36-41."""
    d2 = x.shape[-1] // 2
    a, b = x[..., :d2].to(torch.float32), x[..., d2:].to(torch.float32)
    c, s = cos[pos], sin[pos]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(torch.float16)


def rope_append_ref(qkv, cos, sin, pos, k_cache, v_cache, block_table, n_q, n_kv, D, page):
    """Rotate q and k at `pos`, store k (rotated) and v (unchanged) in the paged cache, return
    the rotated q [n_q, D]. reference/ref_ops.py:44-53."""
    q = qkv[: n_q * D].view(n_q, D)
    k = qkv[n_q * D:(n_q + n_kv) * D].view(n_kv, D)
    v = qkv[(n_q + n_kv) * D:].view(n_kv, D)
    q_rot = rope_ref(q, cos, sin, pos)
    k_rot = rope_ref(k, cos, sin, pos)
    phys = int(block_table[pos // page])
    slot = pos % page
    k_cache[phys, :, slot] = k_rot
    v_cache[phys, :, slot] = v
    return q_rot


def gather_kv(k_cache, v_cache, block_table, ctx, page):
    """Paged cache [pages, n_kv, P, D] -> contiguous [ctx, n_kv, D] for K and V.
    reference/ref_ops.py:56-62."""
    used = (ctx + page - 1) // page
    phys = block_table[:used].long()
    n_kv, D = k_cache.shape[1], k_cache.shape[3]
    k = k_cache[phys].transpose(1, 2).reshape(-1, n_kv, D)[:ctx]
    v = v_cache[phys].transpose(1, 2).reshape(-1, n_kv, D)[:ctx]
    return k, v


def attention_contiguous_ref(q, k, v):
    """q [n_q, D]; k, v [ctx, n_kv, D]. Grouped-query attention by repeating each kv head,
    fp32 scores and softmax, fp16 out. reference/ref_ops.py:65-73."""
    n_q, D = q.shape
    rep = n_q // k.shape[1]
    kf = k.to(torch.float32).repeat_interleave(rep, dim=1)
    vf = v.to(torch.float32).repeat_interleave(rep, dim=1)
    scores = torch.einsum("hd,thd->ht", q.to(torch.float32), kf) / math.sqrt(D)
    prob = torch.softmax(scores, dim=-1)
    return torch.einsum("ht,thd->hd", prob, vf).to(torch.float16)


def paged_attention_ref(q, k_cache, v_cache, block_table, ctx, page):
    """reference/ref_ops.py:76-78."""
    k, v = gather_kv(k_cache, v_cache, block_table, ctx, page)
    return attention_contiguous_ref(q, k, v)


def split_softmax_combine_ref(q, k, v, part):
    """Model of the split-K kernels: per partition an un-normalised output, a running max and a
    sum; then the max-rescale merge. reference/ref_ops.py:81-96."""
    n_q, D = q.shape
    rep = n_q // k.shape[1]
    kf = k.to(torch.float32).repeat_interleave(rep, dim=1)
    vf = v.to(torch.float32).repeat_interleave(rep, dim=1)
    qf = q.to(torch.float32)
    outs, maxes, sums = [], [], []
    for start in range(0, k.shape[0], part):
        sc = torch.einsum("hd,thd->ht", qf, kf[start:start + part]) / math.sqrt(D)
        m = sc.amax(dim=-1)
        p = torch.exp(sc - m[:, None])
        outs.append(torch.einsum("ht,thd->hd", p, vf[start:start + part]))
        maxes.append(m)
        sums.append(p.sum(dim=-1))
    m_all = torch.stack(maxes)                    # [S, n_q]
    weight = torch.exp(m_all - m_all.amax(dim=0))
    denom = (weight * torch.stack(sums)).sum(dim=0)
    numer = (weight[..., None] * torch.stack(outs)).sum(dim=0)
    return (numer / denom[:, None]).to(torch.float16)


# ---- additions for shapes the reference does not have (they loop over the functions above) ----

def paged_attention_batched_ref(q, k_cache, v_cache, block_tables, ctxs, page):
    """q [B, n_q, D]; block_tables [B, max_pages]; ctxs: B context lengths. One sequence at a time
    through paged_attention_ref."""
    return torch.stack([paged_attention_ref(q[b], k_cache, v_cache, block_tables[b], int(ctxs[b]), page)
                        for b in range(q.shape[0])])


def argmax_ref(logits):
    """Index of the largest fp16 logit, lowest index on ties (what the reference's ref backend
    gets from `int(logits.float().argmax())`, runtime/model.py:232)."""
    lf = logits.to(torch.float32)
    return int((lf == lf.max()).nonzero()[0])
