"""Tensor-parallel sharding of the decode step's matrices (Megatron style) for one process per GPU.

The reference is single-GPU (it has no collective anywhere); this file is the shard arithmetic for large shapes
(Llama-3-70B on 2/4/8 B200s):

    q, k, v     split by heads   -> each rank keeps n_q/TP query heads and n_kv/TP KV heads; rows [q_r; k_r; v_r]
    gate, up    split by rows    -> rows [gate_r; up_r], so SwiGLU stays rank-local
    o_proj      split by columns -> K slice = this rank's heads x head_dim; partial sums, all-reduce
    down_proj   split by columns -> K slice = I/TP; partial sums, all-reduce
    lm_head     split by rows    -> V/TP logits per rank, all-gather, argmax on every rank (same result everywhere)

RoPE, KV cache and attention are rank-local (a rank owns whole heads). Norm weights, embedding, token, position and
block table are replicated. Column slices are cut at multiples of the quantization group, so for round-to-nearest
"shard then quantize" equals "quantize then shard" bit for bit; GPTQ results (q, scale, zero) are sharded after the
full-matrix calibration with shard_qsz().

Everything here is plain tensor slicing and runs on CPU tensors too (tests/test_tp.py does exactly that over gloo).
"""
import torch


def part(n, rank, world, what="dimension"):
    """[begin, end) of `rank`'s equal share of n."""
    if n % world:
        raise ValueError(f"{what} {n} is not divisible by the tensor-parallel size {world}")
    s = n // world
    return rank * s, (rank + 1) * s


def check(n_q, n_kv, D, I, V, group, world):
    """Raise unless the shape shards into whole heads and whole quantization groups."""
    for n, what in ((n_q, "query heads"), (n_kv, "KV heads"), (I, "intermediate size"), (V, "vocabulary")):
        part(n, 0, world, what)
    if (n_q // world * D) % group or (I // world) % group:
        raise ValueError("a column slice would cut a quantization group")
    if (I // world) % 8:
        raise ValueError("intermediate shard must be a multiple of 8")


def qkv_rows(n_q, n_kv, D, rank, world):
    """Row indices of this rank's [q_r; k_r; v_r] inside the stacked [q; k; v] matrix."""
    q0, q1 = part(n_q, rank, world, "query heads")
    k0, k1 = part(n_kv, rank, world, "KV heads")
    q = torch.arange(q0 * D, q1 * D)
    k = n_q * D + torch.arange(k0 * D, k1 * D)
    v = (n_q + n_kv) * D + torch.arange(k0 * D, k1 * D)
    return torch.cat([q, k, v])


def gate_up_rows(I, rank, world):
    """Row indices of [gate_r; up_r] inside the stacked [gate; up] matrix."""
    a, b = part(I, rank, world, "intermediate size")
    return torch.cat([torch.arange(a, b), I + torch.arange(a, b)])


def shard_rows(w, rows):
    return w.index_select(0, rows.to(w.device)).contiguous()


def shard_cols(w, a, b):
    return w[:, a:b].contiguous()


def shard_weight(kind, w, dims, rank, world):
    """kind in {"qkv", "o", "gu", "down", "lm_head"}; w the full (stacked) fp16 matrix; dims = (n_q, n_kv, D, I, V)."""
    n_q, n_kv, D, I, V = dims
    if world == 1:
        return w
    if kind == "qkv":
        return shard_rows(w, qkv_rows(n_q, n_kv, D, rank, world))
    if kind == "gu":
        return shard_rows(w, gate_up_rows(I, rank, world))
    if kind == "lm_head":
        a, b = part(V, rank, world, "vocabulary")
        return w[a:b].contiguous()
    if kind == "o":
        a, b = part(n_q, rank, world, "query heads")
        return shard_cols(w, a * D, b * D)
    if kind == "down":
        a, b = part(I, rank, world, "intermediate size")
        return shard_cols(w, a, b)
    raise ValueError(kind)


def shard_qsz(kind, qsz, dims, group, rank, world):
    """The same slicing applied to precomputed (q uint8 [N, K], scale [N, K/G], zero [N, K/G])."""
    if world == 1 or qsz is None:
        return qsz
    n_q, n_kv, D, I, V = dims
    q, s, z = qsz
    if kind in ("qkv", "gu", "lm_head"):
        if kind == "qkv":
            rows = qkv_rows(n_q, n_kv, D, rank, world)
        elif kind == "gu":
            rows = gate_up_rows(I, rank, world)
        else:
            rows = torch.arange(*part(V, rank, world, "vocabulary"))
        return tuple(shard_rows(t, rows) for t in (q, s, z))
    a, b = (x * D for x in part(n_q, rank, world)) if kind == "o" else part(I, rank, world)
    if a % group or b % group:
        raise ValueError("a column slice would cut a quantization group")
    return q[:, a:b].contiguous(), s[:, a // group:b // group].contiguous(), z[:, a // group:b // group].contiguous()
