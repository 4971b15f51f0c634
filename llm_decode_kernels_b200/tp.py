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


def shard_packed(kind, psz, dims, group, rank, world):
    """The same slicing applied to a matrix in kernel format: (packed int32 [N, K/8], sz fp16 [N, K/G, 2]). Column
    slices fall on group boundaries, which are word boundaries too (a group is a multiple of 8 weights)."""
    if world == 1 or psz is None:
        return psz
    n_q, n_kv, D, I, V = dims
    packed, sz = psz
    if kind in ("qkv", "gu", "lm_head"):
        if kind == "qkv":
            rows = qkv_rows(n_q, n_kv, D, rank, world)
        elif kind == "gu":
            rows = gate_up_rows(I, rank, world)
        else:
            rows = torch.arange(*part(V, rank, world, "vocabulary"))
        return shard_rows(packed, rows), shard_rows(sz, rows)
    a, b = (x * D for x in part(n_q, rank, world)) if kind == "o" else part(I, rank, world)
    if a % group or b % group:
        raise ValueError("a column slice would cut a quantization group")
    return packed[:, a // 8:b // 8].contiguous(), sz[:, a // group:b // group].contiguous()


# ---- exchange over NVLink peer memory ------------------------------------------------------------------------------
class _RawCuda:
    """Minimal __cuda_array_interface__ carrier, so torch can wrap memory the exchange block owns."""

    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}


class PeerComm:
    """One rank's exchange block plus its mapping of every peer's block (b200_comm_* of the C library).

    `slots` are byte sizes of the data slots (e.g. [2 H, 2 H, 2 V/TP]: o_proj partial, down_proj partial, logit
    shard). The block is allocated by the library (cudaMalloc, so that a CUDA IPC handle names exactly it), the
    handles travel through torch.distributed (all_gather_object on `group`), and every peer block is opened with
    peer access enabled. slot(i) is a torch fp16 tensor over slot i of the LOCAL block: a GEMV that writes its
    output there has published its partial. `peers` is the ctypes array the exchange entry points take."""

    def __init__(self, K, rank, world, slots, device, group=None):
        import ctypes
        import torch.distributed as dist
        self.K, self.rank, self.world, self.group, self.device = K, rank, world, group, device
        align = lambda n: (n + 255) // 256 * 256
        self.offsets, off = [], K.comm_header_bytes()
        for nbytes in slots:
            self.offsets.append(off)
            off += align(nbytes)
        self.slot_bytes, self.nbytes = list(slots), off
        with torch.cuda.device(device):
            self.base = K.comm_alloc(self.nbytes)
            handle = K.comm_export(self.base)
            handles = [None] * world
            dist.all_gather_object(handles, handle, group=group)
            self.mapped = [self.base if r == rank else K.comm_import(handles[r]) for r in range(world)]
        self.peers = (ctypes.c_void_p * world)(*self.mapped)
        self._views = [torch.as_tensor(_RawCuda(self.base + o, n // 2, "<f2"), device=device)
                       for o, n in zip(self.offsets, self.slot_bytes)]
        dist.barrier(group=group)   # nobody signals before everybody has mapped everybody

    def slot(self, i):
        return self._views[i]

    def error(self):
        """0, or the code of a peer wait that ran out on this rank. Synchronises."""
        return self.K.comm_error(self.base)

    def reset(self):
        """Zero flags, step counter and error word on every rank (collective: every rank must call it)."""
        import torch.distributed as dist
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.K.comm_reset(self.base)
        dist.barrier(group=self.group)

    def close(self):
        """Unmap the peers and free the local block (collective: peers must not be inside an exchange)."""
        import torch.distributed as dist
        if self.base is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self._views = []
        for r, p in enumerate(self.mapped):
            if r != self.rank:
                self.K.comm_unimport(p)
        dist.barrier(group=self.group)
        self.K.comm_free(self.base)
        self.base = None
