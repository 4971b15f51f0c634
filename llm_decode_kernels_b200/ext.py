"""Loader and Python face of libb200decode.so.

`load()` returns an object with the six operators of the reference's extension module `decode_kernels`
(built by its runtime/ext.py:9-20, defined in kernels/bindings.cpp:90-98) under the same names, argument
order and keyword names: gemv_w4a16, bw_read, paged_attention, add_rmsnorm, swiglu, rope_append. Each checks its
tensors the way the reference binding does (contiguous CUDA tensors, dtypes, shapes, 16-byte alignment), then
passes raw device pointers and the current torch CUDA stream to the C ABI declared in include/b200decode.h.
Errors surface as RuntimeError before anything is launched. There is no fallback: if the library is missing,
cannot be built, or a tensor is not on a CUDA device, the call raises.

Additional operators (no counterpart in the reference): dequant_w4a16, paged_attention_batched,
rope_append_batched, embed_row, argmax, and the prompt's batched forms gemm_w4a16, add_rmsnorm_batched,
swiglu_batched.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_size_t, c_void_p
from pathlib import Path

import torch

_LIB = None
_OPS = None
LIB_PATH = Path(__file__).resolve().parent / "libb200decode.so"

# name -> argtypes, exactly the declarations of include/b200decode.h (checked by tests/test_abi.py)
SIGNATURES = {
    "b200_gemv_w4a16": [c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                        c_void_p],
    "b200_gemv_w4a16_tile_repack": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "b200_gemv_w4a16_tiled": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "b200_gemv_w4a16_tiled_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int,
                                   c_int, c_void_p],
    "b200_gemv_w4a16_tune": [c_int, c_int, c_int, c_int, c_int],
    "b200_bw_read": [c_void_p, c_size_t, c_void_p, c_int, c_int, c_int, c_void_p],
    "b200_bw_read_bulk": [c_void_p, c_size_t, c_void_p, c_int, c_int, c_int, c_void_p],
    "b200_paged_attention": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "b200_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p],
    "b200_swiglu": [c_void_p, c_void_p, c_int, c_void_p],
    "b200_rope_append": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                         c_void_p],
    "b200_paged_attention_batched": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                     c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "b200_paged_attention_batched_v": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                       c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p],
    "b200_rope_paged_attention": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                  c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p],
    "b200_paged_attention_status": [c_void_p],
    "b200_comm_header_bytes": [],
    "b200_comm_alloc": [c_size_t, c_void_p],
    "b200_comm_free": [c_void_p],
    "b200_comm_export": [c_void_p, c_void_p],
    "b200_comm_import": [c_void_p, c_void_p],
    "b200_comm_unimport": [c_void_p],
    "b200_comm_reset": [c_void_p],
    "b200_comm_error": [c_void_p, c_void_p],
    "b200_comm_set_wait_limit": [c_void_p, ctypes.c_uint],
    "b200_tp_allreduce_add_rmsnorm": [c_void_p, c_int, c_int, c_size_t, c_void_p, c_void_p, c_void_p, c_int, c_float,
                                      c_void_p],
    "b200_tp_allgather": [c_void_p, c_int, c_int, c_size_t, c_void_p, c_int, c_void_p],
    "b200_gemv_w4a16_tiled_allreduce": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_size_t,
                                        c_void_p],
    "b200_gemv_w4a16_tiled_push": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_size_t, c_void_p],
    "b200_tp_pushed_add_rmsnorm": [c_void_p, c_int, c_int, c_size_t, c_void_p, c_void_p, c_void_p, c_int, c_float,
                                   c_void_p],
    "b200_paged_attention_noalloc": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                     c_int, c_void_p, c_void_p],
    "b200_rope_append_batched": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                 c_int, c_int, c_int, c_int, c_void_p],
    "b200_dequant_w4a16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "b200_add_rmsnorm_batched": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "b200_swiglu_batched": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "b200_gemm_w4a16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "b200_gemm_w4a16_max_tokens": [],
    "b200_gemm_w4a16_status": [c_void_p],
    "b200_embed_row": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "b200_argmax": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
}


class StepLayer(ctypes.Structure):
    """b200_step_layer of include/b200decode.h (an array of these is copied to device memory)."""
    _fields_ = [("w", c_void_p * 4), ("sz", c_void_p * 4), ("ln1", c_void_p), ("ln2", c_void_p), ("kc", c_void_p),
                ("vc", c_void_p)]


class StepDesc(ctypes.Structure):
    """b200_step_desc of include/b200decode.h."""
    _fields_ = [("layers", c_void_p), ("L", c_int), ("H", c_int), ("I", c_int), ("n_q", c_int), ("n_kv", c_int),
                ("D", c_int), ("V", c_int), ("log2G", c_int), ("log2P", c_int), ("eps", c_float), ("emb", c_void_p),
                ("norm_f", c_void_p), ("w_head", c_void_p), ("sz_head", c_void_p), ("cos_t", c_void_p),
                ("sin_t", c_void_p), ("bt", c_void_p), ("tok", c_void_p), ("pos", c_void_p), ("history", c_void_p),
                ("logits", c_void_p), ("xchg", c_void_p), ("ctrl", c_void_p), ("ctx_cap", c_int), ("grid", c_int), ("trace", c_void_p)]


def load_library(build_if_missing=True, path=None):
    """dlopen libb200decode.so (building it with nvcc first if it is absent) and declare its symbols. `path` names
    another build of the same library (step_trace.py's instrumented one); it must be given on the first call."""
    global _LIB
    if _LIB is not None:
        if path is not None and Path(path).resolve() != Path(_LIB._name).resolve():
            raise RuntimeError(f"{_LIB._name} is already loaded")
        return _LIB
    if path is None and not LIB_PATH.exists():
        if not build_if_missing:
            raise RuntimeError(f"{LIB_PATH} is missing; run `python -m llm_decode_kernels_b200.build`")
        from . import build as _build
        _build.build()
    lib = ctypes.CDLL(str(path or LIB_PATH))
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError here = the library does not export a declared symbol
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.b200_decode_step.argtypes = [ctypes.POINTER(StepDesc), c_void_p]
    lib.b200_decode_step.restype = c_int
    lib.b200_gemv_w4a16_tiled_bytes.argtypes = [c_int, c_int, c_int]
    lib.b200_gemv_w4a16_tiled_bytes.restype = c_size_t
    lib.b200_tp_gemv_slot_bytes.argtypes = [c_int, c_int]
    lib.b200_tp_gemv_slot_bytes.restype = c_size_t
    lib.b200_decode_step_xchg_bytes.argtypes = [c_int] * 7
    lib.b200_decode_step_xchg_bytes.restype = c_size_t
    lib.b200_version.restype = c_int
    lib.b200_strerror.restype = ctypes.c_char_p
    lib.b200_strerror.argtypes = [c_int]
    lib.b200_last_cuda_error.restype = ctypes.c_char_p
    _LIB = lib
    return lib


def _ilog2_exact(v, what):
    if v <= 0 or v & (v - 1):
        raise RuntimeError(f"{what} must be a power of two, got {v}")
    return v.bit_length() - 1


def _cuda(t, name, dtype=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda or not t.is_contiguous():
        raise RuntimeError(f"{name} must be a contiguous CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")
    return t


def _aligned16(t, name):
    if t.data_ptr() % 16:
        raise RuntimeError(f"{name} must be 16B aligned")


def _stream():
    return torch.cuda.current_stream().cuda_stream


class Ops:
    """The operator set. Every method launches on torch's current CUDA stream and returns None."""

    def __init__(self, lib):
        self.lib = lib

    def _check(self, code, what):
        if code != 0:
            msg = self.lib.b200_strerror(code).decode()
            if code == -4:
                msg += ": " + self.lib.b200_last_cuda_error().decode()
            raise RuntimeError(f"{what}: {msg}")

    # ---- the reference's six operators ------------------------------------------------------------------
    def gemv_w4a16(self, stage, R, warps, pf, packed, sz, x, y, group):
        """y = dequant(packed, sz) @ x. packed int32 [N, K/8], sz fp16 [N, K/group, 2], x fp16 [K], y fp16 [N].
        (stage, R, warps, pf): see b200_gemv_w4a16; pass R=0 for the library's own choice."""
        _cuda(packed, "packed", torch.int32), _cuda(sz, "sz", torch.float16)
        _cuda(x, "x", torch.float16), _cuda(y, "y", torch.float16)
        N, K = packed.shape[0], packed.shape[1] * 8
        if K % 32 or K % group:
            raise RuntimeError("K must be a multiple of 32 and of the group size")
        if group < 32:
            raise RuntimeError("group must be >= 32")
        if x.numel() != K or y.numel() != N or sz.shape[0] != N or sz.shape[1] != K // group:
            raise RuntimeError("gemv_w4a16: inconsistent shapes")
        _aligned16(packed, "packed"), _aligned16(x, "x")
        self._check(self.lib.b200_gemv_w4a16(int(stage), int(R), int(warps), int(pf), packed.data_ptr(),
                                             sz.data_ptr(), x.data_ptr(), y.data_ptr(), N, K,
                                             _ilog2_exact(int(group), "group"), _stream()), "gemv_w4a16")

    def gemv_tile_repack(self, packed, sz, group, gate_up=False):
        """Copy of a quantized matrix in the tile layout of the tensor-core GEMV (uint8 tensor), or None when the
        shape rules it out (K % 128 != 0 or a group size that is not a multiple of 128). gate_up: the matrix is
        [gate; up]; gate row i and up row i share a tile, for gemv_w4a16_tiled(..., swiglu=True)."""
        _cuda(packed, "packed", torch.int32), _cuda(sz, "sz", torch.float16)
        N, K = packed.shape[0], packed.shape[1] * 8
        nbytes = int(self.lib.b200_gemv_w4a16_tiled_bytes(N, K, int(gate_up)))
        if nbytes == 0 or group % 128:
            return None
        out = torch.empty(nbytes, dtype=torch.uint8, device=packed.device)
        self._check(self.lib.b200_gemv_w4a16_tile_repack(packed.data_ptr(), sz.data_ptr(), out.data_ptr(), N, K,
                                                         _ilog2_exact(int(group), "group"), int(gate_up), _stream()),
                    "gemv_tile_repack")
        return out

    def gemv_tune(self, layout, N, K, ksplit, blocks):
        """Launch shape of the tensor-core GEMV for matrices of N x K (b200_gemv_w4a16_tune); ksplit=0 forgets it."""
        self._check(self.lib.b200_gemv_w4a16_tune(int(layout), int(N), int(K), int(ksplit), int(blocks)), "gemv_tune")

    def load_gemv_tunes(self, path):
        """Register every entry of an autotune file (written by llm_decode_kernels_b200.autotune). Returns how many."""
        import json
        from pathlib import Path as _P
        if not _P(path).is_file():
            return 0
        rows = json.load(open(path)).get("gemv", [])
        for r in rows:
            self.gemv_tune(r["layout"], r["N"], r["K"], r["ksplit"], r["blocks"])
        return len(rows)

    def gemv_w4a16_tiled(self, tiled, x, y, N, K, swiglu=False):
        """y[N] = W x from the tile-layout copy. swiglu: the copy is a paired [gate; up] and y[N] = silu(gate) * up."""
        _cuda(tiled, "tiled", torch.uint8), _cuda(x, "x", torch.float16), _cuda(y, "y", torch.float16)
        if x.numel() != K or y.numel() != N:
            raise RuntimeError("gemv_w4a16_tiled: x must hold K and y N values")
        self._check(self.lib.b200_gemv_w4a16_tiled(tiled.data_ptr(), x.data_ptr(), y.data_ptr(), int(N), int(K),
                                                   int(swiglu), _stream()), "gemv_w4a16_tiled")

    def gemv_w4a16_tiled_norm(self, tiled, x_in, delta, norm_w, eps, x_out, y, N, K, swiglu=False):
        """add_rmsnorm + gemv_w4a16_tiled in one launch: x_out = x_in + delta (delta may be None),
        y = W (norm_w * rmsnorm(x_out)); x_out must be a different buffer from x_in."""
        _cuda(tiled, "tiled", torch.uint8)
        for t_, n_ in ((x_in, "x_in"), (norm_w, "norm_w"), (x_out, "x_out"), (y, "y")):
            _cuda(t_, n_, torch.float16)
        if x_in.numel() != K or x_out.numel() != K or norm_w.numel() != K or y.numel() != N:
            raise RuntimeError("gemv_w4a16_tiled_norm: vectors must hold K values and y N")
        d = 0
        if delta is not None:
            _cuda(delta, "delta", torch.float16)
            d = delta.data_ptr()
        self._check(self.lib.b200_gemv_w4a16_tiled_norm(tiled.data_ptr(), x_in.data_ptr(), d, norm_w.data_ptr(),
                                                        float(eps), x_out.data_ptr(), y.data_ptr(), int(N), int(K),
                                                        int(swiglu), _stream()), "gemv_w4a16_tiled_norm")

    def bw_read(self, buf, sink, blocks, threads, unroll):
        _cuda(buf, "buf"), _cuda(sink, "sink"), _aligned16(buf, "buf")
        self._check(self.lib.b200_bw_read(buf.data_ptr(), buf.numel() * buf.element_size(), sink.data_ptr(),
                                          int(blocks), int(threads), int(unroll), _stream()), "bw_read")

    def bw_read_bulk(self, buf, sink, blocks, stage_bytes, stages):
        _cuda(buf, "buf"), _cuda(sink, "sink"), _aligned16(buf, "buf")
        self._check(self.lib.b200_bw_read_bulk(buf.data_ptr(), buf.numel() * buf.element_size(), sink.data_ptr(),
                                               int(blocks), int(stage_bytes), int(stages), _stream()), "bw_read_bulk")

    def paged_attention(self, q, kc, vc, bt, pos, part_size, o_part, m_part, l_part, out, version=2):
        """One sequence, head_dim 64. q [n_q*64], caches [pages, n_kv, P, 64], bt int32 [pages], pos int32 [1],
        scratch o_part fp32 [n_q, max_splits, 64], m_part/l_part fp32 [n_q, max_splits], out fp16 [n_q, 64]."""
        for t, n in ((q, "q"), (kc, "kc"), (vc, "vc"), (out, "out")):
            _cuda(t, n, torch.float16)
        _cuda(bt, "bt", torch.int32), _cuda(pos, "pos", torch.int32)
        for t, n in ((o_part, "o_part"), (m_part, "m_part"), (l_part, "l_part")):
            _cuda(t, n, torch.float32)
        if kc.dim() != 4 or kc.shape[3] != 64 or vc.shape != kc.shape:
            raise RuntimeError("cache must be [pages, n_kv, P, 64]")
        _aligned16(kc, "kc"), _aligned16(vc, "vc")
        n_q, n_kv, P = q.numel() // 64, kc.shape[1], kc.shape[2]
        if n_q % n_kv or n_q // n_kv not in (1, 2, 4, 8):
            raise RuntimeError("heads-per-group must be 1/2/4/8")
        if part_size <= 0:
            raise RuntimeError("part_size must be > 0")
        if not 1 <= version <= 3:
            raise RuntimeError("attention version must be 1, 2 or 3")
        max_splits = o_part.shape[1]
        if o_part.shape[0] != n_q or m_part.shape[1] != max_splits or l_part.shape[1] != max_splits:
            raise RuntimeError("split buffers have inconsistent shapes")
        self._check(self.lib.b200_paged_attention(int(version), q.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                                  bt.data_ptr(), pos.data_ptr(), n_q, n_kv,
                                                  _ilog2_exact(P, "page size"), int(part_size), max_splits,
                                                  o_part.data_ptr(), m_part.data_ptr(), l_part.data_ptr(),
                                                  out.data_ptr(), _stream()), "paged_attention")

    def add_rmsnorm(self, x, delta, w, out, eps):
        _cuda(x, "x", torch.float16), _cuda(w, "w", torch.float16), _cuda(out, "out", torch.float16)
        if x.numel() % 8:
            raise RuntimeError("H must be a multiple of 8")
        _aligned16(x, "x"), _aligned16(w, "w"), _aligned16(out, "out")
        d = 0
        if delta is not None:
            _cuda(delta, "delta", torch.float16), _aligned16(delta, "delta")
            d = delta.data_ptr()
        self._check(self.lib.b200_add_rmsnorm(x.data_ptr(), d, w.data_ptr(), out.data_ptr(), x.numel(), float(eps),
                                              _stream()), "add_rmsnorm")

    def swiglu(self, gu, out):
        _cuda(gu, "gu", torch.float16), _cuda(out, "out", torch.float16)
        if out.numel() % 8 or gu.numel() != 2 * out.numel():
            raise RuntimeError("swiglu: gu must hold 2*I elements, I a multiple of 8")
        _aligned16(gu, "gu"), _aligned16(out, "out")
        self._check(self.lib.b200_swiglu(gu.data_ptr(), out.data_ptr(), out.numel(), _stream()), "swiglu")

    def rope_append(self, qkv, cos_t, sin_t, pos, bt, kc, vc, n_q, n_kv):
        _cuda(qkv, "qkv", torch.float16), _cuda(cos_t, "cos_t", torch.float32), _cuda(sin_t, "sin_t", torch.float32)
        _cuda(kc, "kc", torch.float16), _cuda(vc, "vc", torch.float16)
        _cuda(pos, "pos", torch.int32), _cuda(bt, "bt", torch.int32)
        if qkv.numel() != (n_q + 2 * n_kv) * 64 or cos_t.shape[1] != 32:
            raise RuntimeError("rope_append: head_dim must be 64 (use rope_append_batched for other sizes)")
        self._check(self.lib.b200_rope_append(qkv.data_ptr(), cos_t.data_ptr(), sin_t.data_ptr(), pos.data_ptr(),
                                              bt.data_ptr(), kc.data_ptr(), vc.data_ptr(), int(n_q), int(n_kv),
                                              _ilog2_exact(kc.shape[2], "page size"), _stream()), "rope_append")

    # ---- additions ----------------------------------------------------------------------------------------
    def paged_attention_batched(self, q, kc, vc, bt, pos, part_size, o_part, m_part, l_part, out, version=0):
        """q [B, n_q, D]; bt int32 [B, max_pages]; pos int32 [B]; o_part [B, n_q, S, D]; m/l_part [B, n_q, S];
        out [B, n_q, D]; D = 64 or 128. version: 0 the library's choice, 1..3 as for paged_attention."""
        for t, n in ((q, "q"), (kc, "kc"), (vc, "vc"), (out, "out")):
            _cuda(t, n, torch.float16)
        _cuda(bt, "bt", torch.int32), _cuda(pos, "pos", torch.int32)
        for t, n in ((o_part, "o_part"), (m_part, "m_part"), (l_part, "l_part")):
            _cuda(t, n, torch.float32)
        B, n_q, D = q.shape
        if kc.dim() != 4 or kc.shape[3] != D or vc.shape != kc.shape:
            raise RuntimeError("cache must be [pages, n_kv, P, D]")
        if bt.dim() != 2 or bt.shape[0] != B or pos.numel() != B:
            raise RuntimeError("bt must be [B, max_pages] and pos [B]")
        S = o_part.shape[2]
        if tuple(o_part.shape) != (B, n_q, S, D) or tuple(m_part.shape) != (B, n_q, S) or m_part.shape != l_part.shape:
            raise RuntimeError("split buffers have inconsistent shapes")
        _aligned16(kc, "kc"), _aligned16(vc, "vc")
        self._check(self.lib.b200_paged_attention_batched_v(
            int(version), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), bt.shape[1], pos.data_ptr(), B, n_q,
            kc.shape[1], D, _ilog2_exact(kc.shape[2], "page size"), int(part_size), S, o_part.data_ptr(),
            m_part.data_ptr(), l_part.data_ptr(), out.data_ptr(), _stream()), "paged_attention_batched")

    def rope_paged_attention(self, qkv, cos_t, sin_t, pos, bt, kc, vc, n_q, n_kv, part_size, o_part, m_part, l_part,
                             out, arrive=None):
        """rope_append + paged_attention of one sequence in one partial-kernel launch. qkv fp16 [(n_q + 2 n_kv) D]
        (not modified), caches [pages, n_kv, P, D], o_part fp32 [n_q, S, D], m/l_part [n_q, S], out fp16 [n_q, D].
        arrive: None, or int32 [n_kv] of zeros - the splits are then merged inside the same launch (no combine kernel)."""
        for t_, n_ in ((qkv, "qkv"), (kc, "kc"), (vc, "vc"), (out, "out")):
            _cuda(t_, n_, torch.float16)
        _cuda(cos_t, "cos_t", torch.float32), _cuda(sin_t, "sin_t", torch.float32)
        _cuda(bt, "bt", torch.int32), _cuda(pos, "pos", torch.int32)
        for t_, n_ in ((o_part, "o_part"), (m_part, "m_part"), (l_part, "l_part")):
            _cuda(t_, n_, torch.float32)
        D = kc.shape[3]
        if kc.dim() != 4 or vc.shape != kc.shape or qkv.numel() != (n_q + 2 * n_kv) * D or kc.shape[1] != n_kv:
            raise RuntimeError("rope_paged_attention: inconsistent shapes")
        S = o_part.shape[1]
        if tuple(o_part.shape) != (n_q, S, D) or tuple(m_part.shape) != (n_q, S) or m_part.shape != l_part.shape:
            raise RuntimeError("split buffers have inconsistent shapes")
        if arrive is not None and (_cuda(arrive, "arrive", torch.int32).numel() < n_kv):
            raise RuntimeError("arrive must hold n_kv ints")
        self._check(self.lib.b200_rope_paged_attention(
            qkv.data_ptr(), cos_t.data_ptr(), sin_t.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(),
            pos.data_ptr(), int(n_q), int(n_kv), D, _ilog2_exact(kc.shape[2], "page size"), int(part_size), S,
            o_part.data_ptr(), m_part.data_ptr(), l_part.data_ptr(), out.data_ptr(),
            None if arrive is None else arrive.data_ptr(), _stream()), "rope_paged_attention")

    def paged_attention_status(self):
        """0, or 1 once an attention block gave up a bounded wait for its own copies (outputs invalid). Synchronises."""
        import ctypes
        code = ctypes.c_int(-1)
        self._check(self.lib.b200_paged_attention_status(ctypes.byref(code)), "paged_attention_status")
        return code.value

    # ---- tensor-parallel exchange blocks (see tp.PeerComm for the object that owns them)
    def comm_header_bytes(self):
        return int(self.lib.b200_comm_header_bytes())

    def comm_alloc(self, nbytes):
        p = ctypes.c_void_p()
        self._check(self.lib.b200_comm_alloc(int(nbytes), ctypes.byref(p)), "comm_alloc")
        return p.value

    def comm_free(self, ptr):
        self._check(self.lib.b200_comm_free(ptr), "comm_free")

    def comm_export(self, ptr):
        h = ctypes.create_string_buffer(64)
        self._check(self.lib.b200_comm_export(ptr, h), "comm_export")
        return h.raw

    def comm_import(self, handle):
        p = ctypes.c_void_p()
        self._check(self.lib.b200_comm_import(ctypes.c_char_p(handle), ctypes.byref(p)), "comm_import")
        return p.value

    def comm_unimport(self, ptr):
        self._check(self.lib.b200_comm_unimport(ptr), "comm_unimport")

    def comm_reset(self, base):
        self._check(self.lib.b200_comm_reset(base), "comm_reset")

    def comm_set_wait_limit(self, base, polls):
        """Bound of the exchange kernels' waits for a peer, in polls (0 = default, about four seconds)."""
        self._check(self.lib.b200_comm_set_wait_limit(base, int(polls)), "comm_set_wait_limit")

    def comm_error(self, base):
        code = ctypes.c_int(-1)
        self._check(self.lib.b200_comm_error(base, ctypes.byref(code)), "comm_error")
        return code.value

    def tp_allreduce_add_rmsnorm(self, peers, rank, slot_off, x, w, out, eps):
        """peers: ctypes array of the W block pointers (tp.PeerComm.peers). x, w, out fp16 [H] as add_rmsnorm."""
        _cuda(x, "x", torch.float16), _cuda(w, "w", torch.float16), _cuda(out, "out", torch.float16)
        self._check(self.lib.b200_tp_allreduce_add_rmsnorm(peers, int(rank), len(peers), int(slot_off), x.data_ptr(),
                                                           w.data_ptr(), out.data_ptr(), x.numel(), float(eps),
                                                           _stream()), "tp_allreduce_add_rmsnorm")

    def tp_gemv_slot_bytes(self, N, W):
        """Bytes of the exchange-block region gemv_tiled_allreduce needs for outputs of N rows over W ranks."""
        return int(self.lib.b200_tp_gemv_slot_bytes(int(N), int(W)))

    def gemv_tiled_allreduce(self, tiled, x, y, N, K, peers, rank, slot_off):
        """y[N] = sum over the ranks of (rank's W_r x_r): the row-split GEMV with its all-reduce inside
        (b200_gemv_w4a16_tiled_allreduce). tiled: this rank's column shard in tile layout; y a local fp16 tensor."""
        _cuda(tiled, "tiled", torch.uint8), _cuda(x, "x", torch.float16), _cuda(y, "y", torch.float16)
        if x.numel() != K or y.numel() != N:
            raise RuntimeError("gemv_tiled_allreduce: x must hold K and y N values")
        _aligned16(y, "y")
        self._check(self.lib.b200_gemv_w4a16_tiled_allreduce(tiled.data_ptr(), x.data_ptr(), y.data_ptr(), int(N),
                                                             int(K), peers, int(rank), len(peers), int(slot_off),
                                                             _stream()), "gemv_tiled_allreduce")

    def gemv_tiled_push(self, tiled, x, N, K, peers, rank, slot_off):
        """The row-split GEMV that pushes its partial rows, as tagged words, into every rank's exchange region and
        returns (b200_gemv_w4a16_tiled_push); tp_pushed_add_rmsnorm on every rank consumes them."""
        _cuda(tiled, "tiled", torch.uint8), _cuda(x, "x", torch.float16)
        if x.numel() != K:
            raise RuntimeError("gemv_tiled_push: x must hold K values")
        self._check(self.lib.b200_gemv_w4a16_tiled_push(tiled.data_ptr(), x.data_ptr(), int(N), int(K), peers,
                                                        int(rank), len(peers), int(slot_off), _stream()),
                    "gemv_tiled_push")

    def tp_pushed_add_rmsnorm(self, peers, rank, slot_off, x, w, out, eps):
        """x <- x + (sum over the ranks of the rows pushed into this rank's region), out <- RMSNorm(x) * w."""
        _cuda(x, "x", torch.float16), _cuda(w, "w", torch.float16), _cuda(out, "out", torch.float16)
        self._check(self.lib.b200_tp_pushed_add_rmsnorm(peers, int(rank), len(peers), int(slot_off), x.data_ptr(),
                                                        w.data_ptr(), out.data_ptr(), x.numel(), float(eps),
                                                        _stream()), "tp_pushed_add_rmsnorm")

    def tp_allgather(self, peers, rank, slot_off, dst, n):
        _cuda(dst, "dst", torch.float16)
        if dst.numel() != n * len(peers):
            raise RuntimeError("tp_allgather: dst must hold W shards of n values")
        self._check(self.lib.b200_tp_allgather(peers, int(rank), len(peers), int(slot_off), dst.data_ptr(), int(n),
                                               _stream()), "tp_allgather")

    def paged_attention_noalloc(self, q, kc, vc, bt, pos, part_size, max_splits, out):
        """paged_attention without caller scratch, for callers that cannot allocate: the split-K partials live in a
        fixed ~1 MB array inside the library (n_q <= 64, max_splits <= 32, one sequence, head_dim 64 or 128). Calls on
        one device share that array and must not overlap; make the first call before any stream capture."""
        for t, n in ((q, "q"), (kc, "kc"), (vc, "vc"), (out, "out")):
            _cuda(t, n, torch.float16)
        _cuda(bt, "bt", torch.int32), _cuda(pos, "pos", torch.int32)
        if kc.dim() != 4 or vc.shape != kc.shape:
            raise RuntimeError("cache must be [pages, n_kv, P, D]")
        D, n_kv = kc.shape[3], kc.shape[1]
        if q.numel() % D or out.shape != q.shape:
            raise RuntimeError("q must hold n_q * D values and out have q's shape")
        n_q = q.numel() // D
        if n_q % n_kv or n_q // n_kv not in (1, 2, 4, 8):
            raise RuntimeError("heads-per-group must be 1/2/4/8")
        if part_size <= 0 or max_splits <= 0 or pos.numel() != 1:
            raise RuntimeError("part_size and max_splits must be > 0 and pos hold one position")
        if bt.numel() * kc.shape[2] < min(part_size * max_splits, kc.shape[0] * kc.shape[2]):
            raise RuntimeError("bt does not cover the pages of max_splits * part_size tokens")
        _aligned16(kc, "kc"), _aligned16(vc, "vc")
        self._check(self.lib.b200_paged_attention_noalloc(
            q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), pos.data_ptr(), q.numel() // D, kc.shape[1], D,
            _ilog2_exact(kc.shape[2], "page size"), int(part_size), int(max_splits), out.data_ptr(), _stream()),
            "paged_attention_noalloc")

    def rope_append_batched(self, qkv, cos_t, sin_t, pos, bt, kc, vc, n_q, n_kv):
        """qkv [B, (n_q + 2 n_kv) * D]; bt int32 [B, max_pages]; pos int32 [B]; D = 2 * cos_t.shape[1]."""
        _cuda(qkv, "qkv", torch.float16), _cuda(cos_t, "cos_t", torch.float32), _cuda(sin_t, "sin_t", torch.float32)
        _cuda(kc, "kc", torch.float16), _cuda(vc, "vc", torch.float16)
        _cuda(pos, "pos", torch.int32), _cuda(bt, "bt", torch.int32)
        B, D = qkv.shape[0], 2 * cos_t.shape[1]
        if qkv.dim() != 2 or qkv.shape[1] != (n_q + 2 * n_kv) * D or kc.shape[3] != D or bt.shape[0] != B:
            raise RuntimeError("rope_append_batched: inconsistent shapes")
        self._check(self.lib.b200_rope_append_batched(
            qkv.data_ptr(), cos_t.data_ptr(), sin_t.data_ptr(), pos.data_ptr(), bt.data_ptr(), bt.shape[1],
            kc.data_ptr(), vc.data_ptr(), B, int(n_q), int(n_kv), D, _ilog2_exact(kc.shape[2], "page size"),
            _stream()), "rope_append_batched")

    def dequant_w4a16(self, packed, sz, out, group):
        _cuda(packed, "packed", torch.int32), _cuda(sz, "sz", torch.float16), _cuda(out, "out", torch.float16)
        N, K = packed.shape[0], packed.shape[1] * 8
        if tuple(out.shape) != (N, K) or K % group:
            raise RuntimeError("dequant_w4a16: inconsistent shapes")
        self._check(self.lib.b200_dequant_w4a16(packed.data_ptr(), sz.data_ptr(), out.data_ptr(), N, K,
                                                _ilog2_exact(int(group), "group"), _stream()), "dequant_w4a16")

    # ---- the prompt: T tokens at once --------------------------------------------------------------------
    def gemm_w4a16(self, packed, sz, x, y, group):
        """y[T, N] = x[T, K] @ dequant(packed, sz)^T on the tcgen05 tensor cores. packed int32 [N, K/8], sz fp16
        [N, K/group, 2], x fp16 [T, K], y fp16 [T, N]; K % 64 == 0, group >= 64, T <= gemm_max_tokens()."""
        _cuda(packed, "packed", torch.int32), _cuda(sz, "sz", torch.float16)
        _cuda(x, "x", torch.float16), _cuda(y, "y", torch.float16)
        N, K = packed.shape[0], packed.shape[1] * 8
        if x.dim() != 2 or x.shape[1] != K or tuple(y.shape) != (x.shape[0], N) or K % group:
            raise RuntimeError("gemm_w4a16: inconsistent shapes")
        if tuple(sz.shape) != (N, K // group, 2):
            raise RuntimeError("gemm_w4a16: sz must be [N, K/group, 2]")
        self._check(self.lib.b200_gemm_w4a16(packed.data_ptr(), sz.data_ptr(), x.data_ptr(), y.data_ptr(), x.shape[0],
                                             N, K, _ilog2_exact(int(group), "group"), _stream()), "gemm_w4a16")

    def gemm_max_tokens(self):
        return int(self.lib.b200_gemm_w4a16_max_tokens())

    def gemm_status(self):
        """0, or 1 once a bounded wait inside the GEMM kernel ran out (synchronizes the device)."""
        code = c_int(-1)
        self._check(self.lib.b200_gemm_w4a16_status(ctypes.byref(code)), "gemm_w4a16_status")
        return code.value

    def add_rmsnorm_batched(self, x, delta, w, out, eps):
        """Row-wise add_rmsnorm over x [T, H] (delta [T, H] or None, w [H], out [T, H])."""
        _cuda(x, "x", torch.float16), _cuda(w, "w", torch.float16), _cuda(out, "out", torch.float16)
        if delta is not None:
            _cuda(delta, "delta", torch.float16)
        T, H = x.shape
        if w.numel() != H or tuple(out.shape) != (T, H) or (delta is not None and tuple(delta.shape) != (T, H)):
            raise RuntimeError("add_rmsnorm_batched: inconsistent shapes")
        self._check(self.lib.b200_add_rmsnorm_batched(x.data_ptr(), None if delta is None else delta.data_ptr(),
                                                      w.data_ptr(), out.data_ptr(), T, H, float(eps), _stream()),
                    "add_rmsnorm_batched")

    def swiglu_batched(self, gu, out):
        """out[t] = silu(gu[t, :I]) * gu[t, I:] for gu [T, 2I], out [T, I]."""
        _cuda(gu, "gu", torch.float16), _cuda(out, "out", torch.float16)
        T, I = out.shape
        if tuple(gu.shape) != (T, 2 * I):
            raise RuntimeError("swiglu_batched: gu must be [T, 2I] and out [T, I]")
        self._check(self.lib.b200_swiglu_batched(gu.data_ptr(), out.data_ptr(), T, I, _stream()), "swiglu_batched")

    def embed_row(self, emb, tok, x):
        _cuda(emb, "emb", torch.float16), _cuda(tok, "tok", torch.int64), _cuda(x, "x", torch.float16)
        if emb.dim() != 2 or emb.shape[1] != x.numel():
            raise RuntimeError("embed_row: emb must be [V, H] and x [H]")
        self._check(self.lib.b200_embed_row(emb.data_ptr(), tok.data_ptr(), x.data_ptr(), x.numel(), emb.shape[0],
                                            _stream()), "embed_row")

    def argmax(self, logits, tok, pos=None, history=None):
        """tok <- argmax(logits), lowest index on ties; with pos: history[pos] <- tok (if given), pos += 1."""
        _cuda(logits, "logits", torch.float16), _cuda(tok, "tok", torch.int64)
        p = _cuda(pos, "pos", torch.int32).data_ptr() if pos is not None else 0
        h = _cuda(history, "history", torch.int64).data_ptr() if history is not None else 0
        self._check(self.lib.b200_argmax(logits.data_ptr(), logits.numel(), tok.data_ptr(), p, h, _stream()),
                    "argmax")


    def decode_step_xchg_bytes(self, L, H, I, n_q, n_kv, D, grid):
        return int(self.lib.b200_decode_step_xchg_bytes(L, H, I, n_q, n_kv, D, grid))

    def decode_step(self, desc: "StepDesc"):
        """One whole decode step as one persistent kernel (b200_decode_step) on the current stream."""
        self._check(self.lib.b200_decode_step(ctypes.byref(desc), _stream()), "decode_step")


def load(verbose=False):
    """Return the operator set (reference runtime/ext.py:9). Raises if the library cannot be loaded."""
    global _OPS
    if _OPS is None:
        _OPS = Ops(load_library())
    return _OPS
