"""CPU oracle for the group-wise INT4 weight format (numpy). TEST INFRASTRUCTURE ONLY.

This file restates, in numpy, the arithmetic of the reference quantizer so that the product's own
quantizer and the CUDA dequant/GEMV kernels can be checked against an independent implementation.
It is imported by tests, by the smoke check and by the CPU-baseline leg of the benchmark, never by
the product path.

Parity status: PINNED. Every function here is compared bit-for-bit with the reference's
runtime/quant.py through the committed fixtures in tests/golden/ (produced by
tests/golden/make_golden.py, which imports the reference), and with the known-answer vectors of the
reference's tests/test_quant_local.py (pack([0..7]) == 0x75316420, magic-number extraction).

Rounding contract restated (reference runtime/quant.py:20-48, :93-124):
  scale = fp16( max((max - min) / 15, 1e-6) )      rounded to fp16 BEFORE it is used
  zero  = clamp(round_half_even(-min / scale), 0, 15)
  q     = clamp(round_half_even(w / scale) + zero, 0, 15)
  w_hat = fp16( (q - zero) * scale )               computed in fp32, one rounding
  word j of a row holds elements 8j..8j+7: element 8j+2i in bits [4i, 4i+4), element 8j+2i+1 in
  bits [16+4i, 16+4i+4); the word is stored as a signed int32.
"""
import numpy as np

# Range-shrink factors tried when clip=True (reference runtime/quant.py:17).
CLIP_GRID = (1.0, 0.95, 0.9, 0.85, 0.8, 0.75, 0.7)

_F32 = np.float32


def _round_clamp_q(wf, scale, zero):
    return np.clip(np.round(wf / scale) + zero, _F32(0), _F32(15)).astype(_F32)


def group_params(wf, clip=False):
    """wf float32 [..., G] -> (scale, zero) float32 [..., 1].

    Follows reference runtime/quant.py:20-39. With clip=True each candidate factor shrinks both
    ends of the range; a later candidate replaces the kept one only when its squared error is
    strictly smaller (the `err < best` rule at :36)."""
    wf = np.asarray(wf, dtype=_F32)
    lo0 = wf.min(axis=-1, keepdims=True)
    hi0 = wf.max(axis=-1, keepdims=True)
    kept = None
    for a in (CLIP_GRID if clip else (1.0,)):
        lo, hi = lo0 * _F32(a), hi0 * _F32(a)
        scale = np.maximum((hi - lo) / _F32(15), _F32(1e-6)).astype(np.float16).astype(_F32)
        zero = np.clip(np.round(-lo / scale), _F32(0), _F32(15)).astype(_F32)
        if not clip:
            return scale, zero
        deq = (_round_clamp_q(wf, scale, zero) - zero) * scale
        err = np.square(deq - wf, dtype=_F32).sum(axis=-1, keepdims=True, dtype=_F32)
        if kept is None:
            kept = [err, scale, zero]
        else:
            better = err < kept[0]
            kept = [np.where(better, err, kept[0]), np.where(better, scale, kept[1]),
                    np.where(better, zero, kept[2])]
    return kept[1], kept[2]


def quantize(w, group, clip=False):
    """fp16/fp32 [N, K] -> (q uint8 [N, K], scale fp16 [N, K/G], zero fp16 [N, K/G]).
    Reference runtime/quant.py:42-48."""
    w = np.asarray(w)
    n, k = w.shape
    if k % group:
        raise ValueError(f"K={k} is not a multiple of group={group}")
    wf = w.astype(_F32).reshape(n, k // group, group)
    scale, zero = group_params(wf, clip)
    q = _round_clamp_q(wf, scale, zero)
    return (q.reshape(n, k).astype(np.uint8), scale.reshape(n, -1).astype(np.float16),
            zero.reshape(n, -1).astype(np.float16))


def dequantize(q, scale, zero, group):
    """(q, scale, zero) -> fp16 [N, K], one rounding. Reference runtime/quant.py:93-97."""
    n, k = q.shape
    qf = q.astype(_F32).reshape(n, k // group, group)
    w = (qf - zero.astype(_F32)[..., None]) * scale.astype(_F32)[..., None]
    return w.reshape(n, k).astype(np.float16)


def pack(q):
    """uint8 nibbles [N, K] -> int32 words [N, K/8]. Reference runtime/quant.py:100-109."""
    n, k = q.shape
    if k % 8:
        raise ValueError("K must be a multiple of 8")
    v = q.astype(np.uint32).reshape(n, k // 8, 8)
    word = np.zeros((n, k // 8), dtype=np.uint32)
    for e in range(8):
        shift = 4 * (e // 2) + 16 * (e % 2)
        word |= v[..., e] << np.uint32(shift)
    return word.view(np.int32)


def unpack(packed):
    """int32 words [N, K/8] -> uint8 nibbles [N, K]. Reference runtime/quant.py:112-119."""
    word = np.ascontiguousarray(packed).view(np.uint32)
    n, w = word.shape
    out = np.empty((n, w, 8), dtype=np.uint8)
    for e in range(8):
        shift = 4 * (e // 2) + 16 * (e % 2)
        out[..., e] = ((word >> np.uint32(shift)) & np.uint32(0xF)).astype(np.uint8)
    return out.reshape(n, w * 8)


def pack_scale_zero(scale, zero):
    """[N, K/G] scale and zero -> [N, K/G, 2] fp16 with (scale, zero) adjacent.
    Reference runtime/quant.py:122-124."""
    return np.ascontiguousarray(np.stack([scale, zero], axis=-1).astype(np.float16))


def magic_pairs(word):
    """The four (even, odd) nibble pairs a kernel recovers from one packed word with
    (word >> 4i) & 0x000F000F. Known answer from the reference's tests/test_quant_local.py:12-20:
    word 0x75316420 -> [(0,1),(2,3),(4,5),(6,7)]."""
    word = int(word) & 0xFFFFFFFF
    pairs = []
    for i in range(4):
        t = (word >> (4 * i)) & 0x000F000F
        pairs.append((t & 0xFFFF, t >> 16))
    return pairs


def quantize_gptq(w, H, group, clip=False, damp=0.01, block=128):
    """GPTQ without activation reordering, same output format as quantize().

    Follows reference runtime/quant.py:51-90: dead Hessian columns are zeroed, the diagonal is
    damped by `damp` times its mean, the upper Cholesky factor of the inverse Hessian drives a
    column-by-column error feedback inside blocks of `block` columns, and a group's (scale, zero)
    are taken from the error-updated weights when the group starts. float64 linear algebra is
    NOT used: the reference works in fp32, and so does this."""
    w = np.asarray(w)
    n, k = w.shape
    if k % group or block % group:
        raise ValueError("K and block must be multiples of group")
    W = w.astype(_F32).copy()
    H = np.asarray(H, dtype=_F32).copy()
    d = np.diag(H).copy()
    dead = d == 0
    H[dead, dead] = 1
    W[:, dead] = 0
    H += _F32(damp) * np.diag(H).mean(dtype=_F32) * np.eye(k, dtype=_F32)
    L = np.linalg.cholesky(H.astype(np.float64)).astype(_F32)
    Linv = np.linalg.inv(L.astype(np.float64))
    Hinv_full = (Linv.T @ Linv).astype(_F32)
    U = np.linalg.cholesky(Hinv_full.astype(np.float64)).T.astype(_F32)  # upper factor
    Q = np.zeros((n, k), dtype=np.uint8)
    S = np.zeros((n, k // group), dtype=_F32)
    Z = np.zeros((n, k // group), dtype=_F32)
    scale = zero = None
    for b0 in range(0, k, block):
        b1 = min(b0 + block, k)
        Wb = W[:, b0:b1].copy()
        Eb = np.zeros_like(Wb)
        Ub = U[b0:b1, b0:b1]
        for i in range(b1 - b0):
            c = b0 + i
            if c % group == 0:
                s, z = group_params(Wb[:, i:i + group], clip)
                S[:, c // group], Z[:, c // group] = s[:, 0], z[:, 0]
                scale, zero = s[:, 0], z[:, 0]
            col = Wb[:, i]
            qc = np.clip(np.round(col / scale) + zero, 0, 15).astype(_F32)
            Q[:, c] = qc.astype(np.uint8)
            e = (col - (qc - zero) * scale) / Ub[i, i]
            Wb[:, i:] -= e[:, None] * Ub[i, i:][None, :]
            Eb[:, i] = e
        W[:, b1:] -= Eb @ U[b0:b1, b1:]
    return Q, S.astype(np.float16), Z.astype(np.float16)


class QuantLinear:
    """One quantized matrix in kernel format plus its fp16 dequantized copy.
    Reference runtime/quant.py:127-140."""

    def __init__(self, w, group, keep_ref=True, clip=False, qsz=None):
        self.N, self.K = w.shape
        self.group = group
        q, s, z = qsz if qsz is not None else quantize(w, group, clip)
        self.packed = pack(np.asarray(q))
        self.sz = pack_scale_zero(np.asarray(s), np.asarray(z))
        self.w_ref = dequantize(np.asarray(q), np.asarray(s), np.asarray(z), group) if keep_ref else None

    def nbytes(self):
        return self.packed.size * 4 + self.sz.size * 2
