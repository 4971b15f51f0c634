"""Group-wise asymmetric INT4 weight format (RTN, range-clipped, GPTQ) and its nibble packing.

Host-side half of the W4A16 path: it produces exactly the tensors the CUDA GEMV streams. The public
names and signatures are those of the reference's runtime/quant.py (quantize, quantize_gptq,
dequantize, pack, unpack, pack_scale_zero, group_params, QuantLinear, CLIP_GRID) so code written
against that module runs unchanged; results are bit-identical to it (tests/test_quant.py checks
this against stored outputs of the reference).

Format, for a weight W [N, K] (out x in) and group size G along K:
    scale [N, K/G] fp16   = max((max - min) / 15, 1e-6), rounded to fp16 before it is used
    zero  [N, K/G] fp16   = integer in [0, 15] = round(-min / scale)
    q     [N, K]   uint8  = clamp(round(w / scale) + zero, 0, 15)
    packed [N, K/8] int32 : word j = elements 8j..8j+7; element 8j+2i sits in bits [4i, 4i+4) and
                            element 8j+2i+1 in bits [16+4i, 16+4i+4)
    sz    [N, K/G, 2] fp16: (scale, zero) adjacent, read by kernels as one half2
The bit layout lets a kernel turn `(word >> 4i) & 0x000F000F | 0x64006400` into the half2
(1024 + q[8j+2i], 1024 + q[8j+2i+1]) with no integer-to-float conversion.

All functions run on the device of their input (torch ops). Quantization is offline work; the
decode step itself never calls into this file.
"""
import torch

CLIP_GRID = (1.0, 0.95, 0.9, 0.85, 0.8, 0.75, 0.7)

# bit position of element e (0..7) inside its 32-bit word
_SHIFTS = tuple(4 * (e >> 1) + 16 * (e & 1) for e in range(8))


def _levels(wf, scale, zero):
    return (torch.round(wf / scale) + zero).clamp_(0, 15)


def group_params(wf, clip=False):
    """wf fp32 [..., G] -> (scale, zero) fp32 [..., 1]; scale is fp16-representable, zero integral.

    clip=True evaluates every factor of CLIP_GRID (shrinking both ends of the range) and keeps,
    per group, the first one with the strictly smallest squared rounding error."""
    lo0 = wf.amin(dim=-1, keepdim=True)
    hi0 = wf.amax(dim=-1, keepdim=True)
    factors = CLIP_GRID if clip else (1.0,)
    best_err = best_scale = best_zero = None
    for a in factors:
        lo, hi = lo0 * a, hi0 * a
        scale = ((hi - lo) / 15).clamp(min=1e-6).to(torch.float16).to(torch.float32)
        zero = torch.round(-lo / scale).clamp(0, 15)
        if not clip:
            return scale, zero
        err = (((_levels(wf, scale, zero) - zero) * scale - wf) ** 2).sum(dim=-1, keepdim=True)
        if best_err is None:
            best_err, best_scale, best_zero = err, scale, zero
        else:
            take = err < best_err
            best_err = torch.where(take, err, best_err)
            best_scale = torch.where(take, scale, best_scale)
            best_zero = torch.where(take, zero, best_zero)
    return best_scale, best_zero


def quantize(w: torch.Tensor, group: int, clip: bool = False):
    """[N, K] -> (q uint8 [N, K], scale fp16 [N, K/G], zero fp16 [N, K/G])."""
    N, K = w.shape
    assert K % group == 0, (K, group)
    wf = w.to(torch.float32).reshape(N, K // group, group)
    scale, zero = group_params(wf, clip)
    q = _levels(wf, scale, zero)
    return (q.reshape(N, K).to(torch.uint8), scale.reshape(N, -1).to(torch.float16),
            zero.reshape(N, -1).to(torch.float16))


@torch.no_grad()
def quantize_gptq(w: torch.Tensor, H: torch.Tensor, group: int, clip: bool = False, damp: float = 0.01,
                  block: int = 128):
    """GPTQ (Frantar et al. 2022), no activation reordering, into the same format as quantize().

    H is the layer-input Hessian 2 X^T X / tokens, [K, K]. Columns are fixed left to right; each
    column's rounding error is pushed onto the columns not yet fixed through the upper Cholesky
    factor of H^-1, inside blocks of `block` columns and then onto the rest of the matrix. A group's
    (scale, zero) come from the error-updated weights at the moment the group starts, so groups
    stay contiguous and the GEMV kernel needs no permutation."""
    N, K = w.shape
    assert K % group == 0 and block % group == 0
    W = w.to(torch.float32).clone()
    H = H.to(torch.float32).clone()
    diag = torch.diagonal(H)
    dead = diag == 0
    diag[dead] = 1
    W[:, dead] = 0
    diag += damp * diag.mean()
    U = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(H)), upper=True)
    Q = torch.zeros(N, K, dtype=torch.uint8, device=W.device)
    S = torch.zeros(N, K // group, device=W.device)
    Z = torch.zeros(N, K // group, device=W.device)
    scale = zero = None
    for b0 in range(0, K, block):
        b1 = min(b0 + block, K)
        Wb = W[:, b0:b1].clone()
        Eb = torch.zeros_like(Wb)
        Ub = U[b0:b1, b0:b1]
        for i in range(b1 - b0):
            c = b0 + i
            if c % group == 0:
                s, z = group_params(Wb[:, i:i + group], clip)
                scale, zero = s[:, 0], z[:, 0]
                S[:, c // group], Z[:, c // group] = scale, zero
            col = Wb[:, i]
            qc = (torch.round(col / scale) + zero).clamp(0, 15)
            Q[:, c] = qc.to(torch.uint8)
            e = (col - (qc - zero) * scale) / Ub[i, i]
            Wb[:, i:] -= e[:, None] * Ub[i, i:][None, :]
            Eb[:, i] = e
        W[:, b1:] -= Eb @ U[b0:b1, b1:]
    return Q, S.to(torch.float16), Z.to(torch.float16)


def dequantize(q, scale, zero, group: int):
    """fp16 [N, K] = half((q - zero) * scale), the product formed in fp32 and rounded once. The
    CUDA kernels' per-element weight (hsub2 then hmul2 on fp16) equals this bit for bit."""
    N, K = q.shape
    lv = q.to(torch.float32).reshape(N, K // group, group)
    w = (lv - zero.to(torch.float32)[..., None]) * scale.to(torch.float32)[..., None]
    return w.reshape(N, K).to(torch.float16)


def pack(q: torch.Tensor) -> torch.Tensor:
    """uint8 [N, K] nibbles -> int32 [N, K/8] words (signed storage of the 32-bit pattern)."""
    N, K = q.shape
    assert K % 8 == 0
    sh = torch.tensor(_SHIFTS, dtype=torch.int64, device=q.device)
    word = (q.to(torch.int64).reshape(N, K // 8, 8) << sh).sum(dim=-1)   # fields do not overlap
    word = word - ((word >> 31) << 32)                                    # two's complement fold
    return word.to(torch.int32).contiguous()


def unpack(packed: torch.Tensor) -> torch.Tensor:
    """int32 [N, K/8] -> uint8 [N, K]."""
    N, Wd = packed.shape
    sh = torch.tensor(_SHIFTS, dtype=torch.int64, device=packed.device)
    word = packed.to(torch.int64) & 0xFFFFFFFF
    return ((word[..., None] >> sh) & 0xF).to(torch.uint8).reshape(N, Wd * 8)


def pack_scale_zero(scale, zero):
    """[N, K/G] scale and zero -> [N, K/G, 2] fp16, one half2 (scale, zero) per group."""
    return torch.stack([scale, zero], dim=-1).contiguous()


class QuantLinear:
    """One quantized matrix in kernel format, optionally with its fp16 dequantized copy."""

    def __init__(self, w: torch.Tensor, group: int, keep_ref: bool = True, clip: bool = False, qsz=None):
        """qsz: precomputed (q, scale, zero), e.g. from quantize_gptq; otherwise RTN (clip: with
        per-group range clipping)."""
        self.N, self.K = w.shape
        self.group = group
        if qsz is not None:
            q, s, z = (t.to(w.device) for t in qsz)
        else:
            q, s, z = quantize(w, group, clip)
        self.packed = pack(q)
        self.sz = pack_scale_zero(s, z)
        self.w_ref = dequantize(q, s, z, group) if keep_ref else None

    def nbytes(self):
        return self.packed.numel() * 4 + self.sz.numel() * 2
