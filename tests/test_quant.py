"""Host-side weight format of the product (llm_decode_kernels_b200/quant.py): bit-exact against
outputs stored from the reference and against the independent numpy oracle."""
import numpy as np
import pytest
import torch

from llm_decode_kernels_b200 import quant as PQ
from oracle import quant_oracle as Q

T = torch.from_numpy
bits = lambda t: t.numpy().view(np.uint16)


def test_api_names():
    for name in ("quantize", "quantize_gptq", "dequantize", "pack", "unpack", "pack_scale_zero", "group_params",
                 "QuantLinear", "CLIP_GRID"):
        assert hasattr(PQ, name)
    assert PQ.CLIP_GRID == Q.CLIP_GRID


def test_hand_packed_word():
    w = PQ.pack(torch.arange(8, dtype=torch.uint8)[None])
    assert (int(w[0, 0]) & 0xFFFFFFFF) == 0x75316420
    assert w.dtype == torch.int32


def test_roundtrip():
    torch.manual_seed(0)
    q = torch.randint(0, 16, (64, 2048), dtype=torch.uint8)
    assert torch.equal(PQ.unpack(PQ.pack(q)), q)
    assert np.array_equal(PQ.pack(q).numpy(), Q.pack(q.numpy()))


@pytest.mark.parametrize("G", [64, 128, 256])
@pytest.mark.parametrize("clip", [False, True])
def test_quantize_golden(golden, G, clip):
    g = golden("quant")
    tag = f"g{G}_{'clip' if clip else 'rtn'}"
    q, s, z = PQ.quantize(T(g["w"]), G, clip)
    assert np.array_equal(q.numpy(), g[f"q_{tag}"])
    assert np.array_equal(bits(s), g[f"s_{tag}"].view(np.uint16))
    assert np.array_equal(bits(z), g[f"z_{tag}"].view(np.uint16))
    assert np.array_equal(PQ.pack(q).numpy(), g[f"packed_{tag}"])
    assert np.array_equal(bits(PQ.pack_scale_zero(s, z)), g[f"sz_{tag}"].view(np.uint16))
    assert np.array_equal(bits(PQ.dequantize(q, s, z, G)), g[f"deq_{tag}"].view(np.uint16))
    ql = PQ.QuantLinear(T(g["w"]), G, clip=clip)
    assert np.array_equal(ql.packed.numpy(), g[f"packed_{tag}"])
    assert np.array_equal(bits(ql.w_ref), g[f"deq_{tag}"].view(np.uint16))
    assert ql.nbytes() == ql.packed.numel() * 4 + ql.sz.numel() * 2


@pytest.mark.parametrize("clip", [False, True])
def test_product_equals_oracle_on_fresh_data(clip):
    torch.manual_seed(5)
    w = (torch.randn(48, 1024) * 0.02).half()
    w[7, 256:384] = 0
    for G in (64, 128):
        q, s, z = PQ.quantize(w, G, clip)
        qo, so, zo = Q.quantize(w.numpy(), G, clip)
        assert np.array_equal(q.numpy(), qo) and np.array_equal(bits(s), so.view(np.uint16))
        assert np.array_equal(bits(z), zo.view(np.uint16))


@pytest.mark.parametrize("clip", [False, True])
def test_gptq_golden(golden, clip):
    """Same torch calls as the reference on the same machine class: the stored result is
    reproduced exactly up to LAPACK kernel differences, so allow a vanishing mismatch rate."""
    g = golden("gptq")
    tag = "clip" if clip else "plain"
    q, s, z = PQ.quantize_gptq(T(g["w"]), T(g["H"]), 64, clip=clip, block=128)
    assert (q.numpy() != g[f"q_{tag}"]).mean() < 2e-3
    assert q.dtype == torch.uint8 and int(q.max()) <= 15
    zf = z.float()
    assert torch.equal(zf, zf.round()) and float(zf.min()) >= 0 and float(zf.max()) <= 15


def test_clip_and_gptq_beat_rtn():
    # property test of reference tests/test_quant_local.py:41-60
    torch.manual_seed(0)
    N, K, G = 128, 512, 128
    w = torch.randn(N, K) * 0.02
    w[torch.rand(N, K) < 0.002] *= 8
    w = w.half()
    X = torch.randn(4096, 64) @ torch.randn(64, K)
    X[:, :8] *= 10
    H = 2 * X.t() @ X / X.shape[0]
    out_err = lambda q, s, z: (X @ (PQ.dequantize(q, s, z, G).float() - w.float()).t()).pow(2).mean().item()
    w_err = lambda q, s, z: (PQ.dequantize(q, s, z, G).float() - w.float()).pow(2).mean().item()
    rtn, clip = PQ.quantize(w, G), PQ.quantize(w, G, clip=True)
    gptq = PQ.quantize_gptq(w, H, G)
    assert w_err(*clip) < w_err(*rtn)
    assert out_err(*gptq) < 0.7 * out_err(*rtn)
