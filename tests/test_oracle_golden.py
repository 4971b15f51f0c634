"""Pins the CPU oracle (oracle/*.py) to outputs stored from the reference implementation.

Every comparison is exact (zero difference) unless stated: the oracle restates the reference's
arithmetic with the same rounding points, so on the same inputs it must give the same bits."""
import types

import numpy as np
import pytest
import torch

from oracle import model_oracle as MO
from oracle import ops_oracle as R
from oracle import quant_oracle as Q

T = torch.from_numpy


def test_pack_known_answer():
    # reference tests/test_quant_local.py:12-20
    word = Q.pack(np.arange(8, dtype=np.uint8)[None])
    assert (int(word[0, 0]) & 0xFFFFFFFF) == 0x75316420
    assert Q.magic_pairs(word[0, 0]) == [(0, 1), (2, 3), (4, 5), (6, 7)]


def test_pack_golden(golden):
    g = golden("quant")
    assert np.array_equal(Q.pack(g["kat_q"]), g["kat_packed"])
    assert np.array_equal(Q.unpack(g["kat_packed"]), g["kat_q"])
    assert np.array_equal(Q.pack(np.arange(8, dtype=np.uint8)[None]), g["kat_word_0to7"])


@pytest.mark.parametrize("G", [64, 128, 256])
@pytest.mark.parametrize("clip", [False, True])
def test_quantize_golden(golden, G, clip):
    g = golden("quant")
    tag = f"g{G}_{'clip' if clip else 'rtn'}"
    q, s, z = Q.quantize(g["w"], G, clip)
    assert np.array_equal(q, g[f"q_{tag}"])
    assert np.array_equal(s.view(np.uint16), g[f"s_{tag}"].view(np.uint16))
    assert np.array_equal(z.view(np.uint16), g[f"z_{tag}"].view(np.uint16))
    assert np.array_equal(Q.pack(q), g[f"packed_{tag}"])
    assert np.array_equal(Q.pack_scale_zero(s, z).view(np.uint16), g[f"sz_{tag}"].view(np.uint16))
    assert np.array_equal(Q.dequantize(q, s, z, G).view(np.uint16), g[f"deq_{tag}"].view(np.uint16))
    # integer zero in [0, 15] (reference tests/test_quant_local.py:57-59)
    zf = z.astype(np.float32)
    assert np.array_equal(zf, np.round(zf)) and zf.min() >= 0 and zf.max() <= 15


def test_rtn_error_bound():
    # reference tests/test_quant_local.py:29-38
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((64, 1024)) * 0.02).astype(np.float16)
    for G in (64, 128, 256):
        q, s, z = Q.quantize(w, G)
        err = np.abs(Q.dequantize(q, s, z, G).astype(np.float32) - w.astype(np.float32)).reshape(64, -1, G)
        bound = s.astype(np.float32)[..., None] * 0.5 + 2e-3 * np.abs(w.astype(np.float32)).max()
        assert (err <= bound + 1e-6).all()


@pytest.mark.parametrize("clip", [False, True])
def test_gptq_golden(golden, clip):
    """The oracle's GPTQ uses float64 factorisations where the reference uses fp32 LAPACK calls, so
    a few levels may differ by one step; the stored result must be matched almost everywhere and the
    layer-output error must be as good."""
    g = golden("gptq")
    tag = "clip" if clip else "plain"
    q, s, z = Q.quantize_gptq(g["w"], g["H"], 64, clip=clip, block=128)
    assert (q != g[f"q_{tag}"]).mean() < 0.02
    assert (np.abs(q.astype(int) - g[f"q_{tag}"].astype(int)) <= 1).mean() > 0.999
    Hm, w = g["H"].astype(np.float64), g["w"].astype(np.float64)

    def out_err(q, s, z):
        dw = Q.dequantize(q, s, z, 64).astype(np.float64) - w
        return np.einsum("nk,kj,nj->", dw, Hm, dw)
    assert out_err(q, s, z) < 1.05 * out_err(g[f"q_{tag}"], g[f"s_{tag}"], g[f"z_{tag}"])
    rq, rs, rz = Q.quantize(g["w"], 64, clip)
    assert out_err(q, s, z) < 0.9 * out_err(rq, rs, rz)


def test_ops_golden(golden):
    g = golden("ops")
    eq = lambda a, b: np.array_equal(a.numpy().view(np.uint16), b.view(np.uint16))
    assert eq(R.gemv_ref(T(g["gemv_wref"]), T(g["gemv_x"])), g["gemv_y"])
    x, out = R.add_rmsnorm_ref(T(g["norm_x"]), T(g["norm_delta"]), T(g["norm_w"]), 1e-5)
    assert eq(x, g["norm_xout"]) and eq(out, g["norm_out"])
    assert eq(R.add_rmsnorm_ref(T(g["norm_x"]), None, T(g["norm_w"]), 1e-5)[1], g["norm_out_nodelta"])
    assert eq(R.swiglu_ref(T(g["swiglu_gu"])), g["swiglu_out"])
    for D in (64, 128):
        cos, sin = R.rope_tables(300, D)
        assert np.array_equal(cos.numpy(), g[f"rope_cos_d{D}"]) and np.array_equal(sin.numpy(), g[f"rope_sin_d{D}"])
        kc, vc = T(g[f"ra_kc_d{D}"].copy()), T(g[f"ra_vc_d{D}"].copy())
        bt = T(g[f"ra_bt_d{D}"])
        q = R.rope_append_ref(T(g[f"ra_qkv_d{D}"].copy()), cos, sin, 37, kc, vc, bt, 8, 2, D, 16)
        assert eq(q, g[f"ra_q_out_d{D}"]) and eq(kc, g[f"ra_kc_out_d{D}"]) and eq(vc, g[f"ra_vc_out_d{D}"])
        kc, vc = T(g[f"ra_kc_d{D}"]), T(g[f"ra_vc_d{D}"])
        qa = T(g[f"attn_q_d{D}"])
        assert eq(R.paged_attention_ref(qa, kc, vc, bt, 70, 16), g[f"attn_out_d{D}"])
        k, v = R.gather_kv(kc, vc, bt, 70, 16)
        assert eq(k, g[f"attn_gk_d{D}"]) and eq(v, g[f"attn_gv_d{D}"])
        assert eq(R.split_softmax_combine_ref(qa, k, v, 16), g[f"attn_split_d{D}"])
        # reference tests/test_ref_local.py:18-24: token 37 lives in logical page 2, slot 5
        assert torch.equal(k[37], kc[bt[2], :, 5]) and torch.equal(v[37], vc[bt[2], :, 5])


def test_split_combine_equals_softmax():
    # reference tests/test_ref_local.py:7-16
    torch.manual_seed(0)
    for ctx in (1, 17, 128, 1000):
        for scale in (1.0, 8.0):
            q, k = torch.randn(32, 64).half(), (torch.randn(ctx, 4, 64) * scale).half()
            v = torch.randn(ctx, 4, 64).half()
            ref = R.attention_contiguous_ref(q, k, v)
            for part in (1, 16, 64, 100, 4096):
                err = (R.split_softmax_combine_ref(q, k, v, part).float() - ref.float()).abs().max().item()
                assert err < 2e-3, (ctx, scale, part, err)


def test_batched_attention_is_a_loop():
    torch.manual_seed(1)
    kc, vc = torch.randn(40, 2, 16, 64).half(), torch.randn(40, 2, 16, 64).half()
    bts = torch.stack([torch.randperm(40)[:12] for _ in range(3)]).int()
    q = torch.randn(3, 4, 64).half()
    ctxs = [1, 100, 192]
    out = R.paged_attention_batched_ref(q, kc, vc, bts, ctxs, 16)
    for b in range(3):
        assert torch.equal(out[b], R.paged_attention_ref(q[b], kc, vc, bts[b], ctxs[b], 16))


def test_argmax_lowest_index_on_ties():
    lg = torch.tensor([0.5, 2.0, 2.0, -1.0, 2.0]).half()
    assert R.argmax_ref(lg) == 1


def model_fixture(g):
    sd = {k[4:]: T(v) for k, v in g.items() if k.startswith("sd__")}
    cfg_hf = types.SimpleNamespace(hidden_size=128, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                                   intermediate_size=256, vocab_size=320, rms_norm_eps=1e-5, rope_theta=10000.0)
    return sd, cfg_hf


@pytest.mark.parametrize("quant", ["rtn", "clip"])
def test_model_golden(golden, quant):
    g = golden("model")
    sd, hf = model_fixture(g)
    cfg = types.SimpleNamespace(group=64, quant=quant, qparams=None, max_ctx=64, page=16, shuffle_pages=True)
    m = MO.OracleModel(sd, hf, cfg, block_table=g[f"bt_{quant}"])
    logits = m.teacher_force(g["prompt"].tolist(), collect_logits=True)
    assert np.array_equal(logits.numpy().view(np.uint16), g[f"logits_{quant}"].view(np.uint16))
    assert m.generate(g["prompt"].tolist(), 20) == g[f"tokens_{quant}"].tolist()
    assert np.array_equal(m.kv.numpy().view(np.uint16), g[f"kv_{quant}"].view(np.uint16))
