"""Calibration driver (llm_decode_kernels_b200/gptq.py) on a tiny random HF Llama, mirroring the reference's own
mechanics test (tests/test_quant_local.py:63-81), and against the reference driver's stored behaviour: same keys,
same shapes, weights restored, and quantized outputs that beat round-to-nearest on layer-output error."""
import pytest
import torch

from llm_decode_kernels_b200 import gptq as GQ
from llm_decode_kernels_b200 import quant as PQ

transformers = pytest.importorskip("transformers")


class Tok:
    bos_token_id = 1
    vocab_size = 256


def tiny_llama():
    from transformers import LlamaConfig, LlamaForCausalLM
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=256, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128)
    return LlamaForCausalLM(cfg).eval()


def test_calibration_windows_are_seeded_synthetic_ids():
    a = GQ.calibration_windows(Tok(), n=3, L=16, seed=5)
    b = GQ.calibration_windows(Tok(), n=3, L=16, seed=5)
    assert len(a) == 3 and all(w.shape == (16,) and int(w[0]) == 1 and int(w.max()) < 256 for w in a)
    assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_calibrate_tiny_llama():
    m = tiny_llama()
    before = {k: v.clone() for k, v in m.state_dict().items()}
    out = GQ.calibrate(m, Tok(), group=64, n=8, L=32, log=lambda *a: None)
    assert set(out) == {f"layers.{i}.{k}" for i in range(2) for k in ("qkv", "o", "gu", "down")} | {"lm_head"}
    assert out["layers.0.qkv"][0].shape == (128 + 2 * 64, 128) and out["layers.1.gu"][0].shape == (512, 128)
    assert out["lm_head"][1].shape == (256, 2)
    assert all(torch.equal(before[k], v) for k, v in m.state_dict().items())       # HF weights restored
    for q, s, z in out.values():
        assert q.dtype == torch.uint8 and int(q.max()) <= 15 and s.dtype == torch.float16
        zf = z.float()
        assert torch.equal(zf, zf.round()) and float(zf.min()) >= 0 and float(zf.max()) <= 15


def test_calibrated_first_layer_beats_rtn_on_its_own_inputs():
    """Layer 0's q/k/v see the embedding outputs of the calibration windows directly, so its layer-output error can be
    recomputed here: GPTQ must do better than round-to-nearest on those inputs."""
    m = tiny_llama()
    out = GQ.calibrate(m, Tok(), group=64, n=16, L=32, lm_head=False, log=lambda *a: None)
    wins = GQ.calibration_windows(Tok(), 16, 32)
    l0 = m.model.layers[0]
    X = torch.cat([l0.input_layernorm(m.model.embed_tokens(w[None])).reshape(-1, 128) for w in wins]).float()
    W = torch.cat([l0.self_attn.q_proj.weight, l0.self_attn.k_proj.weight, l0.self_attn.v_proj.weight], 0).detach()
    err = lambda qsz: (X @ (PQ.dequantize(*qsz, 64).float() - W.float()).t()).pow(2).mean().item()
    assert err(out["layers.0.qkv"]) < err(PQ.quantize(W, 64))


def test_qparams_feed_the_oracle_model():
    """The dict plugs into DecodeConfig(quant='pre'): checked with the CPU oracle model (no GPU needed)."""
    import types
    from oracle import model_oracle as MO
    m = tiny_llama()
    qp = GQ.calibrate(m, Tok(), group=64, n=4, L=16, log=lambda *a: None)
    c = m.config
    hf = types.SimpleNamespace(hidden_size=c.hidden_size, num_hidden_layers=c.num_hidden_layers,
                               num_attention_heads=c.num_attention_heads, num_key_value_heads=c.num_key_value_heads,
                               intermediate_size=c.intermediate_size, vocab_size=c.vocab_size,
                               rms_norm_eps=c.rms_norm_eps, head_dim=32)
    cfg = types.SimpleNamespace(group=64, quant="pre", qparams=qp, max_ctx=32, page=16, shuffle_pages=False)
    o = MO.OracleModel(m.state_dict(), hf, cfg)
    toks = o.generate([1, 5, 9], 4)
    assert len(toks) == 4 and all(0 <= t < 256 for t in toks)
