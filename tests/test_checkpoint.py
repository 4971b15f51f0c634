"""Weights on disk: the lazy Hugging Face reader, the kernel-format directory, the GPTQ cache, shard cuts of packed
tensors (all CPU), and on a GPU the round trip Model -> save_quantized -> Model.from_quantized."""
import types

import pytest
import torch

from llm_decode_kernels_b200 import checkpoint as CK
from llm_decode_kernels_b200 import quant as PQ
from llm_decode_kernels_b200 import tp as TP


def _cfg(L=2):
    return types.SimpleNamespace(hidden_size=256, num_hidden_layers=L, num_attention_heads=4, num_key_value_heads=2,
                                 intermediate_size=512, vocab_size=300, rms_norm_eps=1e-5, rope_theta=10000.0)


def _state(c, seed=0):
    from llm_decode_kernels_b200.shapes import random_llama_state
    return random_llama_state(c, "cpu", seed)


def test_hf_checkpoint_reads_single_file_and_shards(tmp_path):
    c = _cfg()
    sd = _state(c)
    for shards in (1, 3):
        d = CK.write_hf_checkpoint(sd, c, tmp_path / f"hf{shards}", shards=shards)
        ck = CK.HFCheckpoint(d)
        assert set(ck.keys()) == set(sd) and "lm_head.weight" in ck and "nope" not in ck
        assert ck.config.hidden_size == 256 and ck.config.rope_theta == 10000.0
        for k in ("model.embed_tokens.weight", "model.layers.1.mlp.down_proj.weight", "model.norm.weight"):
            assert torch.equal(ck[k], sd[k])
    (tmp_path / "empty").mkdir()
    (tmp_path / "empty" / "config.json").write_text("{}")
    with pytest.raises(FileNotFoundError):
        CK.HFCheckpoint(tmp_path / "empty")


def _fake_model(c, sd, group=128):
    """What save_quantized reads from a Model, built on the CPU with the product's quantizer."""
    ql = lambda w: PQ.QuantLinear(w, group, keep_ref=False)
    layers = []
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append({"ln1": sd[p + "input_layernorm.weight"], "ln2": sd[p + "post_attention_layernorm.weight"],
                       "qkv": ql(torch.cat([sd[p + f"self_attn.{n}_proj.weight"] for n in "qkv"], 0)),
                       "o": ql(sd[p + "self_attn.o_proj.weight"]),
                       "gu": ql(torch.cat([sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"]], 0)),
                       "down": ql(sd[p + "mlp.down_proj.weight"])})
    return types.SimpleNamespace(tp=1, emb=sd["model.embed_tokens.weight"], norm_f=sd["model.norm.weight"],
                                 layers=layers, lm_head=ql(sd["lm_head.weight"]),
                                 cfg=types.SimpleNamespace(group=group, quant="rtn"), H=c.hidden_size,
                                 L=c.num_hidden_layers, n_q=c.num_attention_heads, n_kv=c.num_key_value_heads,
                                 I=c.intermediate_size, V_full=c.vocab_size, eps=c.rms_norm_eps, rope_theta=10000.0,
                                 D=c.hidden_size // c.num_attention_heads)


def test_kernel_format_round_trip(tmp_path):
    c = _cfg()
    sd = _state(c, 3)
    m = _fake_model(c, sd)
    d = CK.save_quantized(m, tmp_path / "q")
    c2, group, state, qp = CK.load_quantized(d)
    assert group == 128 and c2.num_hidden_layers == 2 and c2.head_dim == 64 and c2.vocab_size == 300
    assert torch.equal(state["model.embed_tokens.weight"], sd["model.embed_tokens.weight"])
    assert torch.equal(state["model.layers.1.post_attention_layernorm.weight"], m.layers[1]["ln2"])
    for i in range(2):
        for n in CK.MATRICES:
            pk, sz = qp[f"layers.{i}.{n}"]
            assert pk.dtype == torch.int32 and torch.equal(pk, m.layers[i][n].packed) and torch.equal(sz, m.layers[i][n].sz)
    assert torch.equal(qp["lm_head"][0], m.lm_head.packed)
    (d / "meta.json").write_text('{"format": "something else"}')
    with pytest.raises(ValueError, match="not a"):
        CK.load_quantized(d)
    m.tp = 2
    with pytest.raises(ValueError, match="unsharded"):
        CK.save_quantized(m, tmp_path / "q2")


def test_shard_cuts_of_packed_tensors_match_packing_of_shard_cuts():
    """Cutting a tensor-parallel shard out of the kernel format gives the bits of quantizing the shard."""
    torch.manual_seed(0)
    n_q, n_kv, D, I, V, G = 4, 2, 64, 512, 300, 128
    dims = (n_q, n_kv, D, I, V)
    mats = {"qkv": torch.randn((n_q + 2 * n_kv) * D, 256), "gu": torch.randn(2 * I, 256), "o": torch.randn(256, n_q * D),
            "down": torch.randn(256, I), "lm_head": torch.randn(V, 256)}
    for kind, w in mats.items():
        w = (w * 0.05).half()
        full = PQ.QuantLinear(w, G, keep_ref=False)
        for rank in (0, 1):
            pk, sz = TP.shard_packed(kind, (full.packed, full.sz), dims, G, rank, 2)
            want = PQ.QuantLinear(TP.shard_weight(kind, w, dims, rank, 2), G, keep_ref=False)
            assert torch.equal(pk, want.packed) and torch.equal(sz, want.sz), (kind, rank)
    assert TP.shard_packed("o", None, dims, G, 0, 2) is None


def test_qparams_cache(tmp_path):
    calls = []

    def make():
        calls.append(1)
        q = torch.randint(0, 16, (8, 128), dtype=torch.uint8)
        return {"layers.0.qkv": (q, torch.rand(8, 1).half(), torch.rand(8, 1).half()), "lm_head": (q, q.half()[:, :1], q.half()[:, :1])}

    k1 = CK.qparams_key(shape=(8, 128), group=128, clip=True, seed=0)
    a = CK.cached_qparams(tmp_path, k1, make)
    b = CK.cached_qparams(tmp_path, k1, make)
    assert len(calls) == 1 and set(a) == set(b) == {"layers.0.qkv", "lm_head"}
    for n in a:
        assert all(torch.equal(x, y) for x, y in zip(a[n], b[n]))
    assert CK.qparams_key(shape=(8, 128), group=128, clip=True, seed=1) != k1
    CK.cached_qparams(tmp_path, CK.qparams_key(seed=1), make)
    assert len(calls) == 2


@pytest.mark.gpu
def test_model_from_disk_formats(tmp_path):
    """HF directory -> Model (lazy reads) -> kernel-format directory -> Model.from_quantized: same bits all the way,
    and the step built from the kernel format decodes the same logits."""
    from llm_decode_kernels_b200.model import DecodeConfig, Model
    c = types.SimpleNamespace(hidden_size=512, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
                              intermediate_size=1024, vocab_size=1500, rms_norm_eps=1e-5, rope_theta=10000.0)
    sd = {k: (v * 3 if v.dim() == 2 else v) for k, v in _state(c, 5).items()}
    ck = CK.HFCheckpoint(CK.write_hf_checkpoint(sd, c, tmp_path / "hf", shards=2))
    torch.manual_seed(0)
    stream = torch.randint(0, c.vocab_size, (24,)).tolist()
    outs = []
    m = Model(ck, ck.config, DecodeConfig(max_ctx=64, seed=2))
    CK.save_quantized(m, tmp_path / "packed")
    for mm in (m, Model.from_quantized(tmp_path / "packed", DecodeConfig(max_ctx=64, seed=2)),
               Model.from_quantized(tmp_path / "packed", DecodeConfig(max_ctx=64, seed=2), step_kernel="multi",
                                    keep_packed=False)):
        mm.prepare(64, use_graph=True)
        mm.reset(0)
        outs.append(mm.teacher_force(stream, collect_logits=True).cpu())
        assert mm.step_error() == 0
    assert m.persistent and torch.equal(outs[0], outs[1])
    scale = outs[0].float().abs().max().item()
    assert (outs[2].float() - outs[0].float()).abs().max().item() <= 1e-2 * scale     # other step kernel, same weights
    m2 = Model.from_quantized(tmp_path / "packed", DecodeConfig(max_ctx=64))
    assert torch.equal(m2.layers[1]["down"].packed, m.layers[1]["down"].packed) and m2.cfg.quant == "packed"
    with pytest.raises(ValueError, match="qparams"):
        Model(sd, c, DecodeConfig(max_ctx=64, quant="packed"))
