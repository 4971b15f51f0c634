"""Generate tests/golden/*.npz from the reference implementation.

Run once, where the reference checkout is available:
    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/llm-decode-kernels
It imports the reference's runtime/quant.py, reference/ref_ops.py and runtime/model.py (CPU, torch),
feeds them small seeded inputs and stores inputs and outputs. The stored files are what pins the
oracle (oracle/*.py) and the product's host code (llm_decode_kernels_b200/quant.py) to the reference;
nothing at test time needs the reference checkout.
"""
import sys
import types
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent


def np16(t):
    return t.detach().cpu().numpy()


def main(ref_root):
    sys.path.insert(0, ref_root)
    from runtime import quant as RQ          # noqa: E402
    from reference import ref_ops as RR      # noqa: E402
    from runtime.model import Model, DecodeConfig  # noqa: E402

    # ---------------- quantizer + packing ----------------
    g = torch.Generator().manual_seed(1234)
    w = (torch.randn(24, 512, generator=g) * 0.02)
    w[torch.rand(24, 512, generator=g) < 0.004] *= 8      # a few outliers so clipping matters
    w[3, 128:256] = 0.0                                   # an all-zero group: exercises the 1e-6 scale floor
    w[5, :64] = 0.013                                     # a constant group
    w = w.half()
    d = {"w": np16(w)}
    for G in (64, 128, 256):
        for clip in (False, True):
            q, s, z = RQ.quantize(w, G, clip)
            tag = f"g{G}_{'clip' if clip else 'rtn'}"
            d[f"q_{tag}"], d[f"s_{tag}"], d[f"z_{tag}"] = np16(q), np16(s), np16(z)
            d[f"packed_{tag}"] = np16(RQ.pack(q))
            d[f"sz_{tag}"] = np16(RQ.pack_scale_zero(s, z))
            d[f"deq_{tag}"] = np16(RQ.dequantize(q, s, z, G))
    qr = torch.randint(0, 16, (8, 64), generator=g, dtype=torch.uint8)
    d["kat_q"] = np16(qr)
    d["kat_packed"] = np16(RQ.pack(qr))
    d["kat_unpacked"] = np16(RQ.unpack(RQ.pack(qr)))
    d["kat_word_0to7"] = np16(RQ.pack(torch.arange(8, dtype=torch.uint8)[None]))
    np.savez_compressed(OUT / "quant.npz", **d)

    # ---------------- GPTQ ----------------
    g = torch.Generator().manual_seed(77)
    N, K, G = 32, 256, 64
    wg = (torch.randn(N, K, generator=g) * 0.02).half()
    X = torch.randn(1024, 32, generator=g) @ torch.randn(32, K, generator=g)
    X[:, :4] *= 10
    X[:, 17] = 0                                          # a dead input channel
    Hm = 2 * X.t() @ X / X.shape[0]
    d = {"w": np16(wg), "H": np16(Hm)}
    for clip in (False, True):
        q, s, z = RQ.quantize_gptq(wg, Hm, G, clip=clip, block=128)
        tag = "clip" if clip else "plain"
        d[f"q_{tag}"], d[f"s_{tag}"], d[f"z_{tag}"] = np16(q), np16(s), np16(z)
    np.savez_compressed(OUT / "gptq.npz", **d)

    # ---------------- operators ----------------
    g = torch.Generator().manual_seed(4321)
    rn = lambda *s: torch.randn(*s, generator=g)
    d = {}
    wq = RQ.QuantLinear((rn(96, 256) * 0.02).half(), 128)
    x = rn(256).half()
    d["gemv_packed"], d["gemv_sz"], d["gemv_wref"] = np16(wq.packed), np16(wq.sz), np16(wq.w_ref)
    d["gemv_x"], d["gemv_y"] = np16(x), np16(RR.gemv_ref(wq.w_ref, x))
    H = 256
    xn, dl, wn = (rn(H) * 3).half(), rn(H).half(), (1 + 0.1 * rn(H)).half()
    xo, no = RR.add_rmsnorm_ref(xn.clone(), dl, wn, 1e-5)
    d["norm_x"], d["norm_delta"], d["norm_w"], d["norm_xout"], d["norm_out"] = map(np16, (xn, dl, wn, xo, no))
    d["norm_out_nodelta"] = np16(RR.add_rmsnorm_ref(xn.clone(), None, wn, 1e-5)[1])
    gu = (rn(2 * 320) * 2).half()
    d["swiglu_gu"], d["swiglu_out"] = np16(gu), np16(RR.swiglu_ref(gu))
    for D in (64, 128):
        cos, sin = RR.rope_tables(300, D)
        d[f"rope_cos_d{D}"], d[f"rope_sin_d{D}"] = np16(cos), np16(sin)
        n_q, n_kv, page, pos = 8, 2, 16, 37
        pages = 6
        kc, vc = rn(pages, n_kv, page, D).half(), rn(pages, n_kv, page, D).half()
        bt = torch.randperm(pages, generator=g).int()
        qkv = rn((n_q + 2 * n_kv) * D).half()
        kc2, vc2 = kc.clone(), vc.clone()
        qrot = RR.rope_append_ref(qkv.clone(), cos, sin, pos, kc2, vc2, bt, n_q, n_kv, D, page)
        d[f"ra_kc_d{D}"], d[f"ra_vc_d{D}"], d[f"ra_bt_d{D}"], d[f"ra_qkv_d{D}"] = map(np16, (kc, vc, bt, qkv))
        d[f"ra_kc_out_d{D}"], d[f"ra_vc_out_d{D}"], d[f"ra_q_out_d{D}"] = map(np16, (kc2, vc2, qrot))
        ctx = 70
        qa = rn(n_q, D).half()
        d[f"attn_q_d{D}"] = np16(qa)
        d[f"attn_out_d{D}"] = np16(RR.paged_attention_ref(qa, kc, vc, bt, ctx, page))
        k, v = RR.gather_kv(kc, vc, bt, ctx, page)
        d[f"attn_gk_d{D}"], d[f"attn_gv_d{D}"] = np16(k), np16(v)
        d[f"attn_split_d{D}"] = np16(RR.split_softmax_combine_ref(qa, k, v, 16))
    np.savez_compressed(OUT / "ops.npz", **d)

    # ---------------- whole model, reference backend on CPU ----------------
    torch.manual_seed(2024)
    hf_cfg = types.SimpleNamespace(hidden_size=128, num_hidden_layers=2, num_attention_heads=2,
                                   num_key_value_heads=1, intermediate_size=256, vocab_size=320,
                                   rms_norm_eps=1e-5, rope_theta=10000.0)
    Hh, I, V, D = 128, 256, 320, 64
    sd = {"model.embed_tokens.weight": torch.randn(V, Hh) * 0.5, "model.norm.weight": 1 + 0.1 * torch.randn(Hh),
          "lm_head.weight": torch.randn(V, Hh) * 0.1}
    for i in range(2):
        p = f"model.layers.{i}."
        sd[p + "input_layernorm.weight"] = 1 + 0.1 * torch.randn(Hh)
        sd[p + "post_attention_layernorm.weight"] = 1 + 0.1 * torch.randn(Hh)
        sd[p + "self_attn.q_proj.weight"] = torch.randn(2 * D, Hh) * 0.1
        sd[p + "self_attn.k_proj.weight"] = torch.randn(D, Hh) * 0.1
        sd[p + "self_attn.v_proj.weight"] = torch.randn(D, Hh) * 0.1
        sd[p + "self_attn.o_proj.weight"] = torch.randn(Hh, 2 * D) * 0.1
        sd[p + "mlp.gate_proj.weight"] = torch.randn(I, Hh) * 0.1
        sd[p + "mlp.up_proj.weight"] = torch.randn(I, Hh) * 0.1
        sd[p + "mlp.down_proj.weight"] = torch.randn(Hh, I) * 0.1
    sd = {k: v.half() for k, v in sd.items()}
    d = {"sd__" + k: np16(v) for k, v in sd.items()}
    prompt = torch.randint(0, V, (12,))
    d["prompt"] = np16(prompt)
    for quant in ("rtn", "clip"):
        cfg = DecodeConfig(weights="int4", group=64, quant=quant, backend="ref", device="cpu", max_ctx=64,
                           page=16)
        m = Model(sd, hf_cfg, cfg)
        d[f"bt_{quant}"] = np16(m.bt)
        m.reset(0)
        logits = m.teacher_force(prompt, use_graph=False, collect_logits=True)
        d[f"logits_{quant}"] = np16(logits)
        d[f"tokens_{quant}"] = np.asarray(m.generate(prompt, 20), dtype=np.int64)
        d[f"kv_{quant}"] = np16(m.kv)
    np.savez_compressed(OUT / "model.npz", **d)
    for f in sorted(OUT.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
