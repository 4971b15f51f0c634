"""The prompt path: batched W4A16 GEMM on the tcgen05 tensor cores, batched norm / SwiGLU, Model.prefill.

The reference steps through a prompt one token at a time (runtime/model.py:267-276), so the oracle for a prompt of T
tokens is T oracle steps: the GEMM is checked row by row against the oracle's GEMV, prefill() against the oracle
model's teacher-forced logits and, through the cache it leaves behind, against the tokens decoded after the prompt.
"""
import types

import numpy as np
import pytest
import torch

from llm_decode_kernels_b200 import ext, quant as PQ
from llm_decode_kernels_b200.model import DecodeConfig, Model
from oracle import model_oracle as MO
from oracle import ops_oracle as R
from oracle import quant_oracle as Q
from test_model import KERNEL_TOL, check_logits_and_tokens, hf_cfg, packed_of, random_state

pytestmark = pytest.mark.gpu
dev = "cuda"
GEMM_TOL = 2e-3   # fp32 accumulation of exact fp16 products: only the summation order and the final rounding differ


@pytest.fixture(scope="module")
def K():
    return ext.load()


def test_gemm_one_hot_rows_are_the_dequantized_weights(K):
    """X = rows of the identity: Y[t] must be column t of the dequantized matrix, bit for bit."""
    N, Kd, G = 200, 256, 64          # N not a multiple of the 128-row block
    torch.manual_seed(3)
    w = (torch.randn(N, Kd) * 0.05).half()
    q, s, z = PQ.quantize(w, G, False)
    packed, sz = PQ.pack(q).to(dev), PQ.pack_scale_zero(s, z).to(dev)
    want = Q.dequantize(q.numpy(), s.numpy(), z.numpy(), G)                 # [N, K] fp16
    eye = torch.eye(Kd, dtype=torch.half, device=dev)
    for t0, T in ((0, 16), (16, 1), (17, 100), (117, 139)):                # T = 1, ragged, and past one MMA's 16 columns
        y = torch.full((T, N), float("nan"), dtype=torch.half, device=dev)
        K.gemm_w4a16(packed, sz, eye[t0:t0 + T].contiguous(), y, G)
        assert np.array_equal(y.cpu().numpy().view(np.uint16), want[:, t0:t0 + T].T.copy().view(np.uint16)), (t0, T)
    assert K.gemm_status() == 0


@pytest.mark.parametrize("shape", [(2560, 2048, 128, 37), (2048, 5632, 128, 256), (1003, 1024, 64, 16),
                                   (256, 18432, 256, 100), (32000, 2048, 128, 64)])
def test_gemm_against_oracle_rows(K, shape):
    N, Kd, G, T = shape
    torch.manual_seed(N + T)
    ql = PQ.QuantLinear((torch.randn(N, Kd) * 0.02).half().to(dev), G, keep_ref=True)
    x = torch.randn(T, Kd).half()
    y = torch.full((T, N), float("nan"), dtype=torch.half, device=dev)
    K.gemm_w4a16(ql.packed, ql.sz, x.to(dev), y, G)
    w_ref = ql.w_ref.cpu()
    got = y.float().cpu()
    assert torch.isfinite(got).all()
    for t in sorted({0, 1, T // 2, T - 1}):
        ref = R.gemv_ref(w_ref, x[t]).float()
        err = (got[t] - ref).abs().max().item() / ref.abs().max().item()
        assert err <= GEMM_TOL, (shape, t, err)
    assert K.gemm_status() == 0


def test_gemm_rejects_bad_shapes(K):
    pk = torch.zeros(128, 24, dtype=torch.int32, device=dev)           # K = 192
    sz = torch.zeros(128, 3, 2, dtype=torch.half, device=dev)
    x = torch.zeros(4, 192, dtype=torch.half, device=dev)
    y = torch.zeros(4, 128, dtype=torch.half, device=dev)
    K.gemm_w4a16(pk, sz, x, y, 64)
    with pytest.raises(RuntimeError, match="shape"):
        K.gemm_w4a16(pk, torch.zeros(128, 6, 2, dtype=torch.half, device=dev), x, y, 32)    # group below 64
    too_many = K.gemm_max_tokens() + 1
    with pytest.raises(RuntimeError):
        K.gemm_w4a16(pk, sz, torch.zeros(too_many, 192, dtype=torch.half, device=dev),
                     torch.zeros(too_many, 128, dtype=torch.half, device=dev), 64)
    with pytest.raises(RuntimeError, match="inconsistent"):
        K.gemm_w4a16(pk, sz, x, torch.zeros(4, 64, dtype=torch.half, device=dev), 64)


def test_batched_norm_and_swiglu_match_the_single_row_kernels(K):
    torch.manual_seed(5)
    T, H, I = 19, 2048, 5632
    x, d = torch.randn(T, H, device=dev).half(), torch.randn(T, H, device=dev).half()
    w = (1 + 0.1 * torch.randn(H, device=dev)).half()
    xb, out_b = x.clone(), torch.empty(T, H, dtype=torch.half, device=dev)
    K.add_rmsnorm_batched(xb, d, w, out_b, 1e-5)
    gu = torch.randn(T, 2 * I, device=dev).half()
    act_b = torch.empty(T, I, dtype=torch.half, device=dev)
    K.swiglu_batched(gu, act_b)
    for t in (0, 7, T - 1):
        x1, o1 = x[t].clone(), torch.empty(H, dtype=torch.half, device=dev)
        K.add_rmsnorm(x1, d[t].contiguous(), w, o1, 1e-5)
        assert torch.equal(x1, xb[t]) and torch.equal(o1, out_b[t])
        a1 = torch.empty(I, dtype=torch.half, device=dev)
        K.swiglu(gu[t].contiguous(), a1)
        assert torch.equal(a1, act_b[t])
        ref_x, ref_n = R.add_rmsnorm_ref(x[t].cpu(), d[t].cpu(), w.cpu(), 1e-5)
        assert torch.equal(ref_x, xb[t].cpu())
        assert (ref_n.float() - out_b[t].cpu().float()).abs().max() <= 2e-3 * ref_n.float().abs().max()
    xn = x.clone()
    K.add_rmsnorm_batched(xn, None, w, out_b, 1e-5)          # no residual: x untouched
    assert torch.equal(xn, x)


@pytest.mark.parametrize("shape", ["gqa8_d64", "gqa8_d128", "tinyllama_width"])
def test_prefill_against_oracle_model(shape):
    """prefill(prompt) leaves the logits, the cache and the next token that the oracle's token-by-token pass over the
    same prompt produces; decoding then continues from it."""
    if shape == "gqa8_d64":
        c, D, n_prompt = hf_cfg(512, 3, 8, 1, 1536, 4001), None, 70
    elif shape == "gqa8_d128":
        c, D, n_prompt = hf_cfg(1024, 2, 8, 1, 2048, 3000, D=128), 128, 33
    else:
        c, D, n_prompt = hf_cfg(2048, 2, 32, 4, 5632, 32000), None, 48
    sd = random_state(c, 17, D)
    m = Model(sd, c, DecodeConfig(group=128, max_ctx=160, page=16, seed=5))
    ocfg = types.SimpleNamespace(group=128, quant="rtn", qparams=None, max_ctx=160, page=16, shuffle_pages=True)
    o = MO.OracleModel(sd, c, ocfg, packed=packed_of(m), block_table=m.bt.cpu())
    torch.manual_seed(1)
    prompt = torch.randint(0, c.vocab_size, (n_prompt,)).tolist()
    ref_logits = o.teacher_force(prompt, collect_logits=True)
    n_new = 12
    ref_new, step_logits = [o.tok], [ref_logits[-1]]     # step_logits[t]: the logits ref_new[t] was chosen from
    for _ in range(n_new - 1):
        o.step()
        ref_new.append(o.tok)
        step_logits.append(o.logits.clone())
    m.prepare(160, use_graph=True, part_size=32)
    m.reset(0)
    got = m.prefill(prompt, collect_logits=True).cpu()
    check_logits_and_tokens(got, ref_logits)
    assert m.host_pos == n_prompt and int(m.pos) == n_prompt
    # the cache prefill() wrote equals (to rounding of the inputs it was computed from) the one stepping writes
    kv_prefill = m.kv.clone()
    m.kv.zero_()
    m.reset(0)
    m.teacher_force(prompt)
    assert torch.equal((kv_prefill != 0).any(-1), (m.kv != 0).any(-1))       # the same cache rows were written
    scale = m.kv.float().abs().max().item()
    assert (kv_prefill.float() - m.kv.float()).abs().max().item() <= KERNEL_TOL * scale
    # decode after a prefilled prompt (without the per-position logits: last token through the GEMV)
    m.kv.zero_()
    toks = m.generate(prompt, n_new, prefill=True)
    assert m.step_error() == 0 and m.K.gemm_status() == 0
    lscale = ref_logits.float().abs().max().item()
    for t, (a, b) in enumerate(zip(toks, ref_new)):
        if a != b:      # allowed only where the oracle's own margin is inside the noise floor; later tokens differ then
            row = step_logits[t].float()
            assert row[b] - row[a] <= 2 * KERNEL_TOL * lscale, f"diverged at {t} outside the noise floor"
            break


def test_prefill_in_chunks_and_refusals():
    c = hf_cfg(512, 2, 8, 1, 1536, 1000)
    sd = random_state(c, 23)
    m = Model(sd, c, DecodeConfig(group=128, max_ctx=640, page=16, seed=5))
    m.prepare(640, use_graph=False)
    torch.manual_seed(2)
    prompt = torch.randint(0, 1000, (300,)).tolist()        # more than one GEMM call's worth of tokens
    m.reset(0)
    whole = m.prefill(prompt, collect_logits=True).cpu()
    m.kv.zero_()
    m.reset(0)
    a = m.prefill(prompt[:123], collect_logits=True).cpu()  # a prompt continued by a second call
    b = m.prefill(prompt[123:], collect_logits=True).cpu()
    both = torch.cat([a, b])
    scale = whole.float().abs().max().item()
    assert (both.float() - whole.float()).abs().max().item() <= KERNEL_TOL * scale
    assert m.host_pos == 300
    with pytest.raises(RuntimeError, match="exceeds"):
        m.prefill(list(range(400)))
    with pytest.raises(ValueError, match="token ids"):
        m.prefill([1000])
    m2 = Model(sd, c, DecodeConfig(group=128, max_ctx=64, page=16, keep_packed=False))
    with pytest.raises(ValueError, match="keep_packed"):
        m2.prefill([1, 2, 3])
