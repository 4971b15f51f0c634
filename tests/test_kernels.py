"""Numerical gate for every CUDA kernel, through the C ABI, against the CPU oracle.

Mirrors the order and the cases of the reference's tests/test_kernels.py (tiny hand-checkable cases first) and
extends them to what the reference lacks: batches, head_dim 128, 70B and tensor-parallel shard shapes.
Error measure as there: max|out - ref| / max|ref| (normwise). Tolerances are the reference's own
(GEMV 5e-3, attention and fused ops 2e-3, residual / v-cache / dequantized weights exact); the build's
contract is 1e-2, so these are stricter than required.
"""
import math

import numpy as np
import pytest
import torch

from llm_decode_kernels_b200 import ext, quant as PQ
from oracle import ops_oracle as R
from oracle import quant_oracle as Q

pytestmark = pytest.mark.gpu
dev = "cuda"

GEMV_TOL, ATTN_TOL, FUSED_TOL = 5e-3, 2e-3, 2e-3

# (stage, R, warps, pf): the plain kernel, every explicit rows-per-warp configuration, the segmented kernel (R = 16)
# and the library's own choice (R = 0: the tensor-core kernel where K and the group size allow, else the segmented one)
GEMV_CFGS = ([(0, 1, 4, 0), (1, 1, 4, 0)] + [(2, r, w, 0) for r in (1, 2, 4, 8) for w in (1, 4, 8)]
             + [(2, 16, 0, 0), (2, 0, 0, 0)])


@pytest.fixture(scope="module")
def K():
    return ext.load()


def rel_err(out, ref):
    out, ref = out.float().cpu(), ref.float().cpu()
    err = (out - ref).abs().max().item()
    assert math.isfinite(err)
    return err / max(ref.abs().max().item(), 1e-12)


def gemv(K, cfg, packed, sz, x, N, group):
    y = torch.empty(N, dtype=torch.half, device=dev)
    K.gemv_w4a16(cfg[0], cfg[1], cfg[2], cfg[3], packed, sz, x, y, group)
    return y


# ---- 1. closed-form 4-row GEMV and the one-hot nibble sweep (reference tests/test_kernels.py:47-68) ----
@pytest.mark.parametrize("cfg", GEMV_CFGS)
def test_gemv_closed_form_and_onehot(K, cfg):
    N, Kd, G = 4, 128, 128
    q = torch.tensor([[(k + r) % 16 for k in range(Kd)] for r in range(N)], dtype=torch.uint8)
    s = torch.tensor([[(r + 1) * 0.5] for r in range(N)], dtype=torch.half)
    z = torch.full((N, 1), 8.0, dtype=torch.half)
    packed, sz = PQ.pack(q).to(dev), PQ.pack_scale_zero(s, z).to(dev)
    y = gemv(K, cfg, packed, sz, torch.ones(Kd, dtype=torch.half, device=dev), N, G)
    assert y.float().cpu().tolist() == [-32.0, -64.0, -96.0, -128.0]
    eye = torch.eye(Kd, dtype=torch.half, device=dev)
    for k in range(Kd):
        y = gemv(K, cfg, packed, sz, eye[k].contiguous(), N, G).float().cpu()
        want = (q[:, k].float() - 8) * s[:, 0].float()
        assert torch.equal(y, want), (cfg, k)


# ---- 2. dequantized weights are bit-exact --------------------------------------------------------------
@pytest.mark.parametrize("G", [32, 64, 128, 256])
@pytest.mark.parametrize("clip", [False, True])
def test_dequant_bit_exact(K, G, clip):
    torch.manual_seed(G + clip)
    w = (torch.randn(96, 1024) * 0.02).half()
    w[0, :G] = 0                                    # scale floor 1e-6: a subnormal fp16 scale
    w[1, :G] = 3e-6 * torch.randn(G)                # tiny weights: subnormal products must not flush to zero
    q, s, z = PQ.quantize(w, G, clip)
    out = torch.empty(96, 1024, dtype=torch.half, device=dev)
    K.dequant_w4a16(PQ.pack(q).to(dev), PQ.pack_scale_zero(s, z).to(dev), out, G)
    want = Q.dequantize(q.numpy(), s.numpy(), z.numpy(), G)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))


def test_dequant_golden(K, golden):
    g = golden("quant")
    for G in (64, 128, 256):
        for tag in (f"g{G}_rtn", f"g{G}_clip"):
            out = torch.empty(g["w"].shape, dtype=torch.half, device=dev)
            K.dequant_w4a16(torch.from_numpy(g[f"packed_{tag}"]).to(dev), torch.from_numpy(g[f"sz_{tag}"]).to(dev),
                            out, G)
            assert np.array_equal(out.cpu().numpy().view(np.uint16), g[f"deq_{tag}"].view(np.uint16))


# ---- 3. real shapes ------------------------------------------------------------------------------------
SHAPES = {  # TinyLlama, the single-GEMV benchmark case, Llama-3-70B and its 8-way shards
    "qkv": (2560, 2048), "o": (2048, 2048), "gate_up": (11264, 2048), "down": (2048, 5632),
    "lm_head": (32000, 2048), "bench": (5632, 2048),
    "qkv70_tp8": (1280, 8192), "o70_tp8": (8192, 1024), "gu70_tp8": (7168, 8192), "down70_tp8": (8192, 3584),
    "down70_tp2": (8192, 14336), "ragged": (1003, 2048)}


@pytest.mark.parametrize("name", list(SHAPES))
def test_gemv_real_shapes(K, name):
    N, Kd = SHAPES[name]
    torch.manual_seed(0)
    w = (torch.randn(N, Kd) * 0.02).half().to(dev)
    x = torch.randn(Kd, device=dev).half()
    groups = (64, 128, 256) if Kd % 256 == 0 else (64, 128)
    for G in groups:
        ql = PQ.QuantLinear(w, G)
        ref = R.gemv_ref(ql.w_ref.cpu(), x.cpu())
        cfgs = GEMV_CFGS if (G == 128 and N <= 12000) else [(0, 1, 4, 0), (2, 4, 4, 0), (2, 8, 2, 0), (2, 16, 0, 0),
                                                             (2, 0, 0, 0)]
        for cfg in cfgs:
            e = rel_err(gemv(K, cfg, ql.packed, ql.sz, x, N, G), ref)
            assert e <= GEMV_TOL, (name, G, cfg, e)


@pytest.mark.parametrize("name", ["qkv", "down", "lm_head", "o70_tp8", "down70_tp2", "ragged"])
def test_gemv_tile_layout(K, name):
    """The tensor-core GEMV from the repacked copy: same numbers as from the quantizer's tensors, bit for bit (same
    arithmetic in the same order, only the addresses differ), and within tolerance of the oracle."""
    N, Kd = SHAPES[name]
    torch.manual_seed(1)
    w = (torch.randn(N, Kd) * 0.02).half().to(dev)
    x = torch.randn(Kd, device=dev).half()
    for layout in (0, 1):     # "same order" needs the same launch shape: forget a measured one an earlier test's Model
        K.gemv_tune(layout, N, Kd, 0, 0)   # may have registered for this matrix shape (the table is per process)
    for G in (128, 256) if Kd % 256 == 0 else (128,):
        ql = PQ.QuantLinear(w, G)
        tiled = K.gemv_tile_repack(ql.packed, ql.sz, G)
        assert tiled is not None and tiled.numel() == ((N + 15) // 16) * (Kd // 128) * 1088
        y = torch.full((N,), float("nan"), dtype=torch.half, device=dev)
        K.gemv_w4a16_tiled(tiled, x, y, N, Kd)
        assert torch.equal(y, gemv(K, (2, 0, 0, 0), ql.packed, ql.sz, x, N, G)), (name, G)
        assert rel_err(y, R.gemv_ref(ql.w_ref.cpu(), x.cpu())) <= GEMV_TOL
    assert K.gemv_tile_repack(ql.packed, ql.sz, 64) is None      # groups below 128 have no tile layout


@pytest.mark.parametrize("I,Kd", [(5632, 2048), (1003, 1024), (3584, 8192)])
def test_gemv_swiglu_epilogue(K, I, Kd):
    """[gate; up] in the paired tile layout: one launch gives exactly what the GEMV followed by the SwiGLU kernel
    gives (same sums, same rounding points), and matches the oracle's gemv + swiglu."""
    torch.manual_seed(2)
    w = (torch.randn(2 * I, Kd) * 0.02).half().to(dev)
    x = torch.randn(Kd, device=dev).half()
    # "same sums" needs the same launch shape (the K split decides the order of the partial sums): forget measured
    # shapes an earlier test's Model may have registered for these matrices (the table is per process)
    K.gemv_tune(2, I, Kd, 0, 0)
    for layout in (0, 1):
        K.gemv_tune(layout, 2 * I, Kd, 0, 0)
    ql = PQ.QuantLinear(w, 128)
    paired = K.gemv_tile_repack(ql.packed, ql.sz, 128, gate_up=True)
    assert paired.numel() == ((I + 7) // 8) * (Kd // 128) * 1088
    act = torch.full((I,), float("nan"), dtype=torch.half, device=dev)
    K.gemv_w4a16_tiled(paired, x, act, I, Kd, swiglu=True)
    gu = gemv(K, (2, 0, 0, 0), ql.packed, ql.sz, x, 2 * I, 128)
    if I % 8 == 0:
        two = torch.empty(I, dtype=torch.half, device=dev)
        K.swiglu(gu, two)
        assert torch.equal(act, two)
    ref = R.swiglu_ref(R.gemv_ref(ql.w_ref.cpu(), x.cpu()))
    assert rel_err(act, ref) <= GEMV_TOL


@pytest.mark.parametrize("N,Kd,swiglu", [(2560, 2048, False), (5632, 2048, True), (3000, 1024, False)])
def test_gemv_with_norm_prologue(K, N, Kd, swiglu):
    """Residual add + RMSNorm inside the GEMV's staging: the residual it stores is bit-identical to add_rmsnorm's,
    the product within tolerance of oracle add_rmsnorm -> gemv (-> swiglu); with and without a delta."""
    torch.manual_seed(3)
    rows = 2 * N if swiglu else N
    ql = PQ.QuantLinear((torch.randn(rows, Kd) * 0.02).half().to(dev), 128)
    tiled = K.gemv_tile_repack(ql.packed, ql.sz, 128, gate_up=swiglu)
    nw = (1 + 0.1 * torch.randn(Kd, device=dev)).half()
    for with_delta in (True, False):
        x_in = torch.randn(Kd, device=dev).half()
        delta = (0.5 * torch.randn(Kd, device=dev)).half() if with_delta else None
        x_out = torch.full((Kd,), float("nan"), dtype=torch.half, device=dev)
        y = torch.full((N,), float("nan"), dtype=torch.half, device=dev)
        K.gemv_w4a16_tiled_norm(tiled, x_in, delta, nw, 1e-5, x_out, y, N, Kd, swiglu=swiglu)
        xr, normed = x_in.clone(), torch.empty(Kd, dtype=torch.half, device=dev)
        K.add_rmsnorm(xr, delta, nw, normed, 1e-5)
        assert torch.equal(x_out, xr)
        rx, rn = R.add_rmsnorm_ref(x_in.cpu(), None if delta is None else delta.cpu(), nw.cpu(), 1e-5)
        ref = R.gemv_ref(ql.w_ref.cpu(), rn)
        ref = R.swiglu_ref(ref) if swiglu else ref
        assert rel_err(y, ref) <= GEMV_TOL, (N, Kd, swiglu, with_delta)
    with pytest.raises(RuntimeError):
        K.gemv_w4a16_tiled_norm(tiled, x_in, None, nw, 1e-5, x_in, y, N, Kd, swiglu=swiglu)   # x_out must differ


def test_gemv_golden(K, golden):
    g = golden("ops")
    y = gemv(K, (2, 0, 0, 0), torch.from_numpy(g["gemv_packed"]).to(dev), torch.from_numpy(g["gemv_sz"]).to(dev),
             torch.from_numpy(g["gemv_x"]).to(dev), 96, 128)
    assert rel_err(y, torch.from_numpy(g["gemv_y"])) <= GEMV_TOL


def test_gemv_large_activations_do_not_overflow(K):
    """|x| in the hundreds: partial sums stay finite because the kernel pre-scales x."""
    torch.manual_seed(3)
    w = (torch.randn(512, 4096) * 0.02).half().to(dev)
    x = (torch.randn(4096, device=dev) * 300).half()
    ql = PQ.QuantLinear(w, 128)
    e = rel_err(gemv(K, (2, 0, 0, 0), ql.packed, ql.sz, x, 512, 128), R.gemv_ref(ql.w_ref.cpu(), x.cpu()))
    assert e <= GEMV_TOL


# ---- 4/5. paged attention ------------------------------------------------------------------------------
def make_cache(ctx, n_kv, page, D=64, peaky=1.0, spare=3):
    n_pages = (ctx + page - 1) // page + spare
    kc = (torch.randn(n_pages, n_kv, page, D, device=dev) * peaky).half()
    vc = torch.randn(n_pages, n_kv, page, D, device=dev).half()
    bt = torch.randperm(n_pages, device=dev).int()
    return kc, vc, bt


def run_attn(K, q, kc, vc, bt, ctx, PS, version=2, spare=0):
    n_q = q.numel() // 64
    max_splits = max(1, (ctx + PS - 1) // PS) + spare
    o_part = torch.full((n_q, max_splits, 64), float("nan"), device=dev)
    m_part = torch.full((n_q, max_splits), float("nan"), device=dev)
    l_part = torch.full_like(m_part, float("nan"))
    out = torch.empty(n_q, 64, dtype=torch.half, device=dev)
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device=dev)
    K.paged_attention(q, kc, vc, bt, pos, PS, o_part, m_part, l_part, out, version)
    return out


def test_attention_ctx128_all_groupings(K):
    torch.manual_seed(0)
    for n_q, n_kv in ((32, 4), (8, 8), (16, 4), (8, 4)):  # heads per group 8, 1, 4, 2
        for page in (16, 32):
            kc, vc, bt = make_cache(128, n_kv, page)
            q = torch.randn(n_q, 64, device=dev).half()
            k, v = R.gather_kv(kc.cpu(), vc.cpu(), bt.cpu(), 128, page)
            ref = R.attention_contiguous_ref(q.cpu(), k, v)
            for PS in (4096, 64, 32, 48, 16):
                for ver in (1, 2, 3):
                    e = rel_err(run_attn(K, q, kc, vc, bt, 128, PS, ver), ref)
                    assert e <= ATTN_TOL, (n_q, n_kv, page, PS, ver, e)


@pytest.mark.parametrize("ctx", [1, 2, 17, 63, 65, 129, 1000])
def test_attention_odd_contexts(K, ctx):
    torch.manual_seed(ctx)
    kc, vc, bt = make_cache(ctx, 4, 16)
    q = torch.randn(32, 64, device=dev).half()
    ref = R.paged_attention_ref(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), ctx, 16)
    for PS in (8192, 64, 256):
        for ver in (1, 2, 3):
            assert rel_err(run_attn(K, q, kc, vc, bt, ctx, PS, ver), ref) <= ATTN_TOL, (ctx, PS, ver)


@pytest.mark.parametrize("ctx", [512, 1024, 2048, 4096, 8192, 16384])
@pytest.mark.parametrize("peaky", [1.0, 6.0])
def test_attention_real_contexts(K, ctx, peaky):
    torch.manual_seed(ctx)
    kc, vc, bt = make_cache(ctx, 4, 16, peaky=peaky)
    q = torch.randn(32, 64, device=dev).half()
    ref = R.paged_attention_ref(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), ctx, 16)
    for PS in (ctx, 1024, 256, 128, 64):
        for ver in (1, 2, 3):
            assert rel_err(run_attn(K, q, kc, vc, bt, ctx, PS, ver), ref) <= ATTN_TOL, (ctx, peaky, PS, ver)


@pytest.mark.parametrize("ctx", [1, 40, 64, 100, 700, 2048, 5000])
def test_attention_spare_split_buffers(K, ctx):
    """Buffers sized for a larger cap: surplus split blocks exit, combine ignores the unused (NaN-filled) slots,
    and the single-live-split path writes `out` from the partial kernel."""
    torch.manual_seed(ctx)
    kc, vc, bt = make_cache(ctx, 4, 16, peaky=6.0)
    q = torch.randn(32, 64, device=dev).half()
    ref = R.paged_attention_ref(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), ctx, 16)
    for PS in (64, 128, 256):
        for ver in (1, 2, 3):
            assert rel_err(run_attn(K, q, kc, vc, bt, ctx, PS, ver, spare=8), ref) <= ATTN_TOL, (ctx, PS, ver)


@pytest.mark.parametrize("page", [4, 8, 64, 128])
def test_attention_page_sizes_and_poisoned_tail(K, page):
    """Pages of 8..64 tokens take the ring-staged kernel, others the register-load kernel. Cache slots past the
    context (rest of the last page, spare pages) hold NaN: whole pages are copied, none of it may leak."""
    torch.manual_seed(page)
    for ctx in (1, page - 1, page + 3, 333, 1500):
        kc, vc, bt = make_cache(ctx, 4, page)
        q = torch.randn(32, 64, device=dev).half()
        ref = R.paged_attention_ref(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), ctx, page)
        last, used = bt[(ctx - 1) // page].item(), (ctx - 1) % page + 1
        kc[last, :, used:], vc[last, :, used:] = float("nan"), float("nan")
        for spare_page in bt[(ctx + page - 1) // page:].tolist():
            kc[spare_page], vc[spare_page] = float("nan"), float("nan")
        for PS in (128, 256, 2048):
            for ver in (1, 2, 3):
                out = run_attn(K, q, kc, vc, bt, ctx, PS, ver)
                assert torch.isfinite(out).all() and rel_err(out, ref) <= ATTN_TOL, (page, ctx, PS, ver)
    assert K.paged_attention_status() == 0


@pytest.mark.parametrize("D,n_q,n_kv,page", [(64, 32, 4, 16), (128, 8, 2, 16), (64, 8, 8, 32), (64, 16, 4, 4)])
def test_rope_attention_in_one_launch(K, D, n_q, n_kv, page):
    """b200_rope_paged_attention against b200_rope_append(_batched) followed by b200_paged_attention_batched: the
    attention output and both caches bit for bit (page 4: the entry point falls back to the two kernels); and the
    same again with the splits merged inside the launch by the last block to arrive (the count returns to zero)."""
    torch.manual_seed(D + page)
    arrive = torch.zeros(n_kv, dtype=torch.int32, device=dev)
    cos, sin = (t.to(dev) for t in R.rope_tables(3000, D))
    for ctx, PS in ((1, 64), (17, 64), (64, 64), (65, 64), (300, 128), (1000, 256), (2049, 512)):
        n_pages = (ctx + page - 1) // page + 2
        kc = torch.randn(n_pages, n_kv, page, D, device=dev).half()
        vc = torch.randn(n_pages, n_kv, page, D, device=dev).half()
        bt = torch.randperm(n_pages, device=dev).int()
        qkv = torch.randn((n_q + 2 * n_kv) * D, device=dev).half()
        pos = torch.tensor([ctx - 1], dtype=torch.int32, device=dev)
        S = (ctx + PS - 1) // PS + 1
        bufs = lambda: (torch.full((n_q, S, D), float("nan"), device=dev), torch.full((n_q, S), float("nan"), device=dev),
                        torch.full((n_q, S), float("nan"), device=dev), torch.empty(n_q, D, dtype=torch.half, device=dev))
        # reference path: two kernels (rotates q in place, so on a copy)
        q2, kc2, vc2 = qkv.clone(), kc.clone(), vc.clone()
        K.rope_append_batched(q2.view(1, -1), cos, sin, pos, bt.view(1, -1), kc2, vc2, n_q, n_kv)
        o2, m2, l2, out2 = bufs()
        K.paged_attention_batched(q2[: n_q * D].view(1, n_q, D), kc2, vc2, bt.view(1, -1), pos, PS, o2.unsqueeze(0),
                                  m2.unsqueeze(0), l2.unsqueeze(0), out2.view(1, n_q, D))
        # one launch
        q1, kc1, vc1 = qkv.clone(), kc.clone(), vc.clone()
        o1, m1, l1, out1 = bufs()
        K.rope_paged_attention(q1, cos, sin, pos, bt, kc1, vc1, n_q, n_kv, PS, o1, m1, l1, out1)
        assert torch.equal(out1, out2), (D, n_q, n_kv, page, ctx, PS)
        assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2), (ctx, PS)
        if page >= 8:
            assert torch.equal(q1, qkv)      # the fused kernel leaves qkv alone
        q3, kc3, vc3 = qkv.clone(), kc.clone(), vc.clone()
        o3, m3, l3, out3 = bufs()
        out3.fill_(float("nan"))
        K.rope_paged_attention(q3, cos, sin, pos, bt, kc3, vc3, n_q, n_kv, PS, o3, m3, l3, out3, arrive)
        assert torch.equal(out3, out2), ("last-arriver combine", D, n_q, n_kv, page, ctx, PS)
        assert torch.equal(kc3, kc2) and torch.equal(vc3, vc2) and int(arrive.abs().sum()) == 0
    assert K.paged_attention_status() == 0


def test_attention_golden(K, golden):
    g = golden("ops")
    T = lambda k: torch.from_numpy(g[k]).to(dev)
    for ver in (1, 2, 3):
        out = run_attn(K, T("attn_q_d64"), T("ra_kc_d64"), T("ra_vc_d64"), T("ra_bt_d64"), 70, 32, ver)
        assert rel_err(out, torch.from_numpy(g["attn_out_d64"])) <= ATTN_TOL, ver


@pytest.mark.parametrize("D,n_q,n_kv", [(64, 32, 4), (128, 64, 8), (128, 8, 1), (128, 16, 8)])
@pytest.mark.parametrize("B", [1, 8])
def test_attention_batched(K, D, n_q, n_kv, B):
    """Batch of ragged contexts drawn from [128, 8192] (batch 1: each of 128/512/2048/8192 in turn), one shared
    page pool, per-sequence block tables that are disjoint random page sets."""
    torch.manual_seed(B * 1000 + D)
    page = 16
    ctx_sets = [[c] for c in (128, 512, 2048, 8192)] if B == 1 else [torch.randint(128, 8193, (B,)).tolist()]
    for ctxs in ctx_sets:
        max_pages = (max(ctxs) + page - 1) // page
        pool = sum((c + page - 1) // page for c in ctxs) + 5
        kc = torch.randn(pool, n_kv, page, D, device=dev).half()
        vc = torch.randn(pool, n_kv, page, D, device=dev).half()
        perm = torch.randperm(pool)
        bt = torch.zeros(B, max_pages, dtype=torch.int32)
        o = 0
        for b, c in enumerate(ctxs):
            n = (c + page - 1) // page
            bt[b, :n] = perm[o:o + n]
            o += n
        q = torch.randn(B, n_q, D, device=dev).half()
        pos = torch.tensor([c - 1 for c in ctxs], dtype=torch.int32, device=dev)
        ref = R.paged_attention_batched_ref(q.cpu(), kc.cpu(), vc.cpu(), bt, ctxs, page)
        for PS, ver in ((256, 0), (512, 1), (256, 2), (512, 3)):
            S = (max(ctxs) + PS - 1) // PS
            o_part = torch.full((B, n_q, S, D), float("nan"), device=dev)
            m_part = torch.full((B, n_q, S), float("nan"), device=dev)
            l_part = torch.full_like(m_part, float("nan"))
            out = torch.empty(B, n_q, D, dtype=torch.half, device=dev)
            K.paged_attention_batched(q, kc, vc, bt.to(dev), pos, PS, o_part, m_part, l_part, out, version=ver)
            assert rel_err(out, ref) <= ATTN_TOL, (D, n_q, n_kv, ctxs, PS, ver)


# ---- 6. fused operators ---------------------------------------------------------------------------------
@pytest.mark.parametrize("H", [2048, 8192, 128, 4104])
def test_add_rmsnorm(K, H):
    torch.manual_seed(H)
    w = (1 + 0.1 * torch.randn(H, device=dev)).half()
    x = (torch.randn(H, device=dev) * 3).half()
    d = torch.randn(H, device=dev).half()
    xr, outr = R.add_rmsnorm_ref(x.cpu().clone(), d.cpu(), w.cpu(), 1e-5)
    xk, out = x.clone(), torch.empty_like(x)
    K.add_rmsnorm(xk, d, w, out, 1e-5)
    assert torch.equal(xk.cpu(), xr)                               # residual: exact
    assert rel_err(out, outr) <= FUSED_TOL
    xk = x.clone()
    K.add_rmsnorm(xk, None, w, out, 1e-5)
    assert torch.equal(xk, x)                                      # no delta: x untouched
    assert rel_err(out, R.add_rmsnorm_ref(x.cpu(), None, w.cpu(), 1e-5)[1]) <= FUSED_TOL


def test_fused_golden(K, golden):
    g = golden("ops")
    T = lambda k: torch.from_numpy(g[k].copy()).to(dev)
    x, out = T("norm_x"), torch.empty(256, dtype=torch.half, device=dev)
    K.add_rmsnorm(x, T("norm_delta"), T("norm_w"), out, 1e-5)
    assert np.array_equal(x.cpu().numpy().view(np.uint16), g["norm_xout"].view(np.uint16))
    assert rel_err(out, torch.from_numpy(g["norm_out"])) <= FUSED_TOL
    out = torch.empty(320, dtype=torch.half, device=dev)
    K.swiglu(T("swiglu_gu"), out)
    assert rel_err(out, torch.from_numpy(g["swiglu_out"])) <= FUSED_TOL


@pytest.mark.parametrize("I", [5632, 28672, 3584, 8])
def test_swiglu(K, I):
    torch.manual_seed(I)
    gu = (torch.randn(2 * I, device=dev) * 2).half()
    out = torch.empty(I, dtype=torch.half, device=dev)
    K.swiglu(gu, out)
    assert rel_err(out, R.swiglu_ref(gu.cpu())) <= FUSED_TOL


@pytest.mark.parametrize("pos", [0, 1, 37, 2047, 4095])
def test_rope_append_d64(K, pos):
    torch.manual_seed(pos)
    n_q, n_kv, page = 32, 4, 16
    cos, sin = R.rope_tables(4096)
    kc, vc, bt = make_cache(4096, n_kv, page)
    kr, vr = kc.cpu().clone(), vc.cpu().clone()
    qkv = torch.randn((n_q + 2 * n_kv) * 64, device=dev).half()
    qref = R.rope_append_ref(qkv.cpu().clone(), cos, sin, pos, kr, vr, bt.cpu(), n_q, n_kv, 64, page)
    qk = qkv.clone()
    K.rope_append(qk, cos.to(dev), sin.to(dev), torch.tensor([pos], dtype=torch.int32, device=dev), bt, kc, vc, n_q,
                  n_kv)
    assert rel_err(qk[: n_q * 64].view(n_q, 64), qref) <= FUSED_TOL
    assert rel_err(kc, kr) <= FUSED_TOL
    assert torch.equal(vc.cpu(), vr)                               # v is copied: exact
    assert torch.equal(qk[n_q * 64:], qkv[n_q * 64:])              # k, v inside qkv are left alone


@pytest.mark.parametrize("D", [64, 128])
def test_rope_append_batched(K, D):
    torch.manual_seed(D)
    B, n_q, n_kv, page, max_pos = 3, 8, 2, 16, 600
    cos, sin = R.rope_tables(max_pos, D)
    pool = 3 * 40
    kc = torch.randn(pool, n_kv, page, D, device=dev).half()
    vc = torch.randn(pool, n_kv, page, D, device=dev).half()
    bt = torch.randperm(pool).int().view(B, 40)
    poss = [0, 37, 599]
    qkv = torch.randn(B, (n_q + 2 * n_kv) * D, device=dev).half()
    kr, vr = kc.cpu().clone(), vc.cpu().clone()
    qrefs = [R.rope_append_ref(qkv[b].cpu().clone(), cos, sin, poss[b], kr, vr, bt[b], n_q, n_kv, D, page)
             for b in range(B)]
    qk = qkv.clone()
    K.rope_append_batched(qk, cos.to(dev), sin.to(dev), torch.tensor(poss, dtype=torch.int32, device=dev), bt.to(dev),
                          kc, vc, n_q, n_kv)
    for b in range(B):
        assert rel_err(qk[b, : n_q * D].view(n_q, D), qrefs[b]) <= FUSED_TOL
    assert rel_err(kc, kr) <= FUSED_TOL and torch.equal(vc.cpu(), vr)


def test_rope_golden(K, golden):
    g = golden("ops")
    for D in (64, 128):
        T = lambda k: torch.from_numpy(g[f"{k}_d{D}"].copy()).to(dev)
        kc, vc, qkv = T("ra_kc"), T("ra_vc"), T("ra_qkv").view(1, -1)
        K.rope_append_batched(qkv, T("rope_cos"), T("rope_sin"), torch.tensor([37], dtype=torch.int32, device=dev),
                              T("ra_bt").view(1, -1), kc, vc, 8, 2)
        assert rel_err(qkv[0, : 8 * D].view(8, D), torch.from_numpy(g[f"ra_q_out_d{D}"])) <= FUSED_TOL
        assert rel_err(kc, torch.from_numpy(g[f"ra_kc_out_d{D}"])) <= FUSED_TOL
        assert np.array_equal(vc.cpu().numpy().view(np.uint16), g[f"ra_vc_out_d{D}"].view(np.uint16))


def test_exchange_kernels_with_one_rank(K):
    """W = 1: no peer to wait for, so the fused kernels reduce to add_rmsnorm / a copy and run on a single GPU.
    (Two ranks need two GPUs: see tests/test_tp_gpu.py.)"""
    import ctypes
    torch.manual_seed(5)
    H, n = 4096, 1000
    hdr = K.comm_header_bytes()
    off2 = hdr + 2 * H + 256
    base = K.comm_alloc(off2 + 2 * n + 256)
    try:
        peers = (ctypes.c_void_p * 1)(base)
        assert K.comm_error(base) == 0 and len(K.comm_export(base)) == 64
        part = torch.randn(H, device=dev).half()
        shard = torch.randn(n, device=dev).half()
        import llm_decode_kernels_b200.tp as TP
        torch.as_tensor(TP._RawCuda(base + hdr, H, "<f2"), device=dev).copy_(part)
        torch.as_tensor(TP._RawCuda(base + off2, n, "<f2"), device=dev).copy_(shard)
        x0, w = torch.randn(H, device=dev).half(), (1 + 0.1 * torch.randn(H, device=dev)).half()
        for _ in range(3):   # the step counter advances; the result does not change
            x, out = x0.clone(), torch.empty(H, dtype=torch.half, device=dev)
            K.tp_allreduce_add_rmsnorm(peers, 0, hdr, x, w, out, 1e-5)
            xr, ref = x0.clone(), torch.empty(H, dtype=torch.half, device=dev)
            K.add_rmsnorm(xr, part, w, ref, 1e-5)
            assert torch.equal(x, xr) and torch.equal(out, ref)
            dst = torch.zeros(n, dtype=torch.half, device=dev)
            K.tp_allgather(peers, 0, off2, dst, n)
            assert torch.equal(dst, shard)
        assert K.comm_error(base) == 0
        K.comm_reset(base)
    finally:
        K.comm_free(base)


def test_gemv_with_allreduce_inside(K):
    """b200_gemv_w4a16_tiled_allreduce on one GPU. W = 1: no peer, the kernel's push / sum path must give the bits of
    the plain tile-layout GEMV, call after call (the slot's call counter moves on). W = 2 with a second local block
    standing in for a peer that never pushes: the bounded wait runs out, the error word is set, y is left alone."""
    import ctypes
    torch.manual_seed(7)
    hdr = K.comm_header_bytes()
    for N, Kd in ((8192, 1024), (2048, 5632), (1000, 512)):     # 70B TP8 o_proj shard, TinyLlama down, ragged tiles
        ql = PQ.QuantLinear((torch.randn(N, Kd) * 0.05).half(), 128, keep_ref=False)
        tiled = K.gemv_tile_repack(ql.packed.to(dev), ql.sz.to(dev), 128)
        x = torch.randn(Kd, device=dev).half()
        want = torch.empty(N, dtype=torch.half, device=dev)
        K.gemv_w4a16_tiled(tiled, x, want, N, Kd)
        nbytes = hdr + 2 * ((K.tp_gemv_slot_bytes(N, 2) + 255) // 256 * 256)
        mine, silent = K.comm_alloc(nbytes), K.comm_alloc(nbytes)
        try:
            one = (ctypes.c_void_p * 1)(mine)
            for _ in range(3):
                y = torch.zeros(N, dtype=torch.half, device=dev)
                K.gemv_tiled_allreduce(tiled, x, y, N, Kd, one, 0, hdr)
                assert torch.equal(y, want)
            assert K.comm_error(mine) == 0
            two = (ctypes.c_void_p * 2)(mine, silent)
            K.comm_set_wait_limit(mine, 2000)
            y = torch.full((N,), 7.0, dtype=torch.half, device=dev)
            K.gemv_tiled_allreduce(tiled, x, y, N, Kd, two, 0, hdr)
            torch.cuda.synchronize()                              # returns: every wait is bounded
            assert K.comm_error(mine) == 1 and bool((y == 7.0).all())
            K.comm_reset(mine)
            assert K.comm_error(mine) == 0
        finally:
            K.comm_free(mine)
            K.comm_free(silent)
    with pytest.raises(RuntimeError):
        K.gemv_tiled_allreduce(tiled, x, torch.empty(1001, dtype=torch.half, device=dev), 1001, 512,
                               (ctypes.c_void_p * 1)(0), 0, hdr)


def test_gemv_push_and_its_consumer(K):
    """b200_gemv_w4a16_tiled_push + b200_tp_pushed_add_rmsnorm on one GPU. W = 1: the pushed words, summed by the
    consumer, give the bits of GEMV followed by add_rmsnorm, call after call (the tag moves on). W = 2 with a second
    local block standing in for a peer that never pushes: the consumer's bounded poll runs out, the error word is
    set, x and out are left alone."""
    import ctypes
    torch.manual_seed(9)
    hdr = K.comm_header_bytes()
    N, Kd = 2048, 1024
    ql = PQ.QuantLinear((torch.randn(N, Kd) * 0.05).half(), 128, keep_ref=False)
    tiled = K.gemv_tile_repack(ql.packed.to(dev), ql.sz.to(dev), 128)
    w = (1 + 0.1 * torch.randn(N, device=dev)).half()
    nbytes = hdr + 2 * ((K.tp_gemv_slot_bytes(N, 2) + 255) // 256 * 256)
    mine, silent = K.comm_alloc(nbytes), K.comm_alloc(nbytes)
    try:
        one = (ctypes.c_void_p * 1)(mine)
        for it in range(3):
            xin = torch.randn(Kd, device=dev).half()
            resid = torch.randn(N, device=dev).half()
            y = torch.empty(N, dtype=torch.half, device=dev)
            K.gemv_w4a16_tiled(tiled, xin, y, N, Kd)
            x_ref, out_ref = resid.clone(), torch.empty(N, dtype=torch.half, device=dev)
            K.add_rmsnorm(x_ref, y, w, out_ref, 1e-5)
            x_got, out_got = resid.clone(), torch.empty(N, dtype=torch.half, device=dev)
            K.gemv_tiled_push(tiled, xin, N, Kd, one, 0, hdr)
            K.tp_pushed_add_rmsnorm(one, 0, hdr, x_got, w, out_got, 1e-5)
            assert torch.equal(x_got, x_ref) and torch.equal(out_got, out_ref), it
        assert K.comm_error(mine) == 0
        two = (ctypes.c_void_p * 2)(mine, silent)
        K.comm_set_wait_limit(mine, 2000)
        x_got, out_got = torch.full((N,), 3.0, dtype=torch.half, device=dev), torch.full((N,), 7.0, dtype=torch.half, device=dev)
        K.gemv_tiled_push(tiled, xin, N, Kd, two, 0, hdr)       # pushes into both blocks; nobody pushes as rank 1
        K.tp_pushed_add_rmsnorm(two, 0, hdr, x_got, w, out_got, 1e-5)
        torch.cuda.synchronize()                                 # returns: the poll is bounded
        assert K.comm_error(mine) == 1 and bool((x_got == 3.0).all()) and bool((out_got == 7.0).all())
        K.comm_reset(mine)
        assert K.comm_error(mine) == 0
    finally:
        K.comm_free(mine)
        K.comm_free(silent)


def test_exchange_wait_that_runs_out_is_reported(K):
    """A peer that never signals: the exchange kernel gives up after its bound, reports it and leaves the outputs
    alone. Made on one GPU without any fault: the "peer" is a second local block that no kernel ever writes, and the
    bound is set to a few thousand polls (milliseconds) through the block header."""
    import ctypes
    H = 1024
    hdr = K.comm_header_bytes()
    mine, silent = K.comm_alloc(hdr + 2 * H + 256), K.comm_alloc(hdr + 2 * H + 256)
    try:
        peers = (ctypes.c_void_p * 2)(mine, silent)
        K.comm_set_wait_limit(mine, 2000)
        x0 = torch.randn(H, device=dev).half()
        w = torch.ones(H, dtype=torch.half, device=dev)
        x, out = x0.clone(), torch.full((H,), 7.0, dtype=torch.half, device=dev)
        K.tp_allreduce_add_rmsnorm(peers, 0, hdr, x, w, out, 1e-5)
        torch.cuda.synchronize()                                  # the call returns: the wait was bounded
        assert K.comm_error(mine) == 1
        assert torch.equal(x, x0) and bool((out == 7.0).all())    # nothing was computed from a partial that never came
        dst = torch.full((2 * 8,), 3.0, dtype=torch.half, device=dev)
        K.tp_allgather(peers, 0, hdr, dst, 8)
        torch.cuda.synchronize()
        assert bool((dst == 3.0).all())
        K.comm_reset(mine)
        K.comm_reset(silent)
        assert K.comm_error(mine) == 0
    finally:
        K.comm_free(mine)
        K.comm_free(silent)


def test_embed_and_argmax(K):
    torch.manual_seed(0)
    emb = torch.randn(1000, 2048, device=dev).half()
    tok = torch.tensor([613], dtype=torch.int64, device=dev)
    x = torch.empty(2048, dtype=torch.half, device=dev)
    K.embed_row(emb, tok, x)
    assert torch.equal(x, emb[613])
    for V in (32000, 128256, 5, 1025):
        lg = torch.randn(V, device=dev).half()
        i, j = sorted(torch.randperm(V)[:2].tolist())
        lg[i] = lg[j] = 9.0                                        # a tie: the lower index must win
        pos = torch.tensor([41], dtype=torch.int32, device=dev)
        K.argmax(lg, tok, pos)
        assert int(tok) == i == R.argmax_ref(lg.cpu()) and int(pos) == 42
    lg = -torch.rand(77, device=dev).half() - 1                    # all negative
    K.argmax(lg, tok)
    assert int(tok) == R.argmax_ref(lg.cpu())
    lg = torch.randn(4099, device=dev).half()[3:]                  # not 16-byte aligned: the scalar scan
    K.argmax(lg, tok)
    assert int(tok) == R.argmax_ref(lg.cpu())
    # no comparable logit at all: an index inside the vocabulary, never 2^31 - 1
    K.argmax(torch.full((32000,), float("nan"), dtype=torch.half, device=dev), tok)
    assert int(tok) == 0
    lg = torch.full((1000,), float("nan"), dtype=torch.half, device=dev)
    lg[617] = -3.0
    K.argmax(lg, tok)
    assert int(tok) == 617
    # a token id outside the table reads row 0 instead of memory far outside it
    for bad in (1000, -5, 1 << 40):
        tok.fill_(bad)
        K.embed_row(emb, tok, x)
        assert torch.equal(x, emb[0])


def test_bw_read_runs(K):
    buf = torch.ones(64 << 20, dtype=torch.uint8, device=dev)
    sink = torch.zeros(1, dtype=torch.int32, device=dev)
    for unroll in (1, 4, 8):
        K.bw_read(buf, sink, 148 * 8, 512, unroll)
    torch.cuda.synchronize()
    assert int(sink) == 0
