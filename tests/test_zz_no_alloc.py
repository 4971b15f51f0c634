"""The allocation-free attention entry point (b200_paged_attention_noalloc) against the ordinary one.

Who needs it: callers that may not allocate device memory - a plugin inside a host program that owns the
allocator, a latency-critical path where an allocation could synchronise the device, a process with a memory budget
fixed at start-up. They cannot provide the three split-K scratch arrays b200_paged_attention asks for, so this entry
point keeps the partials in a fixed array inside the library. Checked here through the C ABI: same result as the
ordinary entry point (same tolerance as the other attention tests), on two calls in a row that reuse the array with
different shapes, plus the size limit. The file name sorts last so that a run that stops at the first failure has
already run every other test; it passes alone in a fresh process as well."""
import pytest
import torch

from llm_decode_kernels_b200 import ext
from oracle import ops_oracle as R

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _case(K, n_q, n_kv, D, ctx, PS, seed):
    torch.manual_seed(seed)
    page = 16
    pages = (ctx + page - 1) // page + 2
    kc = torch.randn(pages, n_kv, page, D, device="cuda").half()
    vc = torch.randn(pages, n_kv, page, D, device="cuda").half()
    bt = torch.randperm(pages, device="cuda").int()
    q = torch.randn(n_q, D, device="cuda").half()
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device="cuda")
    S = (ctx + PS - 1) // PS
    ref = torch.empty(n_q, D, dtype=torch.half, device="cuda")
    o_part = torch.empty(1, n_q, S, D, device="cuda")
    m_part, l_part = torch.empty(1, n_q, S, device="cuda"), torch.empty(1, n_q, S, device="cuda")
    K.paged_attention_batched(q.view(1, n_q, D), kc, vc, bt.view(1, -1), pos, PS, o_part, m_part, l_part,
                              ref.view(1, n_q, D))
    out = torch.empty_like(ref)
    K.paged_attention_noalloc(q, kc, vc, bt, pos, PS, S, out)
    torch.cuda.synchronize()
    err = (out.float() - ref.float()).abs().max().item() / ref.float().abs().max().item()
    assert err <= TOL, (n_q, n_kv, D, ctx, PS, err)
    # and against the CPU oracle, so that the check does not rest on another kernel of the same library alone
    want = R.paged_attention_ref(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), ctx, page).float()
    err = (out.cpu().float() - want).abs().max().item() / want.abs().max().item()
    assert err <= TOL, ("oracle", n_q, n_kv, D, ctx, PS, err)


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    K = ext.load()
    _case(K, 32, 4, 64, 2000, 64, seed=1)     # 32 live splits: the whole capacity in the split dimension
    _case(K, 64, 8, 128, 300, 128, seed=2)    # other head count and head_dim over the same array, 3 splits
    _case(K, 8, 1, 128, 40, 64, seed=3)       # one live split: the partial kernel writes the output itself


def test_sizes_beyond_the_fixed_array_are_refused():
    K = ext.load()
    kc = torch.zeros(4, 4, 16, 64, dtype=torch.half, device="cuda")
    q = torch.zeros(32, 64, dtype=torch.half, device="cuda")
    bt = torch.arange(4, dtype=torch.int32, device="cuda")
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="capacity"):
        K.paged_attention_noalloc(q, kc, kc, bt, pos, 16, 33, torch.empty_like(q))        # 33 splits > 32
    q128 = torch.zeros(128, 64, dtype=torch.half, device="cuda")
    kc16 = torch.zeros(4, 16, 16, 64, dtype=torch.half, device="cuda")
    with pytest.raises(RuntimeError, match="capacity"):
        K.paged_attention_noalloc(q128, kc16, kc16, bt, pos, 16, 4, torch.empty_like(q128))  # 128 heads > 64
    # the host face checks shapes before the pointer reaches the kernel
    with pytest.raises(RuntimeError, match="shape"):
        K.paged_attention_noalloc(q, kc, kc, bt, pos, 16, 4, torch.empty(16, 64, dtype=torch.half, device="cuda"))
    with pytest.raises(RuntimeError, match="heads-per-group"):
        K.paged_attention_noalloc(q[:12], kc, kc, bt, pos, 16, 4, torch.empty_like(q[:12]))   # 12 / 4 = 3
