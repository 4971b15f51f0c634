"""The C-ABI library builds, loads, and exports exactly what include/b200decode.h declares (no GPU needed:
nothing here launches a kernel)."""
import ctypes
import re
from pathlib import Path

import pytest

from llm_decode_kernels_b200 import ext

HEADER = Path(__file__).resolve().parents[1] / "include" / "b200decode.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return re.findall(r"\b(b200_\w+)\s*\(", text)


def test_header_declares_the_six_reference_ops():
    names = set(declared_functions())
    for op in ("gemv_w4a16", "bw_read", "paged_attention", "add_rmsnorm", "swiglu", "rope_append"):
        assert f"b200_{op}" in names


def test_library_exports_every_declared_symbol():
    lib = ext.load_library()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in b200decode.h but not exported"
    assert lib.b200_version() >= 100
    assert lib.b200_strerror(-1).decode().startswith("bad argument")


def test_python_signatures_cover_the_header():
    names = set(declared_functions()) - {"b200_version", "b200_strerror", "b200_last_cuda_error", "b200_decode_step",
                                         "b200_decode_step_xchg_bytes", "b200_tp_gemv_slot_bytes",
                                         "b200_gemv_w4a16_tiled_bytes"}   # declared on their own
    assert names == set(ext.SIGNATURES), names ^ set(ext.SIGNATURES)
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    for name, argtypes in ext.SIGNATURES.items():
        m = re.search(name + r"\s*\((.*?)\)\s*;", text, flags=re.S)
        assert m, name
        assert len([a for a in m.group(1).split(",") if a.strip() not in ("", "void")]) == len(argtypes), name


def test_exchange_sizes_are_host_arithmetic():
    """Sizes a caller allocates from: the persistent step's exchange area (per layer qkv, J partial attention outputs
    and their log-sum-exp words, o, act, down; J = min(4, grid / n_q) context slices per query head) and the
    tensor-parallel GEMV region (control, reserved flag rows, W x N tagged words)."""
    lib = ext.load_library()
    L, H, I, n_q, n_kv, D, grid = 22, 2048, 5632, 32, 4, 64, 148           # TinyLlama shape on a B200: J = 4
    per_layer = (n_q + 2 * n_kv) * D + 4 * n_q * D + n_q * 8 + H + I + H
    assert lib.b200_decode_step_xchg_bytes(L, H, I, n_q, n_kv, D, grid) == (L * per_layer + grid * 4) * 4
    per_layer_1 = (64 + 2 * 8) * 128 + 2 * 64 * 128 + 64 * 4 + 8192 + 28672 + 8192      # 64 heads on 148 CTAs: J = 2
    assert lib.b200_decode_step_xchg_bytes(1, 8192, 28672, 64, 8, 128, grid) == (per_layer_1 + grid * 4) * 4
    assert lib.b200_decode_step_xchg_bytes(L, H, I, n_q, n_kv, D, 0) == 0
    assert lib.b200_tp_gemv_slot_bytes(8192, 8) == 256 + 1024 * 16 * 4 + 8 * 8192 * 4


def test_bad_arguments_are_refused_on_the_host():
    """Argument checks run before any CUDA call, so they can be exercised without a device."""
    lib = ext.load_library()
    assert lib.b200_gemv_w4a16(2, 0, 0, 0, None, None, None, None, 4, 128, 7, None) == -1       # null pointers
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    assert lib.b200_gemv_w4a16(2, 0, 0, 0, p16, p16, p16, p16, 4, 100, 7, None) == -3           # K % 32 != 0
    assert lib.b200_gemv_w4a16(2, 0, 0, 0, p16, p16, p16, p16, 4, 128, 4, None) == -3           # group 16 < 32
    assert lib.b200_gemv_w4a16(2, 0, 0, 0, p16 + 4, p16, p16, p16, 4, 128, 7, None) == -2       # misaligned weights
    assert lib.b200_add_rmsnorm(p16, None, p16, p16, 12, 1e-5, None) == -3                      # H % 8 != 0
    peers = (ctypes.c_void_p * 2)(p16, p16)
    assert lib.b200_tp_allreduce_add_rmsnorm(peers, 2, 2, 256, p16, p16, p16, 64, 1e-5, None) == -1   # rank >= W
    assert lib.b200_tp_allreduce_add_rmsnorm(peers, 0, 2, 64, p16, p16, p16, 64, 1e-5, None) == -2    # inside header
    assert lib.b200_tp_allreduce_add_rmsnorm(peers, 0, 2, 256, p16, p16, p16, 60, 1e-5, None) == -3   # H % 8 != 0
    assert lib.b200_tp_allgather(peers, 0, 17, 256, p16, 64, None) == -1                              # too many ranks
    assert lib.b200_comm_alloc(16, ctypes.byref(ctypes.c_void_p())) == -1                             # below the header
    assert lib.b200_comm_header_bytes() == 256
    assert lib.b200_add_rmsnorm(p16, None, p16, p16, 65536, 1e-5, None) == -5                   # H over capacity
    assert lib.b200_swiglu(p16, p16, 0, None) == -1
    assert lib.b200_embed_row(p16, p16, p16, 64, 0, None) == -1                                 # empty table
    assert lib.b200_gemv_w4a16_tune(1, 5632, 2048, 3, 148) == -1                                # ksplit not 1/2/4/8
    assert lib.b200_gemv_w4a16_tune(1, 5632, 2048, 4, 176) == 0 and lib.b200_gemv_w4a16_tune(1, 5632, 2048, 0, 0) == 0
    assert lib.b200_paged_attention(7, p16, p16, p16, p16, p16, 32, 4, 4, 64, 1, p16, p16, p16, p16, None) == -1
    assert lib.b200_paged_attention(2, p16, p16, p16, p16, p16, 12, 4, 4, 64, 1, p16, p16, p16, p16, None) == -3
    assert lib.b200_paged_attention_batched(p16, p16, p16, p16, 8, p16, 1, 32, 4, 96, 4, 64, 1, p16, p16, p16, p16,
                                            None) == -3                                         # head_dim 96


def test_python_face_refuses_cpu_tensors():
    import torch
    K = ext.load()
    x = torch.zeros(128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        K.swiglu(torch.zeros(256, dtype=torch.float16), x)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        K.add_rmsnorm(x, None, x, x, 1e-5)
