"""The C-ABI library builds, loads without a GPU and exports what the header declares."""

import ctypes
import os
import re

import pytest

from dpk_b200 import _native as N
from dpk_b200 import build as B

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "dpk_b200.h")


@pytest.fixture(scope="module")
def lib():
    B.build()
    return N.load()


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dpk_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/dpk_b200.h but not exported"
    # and the binding table covers exactly the header
    assert sorted(N.SIGNATURES) == names


def test_version_and_error_text(lib):
    assert lib.dpk_version() >= 100
    assert isinstance(N.last_error(), str)


def test_argument_checks_reject_before_any_launch(lib):
    # NULL tensors / bad shapes are refused on the host, so these calls are safe without a GPU
    rc = lib.dpk_gemm_mn(None, 0, None, None, 0, None, None, None, 0, 8, 256, 128, 2, N.BF16, 0, None)
    assert rc == N.ERR_INVALID and "NULL" in N.last_error()
    with pytest.raises(ValueError):
        N.check(rc)
    buf = (ctypes.c_uint8 * 4096)()
    p = ctypes.addressof(buf)
    p = (p + 255) & ~255
    # N not divisible by NG
    rc = lib.dpk_gemm_mn(p, 128, p, None, 128, p, p, p, 250, 8, 250, 128, 4, N.BF16, 0, None)
    assert rc == N.ERR_INVALID and "divisible" in N.last_error()
    # group width that the tensor-core path does not take
    rc = lib.dpk_gemm_k(p, 96, p, 96, p, p, p, 64, 8, 64, 96, 2, N.BF16, None, 0, None, 0, None)
    assert rc == N.ERR_INVALID and "multiple of 64" in N.last_error()
    # unknown dtype
    rc = lib.dpk_gemm_k(p, 128, p, 128, p, p, p, 64, 8, 64, 128, 2, 7, None, 0, None, 0, None)
    assert rc == N.ERR_INVALID
    # head_dim outside {64,128}
    rc = lib.dpk_attn_prefill(p, p, p, p, p, None, p, 1, 16, 16, 4, 2, 96, 2, 0.1, 1, 0, N.BF16, 0, 0, 0, 0, None)
    assert rc == N.ERR_INVALID and "head_dim" in N.last_error()
    # keep outside [0, NG]
    rc = lib.dpk_topk_mask(p, 4, 8, 9, p, None)
    assert rc == N.ERR_INVALID


def test_workspace_sizes(lib):
    assert lib.dpk_route_workspace_bytes(1, 8192, 112) == 32 * 112 * 4
    assert lib.dpk_route_workspace_bytes(2, 100, 8) == 2 * 1 * 8 * 4
    assert lib.dpk_ffn_workspace_bytes(8192, 4096, 14336, 112) > 8192 * 14336 * 2
    assert lib.dpk_attn_decode_workspace_bytes(64, 32768, 32, 8, 128, 8) == 64 * 32 * 32 * 130 * 4
    assert lib.dpk_gemm_k_workspace_bytes(64, 4096) == 64 * 4096 * 4
    assert lib.dpk_gemm_k_workspace_bytes(8192, 4096) == 0


def test_ops_refuse_cpu_tensors():
    import torch

    from dpk_b200 import ops

    a = torch.zeros(1, 8, 128, dtype=torch.bfloat16)
    w = torch.zeros(256, 128, dtype=torch.bfloat16)
    m = torch.ones(1, 8, 2, dtype=torch.bool)
    with pytest.raises(ValueError, match="CUDA"):
        ops.gemm_mn(a, w, m)
    with pytest.raises(ValueError, match="CUDA"):
        ops.gemm_k(torch.zeros(1, 8, 256, dtype=torch.bfloat16), w.T.contiguous(), m)
