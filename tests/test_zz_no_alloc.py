"""The K-grouped entry point that brings its own scratch memory.

`b200gemm_k_grouped_static_scratch` exists for hosts that cannot give the library device
memory (a runtime that owns all of HBM, or a loop that cannot tolerate cudaMalloc's device-wide
synchronisation).  It must compute exactly what `b200gemm_k_grouped` computes with a
caller-provided workspace.  The check runs two different problems back to back through the new
entry point: the built-in array still holds the first call's plan when the second starts, which
must not matter.  This file sorts last so a run that stops at the first failure has already been
through every other test; it also passes when run on its own in a fresh process."""

import pytest
import torch

import oracle as O
from triton_grouped_gemm_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _problem(seed, sizes, m_dim, n_dim):
    gen = torch.Generator().manual_seed(seed)
    k_tot = sum(sizes)
    a = (torch.randn(k_tot, m_dim, generator=gen) * 0.5).bfloat16().to(DEV)
    b = (torch.randn(k_tot, n_dim, generator=gen) * 0.5).bfloat16().to(DEV)
    return a, b, torch.tensor(sizes, dtype=torch.int64, device=DEV)


def _with_workspace(a, b, sizes):
    lib = _lib.load()
    g, (k_tot, m_dim), n_dim = sizes.numel(), a.shape, b.shape[1]
    c = torch.empty(g, m_dim, n_dim, device=DEV, dtype=a.dtype)
    ws = torch.empty(int(lib.b200gemm_k_grouped_workspace_bytes(g)), dtype=torch.uint8, device=DEV)
    rc = lib.b200gemm_k_grouped(a.data_ptr(), b.data_ptr(), c.data_ptr(), sizes.data_ptr(), 1, None, None, g, k_tot,
                                m_dim, n_dim, 0, ws.data_ptr(), ws.numel(), -1, torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "b200gemm_k_grouped")
    return c


def _static_scratch(a, b, sizes, out):
    g, (k_tot, m_dim), n_dim = sizes.numel(), a.shape, b.shape[1]
    rc = _lib.load().b200gemm_k_grouped_static_scratch(a.data_ptr(), b.data_ptr(), out.data_ptr(), sizes.data_ptr(), 1,
                                                       None, None, g, k_tot, m_dim, n_dim, 0, -1,
                                                       torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "b200gemm_k_grouped_static_scratch")


def _rdiff(x, ref):
    return ((x.float() - ref.float()).abs().sum() / ref.float().abs().sum()).item()


def test_static_scratch_matches_workspace_entry_on_two_calls_in_a_row():
    p1 = _problem(1, [700, 0, 33, 2100, 64, 5, 1290], 512, 768)
    p2 = _problem(2, [16, 1500, 300, 0, 0, 941], 256, 320)
    ref1, ref2 = _with_workspace(*p1), _with_workspace(*p2)
    # outputs are allocated before the calls under test; the calls themselves allocate nothing
    out1 = torch.full_like(ref1, float("nan"))
    out2 = torch.full_like(ref2, float("nan"))
    torch.cuda.synchronize()
    _static_scratch(*p1, out1)
    _static_scratch(*p2, out2)   # the array still holds the plan of the first problem
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    # same kernel, same schedule inputs -> the tolerance of the K-grouped tests (rdiff 2e-4); in
    # fact the results are identical
    assert _rdiff(out1, ref1) < 2e-4 and _rdiff(out2, ref2) < 2e-4
    assert torch.equal(out1, ref1) and torch.equal(out2, ref2)
    # and against the CPU oracle directly, so this file does not lean on the other K-grouped tests
    for (a, b, sizes), out in ((p1, out1), (p2, out2)):
        ref = O.k_grouped_ref(a.cpu(), b.cpu(), sizes.cpu())
        assert _rdiff(out.cpu(), ref) < 2e-4
    # and once more with the first problem, now after the second one used the array
    _static_scratch(*p1, out1)
    torch.cuda.synchronize()
    assert torch.equal(out1, ref1)


def test_static_scratch_rejects_too_many_groups():
    a, b, sizes = _problem(3, [1] * 8, 128, 128)
    out = torch.empty(8, 128, 128, device=DEV, dtype=torch.bfloat16)
    rc = _lib.load().b200gemm_k_grouped_static_scratch(a.data_ptr(), b.data_ptr(), out.data_ptr(), sizes.data_ptr(), 1,
                                                       None, None, 1025, 8, 128, 128, 0, -1, None)
    assert rc == -1
    assert "1024" in _lib.last_error() and "groups" in _lib.last_error()
