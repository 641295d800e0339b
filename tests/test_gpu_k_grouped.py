"""BF16 / FP16 K-grouped GEMM (C[g] = A_g^T B_g) on the GPU against the CPU oracle.
Tolerance: rdiff <= 2e-3 (build target); asserted tighter because only accumulation order
differs from the oracle's fp32-accumulated, once-rounded result."""

import pytest
import torch

import oracle as O
from triton_grouped_gemm_b200 import _lib
from triton_grouped_gemm_b200.gemm.BF16.k_grouped_gemm_TMA import k_grouped_gemm
from triton_grouped_gemm_b200.gemm.BF16 import k_grouped_gemm as k_mod

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True, params=[-1, 1, 0], ids=["auto", "pair", "single"])
def _kernel_form(request):
    """Every case runs with the tile form chosen by size, with CTA pairs (256 x 256 tiles, used
    whenever the call has a workspace) forced, and with them switched off."""
    _lib.load().b200gemm_set_cta_pair(request.param)
    yield
    _lib.load().b200gemm_set_cta_pair(-1)
    assert _lib.device_status() == 0


def test_golden(golden_dir):
    c = torch.load(golden_dir / "k_grouped.pt", weights_only=False)
    out = k_grouped_gemm(c["a"].to(DEV), c["b"].to(DEV), c["sizes"].to(DEV)).cpu()
    assert out.shape == c["out"].shape
    assert O.rdiff(out.float(), c["out"].float()) < 2e-4
    assert torch.all(out[1] == 0)  # empty group -> zeros


@pytest.mark.parametrize("trans", [True, False])
def test_known_answer_single_block(trans):
    """64 tokens, one-hot A: C[g][m, n] = B[token(m), n] exactly."""
    k_tot, m_dim, n_dim = 64, 128, 256
    a = torch.zeros(k_tot, m_dim)
    a[torch.arange(m_dim) % k_tot, torch.arange(m_dim)] = 1.0
    b = ((torch.arange(k_tot)[:, None] * 7 + torch.arange(n_dim)[None, :] * 3) % 101 - 50).float()
    ref = a.t() @ b
    out = k_grouped_gemm(a.bfloat16().to(DEV), b.bfloat16().to(DEV), torch.tensor([k_tot], device=DEV)).cpu()
    assert torch.equal(out[0].float(), ref)


CASES = [
    # sizes, M_DIM, N_DIM
    ([64], 128, 256),
    ([1], 128, 64),
    ([63, 65, 0, 17, 128, 200], 256, 512),
    ([5, 0, 0, 300], 136, 72),          # M_DIM / N_DIM not multiples of the tile
    ([1000, 24, 40], 2048, 768),
    ([16] * 20, 128, 128),
    ([0, 0], 128, 128),
]


@pytest.mark.parametrize("sizes,m_dim,n_dim", CASES)
@pytest.mark.parametrize("size_dtype", [torch.int32, torch.int64])
def test_ragged_vs_oracle(sizes, m_dim, n_dim, size_dtype):
    gen = torch.Generator().manual_seed(m_dim + n_dim + len(sizes))
    k_tot = sum(sizes)
    extra = 9  # rows after the last group must not leak into it
    a = (torch.randn(k_tot + extra, m_dim, generator=gen) * 0.5).bfloat16()
    b = (torch.randn(k_tot + extra, n_dim, generator=gen) * 0.5).bfloat16()
    ref = O.k_grouped_ref(a[:k_tot], b[:k_tot], sizes, fp32_accumulate_explicit=True)
    out = k_grouped_gemm(a.to(DEV), b.to(DEV), torch.tensor(sizes, dtype=size_dtype, device=DEV)).cpu()
    assert out.shape == ref.shape
    assert not torch.isnan(out.float()).any()
    assert O.rdiff(out.float(), ref.float()) < 2e-4
    for g, s in enumerate(sizes):
        if s == 0:
            assert torch.all(out[g] == 0)


def test_tail_rows_of_next_group_do_not_leak_even_if_nonfinite():
    """The k-block holding a group's tail also holds the next group's first rows; they are
    zeroed in shared memory, so even Inf/NaN there must not reach this group's result."""
    sizes = [40, 50]
    gen = torch.Generator().manual_seed(3)
    a = torch.randn(90, 128, generator=gen).bfloat16()
    b = torch.randn(90, 128, generator=gen).bfloat16()
    a[40:48] = float("inf")
    b[40:48] = float("nan")
    out = k_grouped_gemm(a.to(DEV), b.to(DEV), torch.tensor(sizes, device=DEV)).cpu()
    ref0 = (a[:40].float().t() @ b[:40].float()).bfloat16()
    assert torch.isfinite(out[0].float()).all()
    assert O.rdiff(out[0].float(), ref0.float()) < 2e-4


def test_explicit_group_ranges_and_fp16_and_alias_module():
    gen = torch.Generator().manual_seed(11)
    sizes = torch.tensor([70, 30, 100])
    a = torch.randn(200, 128, generator=gen).half()
    b = torch.randn(200, 192, generator=gen).half()
    ref = O.k_grouped_ref(a, b, sizes, fp32_accumulate_explicit=True)
    ends = sizes.cumsum(0)
    starts = ends - sizes
    out = k_grouped_gemm(a.to(DEV), b.to(DEV), sizes.to(DEV), starts.to(DEV), ends.to(DEV)).cpu()
    assert O.rdiff(out.float(), ref.float()) < 2e-4
    out2 = k_mod.k_grouped_gemm(a.to(DEV), b.to(DEV), sizes.to(DEV)).cpu()
    assert torch.equal(out, out2)


def _k_grouped_abi(a, b, sizes, workspace):
    """Direct C-ABI call: workspace=None -> fixed round-robin tiles, tensor -> balanced scheduler."""
    g, (k_tot, m_dim), n_dim = sizes.numel(), a.shape, b.shape[1]
    c = torch.empty(g, m_dim, n_dim, device=DEV, dtype=a.dtype)
    rc = _lib.load().b200gemm_k_grouped(a.data_ptr(), b.data_ptr(), c.data_ptr(), sizes.data_ptr(), 1, None, None, g,
                                        k_tot, m_dim, n_dim, 0, workspace.data_ptr() if workspace is not None else None,
                                        workspace.numel() if workspace is not None else 0, -1,
                                        torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "b200gemm_k_grouped")
    return c


def test_balanced_and_round_robin_schedules_agree():
    """Groups of very different length: the balanced scheduler (scratch buffer, longest groups
    first) and the fixed assignment must produce the same bits; scratch is reusable as is."""
    sizes = [900, 3, 0, 64, 2500, 130, 1, 700, 0, 333]
    gen = torch.Generator().manual_seed(5)
    k_tot = sum(sizes)
    a = (torch.randn(k_tot, 512, generator=gen) * 0.5).bfloat16().to(DEV)
    b = (torch.randn(k_tot, 768, generator=gen) * 0.5).bfloat16().to(DEV)
    st = torch.tensor(sizes, dtype=torch.int64, device=DEV)
    need = int(_lib.load().b200gemm_k_grouped_workspace_bytes(len(sizes)))
    assert need == (64 + 3 * len(sizes)) * 4
    ws = torch.full((need,), 0xAB, dtype=torch.uint8, device=DEV)  # garbage on purpose: the plan kernel initialises it
    c_static = _k_grouped_abi(a, b, st, None)
    c_bal = _k_grouped_abi(a, b, st, ws)
    c_bal2 = _k_grouped_abi(a, b, st, ws)  # second call on the same scratch
    assert torch.equal(c_static, c_bal) and torch.equal(c_bal, c_bal2)
    ref = O.k_grouped_ref(a.cpu(), b.cpu(), sizes, fp32_accumulate_explicit=True)
    assert O.rdiff(c_bal.cpu().float(), ref.float()) < 2e-4
    rc = _lib.load().b200gemm_k_grouped(a.data_ptr(), b.data_ptr(), c_bal.data_ptr(), st.data_ptr(), 1, None, None,
                                        len(sizes), k_tot, 512, 768, 0, ws.data_ptr(), 16, -1, None)
    assert rc == -1 and "too small" in _lib.last_error()


def test_input_checks():
    a = torch.zeros(16, 128, dtype=torch.bfloat16, device=DEV)
    b = torch.zeros(16, 128, dtype=torch.bfloat16, device=DEV)
    s = torch.tensor([16], device=DEV)
    with pytest.raises(AssertionError, match="trans_b=True path has been removed"):
        k_grouped_gemm(a, b, s, trans_b=True)
    with pytest.raises(AssertionError, match="must equal"):
        k_grouped_gemm(a, b[:8], s)
    with pytest.raises(AssertionError, match="int32 or int64"):
        k_grouped_gemm(a, b, s.float())


def test_full_size_properties():
    """Benchmark size (G=128, K_total ~ 663k, 2048 x 768): sampled groups against the oracle and
    exact linearity in B over the whole output."""
    sizes = O.routing_sizes(128, 655360, seed=2026)
    k_tot = int(sizes.sum())
    gen = torch.Generator(device=DEV).manual_seed(2)
    a = (torch.randn(k_tot, 2048, device=DEV, generator=gen) * 0.02).bfloat16()
    b = (torch.randn(k_tot, 768, device=DEV, generator=gen) * 0.02).bfloat16()
    sz = sizes.to(DEV)
    c1 = k_grouped_gemm(a, b, sz)
    c2 = k_grouped_gemm(a, b * 2, sz)
    assert torch.equal(c1 * 2, c2)
    starts = torch.cumsum(sizes, 0) - sizes
    # every group against real arithmetic on the host: a 16 x 16 patch of its output (all of the
    # group's tokens enter every element), at a position that moves with the group
    for g in range(128):
        s, e = int(starts[g]), int(starts[g] + sizes[g])
        r0, c0 = (g * 16) % 2048, (g * 48) % 768
        ref = (a[s:e, r0:r0 + 16].cpu().float().t() @ b[s:e, c0:c0 + 16].cpu().float()).bfloat16()
        assert O.rdiff(c1[g, r0:r0 + 16, c0:c0 + 16].float().cpu(), ref.float()) < 2e-3, f"group {g}"
    for g in (0, 77, 127):
        s, e = int(starts[g]), int(starts[g] + sizes[g])
        ref = (a[s:e].float().t() @ b[s:e].float()).bfloat16()  # fp32 on the GPU as a cross-check only
        assert O.rdiff(c1[g].float().cpu(), ref.float().cpu()) < 1e-3
    g = 5
    s, e = int(starts[g]), int(starts[g] + sizes[g])
    ref = (a[s:e].cpu().float().t() @ b[s:e].cpu().float()).bfloat16()
    assert O.rdiff(c1[g].float().cpu(), ref.float()) < 2e-4
