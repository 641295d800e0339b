"""BF16 / FP16 M-grouped and masked M-grouped GEMM on the GPU against the CPU oracle.

Tolerance (from the build target): rdiff = sum|a-b| / sum|b| <= 2e-3 against the oracle's
fp32-accumulated, once-rounded result; in practice the two differ only by accumulation
order, so a much tighter bound (2e-4) is asserted as well where noted."""

import pytest
import torch

import oracle as O
from triton_grouped_gemm_b200 import _lib
from triton_grouped_gemm_b200.gemm.BF16.m_grouped_gemm_TMA import _m_grouped_gemm_launch, m_grouped_gemm
from triton_grouped_gemm_b200.gemm.BF16.m_grouped_gemm_masked_TMA import m_grouped_gemm_masked

pytestmark = pytest.mark.gpu
DEV = "cuda"
RDIFF_TOL = 2e-3


@pytest.fixture(autouse=True)
def _reset_tuning():
    yield
    _lib.load().b200gemm_set_block_n(0)
    _lib.load().b200gemm_set_cta_pair(-1)
    assert _lib.device_status() == 0


def _run(a, b, sizes, trans_b, block_n=0, size_dtype=torch.int64, pair=-1):
    _lib.load().b200gemm_set_block_n(block_n)
    _lib.load().b200gemm_set_cta_pair(pair)
    n = b.shape[1] if trans_b else b.shape[2]
    c = torch.full((a.shape[0], n), float("nan"), device=DEV, dtype=a.dtype)
    _m_grouped_gemm_launch(a.to(DEV), b.to(DEV), c, sizes.to(DEV, size_dtype), trans_b)
    torch.cuda.synchronize()
    return c.cpu()


def _check(out, ref, rows_written, tol=RDIFF_TOL):
    assert not torch.isnan(out[:rows_written].float()).any(), "unwritten / NaN outputs inside groups"
    r = O.rdiff(out[:rows_written].float(), ref[:rows_written].float())
    assert r <= tol, f"rdiff {r:.3e} > {tol}"
    # rows past the last group must not have been touched
    assert torch.isnan(out[rows_written:].float()).all()


@pytest.mark.parametrize("block_n", [64, 128, 256])
@pytest.mark.parametrize("trans_b", [True, False])
def test_single_tile_known_answer(block_n, trans_b):
    """One 128-row group, K = 64: A selects one k per row, B holds small integers, so every
    output is exact and a wrong descriptor / swizzle shows up as a wrong integer."""
    m, n, k = 128, 256, 64
    a = torch.zeros(m, k)
    a[torch.arange(m), torch.arange(m) % k] = 1.0
    b_nk = ((torch.arange(n)[:, None] * 3 + torch.arange(k)[None, :] * 5) % 97 - 48).float()
    b = b_nk if trans_b else b_nk.t().contiguous()
    ref = a @ b_nk.t()
    out = _run(a.bfloat16(), b.bfloat16()[None].contiguous(), torch.tensor([m]), trans_b, block_n)
    assert torch.equal(out.float(), ref), f"max abs err {(out.float() - ref).abs().max()}"


@pytest.mark.parametrize("name,trans_b", [("small_nt", True), ("small_nn", False), ("small_nt_fp16", True)])
def test_golden_small(golden_dir, name, trans_b):
    c = torch.load(golden_dir / "m_grouped.pt", weights_only=False)[name]
    out = _run(c["a"], c["b"], c["sizes"], trans_b)
    _check(out, c["out"], int(c["sizes"].sum()), tol=2e-4)


def test_config0_golden_and_oracle(golden_dir):
    g = torch.load(golden_dir / "m_grouped.pt", weights_only=False)["config0"]
    a, b, sizes = O.config0_inputs(0)
    out = _run(a, b, sizes, True)
    _check(out, g["out"], a.shape[0], tol=2e-4)
    _check(out, O.m_grouped_ref(a, b, sizes, True, fp32_accumulate_explicit=True), a.shape[0], tol=2e-4)
    # through the registered custom op as a user would call it
    out2 = m_grouped_gemm(a.to(DEV), b.to(DEV), sizes.to(DEV), True).cpu()
    assert torch.equal(out2, out)
    out3 = torch.ops.moe.m_grouped_gemm(a.to(DEV), b.to(DEV), sizes.to(DEV), True, -1).cpu()
    assert torch.equal(out3, out)


CASES = [
    # sizes, n, k
    ([128, 256, 384], 256, 128),
    ([1, 127, 129, 0, 255, 0, 0, 64], 264, 200),   # ragged rows, n and k tails, empty groups
    ([0, 0, 5], 8, 8),
    ([300], 1536, 2048),
    ([5, 1, 1, 1, 700, 3], 72, 1024),
    ([130] * 40, 512, 320),
]


@pytest.mark.parametrize("block_n", [0, 64, 128, 256])
@pytest.mark.parametrize("trans_b", [True, False])
@pytest.mark.parametrize("sizes,n,k", CASES)
def test_ragged_vs_oracle(sizes, n, k, trans_b, block_n):
    gen = torch.Generator().manual_seed(n * 31 + k + len(sizes))
    m = sum(sizes)
    extra = 7  # rows past the last group: must stay untouched
    a = (torch.randn(m + extra, k, generator=gen) * 0.5).bfloat16()
    g = len(sizes)
    b = (torch.randn(g, n, k, generator=gen) * 0.5).bfloat16()
    ref = O.m_grouped_ref(a[:m], b, sizes, True, fp32_accumulate_explicit=True)
    bb = b if trans_b else b.transpose(1, 2).contiguous()
    out = _run(a, bb, torch.tensor(sizes), trans_b, block_n)
    _check(out, ref, m, tol=2e-4)


@pytest.mark.parametrize("trans_b", [True, False])
def test_pair_kernel_known_answer(trans_b):
    """CTA-pair kernel on one 256 x 256 x 64 tile with exact integer data."""
    m, n, k = 256, 256, 64
    a = torch.zeros(m, k)
    a[torch.arange(m), torch.arange(m) % k] = 1.0
    a[128:, 0] += 2.0
    b_nk = ((torch.arange(n)[:, None] * 3 + torch.arange(k)[None, :] * 5) % 97 - 48).float()
    b = b_nk if trans_b else b_nk.t().contiguous()
    ref = a @ b_nk.t()
    out = _run(a.bfloat16(), b.bfloat16()[None].contiguous(), torch.tensor([m]), trans_b, pair=1)
    assert torch.equal(out.float(), ref), f"max abs err {(out.float() - ref).abs().max()}"


@pytest.mark.parametrize("trans_b", [True, False])
@pytest.mark.parametrize("sizes,n,k", CASES + [([256, 512, 130, 0, 384, 127], 512, 256), ([1000, 3000], 1536, 512)])
def test_pair_kernel_vs_oracle(sizes, n, k, trans_b):
    gen = torch.Generator().manual_seed(n * 31 + k + len(sizes))
    m = sum(sizes)
    extra = 7
    a = (torch.randn(m + extra, k, generator=gen) * 0.5).bfloat16()
    b = (torch.randn(len(sizes), n, k, generator=gen) * 0.5).bfloat16()
    ref = O.m_grouped_ref(a[:m], b, sizes, True, fp32_accumulate_explicit=True)
    bb = b if trans_b else b.transpose(1, 2).contiguous()
    out = _run(a, bb, torch.tensor(sizes), trans_b, pair=1)
    _check(out, ref, m, tol=2e-4)


def test_pair_kernel_masked():
    g, e, n, k = 6, 512, 512, 192
    gen = torch.Generator().manual_seed(17)
    lhs = (torch.randn(g * e, k, generator=gen) * 0.5).bfloat16()
    rhs = (torch.randn(g, n, k, generator=gen) * 0.5).bfloat16()
    masked = torch.tensor([512, 0, 129, 300, 1, 256])
    init = torch.full((g * e, n), 3.0, dtype=torch.bfloat16)
    ref = O.m_grouped_masked_ref(lhs, rhs, init, masked, e, fp32_accumulate_explicit=True)
    out = init.clone().to(DEV)
    _lib.load().b200gemm_set_cta_pair(1)
    m_grouped_gemm_masked(lhs.to(DEV), rhs.to(DEV), out, masked.to(DEV), e, True)
    torch.cuda.synchronize()
    out = out.cpu()
    assert O.rdiff(out.float(), ref.float()) < 2e-4
    for i, mm in enumerate(masked.tolist()):
        assert torch.all(out[i * e + mm:(i + 1) * e] == 3.0)


@pytest.mark.parametrize("size_dtype", [torch.int32, torch.int64])
def test_size_dtypes_and_fp16(size_dtype):
    gen = torch.Generator().manual_seed(5)
    sizes = [200, 56, 128]
    a = torch.randn(sum(sizes), 256, generator=gen).half()
    b = torch.randn(3, 128, 256, generator=gen).half()
    ref = O.m_grouped_ref(a, b, sizes, True, fp32_accumulate_explicit=True)
    out = _run(a, b, torch.tensor(sizes), True, size_dtype=size_dtype)
    _check(out, ref, sum(sizes), tol=2e-4)


def test_num_sms_argument():
    gen = torch.Generator().manual_seed(6)
    sizes = torch.tensor([256, 256, 100])
    a = torch.randn(612, 128, generator=gen).bfloat16().to(DEV)
    b = torch.randn(3, 512, 128, generator=gen).bfloat16().to(DEV)
    full = m_grouped_gemm(a, b, sizes.to(DEV), True)
    few = m_grouped_gemm(a, b, sizes.to(DEV), True, 3)
    one = m_grouped_gemm(a, b, sizes.to(DEV), True, 1)
    assert torch.equal(full, few) and torch.equal(full, one)


@pytest.mark.parametrize("trans_b", [True, False])
def test_masked_golden(golden_dir, trans_b):
    c = torch.load(golden_dir / "masked.pt", weights_only=False)
    e = c["expected_m"]
    rhs = c["rhs"] if trans_b else c["rhs"].transpose(1, 2).contiguous()
    out = torch.full(c["full"].shape, 7.0, dtype=torch.bfloat16, device=DEV)
    assert m_grouped_gemm_masked(c["lhs"].to(DEV), rhs.to(DEV), out, c["masked_m"].to(DEV), e, trans_b) is None
    torch.cuda.synchronize()
    out = out.cpu()
    for g, m in enumerate(c["masked_m"].tolist()):
        if m:
            assert O.rdiff(out[g * e:g * e + m].float(), c["full"][g * e:g * e + m].float()) < 2e-4
        assert torch.all(out[g * e + m:(g + 1) * e] == 7.0), "rows past masked_m were written"


@pytest.mark.parametrize("g,e,n,k", [(16, 256, 3072, 512), (5, 128, 64, 64), (4, 384, 200, 136), (3, 100, 128, 64)])
def test_masked_vs_oracle(g, e, n, k):
    gen = torch.Generator().manual_seed(g * e + n)
    lhs = (torch.randn(g * e, k, generator=gen) * 0.5).bfloat16()
    rhs = (torch.randn(g, n, k, generator=gen) * 0.5).bfloat16()
    masked = torch.randint(0, e + 1, (g,), generator=gen)
    masked[0] = e
    if g > 2:
        masked[1] = 0
    init = torch.full((g * e, n), 3.0, dtype=torch.bfloat16)
    ref = O.m_grouped_masked_ref(lhs, rhs, init, masked, e, fp32_accumulate_explicit=True)
    out = init.clone().to(DEV)
    m_grouped_gemm_masked(lhs.to(DEV), rhs.to(DEV), out, masked.to(DEV), e, True)
    torch.cuda.synchronize()
    out = out.cpu()
    assert O.rdiff(out.float(), ref.float()) < 2e-4
    untouched = torch.ones(g * e, dtype=torch.bool)
    for i, m in enumerate(masked.tolist()):
        untouched[i * e:i * e + m] = False
    assert torch.all(out[untouched] == 3.0)


def test_full_size_properties():
    """Benchmark-size problem (G=128, 655360+ rows, K=2048, N=1536): the oracle is checked on a
    sample of groups, and the whole result through linearity: C(A, B) + C(A, B) == C(A, 2B)."""
    sizes = O.routing_sizes(128, 655360, seed=2026)
    m = int(sizes.sum())
    gen = torch.Generator(device=DEV).manual_seed(1)
    a = (torch.randn(m, 2048, device=DEV, generator=gen) * 0.02).bfloat16()
    b = (torch.randn(128, 1536, 2048, device=DEV, generator=gen) * 0.02).bfloat16()
    sz = sizes.to(DEV)
    c1 = m_grouped_gemm(a, b, sz, True)
    c2 = m_grouped_gemm(a, b * 2, sz, True)
    assert torch.equal(c1 * 2, c2)  # exact: scaling by 2 commutes with every rounding
    starts = torch.cumsum(sizes, 0) - sizes
    # every group against real arithmetic: its first, a middle and its last rows (8 each), so a
    # group that read another expert's weights or the wrong row block cannot hide behind linearity
    for g in range(128):
        s0, sz_g = int(starts[g]), int(sizes[g])
        rows = torch.cat([torch.arange(0, 8), torch.arange(sz_g // 2, sz_g // 2 + 8), torch.arange(sz_g - 8, sz_g)]) + s0
        ref = (a[rows.to(DEV)].cpu().float() @ b[g].cpu().float().t()).bfloat16()
        assert O.rdiff(c1[rows.to(DEV)].cpu().float(), ref.float()) < 2e-4, f"group {g}"
    for g in (0, 63, 127):
        s, n_rows = int(starts[g]), min(int(sizes[g]), 256)
        ref = (a[s:s + n_rows].cpu().float() @ b[g].cpu().float().t()).bfloat16()
        assert O.rdiff(c1[s:s + n_rows].cpu().float(), ref.float()) < 2e-4
    # trans_b=False on the same data gives the same result
    c3 = m_grouped_gemm(a, b.transpose(1, 2).contiguous(), sz, False)
    assert O.rdiff(c3.float().cpu(), c1.float().cpu()) < 1e-5


def test_host_operand_pipeline_matches_single_launch():
    """m_grouped_gemm_host (chunked copies and launches on three streams) returns the same bits as
    one launch on device-resident operands."""
    from triton_grouped_gemm_b200.host import m_grouped_gemm_host

    gen = torch.Generator().manual_seed(12)
    sizes = torch.tensor([300, 0, 129, 1000, 64, 77, 512, 5])
    m = int(sizes.sum())
    a = (torch.randn(m, 256, generator=gen) * 0.5).bfloat16().pin_memory()
    b = (torch.randn(8, 384, 256, generator=gen) * 0.5).bfloat16().pin_memory()
    ref = m_grouped_gemm(a.to(DEV), b.to(DEV), sizes.to(DEV), True).cpu()
    for chunks in (1, 3, 8):
        out = m_grouped_gemm_host(a, b, sizes, True, chunks=chunks)
        torch.cuda.synchronize()
        assert torch.equal(out, ref)


def test_device_layout_builders_match_host_layouts():
    """gemm.layout on CUDA sizes (library kernels) against the same functions on host sizes."""
    from triton_grouped_gemm_b200.gemm import layout as L

    for sizes in ([5, 0, 128, 129, 1, 300], [128] * 7, [0, 0, 3], list(range(0, 700, 7))):
        for dt in (torch.int32, torch.int64):
            host = torch.tensor(sizes, dtype=dt)
            dev = host.to(DEV)
            for block_m in (128, 64):
                assert L.make_group_starts(dev, block_m=block_m).cpu().tolist() == L.make_group_starts(host, block_m=block_m).tolist()
                assert (L.make_group_starts(dev, padded=True, block_m=block_m).cpu().tolist()
                        == L.make_group_starts(host, padded=True, block_m=block_m).tolist())
                assert (L.make_deep_gemm_psum_layout(dev, block_m=block_m).cpu().tolist()
                        == L.make_deep_gemm_psum_layout(host, block_m=block_m).tolist())
                a = L.make_deep_gemm_grouped_layout(dev, block_m=block_m).cpu()
                b = L.make_deep_gemm_grouped_layout(host, block_m=block_m)
                assert a.dtype == b.dtype and torch.equal(a, b)


def test_launch_is_cuda_graph_capturable():
    """The entry points never synchronise or allocate, and group sizes stay on the device, so a
    captured launch can be replayed after the sizes and the operands changed in place."""
    from triton_grouped_gemm_b200.gemm.BF16.m_grouped_gemm_TMA import _m_grouped_gemm_launch

    gen = torch.Generator().manual_seed(9)
    g, n, k, m = 6, 256, 192, 1024
    a = (torch.randn(m, k, generator=gen) * 0.5).bfloat16().to(DEV)
    b = (torch.randn(g, n, k, generator=gen) * 0.5).bfloat16().to(DEV)
    c = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    sizes = torch.tensor([100, 0, 300, 24, 200, 400], dtype=torch.int64, device=DEV)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        _m_grouped_gemm_launch(a, b, c, sizes, True)          # warm-up outside capture
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        _m_grouped_gemm_launch(a, b, c, sizes, True)
    # new routing and new activations in the same buffers, then replay
    sizes.copy_(torch.tensor([1, 500, 0, 123, 300, 100], dtype=torch.int64))
    a.copy_((torch.randn(m, k, generator=gen) * 0.5).bfloat16())
    c.zero_()
    graph.replay()
    torch.cuda.synchronize()
    ref = O.m_grouped_ref(a.cpu(), b.cpu(), sizes.cpu(), True)
    assert O.rdiff(c.cpu().float(), ref.float()) < 2e-4


@pytest.mark.parametrize("pair", [0, 1], ids=["single", "pair"])
@pytest.mark.parametrize("trans_b", [True, False])
def test_sizes_summing_past_m_rows_are_cut_off_and_flagged(pair, trans_b):
    """A routing vector whose sum exceeds the rows A and C really have (sizes live on the device, the
    host cannot check them): the group that runs over is cut at m_rows, later groups get nothing,
    memory past the end of C stays untouched and the status word says so.  C sits inside a larger
    allocation of this test, so an overrun would be seen, not faulted on."""
    sizes_bad = [100, 200, 300, 64]
    m_rows, n, k = 450, 512, 192
    gen = torch.Generator().manual_seed(3)
    a = (torch.randn(m_rows, k, generator=gen) * 0.5).bfloat16()
    b_nk = (torch.randn(4, n, k, generator=gen) * 0.5).bfloat16()
    b = b_nk if trans_b else b_nk.transpose(1, 2).contiguous()
    c_big = torch.full((m_rows + 512, n), 7.0, device=DEV, dtype=torch.bfloat16)
    _lib.load().b200gemm_set_cta_pair(pair)
    _m_grouped_gemm_launch(a.to(DEV), b.to(DEV), c_big[:m_rows], torch.tensor(sizes_bad, device=DEV), trans_b)
    status = _lib.device_status()
    assert status == 0x10, f"status {status:#x}"
    out = c_big.cpu()
    assert torch.all(out[m_rows:] == 7.0), "rows past m_rows were written"
    ref = O.m_grouped_ref(a, b, torch.tensor([100, 200, 150, 0]), trans_b)
    assert O.rdiff(out[:m_rows].float(), ref.float()) < 2e-4
