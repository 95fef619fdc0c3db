"""The tcgen05 GEMM (C ABI sru_b200_gemm) against an fp32 matmul of the same 16-bit operands.

Tolerance: the products are exact in fp32 and accumulation is fp32 in tensor memory, so an fp32
output must agree with a float32 library matmul to 1e-4 relative; a 16-bit output adds one
rounding (bf16 2^-9, fp16 2^-11 relative), bound 1e-2 / 2e-3.  The 16-bit GEMM has no pinned
result in the reference (it calls a vendor library), so the fp32 matmul is the checker here.
"""
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _gemm():
    from sru_b200.projection import gemm
    return gemm


def _ref(a, b, ta, tb):
    A = a.float().t() if ta else a.float()
    B = b.float().t() if tb else b.float()
    return A @ B


SIZES = [
    # M,    N,    K
    (128,  256,  64),
    (256,  512,  128),
    (640,  384,  128),      # first benchmark configuration's projection
    (200,  264,  120),      # ragged M, N % 256 != 0, K % 64 != 0 (fbank-like input width 120)
    (1000, 6144, 2048),     # one row block of the speech-style layer
    (2048, 6144, 1000),     # weight-gradient shape: long reduction
    (64,   8,    8),
    (4096, 3072, 1024),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("layout", ["nn", "nt", "tn"])
@pytest.mark.parametrize("size", SIZES)
def test_gemm_layouts(size, layout, dtype):
    """nn: U = x W (A K-major, B N-major); nt: grad_x = grad_U W^T; tn: grad_W = x^T grad_U."""
    gemm = _gemm()
    M, N, K = size
    g = torch.Generator().manual_seed(M + N + K)
    ta, tb = layout[0] == "t", layout[1] == "t"
    a = (torch.randn((K, M) if ta else (M, K), generator=g) * 0.5).to(dtype).to(DEV)
    b = (torch.randn((N, K) if tb else (K, N), generator=g) * 0.5).to(dtype).to(DEV)
    ref = _ref(a, b, ta, tb)
    out32 = gemm(a, b, trans_a=ta, trans_b=tb, out_dtype=torch.float32)
    out16 = gemm(a, b, trans_a=ta, trans_b=tb)
    torch.cuda.synchronize()
    from sru_b200 import _lib
    _lib.check_device_error()
    assert out16.dtype == dtype and out32.dtype == torch.float32
    assert rel_err(out32, ref) <= 1e-4, rel_err(out32, ref)
    assert rel_err(out16, ref) <= (1e-2 if dtype == torch.bfloat16 else 2e-3), rel_err(out16, ref)


def test_gemm_bias_and_accumulate():
    gemm = _gemm()
    g = torch.Generator().manual_seed(3)
    M, N, K = 300, 520, 192
    a = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    b = torch.randn(K, N, generator=g).bfloat16().to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    ref = a.float() @ b.float()
    out = gemm(a, b, out_dtype=torch.float32, col_bias=bias)
    assert rel_err(out, ref + bias) <= 1e-4
    base = torch.randn(M, N, generator=g).to(DEV)
    acc = base.clone()
    gemm(a, b, out=acc, accumulate=True)
    assert rel_err(acc, ref + base) <= 1e-4
    # strided output / operands: leading dimensions larger than the logical width
    big_a = torch.zeros(M, K + 64, dtype=torch.bfloat16, device=DEV)
    big_a[:, :K] = a
    big_c = torch.full((M, N + 8), 7.0, device=DEV)
    gemm(big_a[:, :K], b, out=big_c[:, :N])
    assert rel_err(big_c[:, :N], ref) <= 1e-4
    assert torch.all(big_c[:, N:] == 7.0)


def test_gemm_many_tiles_persistent():
    """More tiles than SMs: every CTA walks several tiles through both accumulators."""
    gemm = _gemm()
    g = torch.Generator().manual_seed(5)
    M, N, K = 128 * 37, 256 * 9, 320
    a = (torch.randn(M, K, generator=g) * 0.3).bfloat16().to(DEV)
    b = (torch.randn(N, K, generator=g) * 0.3).bfloat16().to(DEV)
    out = gemm(a, b, trans_b=True, out_dtype=torch.float32)
    assert rel_err(out, a.float() @ b.float().t()) <= 1e-4


def test_projection_autograd_matches_library():
    """project() (tcgen05 forward / dgrad / wgrad) against torch.mm autograd on the same bf16 data."""
    from sru_b200 import projection
    from sru_b200.projection import project
    before = projection.gemm_backend()
    projection.set_gemm_backend("tcgen05")
    try:
        g = torch.Generator().manual_seed(8)
        x = torch.randn(384, 256, generator=g).bfloat16().to(DEV).requires_grad_(True)
        w = (torch.randn(256, 768, generator=g) * 0.1).bfloat16().to(DEV).requires_grad_(True)
        gu = torch.randn(384, 768, generator=g).bfloat16().to(DEV)
        u = project(x, w)
        u.backward(gu)
        xr = x.detach().float().requires_grad_(True)
        wr = w.detach().float().requires_grad_(True)
        ur = xr @ wr
        ur.backward(gu.float())
        assert rel_err(u, ur) <= 1e-2 and rel_err(x.grad, xr.grad) <= 1e-2 and rel_err(w.grad, wr.grad) <= 1e-2
    finally:
        projection.set_gemm_backend(before)


@pytest.mark.parametrize("force", [None, 4])
def test_gemm_split_k(force):
    """Weight-gradient shape that under-fills the GPU (narrow input layer, long reduction): the K slabs'
    fp32 partials plus the reduction kernel must give the same product; also with accumulation."""
    from sru_b200 import _lib
    gemm = _gemm()
    g = torch.Generator().manual_seed(21)
    M, N, K = 120, 1024, 8192
    a = (torch.randn(K, M, generator=g) * 0.1).bfloat16().to(DEV)
    b = (torch.randn(K, N, generator=g) * 0.1).bfloat16().to(DEV)
    ref = a.float().t() @ b.float()
    with _lib.options(gemm_ksplit=force):
        out = gemm(a, b, trans_a=True, out_dtype=torch.float32)
        out16 = gemm(a, b, trans_a=True)
        base = torch.randn(M, N, generator=g).to(DEV)
        acc = base.clone()
        gemm(a, b, trans_a=True, out=acc, accumulate=True)
    assert rel_err(out, ref) <= 1e-4 and rel_err(out16, ref) <= 1e-2 and rel_err(acc, ref + base) <= 1e-4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("size", [
    # M,    N,    K       ragged rows / a second store box partly or wholly outside N / eight and four epilogue warps
    (1000, 6144, 2048), (4096, 3072, 1024), (777, 264, 120), (2500, 200, 64), (300, 520, 1280), (256 * 9, 256 * 5 + 72, 512)])
def test_gemm_tma_store_epilogue(size, dtype):
    """16-bit output of the pair kernel through tiled bulk stores from shared memory (default) against the same
    kernel writing with warp stores: bit-identical, with a column bias, when accumulating onto C, and into a strided
    output whose guard columns and rows stay untouched."""
    from sru_b200 import _lib
    gemm = _gemm()
    M, N, K = size
    g = torch.Generator().manual_seed(M * 3 + N + K)
    a = (torch.randn(M, K, generator=g) * 0.5).to(dtype).to(DEV)
    b = (torch.randn(K, N, generator=g) * 0.5).to(dtype).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    base = torch.randn(M, N, generator=g).to(dtype).to(DEV)
    got = {}
    for tma in (0, 1):
        with _lib.options(gemm_2sm=1, gemm_tma_store=tma):
            plain = gemm(a, b)
            biased = gemm(a, b, col_bias=bias)
            acc = base.clone()
            gemm(a, b, out=acc, accumulate=True)
            big = torch.full((M + 3, N + 24), 7.0, dtype=dtype, device=DEV)
            gemm(a, b, out=big[:M, 8:8 + N])
            got[tma] = (plain, biased, acc, big)
    torch.cuda.synchronize()
    _lib.check_device_error()
    ref = a.float() @ b.float()
    tol = 1e-2 if dtype == torch.bfloat16 else 2e-3
    assert rel_err(got[1][0], ref) <= tol and rel_err(got[1][1], ref + bias) <= tol
    assert rel_err(got[1][2], ref + base.float()) <= tol
    for x, y in zip(got[0], got[1]):
        assert torch.equal(x, y)
    big = got[1][3]
    assert torch.all(big[M:] == 7.0) and torch.all(big[:, :8] == 7.0) and torch.all(big[:, 8 + N:] == 7.0)


@pytest.mark.parametrize("layout", ["nn", "nt", "tn"])
@pytest.mark.parametrize("size", [(4096, 3072, 1024), (256 * 37, 256 * 9, 320), (2048, 6144, 64), (1000, 6144, 2048)])
def test_gemm_dynamic_tile_order(size, layout):
    """Option gemm_dynamic: the CTA pairs take their tiles from a global counter (posted through a mailbox to
    both CTAs and all roles) instead of a fixed stride.  Same results, bit for bit: a tile is computed whole by
    whichever pair takes it.  Shapes with many rounds, with one k-block per tile, and with ragged edges."""
    from sru_b200 import _lib
    gemm = _gemm()
    M, N, K = size
    g = torch.Generator().manual_seed(M + K)
    ta, tb = layout[0] == "t", layout[1] == "t"
    a = (torch.randn((K, M) if ta else (M, K), generator=g) * 0.5).bfloat16().to(DEV)
    b = (torch.randn((N, K) if tb else (K, N), generator=g) * 0.5).bfloat16().to(DEV)
    static = gemm(a, b, trans_a=ta, trans_b=tb)
    assert _lib.lib().sru_b200_gemm_workspace_bytes(M, N, K, 0) == 0
    with _lib.options(gemm_dynamic=1):
        # counter and mailboxes live in the caller's workspace: a product with several rounds of tiles asks for it
        if ((M + 255) // 256) * ((N + 255) // 256) > 74:
            assert _lib.lib().sru_b200_gemm_workspace_bytes(M, N, K, 0) > 0
        for _ in range(3):       # several launches: the scheduler words are refilled per launch
            dyn = gemm(a, b, trans_a=ta, trans_b=tb)
            dyn32 = gemm(a, b, trans_a=ta, trans_b=tb, out_dtype=torch.float32)
    torch.cuda.synchronize()
    _lib.check_device_error()
    assert torch.equal(dyn, static)
    assert rel_err(dyn32, _ref(a, b, ta, tb)) <= 1e-4


def test_first_layer_products_full_size():
    """The two products of benchmark configuration 5's first layer (120 -> 2048 per direction x 2, k = 4) at full
    size: forward 256 000 x 8192 over K = 120 (two 64-wide k-blocks, the second partly out of range), and its weight
    gradient 120 x 8192 over K = 256 000, which the library cuts into K slabs (fp32 partials + reduction kernel)."""
    from conftest import check_parity
    from sru_b200 import _lib
    gemm = _gemm()
    g = torch.Generator(device=DEV).manual_seed(17)
    M, N, K = 256000, 8192, 120
    a = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(K, N, device=DEV, generator=g) * 0.15).bfloat16()
    out = gemm(a, w)
    rows = torch.tensor([0, 63, 64, 128, 255, 256, 131071, 255999], device=DEV)
    check_parity("gemm 256000x8192x120 fwd", "U rows", out[rows], a[rows].float() @ w.float(), 1e-2)
    gu = (torch.randn(M, N, device=DEV, generator=g) * 0.1).bfloat16()
    assert _lib.lib().sru_b200_gemm_workspace_bytes(K, N, M, 0) > 0      # a split is planned for this shape
    gw = gemm(a, gu, trans_a=True, out_dtype=torch.float32)               # (M,120)^T x (M,8192)
    cols = torch.arange(0, N, 257, device=DEV)
    ref = a.float().t() @ gu[:, cols].float()
    check_parity("gemm 120x8192x256000 wgrad", "grad_W cols", gw[:, cols], ref, 1e-3)
    torch.cuda.synchronize()
    _lib.check_device_error()


@pytest.mark.parametrize("layout", ["nn", "nt", "tn"])
@pytest.mark.parametrize("size", [(640, 384, 128), (256, 512, 2048), (8, 8, 8), (1000, 264, 72)])
def test_gemm_f32_split_accuracy(size, layout):
    """float32 product through the three-way bfloat16 split against a float64 product.  The split itself is exact to
    2^-24, but the tensor cores' fp32 accumulation is not rounded like IEEE additions: the error grows with the
    reduction length (3e-6 of the largest element up to K = 128, 3e-5 up to K = 2048; the library's float32 GEMM on
    the same data is recorded beside it).  That is why this path is opt-in."""
    from conftest import record_parity
    from sru_b200.projection import gemm_f32
    M, N, K = size
    g = torch.Generator().manual_seed(M + 3 * K)
    ta, tb = layout[0] == "t", layout[1] == "t"
    a = torch.randn((K, M) if ta else (M, K), generator=g).to(DEV)
    b = torch.randn((N, K) if tb else (K, N), generator=g).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    out = gemm_f32(a, b, trans_a=ta, trans_b=tb, col_bias=bias)
    A, B = (a.t() if ta else a).double(), (b.t() if tb else b).double()
    ref = A @ B + bias.double()
    prior = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        lib32 = (a.t() if ta else a) @ (b.t() if tb else b) + bias
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prior
    e, e_lib = rel_err(out, ref), rel_err(lib32, ref)
    tol = 3e-6 if K <= 128 else 3e-5
    record_parity("gemm_f32 %s %s" % (size, layout), "C", e, tol, "library fp32 GEMM: %.1e" % e_lib)
    assert e <= tol, (e, e_lib)
    from sru_b200 import _lib
    torch.cuda.synchronize()
    _lib.check_device_error()
