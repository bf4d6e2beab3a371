"""GPU parity of the matmul path against the CPU oracle, through the C ABI.

Covers: the two GEMM seams (`Cuda::gemm` / `gemm_batch`) over every operand layout dfdx can hand
over, forced through each kernel family; the four kernel traits forward + backward; the reference's
property tests (matmul/mod.rs:412-527); and the benchmark configurations at full size through
sampled rows of the oracle plus size-independent properties.

Tolerances: relative Frobenius error vs the f64 oracle <= 1e-5 (f32), <= 2e-3 (f16), 1e-12 (f64).
"""
import itertools

import pytest
import torch

import dfdx_b200
from helpers import FROB_TOL, CudaBackend, OracleBackend, d_exp_mean, d_exp_sum, d_sum

pytestmark = pytest.mark.gpu


def gen(seed):
    return torch.Generator().manual_seed(seed)


def make_mat(rows, cols, major, pad, dtype, g, device):
    """(rows x cols) view: major='r' -> strides (cols+pad, 1); 'c' -> strides (1, rows+pad)."""
    if major == "r":
        base = torch.randn(rows, cols + pad, generator=g, dtype=torch.float64).to(dtype).to(device)
        return base[:, :cols]
    base = torch.randn(cols, rows + pad, generator=g, dtype=torch.float64).to(dtype).to(device)
    return base[:, :rows].t()


def frob(oracle, got, want):
    return oracle.rel_frobenius(got, want)


def check_gemm(dev, oracle, m, k, n, la, lb, lc, beta, dtype, pad, seed, poison=True):
    g = gen(seed)
    a = make_mat(m, k, la, pad, dtype, g, dev.device)
    b = make_mat(k, n, lb, pad, dtype, g, dev.device)
    c = make_mat(m, n, lc, pad, dtype, g, dev.device)
    c_base = c._base if c._base is not None else c
    if beta == 0 and poison:
        c_base.fill_(float("nan"))           # beta == 0 must never read the output buffer
    c_before = c_base.clone()
    want, _ = oracle.matmul(a.cpu(), b.cpu())
    if beta:
        want = want + c.cpu().to(torch.float64)
    dev.gemm((m, k, n), a, a.stride(), b, b.stride(), beta, c, c.stride())
    dev.synchronize()
    err = frob(oracle, c, want)
    assert err <= FROB_TOL[dtype], f"m{m} k{k} n{n} {la}{lb}{lc} beta{beta}: rel frobenius {err:.3e}"
    # canary: padding columns / rows of the output buffer are untouched
    mask = torch.ones_like(c_base, dtype=torch.bool)
    (mask[:, :n] if lc == "r" else mask[:, :m]).fill_(False)
    if mask.any():
        same = (c_base[mask] == c_before[mask]) | (c_base[mask].isnan() & c_before[mask].isnan())
        assert bool(same.all()), "GEMM wrote outside the output extent"


# --------------------------------------------------------------------------------- SIMT family
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.float16])
def test_simt_small_shape_sweep(cuda_dev, oracle, dtype):
    """Every small (m,k,n) x 8 transpose combinations x beta, odd leading dimensions included."""
    cuda_dev.set_path(dfdx_b200.PATH_SIMT)
    try:
        sizes = [1, 2, 3, 5, 17, 33, 65]
        seed = 0
        for m, k, n in itertools.product(sizes, repeat=3):
            if (m + k + n) % 3 and max(m, k, n) > 5:    # thin the large combinations
                continue
            for la, lb, lc in itertools.product("rc", repeat=3):
                seed += 1
                check_gemm(cuda_dev, oracle, m, k, n, la, lb, lc, seed % 2, dtype, pad=seed % 3, seed=seed)
    finally:
        cuda_dev.set_path(dfdx_b200.PATH_AUTO)


def test_simt_degenerate_stride_pairs(cuda_dev, oracle):
    """`matrix_strides` accepts [1,1], [0,1] and [1,0] (matmul/mod.rs:318-320): rank-1 reshapes and broadcasts."""
    dev = cuda_dev
    g = gen(7)
    v = torch.randn(6, generator=g, dtype=torch.float64).to(torch.float32).to(dev.device)
    w = torch.randn(6, 4, generator=g, dtype=torch.float64).to(torch.float32).to(dev.device)
    # (1,6) with strides [6,1] x (6,4)
    out = torch.empty(1, 4, device=dev.device)
    dev.gemm((1, 6, 4), v, (6, 1), w, w.stride(), 0.0, out, (4, 1))
    want, _ = oracle.matmul(v.cpu(), w.cpu())
    assert frob(oracle, out.reshape(4), want) < 1e-6
    # broadcast lhs: every row is v -> strides [0,1]
    out = torch.empty(3, 4, device=dev.device)
    dev.gemm((3, 6, 4), v, (0, 1), w, w.stride(), 0.0, out, (4, 1))
    want3, _ = oracle.matmul(v.cpu().expand(3, 6), w.cpu())
    assert frob(oracle, out, want3) < 1e-6
    # outer product: (6,1) strides [1,1] x (1,4) strides [4,1]
    u = torch.randn(4, generator=g, dtype=torch.float64).to(torch.float32).to(dev.device)
    out = torch.empty(6, 4, device=dev.device)
    dev.gemm((6, 1, 4), v, (1, 1), u, (4, 1), 0.0, out, (4, 1))
    want_o, _ = oracle.matmul(v.cpu(), u.cpu())
    assert frob(oracle, out, want_o) < 1e-6
    dev.synchronize()


# --------------------------------------------------------------------------------- tensor-core family
TC_SHAPES = [(128, 64, 64), (128, 64, 256), (200, 136, 72), (264, 520, 104), (64, 1032, 136), (384, 40, 512)]


@pytest.mark.parametrize("store", [pytest.param(0, id="auto"), pytest.param(1, id="rowstore"), pytest.param(2, id="colstore")])
@pytest.mark.parametrize("tile_n", [64, 128, 256])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("layout", ["".join(p) for p in itertools.product("rc", repeat=3)])
def test_tensor_core_layouts(cuda_dev, oracle, dtype, layout, tile_n, store):
    """tcgen05 path forced, every tile width and both epilogue store orientations: K-major / MN-major A
    and B, row-major / transposed C, ragged M, N and K (TMA zero fill), padded leading dimensions,
    beta 0 and 1."""
    cuda_dev.set_path(dfdx_b200.PATH_TENSOR)
    assert cuda_dev.lib.b200_set_tile_n(tile_n) == 0
    assert cuda_dev.lib.b200_set_store_mode(store) == 0
    try:
        before = cuda_dev.lib.b200_tensor_launch_count()
        for i, (m, k, n) in enumerate(TC_SHAPES):
            check_gemm(cuda_dev, oracle, m, k, n, layout[0], layout[1], layout[2], i % 2, dtype, pad=8, seed=100 + i)
        assert cuda_dev.lib.b200_tensor_launch_count() - before == len(TC_SHAPES)
    finally:
        cuda_dev.lib.b200_set_tile_n(0)
        cuda_dev.lib.b200_set_store_mode(0)
        cuda_dev.set_path(dfdx_b200.PATH_AUTO)


BIG_SHAPES = [(256, 64, 256), (512, 192, 512), (296, 136, 264), (264, 520, 392), (1000, 1032, 136 * 2), (384, 40, 520)]


@pytest.mark.parametrize("layout", ["".join(p) for p in itertools.product("rc", repeat=3)])
def test_f16_256x256_tile_kernel(cuda_dev, oracle, layout):
    """The f16 kernel with 256 x 256 tiles per CTA (two accumulators filling TMEM), forced: K-major / MN-major A and B,
    row-major / transposed C, ragged M, N and K, outputs whose second 128-row block is empty or partial, beta 0
    (NaN-poisoned output) and beta 1; plus a batched problem with MultiHeadAttention-like batch strides."""
    dev = cuda_dev
    dev.set_path(dfdx_b200.PATH_TENSOR)
    assert dev.lib.b200_set_tile_n(512) == 0
    try:
        before = dev.lib.b200_tensor_launch_count()
        for i, (m, k, n) in enumerate(BIG_SHAPES):
            check_gemm(dev, oracle, m, k, n, layout[0], layout[1], layout[2], i % 2, torch.float16, pad=8, seed=900 + i)
        assert dev.lib.b200_tensor_launch_count() - before == len(BIG_SHAPES)
        g = gen(77)
        a = (torch.randn(3, 2, 296, 72, generator=g) * 0.3).half().to(dev.device)
        b = (torch.randn(3, 2, 72, 264, generator=g) * 0.3).half().to(dev.device)
        out = dev.matmat_batch4_forward(a, b)
        dev.synchronize()
        want, _ = oracle.matmul(a.cpu(), b.cpu())
        assert frob(oracle, out, want) <= FROB_TOL[torch.float16]
    finally:
        dev.lib.b200_set_tile_n(0)
        dev.set_path(dfdx_b200.PATH_AUTO)


@pytest.mark.parametrize("slices", [2, 5])
@pytest.mark.parametrize("layout", ["".join(p) for p in itertools.product("rc", repeat=3)])
def test_f16_256x256_tile_kernel_k_slices(cuda_dev, oracle, layout, slices):
    """K slices of 256 x 256 tiles (forced): every unit adds its f32 partial tile into the library's scratch through
    bulk reduce-adds and the finalize kernel folds the scratch into the f16 output; every layout (the scratch keeps
    the kernel's orientation whichever way C lies), ragged M, N and K, beta 0 (NaN-poisoned output) and beta 1."""
    dev = cuda_dev
    dev.set_path(dfdx_b200.PATH_TENSOR)
    assert dev.lib.b200_set_tile_n(512) == 0
    assert dev.lib.b200_set_split_k(slices) == 0
    try:
        before, before_all = dev.lib.b200_tensor_launch_count(), dev.lib.b200_launch_count()
        shapes = [(512, 1032, 520), (296, 2056, 264), (264, 4104, 392)]
        for i, (m, k, n) in enumerate(shapes):
            check_gemm(dev, oracle, m, k, n, layout[0], layout[1], layout[2], i % 2, torch.float16, pad=8, seed=950 + i)
        assert dev.lib.b200_tensor_launch_count() - before == len(shapes)
        assert dev.lib.b200_launch_count() - before_all == 2 * len(shapes)      # GEMM + finalize
    finally:
        dev.lib.b200_set_split_k(0)
        dev.lib.b200_set_tile_n(0)
        dev.set_path(dfdx_b200.PATH_AUTO)


@pytest.mark.parametrize("stored", ["kn", "nk"])
@pytest.mark.parametrize("shape", [(4, 256, 264, 520), (3, 136, 1032, 264), (64, 256, 512, 2048), (2, 72, 24, 16)], ids=str)
def test_weight_gradient_added_in_f32(cuda_dev, oracle, shape, stored):
    """`b200_matmat_br_grad_rhs_f32`: the broadcast-rhs weight gradient of f16 operands added in f32 to an f32 buffer
    that already holds values, in both storage orders of the (K, N) gradient (dfdx's Linear keeps (N, K)), whole-K
    tiles and K slices, ragged extents; against the f64 oracle at f32 accuracy (an f16 gradient buffer would be at 5e-4),
    and twice in a row (it accumulates)."""
    dev = cuda_dev
    b, m, k, n = shape
    g = gen(4000 + sum(shape))
    lhs = (torch.randn(b, m, k, generator=g) * 0.5).half().to(dev.device)
    go = (torch.randn(b, m, n, generator=g) * 0.5).half().to(dev.device)
    start = torch.randn(k, n, generator=g)
    buf = (start if stored == "kn" else start.t().contiguous()).to(dev.device)
    view = buf if stored == "kn" else buf.t()
    want = lhs.cpu().double().reshape(-1, k).t() @ go.cpu().double().reshape(-1, n)
    before = dev.lib.b200_launch_count()
    dev.matmat_br_grad_rhs_f32(lhs, go, view)
    dev.synchronize()
    assert dev.lib.b200_launch_count() - before == 1
    # f32 accumulation of b * m products per element (up to 16384 here) and one f32 rounding of start + sum
    err = oracle.rel_frobenius(view.cpu().double() - start.double(), want)
    assert err <= 2e-5, f"rel frobenius {err:.3e}"
    dev.matmat_br_grad_rhs_f32(lhs, go, view)
    dev.synchronize()
    err = oracle.rel_frobenius(view.cpu().double() - start.double(), 2 * want)
    assert err <= 2e-5, f"rel frobenius {err:.3e} after the second call"
    # operands the tensor-core path cannot address are refused before any launch (the caller keeps its f16 route)
    before = dev.lib.b200_launch_count()
    with pytest.raises(dfdx_b200.B200Error) as e:
        dev.matmat_br_grad_rhs_f32(lhs[:, :, 1:], go, view[1:, :])
    assert e.value.status == dfdx_b200._lib.ERR_UNSUPPORTED
    assert dev.lib.b200_launch_count() == before


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("layout", ["".join(p) for p in itertools.product("rc", repeat=3)])
def test_cta_pair_kernels(cuda_dev, oracle, dtype, layout):
    """The cta_group::2 kernels (two CTAs per 256x256 tile), forced: every layout, ragged shapes incl. one
    where the second CTA of the pair has no rows, beta 0 and 1, long K."""
    cuda_dev.set_path(dfdx_b200.PATH_TENSOR)
    assert cuda_dev.lib.b200_set_cta_pair_mode(2) == 0
    try:
        before = cuda_dev.lib.b200_tensor_launch_count()
        shapes = [(256, 256, 264), (520, 136, 776), (104, 264, 304), (384, 2056, 512)]
        for i, (m, k, n) in enumerate(shapes):
            check_gemm(cuda_dev, oracle, m, k, n, layout[0], layout[1], layout[2], i % 2, dtype, pad=8, seed=300 + i)
        assert cuda_dev.lib.b200_tensor_launch_count() - before == len(shapes)
    finally:
        cuda_dev.lib.b200_set_cta_pair_mode(1)
        cuda_dev.set_path(dfdx_b200.PATH_AUTO)


@pytest.mark.parametrize("slices", [2, 5])
@pytest.mark.parametrize("layout", ["rcr", "crr", "rrc", "ccc"])
def test_split_k_f16(cuda_dev, oracle, layout, slices):
    """f16 split-K: K slices accumulate f32 partial sums in the library's scratch, a finalize kernel folds them
    into the f16 output (beta 0 with NaN-poisoned output, beta 1), both store orientations, ragged shapes."""
    cuda_dev.set_path(dfdx_b200.PATH_TENSOR)
    assert cuda_dev.lib.b200_set_split_k(slices) == 0
    try:
        for store in (1, 2):
            cuda_dev.lib.b200_set_store_mode(store)
            for i, (m, k, n) in enumerate([(128, 2048, 256), (200, 2312, 136), (264, 4104, 264)]):
                check_gemm(cuda_dev, oracle, m, k, n, layout[0], layout[1], layout[2], i % 2, torch.float16, pad=8,
                           seed=500 + i)
    finally:
        cuda_dev.lib.b200_set_split_k(0)
        cuda_dev.lib.b200_set_store_mode(0)
        cuda_dev.set_path(dfdx_b200.PATH_AUTO)


@pytest.mark.parametrize("slices", [2, 3, 7])
@pytest.mark.parametrize("layout", ["rcr", "crr", "rrc", "ccc"])
def test_split_k_f32(cuda_dev, oracle, layout, slices):
    """f32 split-K: K slices of one tile are separate work units whose partial results are added atomically;
    beta 0 (output zeroed first, NaN-poisoned here) and beta 1, ragged shapes, both store orientations."""
    cuda_dev.set_path(dfdx_b200.PATH_TENSOR)
    assert cuda_dev.lib.b200_set_split_k(slices) == 0
    try:
        for store in (1, 2):
            cuda_dev.lib.b200_set_store_mode(store)
            for i, (m, k, n) in enumerate([(128, 1024, 256), (200, 1160, 136), (264, 2056, 264)]):
                check_gemm(cuda_dev, oracle, m, k, n, layout[0], layout[1], layout[2], i % 2, torch.float32, pad=8,
                           seed=400 + i)
    finally:
        cuda_dev.lib.b200_set_split_k(0)
        cuda_dev.lib.b200_set_store_mode(0)
        cuda_dev.set_path(dfdx_b200.PATH_AUTO)


@pytest.mark.parametrize("tile_n", [0, 64, 128])
@pytest.mark.parametrize("layout", ["rcr", "crr", "rrc", "ccc"])
def test_stream_k_f32(cuda_dev, oracle, layout, tile_n):
    """f32 stream-K forced: every CTA takes one contiguous range of the (tile, k-block) space; ranges that cut a
    tile add their partial sums atomically.  Few tiles (ranges shorter than a tile), many tiles (several whole tiles
    per range plus two cut ones), ragged shapes, beta 0 (NaN-poisoned output) and beta 1, both store orientations."""
    cuda_dev.set_path(dfdx_b200.PATH_TENSOR)
    assert cuda_dev.lib.b200_set_split_k(-1) == 0
    assert cuda_dev.lib.b200_set_tile_n(tile_n) == 0
    try:
        for store in (1, 2):
            cuda_dev.lib.b200_set_store_mode(store)
            shapes = [(128, 1024, 256), (200, 1160, 136), (1160, 264, 2056), (4104, 520, 1032)]
            for i, (m, k, n) in enumerate(shapes):
                check_gemm(cuda_dev, oracle, m, k, n, layout[0], layout[1], layout[2], i % 2, torch.float32, pad=8,
                           seed=450 + i)
    finally:
        cuda_dev.lib.b200_set_split_k(0)
        cuda_dev.lib.b200_set_tile_n(0)
        cuda_dev.lib.b200_set_store_mode(0)
        cuda_dev.set_path(dfdx_b200.PATH_AUTO)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_tensor_core_long_k_accuracy(cuda_dev, oracle, dtype):
    """The stated bound must hold where accumulation is longest: K = 16384."""
    cuda_dev.set_path(dfdx_b200.PATH_TENSOR)
    try:
        check_gemm(cuda_dev, oracle, 128, 16384, 64, "r", "c", "r", 0, dtype, pad=0, seed=5)
        check_gemm(cuda_dev, oracle, 96, 4096, 128, "c", "r", "r", 1, dtype, pad=0, seed=6)
    finally:
        cuda_dev.set_path(dfdx_b200.PATH_AUTO)


def test_tensor_core_rejects_unaddressable_operands(cuda_dev):
    """Forced tensor path reports B200_ERR_UNSUPPORTED (no silent fallback) for an odd leading dimension."""
    dev = cuda_dev
    a = torch.zeros(64, 67, device=dev.device)[:, :64]
    b = torch.zeros(64, 64, device=dev.device)
    c = torch.zeros(64, 64, device=dev.device)
    dev.set_path(dfdx_b200.PATH_TENSOR)
    try:
        with pytest.raises(dfdx_b200.B200Error) as e:
            dev.gemm((64, 64, 64), a, a.stride(), b, b.stride(), 0.0, c, c.stride())
        assert e.value.status == dfdx_b200._lib.ERR_UNSUPPORTED
    finally:
        dev.set_path(dfdx_b200.PATH_AUTO)
    # AUTO serves the same call from the SIMT family
    dev.gemm((64, 64, 64), a, a.stride(), b, b.stride(), 0.0, c, c.stride())
    dev.synchronize()


# --------------------------------------------------------------------------------- kernel traits
def _trait_case(cuda_dev, oracle, dtype, a_shape, b_shape, a_perm=None, b_perm=None, path=dfdx_b200.PATH_AUTO,
                seed=0, loss=d_exp_mean, scale=1.0):
    cb, ob = CudaBackend(cuda_dev, dtype), OracleBackend(oracle, dtype)
    g = gen(seed)
    a = (torch.randn(*a_shape, generator=g, dtype=torch.float64) * scale).to(dtype)
    b = (torch.randn(*b_shape, generator=g, dtype=torch.float64) * scale).to(dtype)
    av = a if a_perm is None else a.permute(*a_perm)
    bv = b if b_perm is None else b.permute(*b_perm)
    want, obwd = ob.matmul(av, bv)
    ad, bd = a.to(cuda_dev.device), b.to(cuda_dev.device)
    avd = ad if a_perm is None else ad.permute(*a_perm)
    bvd = bd if b_perm is None else bd.permute(*b_perm)
    cuda_dev.set_path(path)
    try:
        got, cbwd = cb.matmul(avd, bvd)
        go = loss(want)
        gla, glb = cbwd(go)
        cuda_dev.synchronize()
    finally:
        cuda_dev.set_path(dfdx_b200.PATH_AUTO)
    wla, wlb = obwd(go.to(dtype))
    tol = FROB_TOL[dtype]
    assert frob(oracle, got, want) <= tol
    assert frob(oracle, gla, wla) <= tol
    assert frob(oracle, glb, wlb) <= tol


PATHS = [pytest.param(dfdx_b200.PATH_SIMT, id="simt"), pytest.param(dfdx_b200.PATH_AUTO, id="auto")]


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.float64])
def test_matmat_kernel(cuda_dev, oracle, dtype, path):
    _trait_case(cuda_dev, oracle, dtype, (136, 72), (72, 200), path=path, seed=1, scale=0.3)
    _trait_case(cuda_dev, oracle, dtype, (72, 136), (72, 200), a_perm=(1, 0), path=path, seed=2, scale=0.3)
    _trait_case(cuda_dev, oracle, dtype, (136, 72), (200, 72), b_perm=(1, 0), path=path, seed=3, scale=0.3)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.float64])
def test_matmat_br_kernel(cuda_dev, oracle, dtype, path):
    """Linear-layer shape: rhs is a permuted (O, I) weight; grad_rhs reduces over the batch in one launch."""
    _trait_case(cuda_dev, oracle, dtype, (5, 40, 72), (72, 136), path=path, seed=4, scale=0.3)
    _trait_case(cuda_dev, oracle, dtype, (6, 48, 64), (136, 64), b_perm=(1, 0), path=path, seed=5, scale=0.3)
    _trait_case(cuda_dev, oracle, dtype, (3, 64, 40), (72, 64), a_perm=(0, 2, 1), b_perm=(1, 0), path=path, seed=6,
                scale=0.3)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.float64])
def test_matmat_batch3_kernel(cuda_dev, oracle, dtype, path):
    _trait_case(cuda_dev, oracle, dtype, (5, 40, 72), (5, 72, 136), path=path, seed=7, scale=0.3, loss=d_exp_sum)
    _trait_case(cuda_dev, oracle, dtype, (5, 40, 72), (5, 136, 72), b_perm=(0, 2, 1), path=path, seed=8, scale=0.3)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.float64])
def test_matmat_batch4_kernel(cuda_dev, oracle, dtype, path):
    _trait_case(cuda_dev, oracle, dtype, (3, 4, 40, 72), (3, 4, 72, 136), path=path, seed=9, scale=0.3, loss=d_exp_sum)
    # MultiHeadAttention's views (multi_head_attention.rs:123-133): (b,s,h,d) buffers seen as
    # (b,h,s,d) for q / v and (b,h,d,s) for k.
    _trait_case(cuda_dev, oracle, dtype, (2, 40, 3, 64), (2, 48, 3, 64), a_perm=(0, 2, 1, 3), b_perm=(0, 2, 3, 1),
                path=path, seed=10, scale=0.3)
    _trait_case(cuda_dev, oracle, dtype, (2, 3, 40, 48), (2, 48, 3, 64), b_perm=(0, 2, 1, 3), path=path, seed=11,
                scale=0.3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_rank1_operands(cuda_dev, oracle, dtype):
    _trait_case(cuda_dev, oracle, dtype, (9,), (9, 7), seed=12)
    _trait_case(cuda_dev, oracle, dtype, (5,), (3,), seed=13)
    _trait_case(cuda_dev, oracle, dtype, (6, 9), (9,), seed=14)
    _trait_case(cuda_dev, oracle, dtype, (1030,), (1030, 520), seed=15, scale=0.1)


# --------------------------------------------------------------------------------- reference properties
def test_matmul_transpose_property(cuda_dev):
    """matmul/mod.rs:412-426."""
    cb = CudaBackend(cuda_dev, torch.float32)
    g = gen(20)
    a, b = cb.randn(4, 3, gen=g), cb.randn(3, 2, gen=g)
    c, bwd = cb.matmul(a, b)
    ga1, gb1 = bwd(d_exp_mean(cb.host(c)))
    c2, bwd2 = cb.matmul(b.permute(1, 0), a.permute(1, 0))
    gb2, ga2 = bwd2(d_exp_mean(cb.host(c2)))
    assert (cb.host(ga1) - cb.host(ga2).permute(1, 0)).abs().max() <= 1e-6
    assert (cb.host(gb1) - cb.host(gb2).permute(1, 0)).abs().max() <= 1e-6


def test_matmul_broadcast_property(cuda_dev):
    """matmul/mod.rs:428-452: broadcast-rhs equals per-item matmuls; rhs gradient is their sum."""
    cb = CudaBackend(cuda_dev, torch.float32)
    g = gen(21)
    a, b = cb.randn(5, 4, 3, gen=g), cb.randn(3, 2, gen=g)
    r, bwd = cb.matmul(a, b)
    ga, gb = bwd(d_sum(cb.host(r)))
    acc = torch.zeros(3, 2, dtype=torch.float64)
    for i in range(5):
        ri, bwdi = cb.matmul(a[i].contiguous(), b)
        assert (cb.host(ri) - cb.host(r[i])).abs().max() <= 1e-6
        gai, gbi = bwdi(d_sum(cb.host(ri)))
        assert (cb.host(gai) - cb.host(ga[i])).abs().max() <= 1e-6
        acc += cb.host(gbi)
    assert (acc - cb.host(gb)).abs().max() <= 1e-6


def test_matmul_broadcast_actual_property(cuda_dev):
    """matmul/mod.rs:454-473: a materialised broadcast through the batch-3 kernel gives identical
    outputs; its per-item rhs gradients sum to the broadcast kernel's."""
    cb = CudaBackend(cuda_dev, torch.float32)
    g = gen(22)
    a, b = cb.randn(5, 4, 3, gen=g), cb.randn(3, 2, gen=g)
    b_up = b.expand(5, 3, 2).contiguous()
    r1, bwd1 = cb.matmul(a, b_up)
    r2, bwd2 = cb.matmul(a, b)
    assert torch.equal(cb.host(r1), cb.host(r2))
    ga1, gb1 = bwd1(d_exp_mean(cb.host(r1)))
    ga2, gb2 = bwd2(d_exp_mean(cb.host(r2)))
    assert torch.equal(cb.host(ga1), cb.host(ga2))
    assert (cb.host(gb1).sum(0) - cb.host(gb2)).abs().max() <= 1e-6


def test_shape_mismatch_panics(cuda_dev):
    """matmul/mod.rs:704-767: inner / batch dimension mismatches are rejected before any launch."""
    dev = cuda_dev
    z = lambda *s: torch.zeros(*s, device=dev.device)
    for a, b in [(z(3, 3), z(4, 4)), (z(1, 3, 3), z(4, 4)), (z(1, 3, 3), z(1, 4, 4)), (z(1, 5, 3, 3), z(1, 5, 4, 4))]:
        with pytest.raises(dfdx_b200.ShapeMismatch, match="left: 3\n right: 4"):
            dev.matmul(a, b)
    for a, b in [(z(1, 2, 3), z(2, 3, 4)), (z(1, 1, 2, 3), z(2, 1, 3, 4)), (z(1, 1, 2, 3), z(1, 2, 3, 4))]:
        with pytest.raises(dfdx_b200.ShapeMismatch, match="left: 1\n right: 2"):
            dev.matmul(a, b)


# --------------------------------------------------------------------------------- benchmark configurations, full size
def _rows_check(oracle, got_rows, a_rows, b, tol):
    want, _ = oracle.matmul(a_rows, b)
    err = oracle.rel_frobenius(got_rows, want)
    assert err <= tol, f"rel frobenius {err:.3e}"


def test_config1_matmul_1024_f32(cuda_dev, oracle):
    """A[1024,1024] x B[1024,1024], U(-1,1), dC ~ N(0,1): forward + both gradients vs the oracle (full)."""
    dev = cuda_dev
    g = gen(0xD0FD + 1)
    a = (torch.rand(1024, 1024, generator=g, dtype=torch.float64) * 2 - 1).to(torch.float32)
    b = (torch.rand(1024, 1024, generator=g, dtype=torch.float64) * 2 - 1).to(torch.float32)
    dc = torch.randn(1024, 1024, generator=g, dtype=torch.float64).to(torch.float32)
    before = dev.lib.b200_tensor_launch_count()
    c, bwd = dev.matmul(a.to(dev.device), b.to(dev.device))
    ga, gb = bwd(dc.to(dev.device))
    dev.synchronize()
    assert dev.lib.b200_tensor_launch_count() - before == 3      # all three GEMMs on tensor cores
    want, obwd = oracle.matmul(a, b)
    wga, wgb = obwd(dc)
    for got, w in ((c, want), (ga, wga), (gb, wgb)):
        assert oracle.rel_frobenius(got, w) <= 1e-5


def test_config2_linear_shape_f32(cuda_dev, oracle):
    """X[64,256,1024] x W^T with W stored [4096,1024]: sampled rows / columns against the oracle, and
    the batch-reduction property gW == sum of per-item gradients on a sub-batch."""
    dev = cuda_dev
    g = gen(0xD0FD + 2)
    B, S, K, N = 64, 256, 1024, 4096
    x = torch.randn(B, S, K, generator=g, dtype=torch.float32)
    w = ((torch.rand(N, K, generator=g, dtype=torch.float64) * 2 - 1) / 32.0).to(torch.float32)
    dy = torch.randn(B, S, N, generator=g, dtype=torch.float32)
    xd, wd, dyd = x.to(dev.device), w.to(dev.device), dy.to(dev.device)
    y, bwd = dev.matmul(xd, wd.permute(1, 0))
    gx, gw_view = bwd(dyd)
    dev.synchronize()
    gw = gw_view.permute(1, 0)                                   # (N, K) base layout
    idx = torch.randint(0, B * S, (48,), generator=g)
    x2, y2, dy2, gx2 = x.reshape(-1, K), y.reshape(-1, N), dy.reshape(-1, N), gx.reshape(-1, K)
    _rows_check(oracle, y2[idx.to(dev.device)], x2[idx], w.permute(1, 0), 1e-5)
    _rows_check(oracle, gx2[idx.to(dev.device)], dy2[idx], w, 1e-5)
    # gW[n_idx, k_idx] = sum_rows dy[:, n_idx]^T x[:, k_idx]
    n_idx = torch.randint(0, N, (24,), generator=g)
    k_idx = torch.randint(0, K, (96,), generator=g)
    want, _ = oracle.matmul(dy2[:, n_idx].permute(1, 0).contiguous(), x2[:, k_idx].contiguous())
    got = gw[n_idx.to(dev.device)][:, k_idx.to(dev.device)]
    assert oracle.rel_frobenius(got, want) <= 1e-5
    # linearity in the upstream gradient: bwd(2*dy) == 2*bwd(dy) (power-of-two scaling: equal up to the order in
    # which the partial sums of K-split tiles are added, which differs from run to run in the last bits)
    gx_b, gw_b = bwd(dyd * 2.0)
    dev.synchronize()
    assert oracle.rel_frobenius(gx_b, gx.double() * 2.0) <= 1e-6
    assert oracle.rel_frobenius(gw_b, gw_view.double() * 2.0) <= 1e-6
    # with the K splits switched off the same property holds bit for bit
    dev.lib.b200_set_tail_split(1)
    dev.lib.b200_set_split_k(1)
    try:
        gx_c, gw_c = bwd(dyd)
        gx_d, gw_d = bwd(dyd * 2.0)
        dev.synchronize()
    finally:
        dev.lib.b200_set_tail_split(0)
        dev.lib.b200_set_split_k(0)
    assert torch.equal(gx_d, gx_c * 2.0) and torch.equal(gw_d, gw_c * 2.0)


def test_config3_attention_matmuls_f16(cuda_dev, oracle):
    """Q[16,16,512,64] x K^T -> [16,16,512,512]; softmax(S/8) x V: both rank-4 matmuls forward + backward,
    checked on sampled (batch, head) pairs, contiguous and MultiHeadAttention-strided."""
    dev = cuda_dev
    g = gen(0xD0FD + 3)
    Bn, H, S, D = 16, 16, 512, 64
    q, k, v = (torch.randn(Bn, H, S, D, generator=g, dtype=torch.float32).to(torch.float16) for _ in range(3))
    qd, kd, vd = q.to(dev.device), k.to(dev.device), v.to(dev.device)
    s, bwd_s = dev.matmul(qd, kd.permute(0, 1, 3, 2))
    p = torch.softmax(s.float() / 8.0, dim=-1).to(torch.float16)     # plain elementwise op, not on the path
    o, bwd_o = dev.matmul(p, vd)
    do = torch.randn(Bn, H, S, D, generator=g, dtype=torch.float32).to(torch.float16).to(dev.device)
    dp, dv = bwd_o(do)
    ds = torch.randn(Bn, H, S, S, generator=g, dtype=torch.float32).to(torch.float16).to(dev.device)
    dq, dk_view = bwd_s(ds)
    dev.synchronize()
    dk = dk_view.permute(0, 1, 3, 2)
    tol = 2e-3
    for (b, h) in [(0, 0), (7, 11), (15, 15)]:
        ws, obwd_s = oracle.matmul(q[b, h], k[b, h].permute(1, 0))
        assert oracle.rel_frobenius(s[b, h], ws) <= tol
        wo, obwd_o = oracle.matmul(p[b, h].cpu(), v[b, h])
        assert oracle.rel_frobenius(o[b, h], wo) <= tol
        wdp, wdv = obwd_o(do[b, h].cpu())
        assert oracle.rel_frobenius(dp[b, h], wdp) <= tol and oracle.rel_frobenius(dv[b, h], wdv) <= tol
        wdq, wdk = obwd_s(ds[b, h].cpu())
        assert oracle.rel_frobenius(dq[b, h], wdq) <= tol
        assert oracle.rel_frobenius(dk[b, h], wdk.permute(1, 0)) <= tol
    # same numbers through MHA's strides: (b,s,h,d) buffers viewed as (b,h,s,d) / (b,h,d,s)
    q2 = qd.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    k2 = kd.permute(0, 2, 1, 3).contiguous().permute(0, 2, 3, 1)
    s2, _ = dev.matmul(q2, k2)
    dev.synchronize()
    assert torch.equal(s2, s)


@pytest.mark.parametrize("layout", ["rrr", "rcr", "crr"])
def test_tail_split_f32(cuda_dev, oracle, layout):
    """150 tiles on 148 SMs: the two tiles of the second round are cut along K over all SMs and summed atomically
    (beta 0: those tiles are zeroed first, the output is NaN-poisoned; beta 1), ragged edges included; problems with
    less than one round of tiles and beta 1; the same problems with the tail split switched off give the same results
    within the tolerance."""
    dev = cuda_dev
    dev.set_path(dfdx_b200.PATH_TENSOR)
    assert dev.lib.b200_set_tile_n(256) == 0
    try:
        for mode in (0, 1):
            assert dev.lib.b200_set_tail_split(mode) == 0
            for i, (m, k, n) in enumerate([(640, 256, 7680), (5 * 128 - 24, 264, 30 * 256 - 40)]):
                for beta in (0, 1):
                    l0 = dev.lib.b200_launch_count()
                    check_gemm(dev, oracle, m, k, n, layout[0], layout[1], layout[2], beta, torch.float32, pad=8,
                               seed=700 + i)
                    assert dev.lib.b200_launch_count() - l0 == 1
            # less than one round of tiles (100 and 96 on 148 SMs), long K, an output that is added to: the whole
            # (tile, k-block) space is dealt out over the SMs
            for i, (m, k, n) in enumerate([(640, 1024, 5120), (3 * 128 - 24, 1032, 32 * 256 - 40)]):
                l0 = dev.lib.b200_launch_count()
                check_gemm(dev, oracle, m, k, n, layout[0], layout[1], layout[2], 1, torch.float32, pad=8, seed=720 + i)
                assert dev.lib.b200_launch_count() - l0 == 1
    finally:
        dev.lib.b200_set_tail_split(0)
        dev.lib.b200_set_tile_n(0)
        dev.set_path(dfdx_b200.PATH_AUTO)
    assert dev.lib.b200_set_tail_split(2) == dfdx_b200._lib.ERR_UNSUPPORTED


# --------------------------------------------------------------------------------- streams, capture, bounded waits
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_backward_on_two_streams(cuda_dev, oracle, dtype):
    """The backward entry points with a second stream, as dfdx drives them (matmul/cuda_kernel.rs:282-310):
    grad_lhs on `par_stream`, grad_rhs on the default stream, joins on the caller's side."""
    cuda_dev.par_stream = torch.cuda.Stream(cuda_dev.device)
    try:
        _trait_case(cuda_dev, oracle, dtype, (264, 520), (520, 392), seed=21, scale=0.3)                    # MatMat
        _trait_case(cuda_dev, oracle, dtype, (6, 48, 64), (136, 64), b_perm=(1, 0), seed=22, scale=0.3)     # MatMatBr
        _trait_case(cuda_dev, oracle, dtype, (5, 40, 72), (5, 72, 136), seed=23, scale=0.3)                 # Batch3
        _trait_case(cuda_dev, oracle, dtype, (2, 40, 3, 64), (2, 48, 3, 64), a_perm=(0, 2, 1, 3), b_perm=(0, 2, 3, 1),
                    seed=24, scale=0.3)                                                                     # Batch4
        # long K, few tiles: both gradient GEMMs of the f16 case take split-K and so share the device's scratch
        _trait_case(cuda_dev, oracle, dtype, (128, 4096), (4096, 256), seed=25, scale=0.1)
    finally:
        cuda_dev.par_stream = None


def test_bounded_wait_runs_out_and_kernel_returns(cuda_dev, oracle):
    """A device-side wait that runs out.  First the mechanism alone: a one-CTA kernel waits, with the GEMM kernels'
    bounded wait, on a barrier that nothing completes; it must come back, report B200_ERR_DEVICE_TIMEOUT once, and
    leave the device healthy.  Then a real GEMM: with a clock budget far below what one long-K tile needs, the
    epilogue's wait for the accumulator gives up, the kernel drains, frees its tensor memory and returns."""
    import ctypes as C
    dev = cuda_dev
    TIMEOUT = dfdx_b200._lib.ERR_DEVICE_TIMEOUT
    assert dev.device_status() == 0
    waited = C.c_longlong(0)
    assert dev.lib.b200_selftest_bounded_wait(200000, C.byref(waited), dev._stream()) == 0
    assert waited.value >= 200000
    assert dev.device_status() == TIMEOUT
    assert dev.device_status() == 0                         # reading the status clears it
    assert dev.lib.b200_selftest_bounded_wait(0, None, dev._stream()) == 0
    assert dev.device_status() == TIMEOUT
    check_gemm(dev, oracle, 200, 264, 136, "r", "c", "r", 1, torch.float16, pad=8, seed=30)
    assert dev.device_status() == 0

    # a real kernel: 128 x 256 f16 outputs over K = 2^19.  The epilogue warps wait for the whole main loop (about 3 ms)
    # with a budget of 2000 clocks; how long the 64 unconditional polls in front of the budgeted ones last is up to the
    # hardware (measured on a busy SM: between 0.2 and 0.8 ms), hence the long K.
    k = 1 << 19
    g = gen(31)
    a = (torch.randn(128, k, generator=g) * 0.05).half().to(dev.device)
    b = (torch.randn(k, 256, generator=g) * 0.05).half().to(dev.device)
    c = torch.zeros(128, 256, dtype=torch.float16, device=dev.device)
    dev.set_path(dfdx_b200.PATH_TENSOR)
    assert dev.lib.b200_set_split_k(1) == 0                 # one unit walks the whole K
    try:
        assert dev.lib.b200_set_wait_limit(2000) == 0
        dev.gemm((128, k, 256), a, a.stride(), b, b.stride(), 0.0, c, c.stride())
        torch.cuda.synchronize(dev.device)                  # the kernel came back
        assert dev.device_status() == TIMEOUT
        assert dev.device_status() == 0
    finally:
        dev.lib.b200_set_wait_limit(0)
        dev.lib.b200_set_split_k(0)
        dev.set_path(dfdx_b200.PATH_AUTO)
    del a, b, c
    dev.set_path(dfdx_b200.PATH_TENSOR)
    try:
        check_gemm(dev, oracle, 128, 4096, 256, "r", "r", "r", 0, torch.float32, pad=0, seed=32)
        check_gemm(dev, oracle, 128, 4096, 256, "r", "r", "r", 0, torch.float16, pad=0, seed=33)
    finally:
        dev.set_path(dfdx_b200.PATH_AUTO)
    assert dev.device_status() == 0


def test_captured_split_k_f16_next_to_an_eager_one(cuda_dev, oracle):
    """An f16 GEMM that takes split-K when run eagerly is recorded into a CUDA graph (where it runs unsplit, because
    a replay cannot take part in the event ordering of the device's one split-K scratch) and replayed on one stream
    while an eager split-K GEMM runs on another; both must match the oracle."""
    dev = cuda_dev
    g = gen(41)
    m, k, n = 128, 8192, 256
    a1 = (torch.randn(m, k, generator=g) * 0.1).half().to(dev.device)
    b1 = (torch.randn(k, n, generator=g) * 0.1).half().to(dev.device)
    a2 = (torch.randn(m, k, generator=g) * 0.1).half().to(dev.device)
    b2 = (torch.randn(k, n, generator=g) * 0.1).half().to(dev.device)
    c1 = torch.zeros(m, n, dtype=torch.float16, device=dev.device)
    c2 = torch.zeros(m, n, dtype=torch.float16, device=dev.device)
    want1, _ = oracle.matmul(a1.cpu(), b1.cpu())
    want2, _ = oracle.matmul(a2.cpu(), b2.cpu())
    dev.set_path(dfdx_b200.PATH_TENSOR)
    try:
        l0 = dev.lib.b200_launch_count()
        dev.gemm((m, k, n), a1, a1.stride(), b1, b1.stride(), 0.0, c1, c1.stride())        # eager warm-up: split-K
        assert dev.lib.b200_launch_count() - l0 == 2, "expected the split-K pair of launches (GEMM + finalize)"
        torch.cuda.synchronize(dev.device)
        sa, sb = torch.cuda.Stream(dev.device), torch.cuda.Stream(dev.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(sa):
            l0 = dev.lib.b200_launch_count()
            with torch.cuda.graph(graph, stream=sa):
                dev.gemm((m, k, n), a1, a1.stride(), b1, b1.stride(), 0.0, c1, c1.stride())
            assert dev.lib.b200_launch_count() - l0 == 1, "a captured GEMM must run unsplit"
        c1.fill_(float("nan"))
        torch.cuda.synchronize(dev.device)
        for _ in range(4):
            with torch.cuda.stream(sa):
                graph.replay()
            with torch.cuda.stream(sb):
                dev.gemm((m, k, n), a2, a2.stride(), b2, b2.stride(), 0.0, c2, c2.stride())
        torch.cuda.synchronize(dev.device)
    finally:
        dev.set_path(dfdx_b200.PATH_AUTO)
    assert frob(oracle, c1, want1) <= FROB_TOL[torch.float16]
    assert frob(oracle, c2, want2) <= FROB_TOL[torch.float16]
    assert dev.device_status() == 0
