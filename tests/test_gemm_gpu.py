"""ct_matmul / fused GEMM entry points against a plain PyTorch fp32 product of the same operands,
on both GPU paths (tcgen05 and the shape-generic SIMT kernel), for every operand orientation."""

import pytest
import torch

from causal_tuner_b200 import _lib
from causal_tuner_b200.kernels import linear

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("gpu_guard")]

# name -> (GEMM path, CTAs per tile (CT_B200_GEMM_CTAS), row halves per CTA (CT_B200_GEMM_MH), tensor-map store
# epilogue (CT_B200_GEMM_TMA_STORE)); None leaves the library's own choice
PATHS = {"simt": (_lib.PATH_SIMT, None, None, None),
         "tcgen05": (_lib.PATH_TCGEN05, "1", None, None),
         "tcgen05_pair": (_lib.PATH_TCGEN05, "2", "1", None),
         "tcgen05_pair_register_store": (_lib.PATH_TCGEN05, "2", "1", "0"),
         "tcgen05_wide": (_lib.PATH_TCGEN05, "2", "2", None),
         "tcgen05_wide_register_store": (_lib.PATH_TCGEN05, "2", "2", "0")}


@pytest.fixture(params=list(PATHS))
def path(request, monkeypatch):
    choice, ctas, halves, tma_store = PATHS[request.param]
    monkeypatch.setattr(_lib, "gemm_path", choice)
    for name, value in (("CT_B200_GEMM_CTAS", ctas), ("CT_B200_GEMM_MH", halves), ("CT_B200_GEMM_TMA_STORE", tma_store)):
        if value is not None:
            monkeypatch.setenv(name, value)
        else:
            monkeypatch.delenv(name, raising=False)
    return request.param


def relative(actual, expected):
    actual, expected = actual.float(), expected.float()
    return ((actual - expected).norm() / expected.norm().clamp_min(1e-20)).item()


def operand(rows, cols, major, dtype=torch.bfloat16):
    """A [rows, cols] matrix whose storage is row-major ("K") or column-major ("MN")."""
    if major == "K":
        return torch.randn(rows, cols, device="cuda").to(dtype)
    return torch.randn(cols, rows, device="cuda").to(dtype).T


# (M, N, K): one exact tile; ragged in every dimension; more tiles than SMs; a long contraction
SHAPES = [(128, 256, 64), (304, 520, 200), (2048, 4096, 128), (96, 72, 2048), (1, 8, 8), (1096, 328, 520)]


@pytest.mark.parametrize("a_major,b_major", [("K", "K"), ("K", "MN"), ("MN", "K"), ("MN", "MN")])
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_matmul_orientations(path, shape, a_major, b_major, out_dtype):
    m, n, k = shape
    if path.startswith("tcgen05") and min(m, n, k) < 8:
        pytest.skip("degenerate extents go to the SIMT kernel")
    left = operand(m, k, a_major)             # A(m, k): "K" = k contiguous
    right = operand(n, k, b_major).T          # B(k, n): "K" = k contiguous
    out = torch.full((m, n), float("nan"), device="cuda", dtype=out_dtype)
    linear.matmul(left, right, out=out)
    expected = left.float() @ right.float()
    assert torch.isfinite(out).all()
    assert relative(out, expected) < (4e-3 if out_dtype == torch.bfloat16 else 1e-5)
    if out_dtype == torch.float32:
        linear.matmul(left, right, out=out, add=True)
        assert relative(out, 2 * expected) < 1e-5


def test_matmul_exact_on_small_integers(path):
    # Integer-valued operands: every product and partial sum is exact in fp32, so any layout
    # mistake shows up as a nonzero difference.
    m, n, k = 256, 512, 192
    left = torch.randint(-3, 4, (m, k), device="cuda").bfloat16()
    right = torch.randint(-3, 4, (k, n), device="cuda").bfloat16()
    out = torch.empty(m, n, device="cuda", dtype=torch.float32)
    linear.matmul(left, right, out=out)
    assert torch.equal(out, left.float() @ right.float())
    linear.matmul(left.T.contiguous().T, right.T.contiguous().T, out=out)
    assert torch.equal(out, left.float() @ right.float())


@pytest.mark.parametrize("rows,inner,outer,rank", [(300, 256, 520, 16), (37, 32, 24, 8), (1024, 512, 768, 256)])
@pytest.mark.parametrize("with_bias,with_residual", [(False, False), (True, True)])
def test_forward_linear_concatenated_contraction(path, rows, inner, outer, rank, with_bias, with_residual):
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    w = (torch.randn(outer, inner, device="cuda") * .05).bfloat16()
    a = (torch.randn(rank, inner, device="cuda") * .05).bfloat16()
    b = (torch.randn(outer, rank, device="cuda") * .05).bfloat16()
    bias = torch.randn(outer, device="cuda").bfloat16() if with_bias else None
    residual = torch.randn(rows, outer, device="cuda").bfloat16() if with_residual else None
    out = torch.full((rows, outer), float("nan"), device="cuda", dtype=torch.bfloat16)
    xa = torch.full((rows, rank), float("nan"), device="cuda", dtype=torch.bfloat16)
    linear.forward_linear(x, w, a, b, out=out, xa=xa, bias=bias, residual=residual)
    expected_xa = (x.float() @ a.float().T).bfloat16()
    assert relative(xa, expected_xa) < 4e-3
    expected = x.float() @ w.float().T + xa.float() @ b.float().T
    if bias is not None:
        expected = expected + bias.float()
    expected = expected.bfloat16()
    if residual is not None:
        expected = (expected.float() + residual.float()).bfloat16()
    assert relative(out, expected) < 4e-3
    # the residual add must equal a separate rounded add of the unfused output
    if residual is not None:
        plain = torch.empty_like(out)
        linear.forward_linear(x, w, a, b, out=plain, xa=xa, bias=bias)
        assert torch.equal(out, (plain.float() + residual.float()).bfloat16())


@pytest.mark.parametrize("rows,inner,outer,rank", [(300, 256, 520, 16), (1024, 512, 768, 256)])
def test_input_gradient_and_parameter_gradients(path, rows, inner, outer, rank):
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    dy = torch.randn(rows, outer, device="cuda").bfloat16()
    w = (torch.randn(outer, inner, device="cuda") * .05).bfloat16()
    a = (torch.randn(rank, inner, device="cuda") * .05).bfloat16()
    b = (torch.randn(outer, rank, device="cuda") * .05).bfloat16()
    dx = torch.full((rows, inner), float("nan"), device="cuda", dtype=torch.bfloat16)
    low = torch.full((rows, rank), float("nan"), device="cuda", dtype=torch.bfloat16)
    linear.input_gradient(dy, w, a, b, dx, low)
    expected_low = (dy.float() @ b.float()).bfloat16()
    assert relative(low, expected_low) < 4e-3
    expected_dx = dy.float() @ w.float() + low.float() @ a.float()
    assert relative(dx, expected_dx) < 4e-3
    before = dx.clone()
    linear.input_gradient(dy, w, a, b, dx, low, add=True)
    assert relative(dx, before.float() + expected_dx) < 6e-3
    xa = (x.float() @ a.float().T).bfloat16()
    da = torch.full((rank, inner), float("nan"), device="cuda")
    db = torch.full((outer, rank), float("nan"), device="cuda")
    linear.parameter_gradients(x, dy, da, db, low, xa, add=False)
    expected_da, expected_db = low.float().T @ x.float(), dy.float().T @ xa.float()
    assert relative(da, expected_da) < 1e-5 and relative(db, expected_db) < 1e-5
    first = (da.clone(), db.clone())
    linear.parameter_gradients(x, dy, da, db, low, xa, add=False)
    assert torch.equal(da, first[0]) and torch.equal(db, first[1])  # fixed summation order
    linear.parameter_gradients(x, dy, da, db, low, xa, add=True)
    assert relative(da, 2 * expected_da) < 1e-5 and relative(db, 2 * expected_db) < 1e-5


def test_split_contraction_matches_single_pass_and_is_repeatable(monkeypatch):
    # rank-16 adapter over 4096 tokens: dA has a single output tile, so the token contraction is
    # cut into several slices that are summed in slice order.
    monkeypatch.setattr(_lib, "gemm_path", _lib.PATH_TCGEN05)
    rows, inner, outer, rank = 4096, 256, 512, 16
    assert _lib.load().ct_parameter_gradients_workspace(rows, inner, outer, rank, _lib.BF16, _lib.PATH_TCGEN05) > 0
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    dy = torch.randn(rows, outer, device="cuda").bfloat16()
    low = torch.randn(rows, rank, device="cuda").bfloat16()
    xa = torch.randn(rows, rank, device="cuda").bfloat16()
    da, db = torch.empty(rank, inner, device="cuda"), torch.empty(outer, rank, device="cuda")
    linear.parameter_gradients(x, dy, da, db, low, xa, add=False)
    assert relative(da, low.float().T @ x.float()) < 1e-5
    assert relative(db, dy.float().T @ xa.float()) < 1e-5
    again = (torch.empty_like(da), torch.empty_like(db))
    linear.parameter_gradients(x, dy, *again, low, xa, add=False)
    assert torch.equal(da, again[0]) and torch.equal(db, again[1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_accumulate_first_write_ignores_uninitialised_storage(dtype):
    left = torch.randn(19, 37, device="cuda", dtype=dtype)
    right = torch.randn(37, 23, device="cuda", dtype=dtype)
    output = torch.full((19, 23), float("nan"), device="cuda")
    expected = left.float() @ right.float()
    linear.accumulate(output, left, right, add=False)
    torch.testing.assert_close(output, expected, rtol=1e-5, atol=1e-5)
    linear.accumulate(output, left, right, add=True)
    torch.testing.assert_close(output, expected * 2, rtol=1e-5, atol=1e-5)


def test_fp32_operands_use_the_simt_kernel():
    before = _lib.tcgen05_launch_count()
    left, right = torch.randn(130, 70, device="cuda"), torch.randn(70, 90, device="cuda")
    out = torch.empty(130, 90, device="cuda")
    linear.matmul(left, right, out=out)
    torch.testing.assert_close(out, left @ right, rtol=1e-5, atol=1e-5)
    assert _lib.tcgen05_launch_count() == before


def test_auto_path_picks_tcgen05_for_aligned_bf16():
    before = _lib.tcgen05_launch_count()
    left, right = torch.randn(256, 128, device="cuda").bfloat16(), torch.randn(128, 512, device="cuda").bfloat16()
    out = torch.empty(256, 512, device="cuda", dtype=torch.bfloat16)
    linear.matmul(left, right, out=out)
    assert _lib.tcgen05_launch_count() == before + 1
    assert relative(out, left.float() @ right.float()) < 4e-3


@pytest.mark.parametrize("shapes", [((32, 8, 8), (8, 8, 16)), ((4096, 128, 128), (256, 256, 256)), ((520, 520), (16, 24))])
def test_grouped_input_gradient_equals_the_sum_of_the_projections(path, shapes):
    outers, ranks = shapes
    rows, inner = 300 if outers[0] != 4096 else 1024, 32 if outers[0] == 32 else 512
    dys = [torch.randn(rows, n, device="cuda").bfloat16() for n in outers]
    weights = [(torch.randn(n, inner, device="cuda") * .05).bfloat16() for n in outers]
    a_list = [(torch.randn(r, inner, device="cuda") * .05).bfloat16() for r in ranks]
    b_list = [(torch.randn(n, r, device="cuda") * .05).bfloat16() for n, r in zip(outers, ranks)]
    lows = [torch.full((rows, r), float("nan"), device="cuda", dtype=torch.bfloat16) for r in ranks]
    dx = torch.full((rows, inner), float("nan"), device="cuda", dtype=torch.bfloat16)
    linear.input_gradient_group(dys, weights, a_list, b_list, dx, lows)
    expected = torch.zeros(rows, inner, device="cuda")
    for dy, w, a, b, low in zip(dys, weights, a_list, b_list, lows):
        assert relative(low, (dy.float() @ b.float()).bfloat16()) < 4e-3
        expected += dy.float() @ w.float() + low.float() @ a.float()
    assert relative(dx, expected) < 4e-3
    separate = torch.empty_like(dx)
    scratch = [torch.empty_like(low) for low in lows]
    for index, (dy, w, a, b) in enumerate(zip(dys, weights, a_list, b_list)):
        linear.input_gradient(dy, w, a, b, separate, scratch[index], add=index > 0)
    assert relative(dx, separate) < 8e-3
    before = dx.clone()
    linear.input_gradient_group(dys, weights, a_list, b_list, dx, lows, add=True)
    assert relative(dx, before.float() + expected) < 6e-3


@pytest.mark.parametrize("rows,inner,outers", [(1024, 1024, (1536, 128)), (300, 520, (136,)), (512, 2048, (1024, 1024))])
def test_input_gradient_from_transposed_weights_is_bit_identical(path, rows, inner, outers):
    """The `.T` view of a weight stored transposed (what `materialize_for_gradient` returns) gives every
    input-gradient entry point the very results of the row-major weight: same products, same order."""
    ranks = [16] * len(outers)
    dys = [torch.randn(rows, n, device="cuda").bfloat16() for n in outers]
    weights = [(torch.randn(n, inner, device="cuda") * .05).bfloat16() for n in outers]
    views = [w.T.contiguous().T for w in weights]
    assert all(v.stride(0) == 1 and torch.equal(v, w) for v, w in zip(views, weights))
    a_list = [(torch.randn(r, inner, device="cuda") * .05).bfloat16() for r in ranks]
    b_list = [(torch.randn(n, r, device="cuda") * .05).bfloat16() for n, r in zip(outers, ranks)]
    results = []
    for operands in (weights, views):
        lows = [torch.empty(rows, r, device="cuda", dtype=torch.bfloat16) for r in ranks]
        grouped = torch.full((rows, inner), float("nan"), device="cuda", dtype=torch.bfloat16)
        linear.input_gradient_group(dys, operands, a_list, b_list, grouped, lows)
        single = torch.full((rows, inner), float("nan"), device="cuda", dtype=torch.bfloat16)
        linear.input_gradient(dys[0], operands[0], a_list[0], b_list[0], single, lows[0])
        given = torch.full((rows, inner), float("nan"), device="cuda", dtype=torch.bfloat16)
        linear.input_gradient_with(dys[0], operands[0], a_list[0], lows[0], given)
        linear.input_gradient_with(dys[0], operands[0], a_list[0], lows[0], given, add=True)
        results.append((grouped, single, given))
    for natural, transposed in zip(*results):
        assert torch.isfinite(transposed.float()).all()
        assert torch.equal(natural, transposed)


@pytest.mark.parametrize("tokens,rows,cols", [(4096, 768, 512), (300, 24, 520), (1024, 16, 256), (16384, 512, 128)])
def test_token_gradient_of_stacked_low_matrices(path, tokens, rows, cols):
    # out = left^T @ right over the tokens, fp32, fixed slice order; `left` holds several projections'
    # low matrices side by side, so row blocks of `out` are their separate dA.
    left = torch.randn(tokens, rows, device="cuda").bfloat16()
    right = torch.randn(tokens, cols, device="cuda").bfloat16()
    out = torch.full((rows, cols), float("nan"), device="cuda")
    linear.token_gradient(left, right, out)
    expected = left.float().T @ right.float()
    assert relative(out, expected) < 1e-5
    again = torch.empty_like(out)
    linear.token_gradient(left, right, again)
    assert torch.equal(out, again)
    linear.token_gradient(left, right, out, add=True)
    assert relative(out, 2 * expected) < 1e-5
    # a column slice of a wider buffer as the left operand (leading dimension != width)
    third = rows // 3 if rows >= 24 else rows
    part = torch.empty(third, cols, device="cuda")
    linear.token_gradient(left[:, :third], right, part)
    assert relative(part, expected[:third]) < 1e-5
    with pytest.raises(ValueError):
        linear.token_gradient(left, right, torch.empty(rows, cols, device="cuda", dtype=torch.bfloat16))


@pytest.mark.parametrize("tokens,shapes", [(4096, [(768, 512), (512, 256), (128, 256), (128, 256)]),      # one slice each
                                           (2048, [(256, 512), (512, 256)]),                              # sliced
                                           (304, [(24, 520), (520, 24), (16, 8)]),                        # ragged
                                           (8192, [(512, 1024), (1024, 256), (1024, 256), (256, 1024), (1024, 256)])])
def test_grouped_token_gradients_equal_the_separate_products(path, tokens, shapes):
    """ct_token_gradients_group: several left^T @ right products over the same tokens in one launch (the stacked
    dA and every dB of an operator). Each result within 1e-5 of an fp32 product and of the one-by-one route,
    bit-identical when repeated (one slice count per group, planes summed in slice order), beta honoured."""
    problems = []
    for rows, cols in shapes:
        left = torch.randn(tokens, rows, device="cuda").bfloat16()
        right = torch.randn(tokens, cols, device="cuda").bfloat16()
        problems.append((left, right, torch.full((rows, cols), float("nan"), device="cuda")))
    launches = _lib.tcgen05_launch_count()
    linear.token_gradients(problems)
    used = _lib.tcgen05_launch_count() - launches
    if path.startswith("tcgen05") and tokens != 304:
        assert used == 1                       # one persistent launch for the whole group
    expected = [left.float().T @ right.float() for left, right, _ in problems]
    for (left, right, out), reference in zip(problems, expected):
        assert relative(out, reference) < 1e-5
        alone = torch.empty_like(out)
        linear.token_gradient(left, right, alone)
        assert relative(out, alone) < 1e-5
    again = [(left, right, torch.empty_like(out)) for left, right, out in problems]
    linear.token_gradients(again)
    assert all(torch.equal(a[2], b[2]) for a, b in zip(problems, again))
    linear.token_gradients(problems, add=True)
    for (_, _, out), reference in zip(problems, expected):
        assert relative(out, 2 * reference) < 1e-5


@pytest.mark.parametrize("rows,inner,outer", [(512, 4096, 1024), (300, 256, 520), (2051, 1024, 776), (64, 64, 8)])
def test_decode_inside_the_gemm_is_bit_identical_to_decode_then_gemm(rows, inner, outer):
    """ct_matmul_nf4: the NF4 decode as a stage of the tcgen05 kernel (decode warps fill the swizzled B tiles).
    Same decoded values, same MMA sequence per tile -> the very bits of ct_nf4_decode followed by ct_matmul."""
    from causal_tuner_b200.kernels.nf4_cuda import dequantize_nf4
    from causal_tuner_b200.quant import quantize_nf4
    torch.manual_seed(rows)
    weight = (torch.randn(outer, inner, device="cuda") * .05).bfloat16()
    packed, state = quantize_nf4(weight, blocksize=64, nested=False)
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    dense = dequantize_nf4(packed, state, torch.bfloat16)
    expected = torch.empty(rows, outer, device="cuda", dtype=torch.bfloat16)
    linear.matmul(x, dense.T, out=expected)
    actual = torch.full((rows, outer), float("nan"), device="cuda", dtype=torch.bfloat16)
    before = _lib.tcgen05_launch_count()
    linear.matmul_nf4(x, packed, state, out=actual)
    assert _lib.tcgen05_launch_count() == before + 1
    assert torch.equal(actual, expected)
    assert relative(actual, x.float() @ dense.float().T) < 4e-3
    nested_packed, nested_state = quantize_nf4(weight, blocksize=64, nested=True)
    with pytest.raises(NotImplementedError):
        linear.matmul_nf4(x, nested_packed, nested_state, out=actual)


@pytest.mark.parametrize("rows,inner,outer,rank", [(300, 256, 520, 16), (1024, 512, 768, 256)])
def test_projection_pieces_equal_the_fused_calls(path, rows, inner, outer, rank):
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    dy = torch.randn(rows, outer, device="cuda").bfloat16()
    w = (torch.randn(outer, inner, device="cuda") * .05).bfloat16()
    a = (torch.randn(rank, inner, device="cuda") * .05).bfloat16()
    b = (torch.randn(outer, rank, device="cuda") * .05).bfloat16()
    bias = torch.randn(outer, device="cuda").bfloat16()
    out, xa = torch.empty(rows, outer, device="cuda", dtype=torch.bfloat16), torch.empty(rows, rank, device="cuda", dtype=torch.bfloat16)
    linear.forward_linear(x, w, a, b, out=out, xa=xa, bias=bias)
    # low-rank input computed apart, as a column slice of a stacked buffer
    stacked = torch.full((rows, rank + 8), float("nan"), device="cuda", dtype=torch.bfloat16)
    linear.matmul(x, a.T, out=stacked[:, 8:])
    assert torch.equal(stacked[:, 8:], xa)
    apart = torch.empty_like(out)
    linear.apply_projection(x, w, b, stacked[:, 8:], out=apart, bias=bias)
    assert torch.equal(apart, out)
    dx, low = torch.empty(rows, inner, device="cuda", dtype=torch.bfloat16), torch.empty_like(xa)
    linear.input_gradient(dy, w, a, b, dx, low)
    low_apart = torch.empty_like(low)
    linear.matmul(dy, b, out=low_apart)
    dx_apart = torch.empty_like(dx)
    linear.input_gradient_with(dy, w, a, low_apart, dx_apart)
    assert torch.equal(low_apart, low) and torch.equal(dx_apart, dx)
