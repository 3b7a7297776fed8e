"""GPU parity, tensor-core modes (tcgen05 bf16 / tf32 forward).  Tolerance:
rel-L2 <= 2e-3.  In bf16 mode the coefficients are stored in bf16, so the
oracle evaluates with the same bf16-rounded coefficients (activations stay
fp32 in the oracle)."""
import pytest
import torch

import kan_b200
from kan_b200 import ops
from oracle import chebykan_oracle as o
from _util import TC_TOL, assert_guards_intact, guarded, make_case

pytestmark = pytest.mark.gpu

SHAPES = [
    # B, in, out, deg, dist
    (256, 64, 128, 4, "normal"),          # one tile, BN = 128
    (4096, 1024, 1024, 8, "normal"),      # configuration 3 at reduced batch, BN = 256
    (2048, 2048, 2048, 4, "normal"),      # configuration 4 layer at reduced batch
    (8192, 64, 64, 32, "uniform3"),       # configuration 5 layer
    (256, 784, 64, 4, "sparse"),          # in not a multiple of 64, out padded to 128
    (256, 64, 10, 4, "normal"),           # out < 16
    (100, 13, 7, 3, "normal"),            # in not a multiple of 4: scalar loads
    (1000, 96, 300, 8, "normal"),         # ragged rows and three N tiles of 128
    (129, 32, 256, 0, "normal"),          # degree 0
    (20000, 128, 256, 2, "normal"),       # more tiles than SMs: persistent loop, both accumulators
    # 512 or more padded outputs and more than 128 rows: CTA pairs (cta_group::2)
    (130, 64, 512, 3, "normal"),          # the pair's odd CTA holds 2 real rows
    (257, 100, 640, 4, "normal"),         # second pair: only the even CTA has rows; ragged second N tile
    (1000, 45, 520, 5, "normal"),         # in not a multiple of 4 (no x prefetch) with pairs
    (40000, 64, 512, 1, "normal"),        # more pairs than SM pairs: persistent loop over pair tiles
    (128, 64, 512, 3, "normal"),          # exactly 128 rows: single-CTA kernel on a wide layer
]


def oracle_y(x, coeffs, mode):
    c = coeffs.bfloat16().float() if mode == "bf16" else coeffs
    return o.forward(x, c)


def run_fwd(x, coeffs, mode):
    n_in, n_out, dp1 = coeffs.shape
    xd, cd = x.cuda(), coeffs.cuda()
    packed = ops.pack_coeffs(cd, mode)
    y, yw = guarded((x.shape[0], n_out))
    ops.forward(xd, packed, n_in, n_out, dp1 - 1, mode, out=y)
    torch.cuda.synchronize()
    ops.check_status()
    assert_guards_intact(y, yw)
    return y.cpu()


@pytest.mark.parametrize("mode", ["bf16", "tf32"])
@pytest.mark.parametrize("B,n_in,n_out,deg,dist", SHAPES)
def test_tc_forward_vs_oracle(mode, B, n_in, n_out, deg, dist):
    x, coeffs, _ = make_case(B, n_in, n_out, deg, dist, seed=B + n_in + deg)
    y = run_fwd(x, coeffs, mode)
    err = o.rel_l2(y, oracle_y(x, coeffs, mode))
    assert err <= TC_TOL, err
    # and it is a real tensor-core result, not the fp32 path: some rounding must be visible
    if deg > 0:
        assert err > 1e-6


# Narrow layers (at most 128 outputs, inputs a multiple of 4) run the kernel that keeps the generated basis tile in
# tensor memory (tcgen05.st by the producers, tcgen05.mma with the A operand in TMEM): 64- and 128-column accumulators,
# one (bf16) or two (tf32) row sub-tiles of 128 rows per CTA, x tiles by 128B-swizzled TMA boxes of 32 inputs.
NARROW_SHAPES = [
    # B, in, out, deg, dist
    (1, 4, 16, 1, "normal"),              # a single row, one chunk of inputs
    (127, 64, 64, 32, "uniform3"),        # less than one sub-tile
    (129, 64, 64, 32, "uniform3"),        # second sub-tile holds one row
    (257, 32, 64, 7, "normal"),           # third sub-tile (second CTA tile in tf32 mode)
    (1000, 100, 65, 5, "normal"),         # ragged input block (100 = 3 x 32 + 4), 128-column accumulator, odd out
    (1000, 64, 128, 9, "normal"),         # full 128 outputs
    (3000, 200, 40, 0, "normal"),         # degree 0: one K block per input block
    (3000, 36, 96, 1, "normal"),          # degree 1
    (50000, 64, 64, 6, "normal"),         # more tiles than SMs: persistent loop, both accumulator buffers
    (20000, 784, 64, 4, "sparse"),        # configuration 2's first layer shape at a large batch: 25 (13) input blocks
    (70000, 64, 64, 32, "uniform3"),      # configuration 5's layer
    (4096, 8, 8, 63, "normal"),           # highest tested degree: 64 K blocks from one input block
]


@pytest.mark.parametrize("mode", ["bf16", "tf32"])
@pytest.mark.parametrize("B,n_in,n_out,deg,dist", NARROW_SHAPES)
def test_narrow_forward_with_basis_in_tensor_memory(mode, B, n_in, n_out, deg, dist):
    x, coeffs, _ = make_case(B, n_in, n_out, deg, dist, seed=B + n_in + deg)
    y = run_fwd(x, coeffs, mode)
    err = o.rel_l2(y, oracle_y(x, coeffs, mode))
    assert err <= TC_TOL, err
    if deg > 0:
        assert err > 1e-6
    # a block of rows that starts on a 256-row boundary gives the same bits as inside the full batch
    if B >= 1024:
        blk = run_fwd(x[512:1024].contiguous(), coeffs, mode)
        assert torch.equal(y[512:1024], blk)


@pytest.mark.parametrize("mode", ["bf16", "tf32"])
def test_narrow_forward_propagates_nan_rows(mode):
    """A NaN input poisons exactly its own row (the tf32 rounding increment must not turn it into a number)."""
    x, coeffs, _ = make_case(600, 64, 64, 5, seed=3)
    x[17, 5] = float("nan")
    x[300, 63] = float("nan")
    xd = x.cuda()
    y = ops.forward(xd, ops.pack_coeffs(coeffs.cuda(), mode), 64, 64, 5, mode).cpu()
    bad = torch.isnan(y).any(dim=1)
    assert bad[17] and bad[300] and int(bad.sum()) == 2
    ok = ~bad
    assert o.rel_l2(y[ok], oracle_y(x[ok], coeffs, mode)) <= TC_TOL


@pytest.mark.parametrize("mode", ["bf16", "tf32"])
def test_tc_bitwise_repeatable_and_row_block_invariant(mode):
    x, coeffs, _ = make_case(3000, 128, 256, 4, seed=77)
    a = run_fwd(x, coeffs, mode)
    b = run_fwd(x, coeffs, mode)
    assert torch.equal(a, b)
    # a block of rows starting on a tile boundary gives the same bits as the full batch
    c = run_fwd(x[1280:2560].contiguous(), coeffs, mode)
    assert torch.equal(a[1280:2560], c)


def test_tc_layer_autograd_mixes_with_fp32_backward():
    """math_mode='bf16': tensor-core forward, fp32 backward kernels; gradients within the tensor-core tolerance."""
    torch.manual_seed(4)
    layer = kan_b200.ChebyKANLayer(128, 64, 8, math_mode="bf16").cuda()
    x = torch.randn(512, 128, device="cuda", requires_grad=True)
    y = layer(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    ops.check_status()
    y_ref, dC_ref, dx_ref = o.forward_backward(x.detach().cpu(), layer.cheby_coeffs.detach().cpu(), dy.cpu())
    assert o.rel_l2(y.detach().cpu(), y_ref) <= 3e-3      # against fp32-weight oracle: bf16 storage included
    assert o.rel_l2(layer.cheby_coeffs.grad.cpu(), dC_ref) <= TC_TOL
    assert o.rel_l2(x.grad.cpu(), dx_ref) <= TC_TOL


def test_tc_repack_after_optimizer_step():
    torch.manual_seed(6)
    layer = kan_b200.ChebyKANLayer(64, 128, 4, math_mode="bf16").cuda()
    x = torch.randn(256, 64, device="cuda")
    opt = kan_b200.optim.SGD(layer.parameters(), lr=0.5)
    y0 = layer(x)
    y0.sum().backward()
    opt.step()
    y1 = layer(x).detach()
    ref = o.forward(x.cpu(), layer.cheby_coeffs.detach().cpu().bfloat16().float())
    assert o.rel_l2(y1.cpu(), ref) <= TC_TOL          # the packed copy followed the update
    assert not torch.equal(y0.detach(), y1)


@pytest.mark.parametrize("mode", ["bf16", "tf32"])
def test_full_size_properties(mode):
    """Configuration 3 at full size (65536 x 1024 -> 1024, degree 8) through
    properties that need no CPU oracle run of that size."""
    B, n_in, n_out, deg = 65536, 1024, 1024, 8
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(B, n_in, device="cuda", generator=g)
    coeffs = torch.randn(n_in, n_out, deg + 1, device="cuda", generator=g) / (n_in * (deg + 1))
    packed = ops.pack_coeffs(coeffs, mode)
    y = ops.forward(x, packed, n_in, n_out, deg, mode)
    # (1) any row block recomputed alone gives the same bits
    y_blk = ops.forward(x[32768:32768 + 256].contiguous(), packed, n_in, n_out, deg, mode)
    assert torch.equal(y[32768:32768 + 256], y_blk)
    # (2) a CPU oracle on a 64-row sample of the full-size result
    rows = torch.tensor([0, 1, 127, 128, 4095, 32767, 32768, 65535] + list(range(50000, 50056)))
    c_cpu = coeffs.cpu()
    y_ref = oracle_y(x[rows.cuda()].cpu(), c_cpu, mode)
    assert o.rel_l2(y[rows.cuda()].cpu(), y_ref) <= TC_TOL
    # (3) linearity in the coefficients: y(C) + y(-C) == 0 exactly (sign flips commute with rounding)
    packed_neg = ops.pack_coeffs(-coeffs, mode)
    y_neg = ops.forward(x, packed_neg, n_in, n_out, deg, mode)
    assert torch.equal(y, -y_neg)
    # (4) degree-0-only coefficients: every row equals sum_i C[i,o,0]
    c0 = torch.zeros_like(coeffs)
    c0[:, :, 0] = coeffs[:, :, 0]
    y0 = ops.forward(x, ops.pack_coeffs(c0, mode), n_in, n_out, deg, mode)
    expect = (c0[:, :, 0].bfloat16().float() if mode == "bf16" else c0[:, :, 0]).sum(0)
    assert o.rel_l2(y0[::997].cpu(), expect.cpu().expand(y0[::997].shape[0], n_out)) <= TC_TOL
    torch.cuda.synchronize()
    ops.check_status()


DC_SHAPES = [
    # B, in, out, deg, dist
    (8192, 64, 64, 32, "uniform3"),      # configuration 5 layer: 3 inputs per tile, BN = 64
    (4096, 1024, 1024, 8, "normal"),     # configuration 3 shape: 14 inputs per tile, four N tiles of 256
    (256, 784, 64, 4, "sparse"),         # configuration 2 first layer: 25 inputs per tile
    (100, 16, 12, 3, "normal"),          # out < 32: second half of the 64-wide tile is out of bounds
    (300, 13, 20, 8, "normal"),          # ragged inputs and rows
    (5000, 40, 132, 5, "normal"),        # BN = 256 with a ragged N tile
    (40000, 8, 8, 7, "normal"),          # batch split over many CTAs (workspace + reduction)
    (1, 4, 4, 2, "normal"),              # single row
    # more than 256 outputs: 512-column tiles, CTA pairs over neighbouring input tiles
    (700, 45, 300, 2, "normal"),         # 28 inputs per tile: two tiles = one pair; second half-tile ragged
    (3000, 70, 520, 8, "normal"),        # 14 per tile: five tiles padded to six (an empty tile); two N tiles
    (20000, 20, 512, 6, "normal"),       # pairs with the batch split over CTAs (workspace + reduction)
    (500, 10, 260, 20, "normal"),        # a single input tile with 512-column tiles: no pair
]


@pytest.mark.parametrize("mode", ["tf32", "bf16"])
@pytest.mark.parametrize("B,n_in,n_out,deg,dist", DC_SHAPES)
def test_tc_dcoeff_vs_oracle(mode, B, n_in, n_out, deg, dist):
    x, coeffs, dy = make_case(B, n_in, n_out, deg, dist, seed=B + n_in + deg)
    _, dC_ref, _ = o.forward_backward(x, coeffs, dy, need_dx=False)
    dC, dCw = guarded((n_in, n_out, deg + 1))
    ops.bwd_dcoeff(x.cuda(), dy.cuda(), n_in, n_out, deg, mode, out=dC)
    torch.cuda.synchronize()
    ops.check_status()
    assert_guards_intact(dC, dCw)
    err = o.rel_l2(dC.cpu(), dC_ref)
    assert err <= TC_TOL, err
    assert err > 1e-6            # tf32 operands leave a visible rounding: this is the tensor-core path


# Narrow layers (at most 128 outputs, inputs a multiple of 4) contract in tcgen05 kind::f16 with fp16 operands: the
# basis values as they are, dY scaled by a power of two and transposed by a pre-pass.  fp16 has tf32's 11 significant
# bits, so the error is the tf32 kernel's.
DC_F16_SHAPES = [
    # B, in, out, deg, dist, dY scale
    (70000, 64, 64, 32, "uniform3", 1.0),      # configuration 5 layer, batch split over CTAs, ragged last K block
    (3000, 64, 128, 8, "normal", 1.0),         # 128-column accumulators
    (3000, 100, 96, 5, "normal", 1.0),         # several input tiles, ragged outputs
    (777, 28, 4, 3, "normal", 1.0),            # 28 inputs in one tile (the x tile's 32 columns almost full)
    (63, 8, 8, 63, "normal", 1.0),             # less than one K block; highest tested degree (two inputs per M tile)
    (4096, 64, 64, 32, "uniform3", 3e7),       # large gradients: scaled down into fp16's range
    (4096, 64, 64, 32, "uniform3", 1e-12),     # tiny gradients: scaled up (fp16 alone would flush them to zero)
]


@pytest.mark.parametrize("B,n_in,n_out,deg,dist,dy_scale", DC_F16_SHAPES)
def test_narrow_dcoeff_fp16_operands(B, n_in, n_out, deg, dist, dy_scale):
    x, coeffs, dy = make_case(B, n_in, n_out, deg, dist, seed=B + n_in + deg)
    dy = dy * dy_scale
    _, dC_ref, _ = o.forward_backward(x, coeffs, dy, need_dx=False)
    dC, dCw = guarded((n_in, n_out, deg + 1))
    xd, dyd = x.cuda(), dy.cuda()
    ops.bwd_dcoeff(xd, dyd, n_in, n_out, deg, "tf32", out=dC)
    torch.cuda.synchronize()
    ops.check_status()
    assert_guards_intact(dC, dCw)
    err = o.rel_l2(dC.cpu(), dC_ref)
    assert 1e-6 < err <= TC_TOL, err
    again = ops.bwd_dcoeff(xd, dyd, n_in, n_out, deg, "tf32")
    assert torch.equal(again, dC)                       # fixed summation order: repeatable bit for bit
    acc = dC.clone()
    ops.bwd_dcoeff(xd, dyd, n_in, n_out, deg, "tf32", out=acc, accumulate=True)
    assert o.rel_l2(acc.cpu(), 2 * dC_ref) <= TC_TOL
    # an all-zero gradient gives an all-zero result (no scale can be derived from it)
    z = ops.bwd_dcoeff(xd, torch.zeros_like(dyd), n_in, n_out, deg, "tf32")
    assert float(z.abs().max()) == 0.0


def test_tc_dcoeff_accumulate_and_repeatable():
    x, coeffs, dy = make_case(6000, 24, 64, 8, seed=31)
    _, dC_ref, _ = o.forward_backward(x, coeffs, dy, need_dx=False)
    xd, dyd = x.cuda(), dy.cuda()
    a = ops.bwd_dcoeff(xd, dyd, 24, 64, 8, "tf32")
    b = ops.bwd_dcoeff(xd, dyd, 24, 64, 8, "tf32")
    assert torch.equal(a, b)
    acc = torch.zeros_like(a)
    ops.bwd_dcoeff(xd, dyd, 24, 64, 8, "tf32", out=acc, accumulate=True)
    ops.bwd_dcoeff(xd, dyd, 24, 64, 8, "tf32", out=acc, accumulate=True)
    assert o.rel_l2(acc.cpu(), 2 * dC_ref) <= TC_TOL
    # a shape the tensor-core kernel does not take (out % 4 != 0) falls back to the fp32 kernel
    x, coeffs, dy = make_case(500, 10, 7, 4, seed=32)
    _, dC_ref, _ = o.forward_backward(x, coeffs, dy, need_dx=False)
    got = ops.bwd_dcoeff(x.cuda(), dy.cuda(), 10, 7, 4, "tf32")
    assert o.rel_l2(got.cpu(), dC_ref) <= 1e-5
    ops.check_status()


DX_SHAPES = [
    # B, in, out, deg, dist
    (8192, 64, 64, 32, "uniform3"),      # configuration 5 layer: 7 inputs per 256-slot tile
    (4096, 1024, 1024, 8, "normal"),     # configuration 3 shape: 28 inputs per tile, 32 K blocks
    (256, 64, 12, 4, "normal"),          # configuration 2 second-layer-like, out < 32
    (300, 13, 20, 8, "normal"),          # ragged rows and inputs
    (1000, 51, 40, 4, "normal"),         # 51 inputs x 5 degrees = 255 slots: last TMEM read is shifted
    (129, 5, 36, 63, "normal"),          # degree 63: 4 inputs per tile
    (20000, 8, 8, 7, "normal"),          # more tiles than SMs, both accumulator buffers
    (1, 4, 4, 0, "normal"),              # degree 0: dx is identically zero
]


@pytest.mark.parametrize("mode", ["tf32", "bf16"])
@pytest.mark.parametrize("B,n_in,n_out,deg,dist", DX_SHAPES)
def test_tc_dx_vs_oracle(mode, B, n_in, n_out, deg, dist):
    x, coeffs, dy = make_case(B, n_in, n_out, deg, dist, seed=B + n_in + deg)
    _, _, dx_ref = o.forward_backward(x, coeffs, dy)
    dx, dxw = guarded((B, n_in))
    ops.bwd_dx(x.cuda(), dy.cuda(), coeffs.cuda(), mode, out=dx)
    torch.cuda.synchronize()
    ops.check_status()
    assert_guards_intact(dx, dxw)
    err = o.rel_l2(dx.cpu(), dx_ref)
    assert err <= TC_TOL, err
    if deg > 0:
        assert err > 1e-6            # tf32 operands leave a visible rounding: this is the tensor-core path
    else:
        assert float(dx.abs().max()) == 0.0


@pytest.mark.parametrize("dy_scale,c_scale", [(1.0, 1.0), (1e-9, 1.0), (3e5, 1e-6), (1.0, 4e4)])
@pytest.mark.parametrize("B,n_in,n_out,deg", [
    (700, 40, 512, 8),        # narrowest layer that takes the fp16 operands; ragged rows, eight K blocks of 64 outputs
    (129, 24, 516, 5),        # outputs not a multiple of 64: the last K block ends in zero fill; a CTA pair's second half nearly empty
    (100, 16, 1000, 31),      # one CTA (no pair), 16 K blocks, eight inputs per tile
    (5000, 96, 512, 3),       # more tiles than one wave of pairs
])
def test_wide_dx_fp16_operands(B, n_in, n_out, deg, dy_scale, c_scale):
    """bf16 mode on layers of 512 outputs or more: dY and d * C go to the tensor cores as fp16, each scaled by a power
    of two found from its largest element; the result holds the tensor-core tolerance whatever the magnitudes, and the
    tf32 kernel (same 11 significant bits) lands within the same distance of the oracle."""
    x, coeffs, dy = make_case(B, n_in, n_out, deg, seed=B + n_out + deg)
    dy = dy * dy_scale
    coeffs = coeffs * c_scale
    _, _, dx_ref = o.forward_backward(x, coeffs, dy)
    dx, dxw = guarded((B, n_in))
    ops.bwd_dx(x.cuda(), dy.cuda(), coeffs.cuda(), "bf16", out=dx)
    torch.cuda.synchronize()
    ops.check_status()
    assert_guards_intact(dx, dxw)
    err = o.rel_l2(dx.cpu(), dx_ref)
    err_tf32 = o.rel_l2(ops.bwd_dx(x.cuda(), dy.cuda(), coeffs.cuda(), "tf32").cpu(), dx_ref)
    assert 1e-6 < err <= TC_TOL, err
    assert err <= 2.0 * err_tf32 + 1e-5, (err, err_tf32)
    assert torch.equal(dx, ops.bwd_dx(x.cuda(), dy.cuda(), coeffs.cuda(), "bf16"))     # bitwise repeatable


def test_wide_dx_fp16_operands_zero_and_nan():
    x, coeffs, dy = make_case(300, 8, 512, 4, seed=77)
    zero = ops.bwd_dx(x.cuda(), torch.zeros_like(dy).cuda(), coeffs.cuda(), "bf16")
    assert float(zero.abs().max()) == 0.0
    dy_nan = dy.clone()
    dy_nan[17, 3] = float("nan")
    got = ops.bwd_dx(x.cuda(), dy_nan.cuda(), coeffs.cuda(), "bf16").cpu()
    assert torch.isnan(got[17]).all()                    # the NaN reaches every input of its row
    ops.check_status()


def test_tc_dx_repeatable_and_fallback():
    x, coeffs, dy = make_case(3000, 24, 64, 8, seed=41)
    xd, dyd, cd = x.cuda(), dy.cuda(), coeffs.cuda()
    assert torch.equal(ops.bwd_dx(xd, dyd, cd, "tf32"), ops.bwd_dx(xd, dyd, cd, "tf32"))
    # out % 4 != 0 is not TMA-addressable: the fp32 kernel takes over
    x, coeffs, dy = make_case(500, 10, 7, 4, seed=42)
    _, _, dx_ref = o.forward_backward(x, coeffs, dy)
    got = ops.bwd_dx(x.cuda(), dy.cuda(), coeffs.cuda(), "tf32")
    assert o.rel_l2(got.cpu(), dx_ref) <= 1e-5
    ops.check_status()


def test_bounded_wait_gives_up_and_reports():
    """A wait nothing will ever satisfy runs out after its limit, reports through the status word
    and leaves the GPU context usable (the mechanism that keeps a broken pipeline from hanging)."""
    from kan_b200 import _lib
    lib = _lib.load()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = lib.chebykan_selftest_bounded_wait(st.data_ptr(), 20_000_000, 77, torch.cuda.current_stream().cuda_stream)
    t1.record()
    assert rc == 0
    torch.cuda.synchronize()
    assert int(st.item()) == 77
    assert 15.0 <= t0.elapsed_time(t1) <= 500.0          # about the 20 ms limit, far from the 4 s of the second warp
    # the context still works, and the Python layer turns a non-zero status into an exception
    ops.status_tensor("cuda").fill_(3)
    with pytest.raises(RuntimeError, match="bounded wait"):
        ops.check_status()
    ops.check_status()
    assert lib.chebykan_selftest_bounded_wait(st.data_ptr(), 0, 1, None) == -1
    x, coeffs, _ = make_case(256, 64, 128, 4, seed=1)
    assert o.rel_l2(run_fwd(x, coeffs, "bf16"), oracle_y(x, coeffs, "bf16")) <= TC_TOL


@pytest.mark.parametrize("mode,tol", [("fp32", 1e-5), ("bf16", TC_TOL)])
def test_forward_host_pipelined(mode, tol):
    """Host tensors in and out through the layer's pipelined call: same result as the device call."""
    torch.manual_seed(12)
    layer = kan_b200.ChebyKANLayer(96, 72, 5, math_mode=mode).cuda()
    x = torch.randn(5000, 96).pin_memory()
    y = layer.forward_host(x, chunk_rows=1024)              # 5 blocks, the last one ragged
    assert y.shape == (5000, 72) and not y.is_cuda
    y_dev = layer(x.cuda()).detach().cpu()
    # tensor-core kernels give the same bits for any row blocking; the fp32 kernel splits its contraction over a
    # cluster when a call has few tiles, so there the summation order (not the value) depends on the block size
    same = (lambda a, b: torch.equal(a, b)) if mode != "fp32" else (lambda a, b: o.rel_l2(a, b) <= 1e-6)
    assert same(y, y_dev)
    c = layer.cheby_coeffs.detach().cpu()
    assert o.rel_l2(y, o.forward(x, c.bfloat16().float() if mode == "bf16" else c)) <= tol
    out = torch.empty(5000, 72).pin_memory()
    assert layer.forward_host(x, out=out, chunk_rows=100000) is out and same(out, y)
    # the first and last blocks are shortened (1/8, 1/4, 1/2 of a block): a block size that 8 does not divide
    out.fill_(float("nan"))
    assert same(layer.forward_host(x, out=out, chunk_rows=1030), y)
    # pageable (not pinned) host memory and a block size that does not divide anything: still the same bits
    xp = x[:777].clone()
    assert not xp.is_pinned()
    assert same(layer.forward_host(xp, out=torch.empty(777, 72), chunk_rows=250), y[:777])
    # the C entry point refuses scratch that is too small instead of writing past it
    lib = kan_b200._lib.load()
    packed = ops.pack_coeffs(layer.cheby_coeffs.detach(), mode)
    small = torch.empty(1024, dtype=torch.uint8, device="cuda")
    rc = lib.chebykan_fwd_host_packed(x.data_ptr(), packed.data_ptr(), out.data_ptr(), small.data_ptr(), small.numel(),
                                      5000, 96, 72, 5, ops.MODES[mode], 1024, torch.cuda.current_stream().cuda_stream)
    assert rc == -6                    # CHEBYKAN_EWORKSPACE
    with pytest.raises(RuntimeError):
        layer.forward_host(x.cuda())
    ops.check_status()


@pytest.mark.parametrize("mode", ["bf16", "tf32"])
@pytest.mark.parametrize("widths,deg,B", [((256, 256, 256, 256), 4, 1000), ((200, 136, 72), 3, 333), ((64, 512, 64), 8, 4096),
                                          ((64, 512, 1024, 64), 3, 700)])   # CTA pairs with both fusion sides
def test_fused_layernorm_stack(mode, widths, deg, B):
    """Sequential(Cheby, LN, Cheby, LN, ...) with the LayerNorms folded into the kernels: same output as the
    unfused modules (tight), and within the tensor-core tolerance per layer of the CPU oracle model."""
    from _util import OracleLayer
    torch.manual_seed(widths[0] + deg)
    mods, ref_mods = [], []
    for k in range(len(widths) - 1):
        if k > 0:
            ln = torch.nn.LayerNorm(widths[k])
            with torch.no_grad():                      # a non-trivial affine part
                ln.weight.uniform_(0.5, 1.5)
                ln.bias.uniform_(-0.5, 0.5)
            mods.append(ln)
            ref_ln = torch.nn.LayerNorm(widths[k])
            ref_ln.load_state_dict(ln.state_dict())
            ref_mods.append(ref_ln)
        layer = kan_b200.ChebyKANLayer(widths[k], widths[k + 1], deg, math_mode=mode)
        ref_layer = OracleLayer(widths[k], widths[k + 1], deg)
        c = layer.cheby_coeffs.detach()
        with torch.no_grad():
            ref_layer.cheby_coeffs.copy_(c.bfloat16().float() if mode == "bf16" else c)
        mods.append(layer)
        ref_mods.append(ref_layer)
    model = torch.nn.Sequential(*mods).cuda()
    ref = torch.nn.Sequential(*ref_mods)
    fused = kan_b200.fuse_layernorm(model)
    x = torch.randn(B, widths[0])
    with torch.no_grad():
        y_plain = model(x.cuda()).cpu()
        y_ref = ref(x)
    y_fused = fused(x.cuda()).cpu()
    torch.cuda.synchronize()
    ops.check_status()
    assert y_fused.shape == y_plain.shape
    assert o.rel_l2(y_fused, y_plain) <= 2e-4          # LayerNorm arithmetic order only
    # against the oracle the fused path is as good as the unfused one (rounding accumulates over layers either way)
    err_plain, err_fused = o.rel_l2(y_plain, y_ref), o.rel_l2(y_fused, y_ref)
    assert err_fused <= 1.1 * err_plain + 1e-4
    assert err_fused <= 1.5 * TC_TOL * (len(widths) - 1)
    # parameters are shared, not copied
    assert fused.layers[0].cheby_coeffs is model[0].cheby_coeffs


@pytest.mark.parametrize("mode", ["bf16", "tf32"])
def test_tc_nan_input_propagates(mode):
    """A NaN input poisons exactly its own row of y and its own input's coefficient gradients (degrees >= 1; T_0 is
    the constant 1 here), as a NaN does in the reference's tanh -> acos -> cos chain; everything else is untouched.
    The tf32 paths round finite basis values with an integer add and must not turn the NaN into a finite number."""
    B, n_in, n_out, deg = 300, 40, 520, 5
    x, coeffs, dy = make_case(B, n_in, n_out, deg, seed=91)
    clean = run_fwd(x, coeffs, mode)
    xn = x.clone()
    xn[7, 3] = float("nan")
    y = ops.forward(xn.cuda(), ops.pack_coeffs(coeffs.cuda(), mode), n_in, n_out, deg, mode).cpu()
    ops.check_status()
    assert bool(torch.isnan(y[7]).all())
    keep = torch.ones(B, dtype=torch.bool)
    keep[7] = False
    assert torch.equal(y[keep], clean[keep])
    dC = ops.bwd_dcoeff(xn.cuda(), dy.cuda(), n_in, n_out, deg, mode).cpu()
    ops.check_status()
    assert bool(torch.isnan(dC[3, :, 1:]).all())
    others = torch.ones(n_in, dtype=torch.bool)
    others[3] = False
    assert bool(torch.isfinite(dC[others]).all())


X3_SHAPES = [
    (256, 64, 128, 4, "normal"),          # one 128-wide tile
    (4096, 1024, 1024, 8, "normal"),      # configuration 3 at reduced batch: CTA pairs, 512-column tiles
    (2048, 512, 256, 4, "normal"),        # 256-wide tile, two accumulators
    (8192, 64, 64, 32, "uniform3"),       # configuration 5 layer: 64-wide tile, degree 32
    (100, 13, 7, 3, "normal"),            # in not a multiple of 4: scalar loads
    (1000, 96, 300, 8, "normal"),         # ragged rows, padded outputs
    (130, 64, 512, 3, "normal"),          # pair whose odd CTA holds 2 real rows
    (128, 64, 512, 3, "normal"),          # single-CTA kernel on a wide layer
    (129, 32, 256, 0, "normal"),          # degree 0
]


@pytest.mark.parametrize("B,n_in,n_out,deg,dist", X3_SHAPES)
def test_fp32x3_forward_meets_the_fp32_tolerance(B, n_in, n_out, deg, dist):
    """'fp32x3': three tf32 tensor-core products of head/tail splits; same 1e-5 bound as the FFMA mode."""
    x, coeffs, _ = make_case(B, n_in, n_out, deg, dist, seed=B + n_in + deg)
    y = run_fwd(x, coeffs, "fp32x3")
    err = o.rel_l2(y, o.forward(x, coeffs))
    assert err <= 1e-5, err


@pytest.mark.parametrize("B,n_in,n_out,deg,dist", [
    (8192, 64, 64, 32, "uniform3"), (4096, 1024, 1024, 8, "normal"), (300, 13, 20, 8, "normal"),
    (1000, 51, 40, 4, "normal"), (129, 5, 36, 63, "normal"), (2048, 256, 2048, 3, "normal"), (1, 4, 4, 0, "normal")])
def test_fp32x3_dx_meets_the_fp32_tolerance(B, n_in, n_out, deg, dist):
    """dx in 'fp32x3' mode: the tf32 kernel run on heads and tails of dY and of the coefficients (three launches
    that add into dx), within the 1e-5 bound of the fp32 mode."""
    x, coeffs, dy = make_case(B, n_in, n_out, deg, dist, seed=B + n_in + deg)
    _, _, dx_ref = o.forward_backward(x, coeffs, dy)
    dx, dxw = guarded((B, n_in))
    ops.bwd_dx(x.cuda(), dy.cuda(), coeffs.cuda(), "fp32x3", out=dx)
    torch.cuda.synchronize()
    ops.check_status()
    assert_guards_intact(dx, dxw)
    if deg == 0:
        assert float(dx.abs().max()) == 0.0
    else:
        assert o.rel_l2(dx.cpu(), dx_ref) <= 1e-5


@pytest.mark.parametrize("B,n_in,n_out,deg,dist", [
    (8192, 64, 64, 32, "uniform3"), (4096, 1024, 1024, 8, "normal"), (5000, 40, 132, 5, "normal"),
    (40000, 24, 64, 7, "normal"), (3000, 70, 520, 8, "normal"), (300, 13, 20, 8, "normal"),
    (1024, 1024, 1024, 1, "normal")])      # one batch slice: the three passes add straight into dC
def test_fp32x3_dcoeff_meets_the_fp32_tolerance(B, n_in, n_out, deg, dist):
    """dC in 'fp32x3' mode: the tf32 kernel on basis heads / tails and dY / dY tails over batch slices of at most
    1536 rows, partial sums added in fp32 (small products stay on the fp32 kernel); also with accumulate."""
    x, coeffs, dy = make_case(B, n_in, n_out, deg, dist, seed=B + n_in + deg)
    _, dC_ref, _ = o.forward_backward(x, coeffs, dy, need_dx=False)
    dC, dCw = guarded((n_in, n_out, deg + 1))
    ops.bwd_dcoeff(x.cuda(), dy.cuda(), n_in, n_out, deg, "fp32x3", out=dC)
    torch.cuda.synchronize()
    ops.check_status()
    assert_guards_intact(dC, dCw)
    assert o.rel_l2(dC.cpu(), dC_ref) <= 1e-5
    acc = dC.clone()
    ops.bwd_dcoeff(x.cuda(), dy.cuda(), n_in, n_out, deg, "fp32x3", out=acc, accumulate=True)
    assert o.rel_l2(acc.cpu(), 2 * dC_ref) <= 1e-5


def test_fp32x3_layer_trains_with_fp32_backward():
    torch.manual_seed(5)
    layer = kan_b200.ChebyKANLayer(96, 520, 6, math_mode="fp32x3").cuda()
    x = torch.randn(700, 96, device="cuda", requires_grad=True)
    y = layer(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    ops.check_status()
    y_ref, dC_ref, dx_ref = o.forward_backward(x.detach().cpu(), layer.cheby_coeffs.detach().cpu(), dy.cpu())
    assert o.rel_l2(y.detach().cpu(), y_ref) <= 1e-5
    assert o.rel_l2(layer.cheby_coeffs.grad.cpu(), dC_ref) <= 1e-5
    assert o.rel_l2(x.grad.cpu(), dx_ref) <= 1e-5
    # LayerNorm fusion is a bf16 / tf32 feature: the C entry point refuses this mode
    with pytest.raises(RuntimeError):
        ops.forward_ln(x.detach(), ops.pack_coeffs(layer.cheby_coeffs.detach(), "fp32x3"), 96, 520, 6, "fp32x3",
                       stats_out=torch.zeros(700, 2, device="cuda"))


def test_cta_pair_kernels_replay_from_a_cuda_graph():
    """The wide-layer kernels are cluster launches; captured into a CUDA graph they replay with the same bits."""
    x, coeffs, dy = make_case(600, 48, 520, 4, seed=123)
    xd, cd, dyd = x.cuda(), coeffs.cuda(), dy.cuda()
    packed = ops.pack_coeffs(cd, "bf16")
    y_e = ops.forward(xd, packed, 48, 520, 4, "bf16")
    dc_e = ops.bwd_dcoeff(xd, dyd, 48, 520, 4, "tf32")
    dx_e = ops.bwd_dx(xd, dyd, cd, "tf32")
    y_g, dc_g, dx_g = torch.empty_like(y_e), torch.empty_like(dc_e), torch.empty_like(dx_e)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):                      # warm-up on the capture stream (first-call attribute setup)
        ops.forward(xd, packed, 48, 520, 4, "bf16", out=y_g)
        ops.bwd_dcoeff(xd, dyd, 48, 520, 4, "tf32", out=dc_g)
        ops.bwd_dx(xd, dyd, cd, "tf32", out=dx_g)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ops.forward(xd, packed, 48, 520, 4, "bf16", out=y_g)
        ops.bwd_dcoeff(xd, dyd, 48, 520, 4, "tf32", out=dc_g)
        ops.bwd_dx(xd, dyd, cd, "tf32", out=dx_g)
    for t in (y_g, dc_g, dx_g):
        t.fill_(float("nan"))
    g.replay()
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(y_g, y_e) and torch.equal(dc_g, dc_e) and torch.equal(dx_g, dx_e)



@pytest.mark.parametrize("mode", ["tf32", "bf16"])
def test_graphed_training_step_narrow_layers_equals_eager(mode):
    """Configuration 5's model shape (64 -> 64 -> 64, degree 32) at a small batch: the whole step (narrow-layer
    tensor-memory forward, fp16-operand dC with its pre-pass, dx, fused MSE, SGD) replayed as one CUDA graph leaves
    the coefficients an eager loop leaves, bit for bit."""
    torch.manual_seed(17)
    make = lambda: torch.nn.Sequential(kan_b200.ChebyKANLayer(64, 64, 32, math_mode=mode),
                                       kan_b200.ChebyKANLayer(64, 64, 32, math_mode=mode)).cuda()
    eager, graphed = make(), make()
    graphed.load_state_dict(eager.state_dict())
    B = 4096 + 64
    x = (torch.rand(B, 64, generator=torch.Generator().manual_seed(18)) * 6 - 3).cuda()
    tgt = torch.sin(x).sum(1, keepdim=True).expand(-1, 64).contiguous()
    loss_fn = lambda y, t: kan_b200.mse_loss(y, t, n_mean=B * 64)
    step = kan_b200.graph.GraphedTrainStep(graphed, loss_fn, kan_b200.optim.SGD(list(graphed.parameters()), lr=1e-2),
                                           x, tgt)
    n_done = 3                                           # the constructor's eager warm-up steps
    for _ in range(4):
        step()
        n_done += 1
    buf = kan_b200.dp.FlatGradBuffer(eager.parameters())
    opt = kan_b200.optim.SGD(list(eager.parameters()), lr=1e-2)
    for _ in range(n_done):
        buf.zero()
        loss = loss_fn(eager(x), tgt)
        loss.backward()
        opt.step()
    torch.cuda.synchronize()
    ops.check_status()
    for a, b in zip(eager.parameters(), graphed.parameters()):
        assert torch.equal(a.detach(), b.detach())
    assert torch.equal(step.loss.detach(), loss.detach())
