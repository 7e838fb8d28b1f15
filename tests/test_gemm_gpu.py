"""The tcgen05 matrix product against float64, in both operand arrangements, at ragged sizes."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, seed=0, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).to(torch.bfloat16)


def check(got, want, bf16_out=True):
    got, want = got.cpu().double(), want
    assert torch.isfinite(got).all()
    tolerance = (2 ** -8 if bf16_out else 1e-5) * want.abs().max()
    error = (got - want).abs().max()
    assert error <= tolerance, f"error {float(error):.3e} above {float(tolerance):.3e}"


@pytest.mark.parametrize("m, n, k", [(128, 256, 64), (200, 520, 328), (2048, 1024, 512), (65, 256, 1096), (300, 136, 72)])
def test_tile_shape_bf16_and_float_outputs(m, n, k):
    from hyperion_b200.ops import gemm, raise_on_status

    x, w, b = rnd(m, k, seed=1), rnd(n, k, seed=2, scale=0.1), rnd(n, seed=3)
    want = x.double() @ w.double().t()
    check(gemm.gemm_bf16(x.to(DEV), w.to(DEV)), want)
    check(gemm.gemm_bf16(x.to(DEV), w.to(DEV), b.to(DEV)), want + b.double())
    check(gemm.gemm_bf16(x.to(DEV), w.to(DEV), b.float().to(DEV), epilogue=gemm.EPI_F32), want + b.double(), bf16_out=False)
    raise_on_status(torch.device(DEV))


def test_rows_may_be_strided_views():
    from hyperion_b200.ops import gemm

    big = rnd(70, 400, seed=4)
    x = big.to(DEV)[:, 64:64 + 264]  # row stride 400, offset 128 bytes
    w = rnd(90, 264, seed=5, scale=0.1)
    check(gemm.gemm_bf16(x, w.to(DEV)), big[:, 64:64 + 264].double() @ w.double().t())


@pytest.mark.parametrize("m, inter, k", [(130, 256, 192), (2048, 1280, 256), (7, 128, 64)])
def test_fused_swiglu_epilogue(m, inter, k):
    from hyperion_b200.ops import gemm

    x, gate, up = rnd(m, k, seed=6), rnd(inter, k, seed=7, scale=0.2), rnd(inter, k, seed=8, scale=0.2)
    w = gemm.interleave_gate_up(gate, up)
    got = gemm.gemm_bf16(x.to(DEV), w.to(DEV), epilogue=gemm.EPI_SWIGLU)
    g = (x.double() @ gate.double().t()).to(torch.bfloat16).double()  # the projections are rounded before the activation
    u = (x.double() @ up.double().t()).to(torch.bfloat16).double()
    check(got, g / (1 + torch.exp(-g)) * u)


@pytest.mark.parametrize("m", [1, 8, 16, 17, 33, 64])
@pytest.mark.parametrize("n, k, splits", [(384, 328, 1), (1000, 2048, 3), (128, 64, 1), (3584, 1152, None)])
def test_swapped_shape_for_small_batches(m, n, k, splits):
    from hyperion_b200.ops import gemm, raise_on_status

    x, w, b = rnd(m, k, seed=9), rnd(n, k, seed=10, scale=0.1), rnd(n, seed=11)
    want = x.double() @ w.double().t() + b.double()
    check(gemm.gemm_bf16(x.to(DEV), w.to(DEV), b.to(DEV), splits=splits), want)
    check(gemm.gemm_bf16(x.to(DEV), w.to(DEV), b.float().to(DEV), epilogue=gemm.EPI_F32, splits=splits), want, bf16_out=False)
    raise_on_status(torch.device(DEV))


def test_a_row_does_not_depend_on_its_batch():
    from hyperion_b200.ops import gemm

    x, w = rnd(64, 512, seed=12), rnd(640, 512, seed=13, scale=0.1)
    full = gemm.gemm_bf16(x.to(DEV), w.to(DEV), splits=2)
    for m in (1, 5, 16, 40):
        part = gemm.gemm_bf16(x[:m].to(DEV), w.to(DEV), splits=2)
        assert torch.equal(part, full[:m])


@pytest.mark.parametrize("m, n, k", [(256, 256, 64), (200, 520, 328), (2048, 1024, 512), (65, 272, 1096), (700, 136, 72), (1000, 3584, 640)])
def test_pairs_of_sms_bf16_and_float_outputs(m, n, k):
    """The cta_group::2 kernel: 256-row tiles shared by two SMs, ragged in every extent, several tiles per pair."""
    from hyperion_b200.ops import gemm, raise_on_status

    x, w, b = rnd(m, k, seed=21), rnd(n, k, seed=22, scale=0.1), rnd(n, seed=23)
    want = x.double() @ w.double().t()
    check(gemm.gemm_pair_bf16(x.to(DEV), w.to(DEV)), want)
    check(gemm.gemm_pair_bf16(x.to(DEV), w.to(DEV), b.to(DEV)), want + b.double())
    check(gemm.gemm_pair_bf16(x.to(DEV), w.to(DEV), b.float().to(DEV), epilogue=gemm.EPI_F32), want + b.double(), bf16_out=False)
    raise_on_status(torch.device(DEV))


@pytest.mark.parametrize("m, inter, k", [(130, 256, 192), (2048, 1280, 256), (300, 128, 64)])
def test_pairs_of_sms_fused_swiglu(m, inter, k):
    from hyperion_b200.ops import gemm, raise_on_status

    x, gate, up = rnd(m, k, seed=26), rnd(inter, k, seed=27, scale=0.2), rnd(inter, k, seed=28, scale=0.2)
    w = gemm.interleave_gate_up(gate, up)
    got = gemm.gemm_pair_bf16(x.to(DEV), w.to(DEV), epilogue=gemm.EPI_SWIGLU)
    g = (x.double() @ gate.double().t()).to(torch.bfloat16).double()  # the projections are rounded before the activation
    u = (x.double() @ up.double().t()).to(torch.bfloat16).double()
    check(got, g / (1 + torch.exp(-g)) * u)
    raise_on_status(torch.device(DEV))
