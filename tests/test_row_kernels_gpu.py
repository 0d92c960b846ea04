"""Parity of the CUDA LayerNorm / RMSNorm / softmax kernels (called through the C ABI of libmhlo_cuda.so)
against the fp64 CPU oracle on the same seeded inputs."""
import math

import numpy as np
import pytest
import torch

import oracle
from parity import assert_close, rel_for, to_np

pytestmark = pytest.mark.gpu

DTYPES = [torch.bfloat16, torch.float16, torch.float32]


def cuda_mod():
    from metalhlo_b200 import cuda

    return cuda


def make_rows(rows, hidden, dtype, seed=42, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, hidden, generator=g) * scale).to(dtype)
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
    beta = (0.1 * torch.randn(hidden, generator=g)).to(dtype)
    return x, gamma, beta


@pytest.mark.parametrize("dtype", DTYPES, ids=str)
@pytest.mark.parametrize("rows,hidden", [(64, 4096), (33, 768), (7, 8), (5, 1024), (3, 12288), (2, 65536)])
def test_layer_norm_rms_softmax_vector_path(dtype, rows, hidden):
    cuda = cuda_mod()
    x, gamma, beta = make_rows(rows, hidden, dtype)
    xd, gd, bd = x.cuda(), gamma.cuda(), beta.cuda()
    rel = rel_for(dtype)
    assert_close(to_np(cuda.layer_norm(xd, gd, bd, 1e-5)), oracle.layer_norm(x, gamma, beta, 1e-5), rel, "layer_norm")
    assert_close(to_np(cuda.rms_norm(xd, gd, 1e-5)), oracle.rms_norm(x, gamma, 1e-5), rel, "rms_norm")
    x4 = (x.float() * 4).to(dtype)
    assert_close(to_np(cuda.softmax(x4.cuda())), oracle.softmax(x4), rel, "softmax")


@pytest.mark.parametrize("dtype", DTYPES, ids=str)
@pytest.mark.parametrize("rows,hidden", [(64, 4096), (33, 768), (7, 8), (300, 1024), (3, 12288), (5, 1001), (2, 16384)])
def test_residual_add_fused_into_the_norm(dtype, rows, hidden):
    """sum = x + r must be bit-identical to a separate add in the element type; the norm is that of the rounded sum."""
    cuda = cuda_mod()
    x, gamma, beta = make_rows(rows, hidden, dtype, seed=5)
    r = make_rows(rows, hidden, dtype, seed=6, scale=0.5)[0]
    want_sum = (x.float() + r.float()).to(dtype)
    rel = rel_for(dtype)
    total, out = cuda.add_layer_norm(x.cuda(), r.cuda(), gamma.cuda(), beta.cuda(), 1e-5)
    assert torch.equal(total.cpu().view(torch.uint8), want_sum.view(torch.uint8))
    assert_close(to_np(out), oracle.layer_norm(want_sum, gamma, beta, 1e-5), rel, "add_layer_norm")
    total, out = cuda.add_rms_norm(x.cuda(), r.cuda(), gamma.cuda(), 1e-5)
    assert torch.equal(total.cpu().view(torch.uint8), want_sum.view(torch.uint8))
    assert_close(to_np(out), oracle.rms_norm(want_sum, gamma, 1e-5), rel, "add_rms_norm")


@pytest.mark.parametrize("dtype", DTYPES, ids=str)
@pytest.mark.parametrize("batch,block,hidden", [(8, 64, 768), (3, 5, 1024), (1, 7, 256), (37, 1, 4096), (4, 6, 1001), (2, 3, 16384)])
def test_residual_block_repeated_down_the_rows(dtype, batch, block, hidden):
    """A [block, hidden] residual added to every one of `batch` groups of rows (a position table over the batch)."""
    cuda = cuda_mod()
    x, gamma, beta = make_rows(batch * block, hidden, dtype, seed=15)
    r = make_rows(block, hidden, dtype, seed=16, scale=0.5)[0]
    want_sum = (x.float().view(batch, block, hidden) + r.float()).to(dtype).view(batch * block, hidden)
    rel = rel_for(dtype)
    total, out = cuda.add_layer_norm(x.cuda(), r.cuda(), gamma.cuda(), beta.cuda(), 1e-5)
    assert torch.equal(total.cpu().view(torch.uint8), want_sum.view(torch.uint8))
    assert_close(to_np(out), oracle.layer_norm(want_sum, gamma, beta, 1e-5), rel, "add_layer_norm_rows")
    total, out = cuda.add_rms_norm(x.cuda(), r.cuda(), gamma.cuda(), 1e-5)
    assert torch.equal(total.cpu().view(torch.uint8), want_sum.view(torch.uint8))
    assert_close(to_np(out), oracle.rms_norm(want_sum, gamma, 1e-5), rel, "add_rms_norm_rows")


def test_residual_block_that_does_not_tile_the_rows_is_rejected():
    cuda = cuda_mod()
    x, gamma, beta = make_rows(10, 256, torch.float16)
    r = make_rows(4, 256, torch.float16, seed=3)[0]
    with pytest.raises(cuda.MhloCudaError) as e:
        cuda.add_layer_norm(x.cuda(), r.cuda(), gamma.cuda(), beta.cuda(), 1e-5)
    assert "do not tile" in str(e.value)


@pytest.mark.parametrize("dtype", DTYPES, ids=str)
@pytest.mark.parametrize("rows,hidden", [(9, 1), (4, 7), (3, 1001), (2, 70001), (1, 300000)])
def test_ragged_hidden_takes_the_strided_path(dtype, rows, hidden):
    cuda = cuda_mod()
    x, gamma, beta = make_rows(rows, hidden, dtype, seed=7)
    rel = rel_for(dtype)
    assert_close(to_np(cuda.layer_norm(x.cuda(), gamma.cuda(), beta.cuda())), oracle.layer_norm(x, gamma, beta), rel)
    assert_close(to_np(cuda.rms_norm(x.cuda(), gamma.cuda())), oracle.rms_norm(x, gamma), rel)
    assert_close(to_np(cuda.softmax(x.cuda())), oracle.softmax(x), rel)


@pytest.mark.parametrize("dtype", DTYPES, ids=str)
def test_unaligned_base_pointers(dtype):
    cuda = cuda_mod()
    x, gamma, beta = make_rows(16, 256, dtype, seed=3)
    # one-element offset views: rows stay contiguous but no pointer is 16-byte aligned
    big = torch.empty(16 * 256 + 1, dtype=dtype, device="cuda")
    xd = big[1:].view(16, 256)
    xd.copy_(x)
    gbuf = torch.empty(257, dtype=dtype, device="cuda")
    gd = gbuf[1:]
    gd.copy_(gamma)
    out = torch.empty(16 * 256 + 1, dtype=dtype, device="cuda")[1:].view(16, 256)
    cuda.layer_norm(xd, gd, None, out=out)
    assert_close(to_np(out), oracle.layer_norm(x, gamma, None), rel_for(dtype))


def test_null_affine_parameters():
    cuda = cuda_mod()
    x, gamma, beta = make_rows(8, 512, torch.float32, seed=5)
    assert_close(to_np(cuda.layer_norm(x.cuda(), None, None)), oracle.layer_norm(x), 1e-5)
    assert_close(to_np(cuda.layer_norm(x.cuda(), None, beta.cuda())), oracle.layer_norm(x, None, beta), 1e-5)
    assert_close(to_np(cuda.rms_norm(x.cuda(), None)), oracle.rms_norm(x), 1e-5)


def test_reference_known_answers_on_device():
    # Tests/MetalHLOCoreTests/MetalKernelTests.swift:56-102 (softmax), :173-225 (LayerNorm), :236-274 (RMSNorm)
    cuda = cuda_mod()
    y = cuda.softmax(torch.tensor([[1.0, 2, 3, 4], [0, 0, 0, 0]], device="cuda")).cpu()
    assert abs(float(y[0].sum()) - 1) < 1e-5 and torch.all((y[1] - 0.25).abs() < 1e-5)
    assert y[0, 3] > y[0, 2] > y[0, 1] > y[0, 0]
    y = cuda.layer_norm(torch.tensor([[1.0, 2, 3, 4], [10, 20, 30, 40]], device="cuda"), None, None).cpu()
    for row in y:
        assert abs(float(row.mean())) < 1e-4 and abs(float(row.std(unbiased=False)) - 1) < 1e-4
    y = cuda.rms_norm(torch.tensor([[3.0, 4, 0, 0]], device="cuda"), None).cpu()[0]
    assert abs(float(y[0]) - 1.2) < 1e-4 and abs(float(y[1]) - 1.6) < 1e-4 and abs(float(y[2])) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES, ids=str)
@pytest.mark.parametrize("shape,axis", [((4, 33, 16), 1), ((6, 5, 7), 0), ((2, 3, 64, 8), 2), ((3, 128), 0)])
def test_softmax_over_an_inner_axis(dtype, shape, axis):
    cuda = cuda_mod()
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(*shape, generator=g) * 3).to(dtype)
    assert_close(to_np(cuda.softmax(x.cuda(), axis=axis)), oracle.softmax(x, axis=axis), rel_for(dtype))


def test_empty_inputs_are_a_no_op():
    cuda = cuda_mod()
    x = torch.empty(0, 128, dtype=torch.bfloat16, device="cuda")
    assert cuda.layer_norm(x, None, None).shape == (0, 128)
    assert cuda.softmax(torch.empty(4, 0, device="cuda")).shape == (4, 0)


def test_softmax_extreme_values_stay_finite():
    cuda = cuda_mod()
    x = torch.tensor([[1e4, -1e4, 0.0, 1e4], [-3e38, -3e38, -3e38, -3e38]], dtype=torch.float32)
    got = to_np(cuda.softmax(x.cuda()))
    assert_close(got, oracle.softmax(x), 1e-5)
    assert np.all(np.isfinite(got))


@pytest.mark.parametrize("tuning", [(64, 8, 0), (128, 4, 0), (256, 2, 0), (512, 1, 0), (128, 4, 8), (256, 2, 4),
                                    (1024, 1, 2)])
def test_every_tuning_of_the_vector_kernel_gives_the_same_answer(tuning):
    cuda = cuda_mod()
    x, gamma, beta = make_rows(300, 4096, torch.bfloat16, seed=13)
    base = cuda.layer_norm(x.cuda(), gamma.cuda(), beta.cuda())
    got = cuda.layer_norm(x.cuda(), gamma.cuda(), beta.cuda(), tuning=tuning)
    assert_close(to_np(got), oracle.layer_norm(x, gamma, beta), 2e-2)
    assert torch.equal(got, base) or (got.float() - base.float()).abs().max() < 0.07
    sm = cuda.softmax(x.cuda(), tuning=tuning)
    assert_close(to_np(sm), oracle.softmax(x), 2e-2)


def test_invalid_tuning_is_rejected_with_a_message():
    cuda = cuda_mod()
    x = torch.zeros(4, 4096, dtype=torch.bfloat16, device="cuda")
    for bad in [(100, 4, 0), (128, 3, 0), (32, 1, 0), (512, 8, 0)]:
        with pytest.raises(cuda.MhloCudaError) as e:
            cuda.layer_norm(x, None, None, tuning=bad)
        assert e.value.status == 10


def test_full_size_norm_sweep_properties_and_sampled_parity():
    """The benchmark configuration: [32768, 4096] bf16, eps 1e-5; softmax input scaled by 4."""
    cuda = cuda_mod()
    rows, hidden = 32768, 4096
    x, gamma, beta = make_rows(rows, hidden, torch.bfloat16, seed=42)
    xd, gd, bd = x.cuda(), gamma.cuda(), beta.cuda()
    pick = torch.arange(0, rows, 257)
    ln = cuda.layer_norm(xd, gd, bd)
    assert_close(to_np(ln[pick.cuda()]), oracle.layer_norm(x[pick], gamma, beta), 2e-2, "layer_norm")
    rm = cuda.rms_norm(xd, gd)
    assert_close(to_np(rm[pick.cuda()]), oracle.rms_norm(x[pick], gamma), 2e-2, "rms_norm")
    x4 = (xd.float() * 4).to(torch.bfloat16)
    sm = cuda.softmax(x4)
    assert_close(to_np(sm[pick.cuda()]), oracle.softmax(x4[pick.cuda()].cpu()), 2e-2, "softmax")
    # size-independent properties over every row
    sums = sm.float().sum(dim=1)
    assert float((sums - 1).abs().max()) < 2e-2
    plain = cuda.layer_norm(xd, None, None).float()
    assert float(plain.mean(dim=1).abs().max()) < 1e-2
    assert float((plain.std(dim=1, unbiased=False) - 1).abs().max()) < 1e-2
    # scaling the input leaves LayerNorm unchanged and RMSNorm unchanged (eps aside): linearity check
    ln2 = cuda.layer_norm((xd.float() * 2).to(torch.bfloat16), gd, bd)
    assert float((ln2.float() - ln.float()).abs().max()) < 0.05
