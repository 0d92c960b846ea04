"""The tensor-core GEMM with a pair of CTAs per 256 x 256 tile (tcgen05 cta_group::2), and its other launch knobs, against
the fp64 oracle: every operand major, ragged edges in all three extents, batches, epilogues, more tiles than pairs, and
bit-equality with the one-CTA kernel (the same products are accumulated in the same order)."""
import math

import pytest
import torch

import oracle
from parity import assert_close, to_np

pytestmark = pytest.mark.gpu

PAIR = (256, 0, 2)


def cuda_mod():
    from metalhlo_b200 import cuda

    return cuda


def operands(batch, m, n, k, dtype, trans_a, trans_b, seed=0):
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(*batch, k, m, generator=g) if trans_a else torch.randn(*batch, m, k, generator=g)) / math.sqrt(k)
    b = torch.randn(*batch, n, k, generator=g) if trans_b else torch.randn(*batch, k, n, generator=g)
    return a.to(dtype), b.to(dtype)


def reference(a, b, trans_a, trans_b):
    a3 = a.reshape(-1, *a.shape[-2:])
    b3 = b.reshape(-1, *b.shape[-2:])
    c = oracle.gemm(a3, b3, trans_a=trans_a, trans_b=trans_b)
    return c.reshape(*a.shape[:-2], *c.shape[-2:])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=str)
@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (512, 512, 256), (384, 640, 192), (136, 264, 72), (1000, 776, 328), (130, 300, 64),
                                   (64, 64, 64), (2048, 768, 768)])
def test_pair_kernel_all_operand_majors(dtype, trans_a, trans_b, m, n, k):
    cuda = cuda_mod()
    a, b = operands((), m, n, k, dtype, trans_a, trans_b, seed=m + n + k)
    got = cuda.gemm(a.cuda(), b.cuda(), trans_a=trans_a, trans_b=trans_b, tuning=PAIR)
    assert cuda.device_error() == 0
    assert_close(to_np(got), reference(a, b, trans_a, trans_b), 2e-2, f"pair gemm {m}x{n}x{k}")
    # the same sums in the same order as the one-CTA kernel: equal bit for bit
    one = cuda.gemm(a.cuda(), b.cuda(), trans_a=trans_a, trans_b=trans_b, tuning=(256, 0, 1))
    assert torch.equal(got.view(torch.int16), one.view(torch.int16))


@pytest.mark.parametrize("batch", [(3,), (2, 3)])
def test_pair_kernel_batched_with_bias_and_activation(batch):
    cuda = cuda_mod()
    a, b = operands(batch, 384, 512, 128, torch.bfloat16, False, False, seed=5)
    bias = (0.5 * torch.randn(512, generator=torch.Generator().manual_seed(1))).to(torch.bfloat16)
    got = cuda.gemm(a.cuda(), b.cuda(), bias=bias.cuda(), epilogue="relu", tuning=PAIR)
    assert cuda.device_error() == 0
    import numpy as np

    want = np.maximum(reference(a, b, False, False) + bias.double().numpy(), 0)
    assert_close(to_np(got), want, 2e-2, "pair gemm, batched, bias + relu")


def test_pair_kernel_walks_many_tiles_per_pair():
    """8192 x 4096 x 512: 512 tiles on 74 pairs, so every pair hands its stages, accumulators and barriers on seven times."""
    cuda = cuda_mod()
    g = torch.Generator(device="cuda").manual_seed(3)
    a = (torch.randint(-4, 5, (8192, 512), generator=g, device="cuda").float() / 8).to(torch.bfloat16)
    b = (torch.randint(-4, 5, (512, 4096), generator=g, device="cuda").float() / 8).to(torch.bfloat16)
    got = cuda.gemm(a, b, out_dtype=torch.float32, tuning=PAIR)
    assert cuda.device_error() == 0
    # small integers / 8: every product and partial sum is exact in fp32, so any correct kernel gives the exact result
    assert torch.equal(got, a.float() @ b.float())


@pytest.mark.parametrize("tuning", [(128, 0, 1), (128, 3, 1), (256, 2, 1), (256, 4, 1), (256, 3, 2), (256, 6, 2), (0, 0, 0)])
def test_every_configuration_of_the_knobs_gives_the_same_result(tuning):
    cuda = cuda_mod()
    a, b = operands((), 640, 896, 448, torch.float16, False, True, seed=9)
    got = cuda.gemm(a.cuda(), b.cuda(), trans_b=True, tuning=tuning)
    assert cuda.device_error() == 0
    assert_close(to_np(got), reference(a, b, False, True), 2e-2, f"tuning {tuning}")
    base = cuda.gemm(a.cuda(), b.cuda(), trans_b=True)
    assert torch.equal(got.view(torch.int16), base.view(torch.int16))


def test_configurations_the_kernel_does_not_have_are_refused():
    cuda = cuda_mod()
    a, b = operands((), 256, 256, 64, torch.bfloat16, False, False)
    for bad in [(64, 0, 1), (128, 0, 2), (256, 9, 1), (256, 1, 1), (256, 0, 3)]:
        with pytest.raises(RuntimeError, match="not a configuration"):
            cuda.gemm(a.cuda(), b.cuda(), tuning=bad)
