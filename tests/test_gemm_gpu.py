"""Parity of mhlo_cuda_gemm (tcgen05 tensor-core path and general-layout path) against the fp64 oracle."""
import math

import pytest
import torch

import oracle
from parity import assert_close, to_np

pytestmark = pytest.mark.gpu


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
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (384, 640, 192), (128, 128, 512), (136, 264, 72),
                                   (1000, 776, 328), (64, 64, 64)])
def test_tensor_core_gemm_all_operand_majors(dtype, trans_a, trans_b, m, n, k):
    cuda = cuda_mod()
    a, b = operands((), m, n, k, dtype, trans_a, trans_b, seed=m + n + k)
    got = cuda.gemm(a.cuda(), b.cuda(), trans_a=trans_a, trans_b=trans_b)
    assert cuda.device_error() == 0
    assert_close(to_np(got), reference(a, b, trans_a, trans_b), 2e-2, f"gemm {m}x{n}x{k}")


@pytest.mark.parametrize("batch", [(3,), (2, 3), (64,)])
def test_batched(batch):
    cuda = cuda_mod()
    m, n, k = (256, 256, 128) if batch != (64,) else (128, 256, 128)
    a, b = operands(batch, m, n, k, torch.bfloat16, False, False, seed=5)
    got = cuda.gemm(a.cuda(), b.cuda())
    assert cuda.device_error() == 0
    assert_close(to_np(got), reference(a, b, False, False), 2e-2, "batched gemm")


@pytest.mark.parametrize("epilogue", ["none", "relu", "gelu_tanh", "gelu_erf", "silu", "tanh", "sigmoid"])
def test_bias_and_activation_epilogue(epilogue):
    cuda = cuda_mod()
    m, n, k = 256, 384, 128
    a, b = operands((), m, n, k, torch.bfloat16, False, False, seed=9)
    bias = (0.5 * torch.randn(n, generator=torch.Generator().manual_seed(1))).to(torch.bfloat16)
    got = cuda.gemm(a.cuda(), b.cuda(), bias=bias.cuda(), epilogue=epilogue)
    want = reference(a, b, False, False) + bias.double().numpy()
    import numpy as np

    if epilogue == "relu":
        want = np.maximum(want, 0)
    elif epilogue == "gelu_tanh":
        want = 0.5 * want * (1 + np.tanh(0.7978845608028654 * (want + 0.044715 * want ** 3)))
    elif epilogue == "gelu_erf":
        want = 0.5 * want * (1 + np.vectorize(math.erf)(want / math.sqrt(2)))
    elif epilogue == "silu":
        want = want / (1 + np.exp(-want))
    elif epilogue == "tanh":
        want = np.tanh(want)
    elif epilogue == "sigmoid":
        want = 1 / (1 + np.exp(-want))
    assert_close(to_np(got), want, 2e-2, f"epilogue {epilogue}")


@pytest.mark.parametrize("dtype,out_dtype", [(torch.float16, torch.float16), (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32),
                                             (torch.float32, torch.float32)], ids=str)
@pytest.mark.parametrize("m,n,k,tuning", [(512, 768, 256, None), (300, 264, 72, None), (1024, 512, 128, (256, 6, 2)), (256, 250, 64, None)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_residual_is_added_before_the_rounding(dtype, out_dtype, m, n, k, tuning, with_bias):
    """mhlo_cuda_gemm_residual: A . B + bias + R against the fp64 oracle; n = 250 and fp32 operands take the two-pass route."""
    cuda = cuda_mod()
    a, b = operands((), m, n, k, dtype, False, False, seed=m + n)
    g = torch.Generator().manual_seed(n)
    bias = torch.randn(n, generator=g).to(out_dtype) if with_bias else None
    res = (3 * torch.randn(m, n, generator=g)).to(out_dtype)
    got = cuda.gemm(a.cuda(), b.cuda(), bias=None if bias is None else bias.cuda(), out_dtype=out_dtype, residual=res.cuda(), tuning=tuning)
    assert cuda.device_error() == 0
    want = reference(a, b, False, False) + res.double().numpy() + (0 if bias is None else bias.double().numpy())
    assert_close(to_np(got), want, 1e-5 if out_dtype == torch.float32 and dtype == torch.float32 else 2e-2, f"gemm+residual {m}x{n}x{k}")
    if dtype != torch.float32 and n % 8 == 0:
        # one rounding: the result is the correctly rounded fp32 sum wherever fp32 accumulation is exact enough to tell
        plain = cuda.gemm(a.cuda(), b.cuda(), out_dtype=torch.float32).double().cpu()
        twice = (plain + res.double() + (0 if bias is None else bias.double())).to(out_dtype)
        assert (got.cpu().double() - twice.double()).abs().max() <= 2e-2 * want.__abs__().max()


def test_fp32_output_from_bf16_operands():
    cuda = cuda_mod()
    a, b = operands((), 256, 256, 512, torch.bfloat16, False, True, seed=2)
    got = cuda.gemm(a.cuda(), b.cuda(), trans_b=True, out_dtype=torch.float32)
    assert_close(to_np(got), reference(a, b, False, True), 1e-5, "f32 out")  # fp32 accumulation of exact bf16 products


def test_unaligned_row_stride_of_c_and_odd_n():
    cuda = cuda_mod()
    # vocabulary-sized N that is not a multiple of 8: the epilogue falls back to element stores at the ragged edge
    m, n, k = 256, 50257 // 32 + 1, 768
    a, b = operands((), m, n, k, torch.float16, False, True, seed=3)
    got = cuda.gemm(a.cuda(), b.cuda(), trans_b=True)
    assert_close(to_np(got), reference(a, b, False, True), 2e-2, "odd n")


def test_general_layout_path_fp32_and_tiny():
    cuda = cuda_mod()
    a, b = operands((), 33, 45, 70, torch.float32, False, False, seed=4)
    assert_close(to_np(cuda.gemm(a.cuda(), b.cuda())), reference(a, b, False, False), 1e-5, "fp32 gemm")
    a, b = operands((), 5, 7, 3, torch.bfloat16, False, False, seed=4)
    assert_close(to_np(cuda.gemm(a.cuda(), b.cuda())), reference(a, b, False, False), 2e-2, "tiny")


def test_linearity_at_benchmark_size():
    """8192^3 bf16: too large for the CPU oracle, so use linearity: (A1 + A2) B = A1 B + A2 B with exactly representable
    sums, and a sampled block against the oracle."""
    cuda = cuda_mod()
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(7)
    a1 = (torch.randint(-4, 5, (n, n), generator=g, device="cuda").float() / 8).to(torch.bfloat16)
    a2 = (torch.randint(-4, 5, (n, n), generator=g, device="cuda").float() / 8).to(torch.bfloat16)
    b = (torch.randint(-4, 5, (n, n), generator=g, device="cuda").float() / 8).to(torch.bfloat16)
    c1 = cuda.gemm(a1, b, out_dtype=torch.float32)
    c2 = cuda.gemm(a2, b, out_dtype=torch.float32)
    c12 = cuda.gemm((a1.float() + a2.float()).to(torch.bfloat16), b, out_dtype=torch.float32)
    assert cuda.device_error() == 0
    # small integers / 8: every product and partial sum is exact in fp32, so linearity holds bit for bit
    assert torch.equal(c12, c1 + c2)
    rows = torch.arange(0, n, 1021, device="cuda")
    want = oracle.gemm(a1[rows].cpu(), b.cpu())
    assert_close(to_np(c1[rows]), want, 1e-6, "sampled rows of 8192^3")


def test_batched_benchmark_configuration_against_the_oracle():
    """bf16 [64,2048,128] . [64,128,2048] with operands ~ N(0,1)/sqrt(128): the HBM-limited batched product at exactly its
    benchmark extents, every element of every batch against the fp64 oracle."""
    cuda = cuda_mod()
    g = torch.Generator().manual_seed(42)
    a = (torch.randn(64, 2048, 128, generator=g) / math.sqrt(128)).to(torch.bfloat16)
    b = (torch.randn(64, 128, 2048, generator=g) / math.sqrt(128)).to(torch.bfloat16)
    got = cuda.gemm(a.cuda(), b.cuda())
    assert cuda.device_error() == 0
    assert tuple(got.shape) == (64, 2048, 2048) and got.dtype == torch.bfloat16
    got = got.cpu()
    for i in range(64):
        assert_close(to_np(got[i]), oracle.gemm(a[i], b[i]), 2e-2, f"batch {i} of [64,2048,128].[64,128,2048]")
