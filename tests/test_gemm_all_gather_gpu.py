"""mhlo_cuda_gemm_all_gather: the column-split GEMM whose epilogue stores every tile into all ranks' copies of C.

On one GPU the "ranks" are launched one after the other and the copies of C are separate local buffers: the tile
placement (row pitch, column offset, every copy written) is exactly what runs across GPUs, only the stores stay local.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def run_ranks(cuda, a, b, n_ranks, out_dtype=torch.bfloat16, bias=None, epilogue=0):
    m, k = a.shape
    n = b.shape[1]
    n_local = n // n_ranks
    copies = [torch.full((m, n), float("nan"), device="cuda", dtype=out_dtype) for _ in range(n_ranks)]
    ptrs = (C.c_void_p * n_ranks)(*[c.data_ptr() for c in copies])
    stream = torch.cuda.current_stream().cuda_stream
    for rank in range(n_ranks):
        b_local = b[:, rank * n_local:(rank + 1) * n_local]  # a column block of B, read in place through its strides
        bias_ptr = None if bias is None else bias[rank * n_local:(rank + 1) * n_local].data_ptr()
        cuda.check(cuda.lib.mhlo_cuda_gemm_all_gather(
            cuda.torch_dtype_code(a.dtype), cuda.torch_dtype_code(out_dtype), a.data_ptr(), cuda._i64s([a.stride(0), a.stride(1)]),
            b_local.data_ptr(), cuda._i64s([b_local.stride(0), b_local.stride(1)]), ptrs, n_ranks, rank, m, n_local, k, bias_ptr, epilogue, stream))
    torch.cuda.synchronize()
    assert cuda.device_error() == 0
    return copies


@pytest.mark.parametrize("n_ranks", [1, 2, 4, 8])
@pytest.mark.parametrize("m,n,k", [(512, 1024, 256), (300, 2048, 320), (1024, 4096, 512)])
def test_every_copy_holds_the_full_product(n_ranks, m, n, k):
    from metalhlo_b200 import cuda

    g = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(torch.bfloat16).cuda()
    b = torch.randn(k, n, generator=g).to(torch.bfloat16).cuda()
    copies = run_ranks(cuda, a, b, n_ranks)
    want = cuda.gemm(a, b)  # the single-GPU product of the same operands
    for c in copies:
        assert torch.equal(c.view(torch.int16), want.view(torch.int16))
    ref = (a.double() @ b.double())
    assert (copies[0].double() - ref).abs().max() <= 2e-2 * ref.abs().max()


def test_bias_and_activation_travel_with_the_tiles():
    from metalhlo_b200 import cuda

    g = torch.Generator().manual_seed(3)
    a = (torch.randn(256, 128, generator=g) / 11).to(torch.float16).cuda()
    b = torch.randn(128, 1024, generator=g).to(torch.float16).cuda()
    bias = torch.randn(1024, generator=g).to(torch.float16).cuda()
    copies = run_ranks(cuda, a, b, 4, out_dtype=torch.float16, bias=bias, epilogue=cuda.EPILOGUES["relu"])
    want = torch.relu(a.float() @ b.float() + bias.float())
    for c in copies:
        assert torch.equal(c, copies[0])
        assert (c.float() - want).abs().max() <= 2e-2 * want.abs().max()


def test_bad_rank_counts_are_refused():
    from metalhlo_b200 import cuda

    x = torch.zeros(128, 128, device="cuda", dtype=torch.bfloat16)
    ptrs = (C.c_void_p * 1)(x.data_ptr())
    st = cuda._i64s([128, 1])
    assert cuda.lib.mhlo_cuda_gemm_all_gather(cuda.BF16, cuda.BF16, x.data_ptr(), st, x.data_ptr(), st, ptrs, 9, 0, 128, 128, 128, None, 0, None) == 10
    assert cuda.lib.mhlo_cuda_gemm_all_gather(cuda.BF16, cuda.BF16, x.data_ptr(), st, x.data_ptr(), st, ptrs, 1, 1, 128, 128, 128, None, 0, None) == 10
    f = torch.zeros(128, 128, device="cuda")
    pf = (C.c_void_p * 1)(f.data_ptr())
    assert cuda.lib.mhlo_cuda_gemm_all_gather(cuda.F32, cuda.F32, f.data_ptr(), st, f.data_ptr(), st, pf, 1, 0, 128, 128, 128, None, 0, None) == 4
