"""mhlo_cuda_convert_many: many dense dtype conversions in one launch, bit-exact against torch's round-to-nearest-even
casts; sizes straddle the 4096-element tile, pointers are both aligned and off by one element, and more jobs than one
launch table holds are given."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

PAIRS = [(torch.float32, torch.float16), (torch.float32, torch.bfloat16), (torch.float16, torch.float32),
         (torch.bfloat16, torch.float32), (torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)]
SIZES = [0, 1, 15, 16, 4095, 4096, 4097, 12288, 50_000, 1_000_003]


def test_every_pair_size_and_alignment_bit_exact():
    from metalhlo_b200 import cuda

    g = torch.Generator().manual_seed(9)
    jobs, checks = [], []
    for si, n in enumerate(SIZES + SIZES):
        for pi, (sd, dd) in enumerate(PAIRS):
            shift = (si + pi) % 2  # every other job starts one element past a 16-byte boundary
            src_store = (torch.randn(n + 1, generator=g) * 300).to(sd).cuda()
            dst_store = torch.full((n + 1,), 7.0, dtype=dd, device="cuda")
            src, dst = src_store[shift:shift + n], dst_store[shift:shift + n]
            jobs.append(cuda.ConvertJob(src.data_ptr() if n else None, dst.data_ptr() if n else None, n, cuda.torch_dtype_code(sd),
                                        cuda.torch_dtype_code(dd)))
            checks.append((src, dst, dst_store, shift, n, dd))
    assert len(jobs) > 96  # more than one launch table
    table = (cuda.ConvertJob * len(jobs))(*jobs)
    cuda.check(cuda.lib.mhlo_cuda_convert_many(table, len(jobs), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    for src, dst, store, shift, n, dd in checks:
        assert torch.equal(dst.view(torch.uint8), src.to(dd).view(torch.uint8)), (n, dd)
        # the elements around the job are untouched
        assert float(store[0 if shift else n]) == 7.0


def test_bad_jobs_are_refused():
    from metalhlo_b200 import cuda

    x = torch.zeros(8, device="cuda")
    bad_pair = (cuda.ConvertJob * 1)(cuda.ConvertJob(x.data_ptr(), x.data_ptr(), 8, cuda.F16, cuda.BF16))
    assert cuda.lib.mhlo_cuda_convert_many(bad_pair, 1, None) == 4          # MHLO_CUDA_UNSUPPORTED
    null_ptr = (cuda.ConvertJob * 1)(cuda.ConvertJob(None, x.data_ptr(), 8, cuda.F32, cuda.F32))
    assert cuda.lib.mhlo_cuda_convert_many(null_ptr, 1, None) == 10         # MHLO_CUDA_INVALID_ARGUMENT
    assert cuda.lib.mhlo_cuda_convert_many(None, 0, None) == 0
