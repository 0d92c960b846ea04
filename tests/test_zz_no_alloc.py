"""mhlo_cuda_reduce_static_scratch: the split reduce on scratch that is part of the library image.

Collected last on purpose (the file name sorts after every other test file): the entry point must give the same
answers in a fresh process and after the whole suite has used the device. Every case calls it through the C ABI
twice in a row and compares each result with mhlo_cuda_reduce on the same input, bit for bit.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SUM, MAX, ARGMAX = 0, 1, 7
UNSUPPORTED = 4


def cuda_mod():
    from metalhlo_b200 import cuda

    return cuda


def view_of(cuda, t):
    v = cuda.View()
    v.base = t.data_ptr()
    v.dtype = cuda.torch_dtype_code(t.dtype)
    v.rank = t.dim()
    for d in range(t.dim()):
        v.shape[d] = t.shape[d]
        v.stride[d] = t.stride(d)
    return v


def both(cuda, x, n_kept, op, out_dtype, splits=0, want_index=False):
    """(existing entry point, [static-scratch call 1, static-scratch call 2]) as host arrays."""
    n_out = int(np.prod(x.shape[:n_kept])) if n_kept else 1
    stream = torch.cuda.current_stream().cuda_stream
    view = view_of(cuda, x)

    def run(fn, extra):
        out = torch.full((n_out,), -77, device="cuda", dtype=out_dtype)
        idx = torch.full((n_out,), -77, device="cuda", dtype=torch.int32)
        cuda.check(fn(C.byref(view), n_kept, op, None, out.data_ptr(), idx.data_ptr() if want_index else None, cuda.I32, *extra, stream))
        torch.cuda.synchronize()
        return (idx if want_index else out).cpu()

    ref = run(cuda.lib.mhlo_cuda_reduce, ())
    return ref, [run(cuda.lib.mhlo_cuda_reduce_static_scratch, (splits,)) for _ in range(2)]


def test_float_sum_matches_the_allocating_entry_point_bit_for_bit():
    cuda = cuda_mod()
    g = torch.Generator().manual_seed(1)
    x = torch.rand(3, 400_000, generator=g).cuda()
    ref, got = both(cuda, x, 1, SUM, torch.float32)
    for r in got:
        assert torch.equal(r.view(torch.int32), ref.view(torch.int32))
    np.testing.assert_allclose(ref.double().numpy(), x.double().sum(dim=1).cpu().numpy(), rtol=1e-6)


def test_bf16_max_and_argmax_with_ties():
    cuda = cuda_mod()
    g = torch.Generator().manual_seed(2)
    x = torch.randn(2, 300_000, generator=g).to(torch.bfloat16)
    x[0, 250_000] = x[0, 17] = 9.0
    x[1, 299_999] = 12.0
    x = x.cuda()
    ref, got = both(cuda, x, 1, MAX, torch.bfloat16)
    for r in got:
        assert torch.equal(r.view(torch.int16), ref.view(torch.int16))
    assert ref.float().tolist() == [9.0, 12.0]
    ref_i, got_i = both(cuda, x, 1, ARGMAX, torch.bfloat16, want_index=True)
    for r in got_i:
        assert torch.equal(r, ref_i)
    assert ref_i.tolist() == [17, 299_999]


def test_integer_sum_is_exact_for_any_segment_count():
    cuda = cuda_mod()
    g = torch.Generator().manual_seed(3)
    x = torch.randint(-1000, 1000, (1, 1_000_000), generator=g, dtype=torch.int32).cuda()
    want = int(x.sum().item())
    for splits in (0, 1, 7, 512, 3000):
        ref, got = both(cuda, x, 1, SUM, torch.int32, splits=splits)
        assert ref.item() == want
        assert [r.item() for r in got] == [want, want]


def test_scalar_result_of_a_strided_view():
    cuda = cuda_mod()
    g = torch.Generator().manual_seed(4)
    x = torch.rand(1024, 2048, generator=g).cuda().t()  # a transposed view: strides (1, 2048)
    ref, got = both(cuda, x, 0, SUM, torch.float32)
    for r in got:
        assert torch.equal(r.view(torch.int32), ref.view(torch.int32))
    np.testing.assert_allclose(ref.item(), x.double().sum().item(), rtol=1e-6)


def test_more_partials_than_the_built_in_scratch_holds_is_refused():
    cuda = cuda_mod()
    x = torch.ones(8, 1 << 20, device="cuda")
    out = torch.zeros(8, device="cuda")
    view = view_of(cuda, x)
    # 8 outputs x 1024 segments x 16 bytes = 131072 bytes > 65536
    rc = cuda.lib.mhlo_cuda_reduce_static_scratch(C.byref(view), 1, SUM, None, out.data_ptr(), None, cuda.I32, 1024, None)
    assert rc == UNSUPPORTED
    msg = cuda.last_error()
    assert "131072" in msg and "65536" in msg
    # the same reduction with 512 segments (exactly 65536 bytes) runs
    cuda.check(cuda.lib.mhlo_cuda_reduce_static_scratch(C.byref(view), 1, SUM, None, out.data_ptr(), None, cuda.I32, 512, None))
    torch.cuda.synchronize()
    assert out.tolist() == [float(1 << 20)] * 8
    rc = cuda.lib.mhlo_cuda_reduce_static_scratch(C.byref(view), 1, SUM, None, out.data_ptr(), None, cuda.I32, -1, None)
    assert rc == 10  # MHLO_CUDA_INVALID_ARGUMENT
