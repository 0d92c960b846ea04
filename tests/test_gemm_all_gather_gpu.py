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


@pytest.mark.parametrize("copy_stores", [1, 2])
@pytest.mark.parametrize("tile_n,cta_group", [(0, 0), (128, 1), (256, 1), (256, 2)])
@pytest.mark.parametrize("n_ranks", [2, 8])
def test_bulk_tensor_stores_write_the_same_copies(n_ranks, tile_n, cta_group, copy_stores):
    """copy_stores = 2: every staged box goes to each copy with one bulk tensor store; the bits are those of the lane stores."""
    from metalhlo_b200 import cuda

    m, n, k = 600, 2048, 320
    g = torch.Generator().manual_seed(17)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(torch.bfloat16).cuda()
    b = torch.randn(k, n, generator=g).to(torch.bfloat16).cuda()
    n_local = n // n_ranks
    copies = [torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(n_ranks)]
    ptrs = (C.c_void_p * n_ranks)(*[c.data_ptr() for c in copies])
    tuning = cuda.GemmTuning(tile_n, 0, cta_group, 0)
    for rank in range(n_ranks):
        b_local = b[:, rank * n_local:(rank + 1) * n_local]
        cuda.check(cuda.lib.mhlo_cuda_gemm_all_gather_tuned(
            cuda.BF16, cuda.BF16, a.data_ptr(), cuda._i64s([k, 1]), b_local.data_ptr(), cuda._i64s([n, 1]), ptrs, n_ranks, rank, m, n_local, k,
            None, 0, C.addressof(tuning), copy_stores, None))
    torch.cuda.synchronize()
    assert cuda.device_error() == 0
    want = run_ranks(cuda, a, b, n_ranks)[0]
    for c in copies:
        assert torch.equal(c.view(torch.int16), want.view(torch.int16))


def test_all_gather_knobs_outside_the_kernel_are_refused():
    from metalhlo_b200 import cuda

    x = torch.zeros(128, 128, device="cuda", dtype=torch.bfloat16)
    ptrs = (C.c_void_p * 1)(x.data_ptr())
    st = cuda._i64s([128, 1])
    call = lambda tuning, stores: cuda.lib.mhlo_cuda_gemm_all_gather_tuned(
        cuda.BF16, cuda.BF16, x.data_ptr(), st, x.data_ptr(), st, ptrs, 1, 0, 128, 128, 128, None, 0, C.addressof(tuning), stores, None)
    assert call(cuda.GemmTuning(0, 0, 0, 0), 3) == 10
    assert call(cuda.GemmTuning(192, 0, 0, 0), 0) == 10
    assert call(cuda.GemmTuning(128, 0, 2, 0), 0) == 10  # a pair of CTAs shares a 256-column tile
    assert call(cuda.GemmTuning(256, 4, 1, 0), 2) == 0
    torch.cuda.synchronize()


def test_peer_barrier_passes_once_every_rank_has_published():
    """One GPU stands for rank 1 of 4; the other ranks' words are written by the host beforehand, as their kernels would."""
    from metalhlo_b200 import cuda

    flags = [torch.zeros(8, dtype=torch.int64, device="cuda") for _ in range(4)]
    flags[1][0] = 7
    flags[1][2] = 7
    flags[1][3] = 9  # a rank that is already one epoch ahead
    ptrs = (C.c_void_p * 4)(*[f.data_ptr() for f in flags])
    torch.cuda.synchronize()
    cuda.check(cuda.lib.mhlo_cuda_peer_barrier(ptrs, 4, 1, 7, 50_000_000, None))
    torch.cuda.synchronize()
    assert cuda.device_error() == 0
    for r in (0, 2, 3):  # rank 1 published its epoch in word 1 of every other rank's array
        assert flags[r].tolist() == [0, 7, 0, 0, 0, 0, 0, 0]
    assert flags[1].tolist() == [7, 0, 7, 9, 0, 0, 0, 0]


def test_peer_barrier_gives_up_after_its_limit():
    """A word that nobody writes: the wait ends after a millisecond, the status word says so and the context stays usable."""
    from metalhlo_b200 import cuda

    flags = [torch.zeros(8, dtype=torch.int64, device="cuda") for _ in range(2)]
    ptrs = (C.c_void_p * 2)(*[f.data_ptr() for f in flags])
    torch.cuda.synchronize()
    cuda.check(cuda.lib.mhlo_cuda_peer_barrier(ptrs, 2, 0, 1, 1_000_000, None))
    torch.cuda.synchronize()
    assert cuda.device_error() == 95
    assert cuda.device_error() == 0  # reading clears it
    assert flags[1].tolist()[0] == 1
    x = torch.ones(4, device="cuda")
    assert float((x + x).sum()) == 8.0


def test_peer_barrier_arguments():
    from metalhlo_b200 import cuda

    f = torch.zeros(8, dtype=torch.int64, device="cuda")
    ptrs = (C.c_void_p * 2)(f.data_ptr(), f.data_ptr())
    assert cuda.lib.mhlo_cuda_peer_barrier(ptrs, 9, 0, 1, 1000, None) == 10
    assert cuda.lib.mhlo_cuda_peer_barrier(ptrs, 2, 2, 1, 1000, None) == 10
    assert cuda.lib.mhlo_cuda_peer_barrier(ptrs, 2, 0, 1, 0, None) == 10
    assert cuda.lib.mhlo_cuda_peer_barrier(ptrs, 2, 0, 1, 3_000_000_000, None) == 10
    odd = (C.c_void_p * 2)(f.data_ptr() + 4, f.data_ptr())
    assert cuda.lib.mhlo_cuda_peer_barrier(odd, 2, 0, 1, 1000, None) == 10
    one = (C.c_void_p * 1)(f.data_ptr())
    assert cuda.lib.mhlo_cuda_peer_barrier(one, 1, 0, 1, 1000, None) == 0  # a single rank has nobody to wait for


def _ipc_rank(rank, world, store_path, copy_stores, result_queue):
    """One process per GPU: C and the flag words live in one allocation that the other rank opens through an IPC handle."""
    import os

    import torch.distributed as dist

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", store=dist.FileStore(store_path, world), rank=rank, world_size=world)
    from metalhlo_b200 import cuda, sharding

    m, n, k = 1024, 4096, 512
    n_local = n // world
    g = torch.Generator().manual_seed(5)  # the same operands on every rank
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(torch.bfloat16).cuda()
    b = torch.randn(k, n, generator=g).to(torch.bfloat16).cuda()
    c_bytes = m * n * 2
    own = C.c_void_p()
    cuda.check(cuda.lib.mhlo_cuda_alloc(c_bytes + 256, C.byref(own)))
    cuda.check(cuda.lib.mhlo_cuda_memset(own, 0, c_bytes + 256, None))
    torch.cuda.synchronize()
    handle = C.create_string_buffer(64)
    cuda.check(cuda.lib.mhlo_cuda_ipc_export(own, handle))
    handles = sharding.exchange_handles(handle.raw, dist)
    bases = []
    for r in range(world):
        if r == rank:
            bases.append(own.value)
        else:
            ptr = C.c_void_p()
            cuda.check(cuda.lib.mhlo_cuda_ipc_open(handles[r], C.byref(ptr)))
            bases.append(ptr.value)
    c_ptrs = (C.c_void_p * world)(*bases)
    flag_ptrs = (C.c_void_p * world)(*[p + c_bytes for p in bases])
    dist.barrier()  # every rank has zeroed its allocation and opened the others'
    ok = True
    for epoch in (1, 2, 3):
        b_local = b[:, rank * n_local:(rank + 1) * n_local]
        cuda.check(cuda.lib.mhlo_cuda_gemm_all_gather_tuned(
            cuda.BF16, cuda.BF16, a.data_ptr(), cuda._i64s([k, 1]), b_local.data_ptr(), cuda._i64s([n, 1]), c_ptrs, world, rank, m, n_local, k,
            None, 0, None, copy_stores, None))
        cuda.check(cuda.lib.mhlo_cuda_peer_barrier(flag_ptrs, world, rank, epoch, 1_000_000_000, None))
        mine = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        cuda.check(cuda.lib.mhlo_cuda_copy(mine.data_ptr(), own, c_bytes, None))  # stream-ordered behind the barrier: no host sync between
        torch.cuda.synchronize()
        ok = ok and cuda.device_error() == 0 and torch.equal(mine.view(torch.int16), cuda.gemm(a, b).view(torch.int16))
        a = (a * 0.5).contiguous()  # the next epoch's product differs, so a stale copy would show
        dist.barrier()  # nobody overwrites a copy that a slower rank is still checking
    result_queue.put((rank, ok))
    dist.barrier()
    for r in range(world):
        if r != rank:
            cuda.check(cuda.lib.mhlo_cuda_ipc_close(C.c_void_p(bases[r])))
    dist.barrier()
    cuda.check(cuda.lib.mhlo_cuda_free(own))
    dist.destroy_process_group()


@pytest.mark.parametrize("copy_stores", [1, 2])
def test_two_ranks_exchange_over_ipc_with_the_device_barrier(copy_stores, tmp_path):
    """Two processes, two GPUs: each rank's epilogue stores into both copies of C, the flag words close the exchange."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ipc_rank, args=(r, 2, str(tmp_path / "store"), copy_stores, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()  # exactly the processes this test started
    assert not alive, "a rank did not finish"
    assert all(p.exitcode == 0 for p in procs)
    results = dict(q.get(timeout=5) for _ in range(2))
    assert results == {0: True, 1: True}
