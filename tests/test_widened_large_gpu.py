"""Sort, pooling, convolution and scatter at sizes the numpy oracle cannot finish: checked through size-independent
properties (sortedness, permutation, stability) and against torch's own CUDA operators as an independent implementation.
The modules are the ones `bench.py --profile-kernel` times."""
import numpy as np
import pytest

import bench
from metalhlo_b200 import capi

pytestmark = pytest.mark.gpu

_client = None


def client():
    global _client
    if _client is None:
        _client = capi.Client()
    return _client


def run_on_device(text, inputs, out_specs):
    """inputs: CUDA torch tensors; out_specs: [(shape, torch dtype)]. Returns the output tensors."""
    import torch

    exe = client().compile(text, 3)
    outs = [torch.empty(shape, dtype=dt, device="cuda") for shape, dt in out_specs]
    torch.cuda.synchronize()
    exe.execute_on_device([t.data_ptr() for t in inputs], [o.data_ptr() for o in outs], torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return outs


@pytest.mark.parametrize("rows,n", [(4096, 4096), (4, 1 << 21), (3, 100003)])
def test_sort_is_a_stable_sorted_permutation(rows, n):
    import torch

    g = torch.Generator(device="cuda").manual_seed(rows + n)
    # few distinct values, so that ties are everywhere and stability is visible
    x = torch.randint(-500, 500, (rows, n), device="cuda", generator=g).float() * 0.25
    vals, order = run_on_device(bench._sort_text(rows, n), [x], [((rows, n), torch.float32), ((rows, n), torch.int32)])
    assert bool((vals[:, 1:] >= vals[:, :-1]).all()), "not sorted"
    assert bool((torch.gather(x, 1, order.long()) == vals).all()), "values do not follow the order"
    ties = vals[:, 1:] == vals[:, :-1]
    assert bool((order[:, 1:][ties] > order[:, :-1][ties]).all()), "ties are not in their original order"
    ref_vals, ref_order = torch.sort(x, dim=1, stable=True)
    assert bool((ref_vals == vals).all()) and bool((ref_order.int() == order).all())


def test_max_pooling_equals_torch():
    import torch

    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn(32, 112, 112, 64, device="cuda", generator=g).to(torch.bfloat16)
    (got,) = run_on_device(bench._pool_text(), [x], [((32, 56, 56, 64), torch.bfloat16)])
    padded = torch.nn.functional.pad(x.permute(0, 3, 1, 2).float(), (0, 1, 0, 1), value=float("-inf"))
    want = torch.nn.functional.max_pool2d(padded, 3, 2).permute(0, 2, 3, 1)
    assert bool((got.float() == want).all())  # a maximum of bf16 values is one of them: bit-exact


def test_convolution_matches_torch_in_fp32():
    import torch

    g = torch.Generator(device="cuda").manual_seed(8)
    x = torch.randn(32, 56, 56, 64, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(3, 3, 64, 64, device="cuda", generator=g) / 24).to(torch.bfloat16)
    (got,) = run_on_device(bench._conv_text(), [x, w], [((32, 56, 56, 64), torch.bfloat16)])
    prev = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        want = torch.nn.functional.conv2d(x.permute(0, 3, 1, 2).float(), w.permute(3, 2, 0, 1).float(), padding=1).permute(0, 2, 3, 1)
    finally:
        torch.backends.cudnn.allow_tf32 = prev
    err = (got.float() - want).abs()
    # bf16 result of an fp32 accumulation over 576 terms: within the 16-bit tolerance of the parity tests (rel 2e-2)
    assert float(err.max()) <= 2e-2 * float(want.abs().max())
    assert float(err.mean()) <= 2e-3 * float(want.abs().mean()) + 1e-6


def test_scatter_add_matches_index_add():
    import torch

    g = torch.Generator(device="cuda").manual_seed(9)
    table = torch.randn(50257, 768, device="cuda", generator=g)
    idx = torch.randint(0, 50257, (32768, 1), device="cuda", generator=g, dtype=torch.int32)
    upd = torch.randn(32768, 768, device="cuda", generator=g)
    (got,) = run_on_device(bench._scatter_text(), [table, idx, upd], [((50257, 768), torch.float32)])
    want = table.double().index_add_(0, idx[:, 0].long(), upd.double())
    # colliding rows are added in an unspecified order: fp32 rounding differs by a few ulp of the partial sums
    assert float((got.double() - want).abs().max()) <= 1e-5 * float(want.abs().max())
    untouched = torch.ones(50257, dtype=torch.bool, device="cuda")
    untouched[idx[:, 0].long()] = False
    assert bool((got[untouched] == table[untouched]).all())
