"""Parity of mhlo_cuda_attention (tcgen05 flash kernel and the general-layout kernel) against the fp64 oracle."""
import math

import numpy as np
import pytest
import torch

import oracle
from parity import assert_close, to_np

pytestmark = pytest.mark.gpu


def cuda_mod():
    from metalhlo_b200 import cuda

    return cuda


def qkv(b, h, sq, sk, d, dtype, layout, seed):
    g = torch.Generator().manual_seed(seed)
    shape = (lambda s: (b, h, s, d)) if layout == "BHSD" else (lambda s: (b, s, h, d))
    return (torch.randn(shape(sq), generator=g).to(dtype), torch.randn(shape(sk), generator=g).to(dtype),
            torch.randn(shape(sk), generator=g).to(dtype))


def reference(q, k, v, scale, causal, layout):
    if layout == "BSHD":
        q, k, v = (t.permute(0, 2, 1, 3).contiguous() for t in (q, k, v))
    o = oracle.attention(q, k, v, scale, causal=causal)
    return o if layout == "BHSD" else np.ascontiguousarray(o.transpose(0, 2, 1, 3))


def magnitude(q, k, v, scale, causal, layout):
    """sum_j p_ij |v_jd|: the scale of the terms the output element contracts (see tests/parity.py)."""
    return reference(q, k, v.abs(), scale, causal, layout)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=str)
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("sq,sk", [(256, 256), (512, 512), (200, 333), (64, 64), (1, 300), (300, 300), (128, 1024), (700, 640)])
def test_tensor_core_attention(dtype, causal, d, sq, sk):
    cuda = cuda_mod()
    q, k, v = qkv(2, 3, sq, sk, d, dtype, "BHSD", seed=sq + sk + d)
    scale = 1 / math.sqrt(d)
    got = cuda.attention(q.cuda(), k.cuda(), v.cuda(), scale, causal=causal)
    assert cuda.device_error() == 0
    assert_close(to_np(got), reference(q, k, v, scale, causal, "BHSD"), 2e-2, f"attention {sq}x{sk} d{d} causal={causal}",
                 magnitude=magnitude(q, k, v, scale, causal, "BHSD"))


@pytest.mark.parametrize("causal", [False, True])
def test_bshd_layout_is_read_and_written_in_place(causal):
    cuda = cuda_mod()
    q, k, v = qkv(2, 4, 384, 384, 64, torch.float16, "BSHD", seed=11)
    got = cuda.attention(q.cuda(), k.cuda(), v.cuda(), 0.125, causal=causal, layout="BSHD")
    assert cuda.device_error() == 0
    assert_close(to_np(got), reference(q, k, v, 0.125, causal, "BSHD"), 2e-2, "BSHD")


@pytest.mark.parametrize("d", [64, 128])
def test_large_scores_trigger_rescaling(d):
    """Growing maxima along the key axis force the lazy rescale of the TMEM accumulator many times."""
    cuda = cuda_mod()
    b, h, s = 1, 2, 512
    g = torch.Generator().manual_seed(3)
    q = torch.randn(b, h, s, d, generator=g)
    k = torch.randn(b, h, s, d, generator=g) * torch.linspace(0.2, 3.0, s).view(1, 1, s, 1)
    v = torch.randn(b, h, s, d, generator=g)
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    got = cuda.attention(q.cuda(), k.cuda(), v.cuda(), 0.5)
    assert cuda.device_error() == 0
    assert_close(to_np(got), reference(q, k, v, 0.5, False, "BHSD"), 2e-2, "rescale")


@pytest.mark.parametrize("jump", [640, 704, 736])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=str)
def test_scores_growing_past_the_carried_reference(dtype, d, jump):
    """After a tile's first key block the kernel works against the maximum carried over from earlier blocks and moves it
    when a block (head dim 128: by its row sums; head dim 64: a 64-key chunk by its own maximum) would leave the range of
    the 16-bit probabilities. Keys whose norm jumps by 40x force that: at a block boundary (640), in the middle of a block
    (704: the block's first chunk of probabilities, already written, has to be scaled down too) and inside a chunk (736)."""
    cuda = cuda_mod()
    b, h, s = 1, 2, 1024
    g = torch.Generator().manual_seed(5)
    q = torch.randn(b, h, s, d, generator=g)
    gain = torch.where(torch.arange(s) < jump, 0.05, 2.0).view(1, 1, s, 1)
    k = torch.randn(b, h, s, d, generator=g) * gain
    v = torch.randn(b, h, s, d, generator=g)
    q, k, v = (t.to(dtype) for t in (q, k, v))
    for causal in (False, True):
        got = cuda.attention(q.cuda(), k.cuda(), v.cuda(), 0.5, causal=causal)
        assert cuda.device_error() == 0
        assert np.isfinite(to_np(got)).all()
        assert_close(to_np(got), reference(q, k, v, 0.5, causal, "BHSD"), 2e-2, f"carried reference causal={causal}")


@pytest.mark.parametrize("causal", [False, True])
def test_more_tiles_than_resident_ctas(causal):
    """320 tiles on at most 148 persistent CTAs: every CTA walks several tiles, so barrier phases, the Q buffers and the
    TMEM accumulators are handed from one tile to the next."""
    cuda = cuda_mod()
    q, k, v = qkv(4, 20, 1024, 1024, 64, torch.bfloat16, "BHSD", seed=21)
    got = cuda.attention(q.cuda(), k.cuda(), v.cuda(), 0.125, causal=causal)
    assert cuda.device_error() == 0
    assert_close(to_np(got), reference(q, k, v, 0.125, causal, "BHSD"), 2e-2, f"many tiles causal={causal}", row_scale=True)


@pytest.mark.parametrize("sq,sk", [(768, 256), (256, 768), (300, 170)])
def test_causal_cut_when_query_and_key_lengths_differ(sq, sk):
    """Under the causal flag key j is visible to query i iff j <= i whatever the two lengths are: the reference kernel
    cuts at `kv_pos > q_pos` (Sources/MetalHLOCore/Metal/Kernels/FlashAttentionKernel.swift:545,578). With more queries
    than keys the late rows see every key; with more keys than queries the keys past the last query are never read.
    Checked against the oracle and against a numpy statement of the rule written out here."""
    cuda = cuda_mod()
    q, k, v = qkv(2, 5, sq, sk, 128, torch.bfloat16, "BHSD", seed=23)
    got = to_np(cuda.attention(q.cuda(), k.cuda(), v.cuda(), 0.1, causal=True))
    assert cuda.device_error() == 0
    assert_close(got, reference(q, k, v, 0.1, True, "BHSD"), 2e-2, "oracle", row_scale=True)
    s = np.einsum("bhqd,bhkd->bhqk", to_np(q), to_np(k)) * 0.1
    s = np.where(np.arange(sk)[None, :] > np.arange(sq)[:, None], -np.inf, s)
    p = np.exp(s - s.max(-1, keepdims=True))
    want = np.einsum("bhqk,bhkd->bhqd", p / p.sum(-1, keepdims=True), to_np(v))
    assert_close(got, want, 2e-2, "kv_pos > q_pos rule", row_scale=True)
    # query 0 sees key 0 only: its output row is V[0] exactly
    np.testing.assert_array_equal(got[:, :, 0, :], to_np(v)[:, :, 0, :])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=str)
def test_general_layout_kernel(dtype):
    cuda = cuda_mod()
    q, k, v = qkv(2, 2, 37, 53, 40, dtype, "BHSD", seed=5)
    for causal in (False, True):
        got = cuda.attention(q.cuda(), k.cuda(), v.cuda(), 0.2, causal=causal)
        assert_close(to_np(got), reference(q, k, v, 0.2, causal, "BHSD"), 1e-5 if dtype == torch.float32 else 2e-2, "general")
    mask = torch.randn(37, 53, generator=torch.Generator().manual_seed(1)).to(dtype)
    got = cuda.attention(q.cuda(), k.cuda(), v.cuda(), 0.2, mask=mask.cuda())
    assert_close(to_np(got), oracle.attention(q, k, v, 0.2, mask=mask), 1e-5 if dtype == torch.float32 else 2e-2, "mask")


@pytest.mark.parametrize("causal", [False, True])
def test_benchmark_shape_sampled_heads_and_properties(causal):
    """B8 H32 S4096 D128 bf16. Oracle on two (batch, head) slices; every row of P sums to one, so with V = 1 the
    output must be one everywhere (a size-independent property over the full tensor)."""
    cuda = cuda_mod()
    b, h, s, d = 8, 32, 4096, 128
    g = torch.Generator(device="cuda").manual_seed(42)
    q = torch.randn(b, h, s, d, generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn(b, h, s, d, generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn(b, h, s, d, generator=g, device="cuda").to(torch.bfloat16)
    scale = 1 / math.sqrt(d)
    got = cuda.attention(q, k, v, scale, causal=causal)
    assert cuda.device_error() == 0
    for bi, hi in [(0, 0), (7, 31)]:
        want = oracle.attention(q[bi, hi].cpu(), k[bi, hi].cpu(), v[bi, hi].cpu(), scale, causal=causal)
        assert_close(to_np(got[bi, hi]), want, 2e-2, f"slice {bi},{hi}", row_scale=True)
    ones = cuda.attention(q, k, torch.ones_like(v), scale, causal=causal)
    assert float((ones.float() - 1).abs().max()) < 2e-2
