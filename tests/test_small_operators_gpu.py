"""Entry points of the small numeric operators called directly: the random-bit generator's stream and its argument checks,
and the residual form of the product on its two-pass route."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def threefry(key, counters):
    """Threefry-2x32-20 on uint64 counters with a uint64 key (numpy, the published algorithm)."""
    k0, k1 = np.uint32(key & 0xFFFFFFFF), np.uint32(key >> 32)
    ks = [k0, k1, k0 ^ k1 ^ np.uint32(0x1BD11BDA)]
    x0 = (counters & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    x1 = (counters >> np.uint64(32)).astype(np.uint32)
    rot = [13, 15, 26, 6, 17, 29, 16, 24]
    with np.errstate(over="ignore"):
        x0, x1 = x0 + ks[0], x1 + ks[1]
        for g in range(5):
            for r in rot[4 * (g % 2):4 * (g % 2) + 4]:
                x0 = x0 + x1
                x1 = ((x1 << np.uint32(r)) | (x1 >> np.uint32(32 - r))) ^ x0
            x0 = x0 + ks[(g + 1) % 3]
            x1 = x1 + ks[(g + 2) % 3] + np.uint32(g + 1)
    return x0, x1


def draw(cuda, state, count, elem_bytes):
    st = torch.from_numpy(state.view(np.int64)).cuda()
    new = torch.zeros(2, dtype=torch.int64, device="cuda")
    out = torch.zeros(max(count * elem_bytes, 1), dtype=torch.uint8, device="cuda")
    cuda.check(cuda.lib.mhlo_cuda_rng_bit_generator(st.data_ptr(), new.data_ptr(), out.data_ptr(), count, elem_bytes, None))
    torch.cuda.synchronize()
    return new.cpu().numpy().view(np.uint64), out.cpu().numpy()[:count * elem_bytes]


def test_known_answer_and_word_order():
    from metalhlo_b200 import cuda

    new, raw = draw(cuda, np.zeros(2, np.uint64), 2, 4)
    assert raw.view(np.uint32).tolist() == [0x6B200159, 0x99BA4EFE]  # Random123 kat_vectors, zero key and counter
    assert new.tolist() == [0, 1]
    _, raw64 = draw(cuda, np.zeros(2, np.uint64), 1, 8)
    assert int(raw64.view(np.uint64)[0]) == 0x6B200159 | (0x99BA4EFE << 32)


@pytest.mark.parametrize("elem_bytes", [1, 2, 4, 8])
def test_a_million_elements_follow_the_counter_across_its_wrap(elem_bytes):
    from metalhlo_b200 import cuda

    count = 1_000_003
    state = np.array([0xDEADBEEFCAFEF00D, 0xFFFFFFFFFFFFFF00], dtype=np.uint64)  # the counter wraps inside the draw
    new, raw = draw(cuda, state, count, elem_bytes)
    blocks = count if elem_bytes == 8 else (count + 1) // 2
    with np.errstate(over="ignore"):
        counters = np.arange(blocks, dtype=np.uint64) + state[1]
    x0, x1 = threefry(int(state[0]), counters)
    if elem_bytes == 8:
        want = x0.astype(np.uint64) | (x1.astype(np.uint64) << np.uint64(32))
        got = raw.view(np.uint64)
    else:
        words = np.stack([x0, x1], 1).reshape(-1)[:count]
        dt = {1: np.uint8, 2: np.uint16, 4: np.uint32}[elem_bytes]
        want, got = words.astype(dt), raw.view(dt)
    np.testing.assert_array_equal(got, want)
    assert int(new[0]) == int(state[0]) and int(new[1]) == (int(state[1]) + blocks) % 2 ** 64
    bits = np.unpackbits(raw[:400_000])
    assert abs(bits.mean() - 0.5) < 2e-3


def test_random_bit_arguments():
    from metalhlo_b200 import cuda

    a = torch.zeros(2, dtype=torch.int64, device="cuda")
    b = torch.zeros(2, dtype=torch.int64, device="cuda")
    o = torch.zeros(64, dtype=torch.uint8, device="cuda")
    f = cuda.lib.mhlo_cuda_rng_bit_generator
    assert f(a.data_ptr(), b.data_ptr(), o.data_ptr(), 4, 3, None) == 10     # element width
    assert f(a.data_ptr(), b.data_ptr(), o.data_ptr(), -1, 4, None) == 10
    assert f(a.data_ptr(), a.data_ptr(), o.data_ptr(), 4, 4, None) == 10     # the new state may not alias the state
    assert f(None, b.data_ptr(), o.data_ptr(), 4, 4, None) == 10
    assert f(a.data_ptr(), b.data_ptr(), None, 0, 4, None) == 0              # an empty draw still copies the state forward
    torch.cuda.synchronize()
    assert b.tolist() == [0, 0]


def test_residual_product_outside_the_tensor_core_path():
    """fp32 operands (general-layout product) and a result pitch off the 16-byte grid take the two-pass route: product, then sum."""
    from metalhlo_b200 import cuda

    g = torch.Generator().manual_seed(9)
    for dtype, m, n, k in ((torch.float32, 70, 50, 33), (torch.float16, 130, 250, 64)):
        a = (torch.randn(m, k, generator=g) / k ** 0.5).to(dtype).cuda()
        b = torch.randn(k, n, generator=g).to(dtype).cuda()
        bias = torch.randn(n, generator=g).to(dtype).cuda()
        res = torch.randn(m, n, generator=g).to(dtype).cuda()
        got = cuda.gemm(a, b, bias=bias, residual=res)
        want = a.double() @ b.double() + bias.double() + res.double()
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert (got.double() - want).abs().max() <= tol * want.abs().max()
    assert cuda.device_error() == 0


RNG_TEXT = """func.func @main(%a: tensor<{dt}>, %b: tensor<{dt}>) -> tensor<{n}x{dt}> {{
  %s = stablehlo.constant dense<[{n}]> : tensor<1xi64>
  %0 = stablehlo.rng %a, %b, %s, distribution = {dist} : (tensor<{dt}>, tensor<{dt}>, tensor<1xi64>) -> tensor<{n}x{dt}>
  return %0 : tensor<{n}x{dt}>
}}"""


def run_rng(dt, np_dt, dist, a, b, n=200_000, level=2):
    from metalhlo_b200 import capi

    c = capi.Client()
    exe = c.compile(RNG_TEXT.format(dt=dt, n=n, dist=dist), level)
    ins = [c.buffer(np.asarray(a, dtype=np_dt)), c.buffer(np.asarray(b, dtype=np_dt))]
    return [exe.execute(ins)[0].to_numpy() for _ in range(3)]


def test_uniform_floats_fill_the_interval_and_every_execution_continues_the_stream():
    draws = run_rng("f32", np.float32, "UNIFORM", -2.0, 6.0)
    for d in draws:
        assert d.min() >= -2.0 and d.max() < 6.0
        assert abs(d.mean() - 2.0) < 0.05 and abs(d.std() - 8 / 12 ** 0.5) < 0.05
        hist = np.histogram(d, bins=16, range=(-2, 6))[0]
        assert hist.min() > 0.9 * d.size / 16 and hist.max() < 1.1 * d.size / 16
    assert not np.array_equal(draws[0], draws[1]) and not np.array_equal(draws[1], draws[2])
    assert len(np.intersect1d(draws[0][:1000], draws[1][:1000])) < 5  # not the same numbers shifted or repeated


def test_normal_floats_have_the_asked_moments():
    for dt, np_dt in (("f32", np.float32), ("f64", np.float64)):
        d = run_rng(dt, np_dt, "NORMAL", 1.5, 0.5)[0].astype(np.float64)
        assert abs(d.mean() - 1.5) < 0.01 and abs(d.std() - 0.5) < 0.01
        z = (d - 1.5) / 0.5
        assert abs((z ** 3).mean()) < 0.05 and abs((z ** 4).mean() - 3.0) < 0.1
        assert 0.66 < (np.abs(z) < 1).mean() < 0.70


def test_uniform_integers_cover_their_range():
    for dt, np_dt in (("i32", np.int32), ("ui8", np.uint8), ("i64", np.int64)):
        d = run_rng(dt, np_dt, "UNIFORM", 3, 13, n=100_000)[0]
        assert d.min() == 3 and d.max() == 12
        counts = np.bincount(d.astype(np.int64) - 3, minlength=10)
        assert counts.min() > 0.9 * d.size / 10 and counts.max() < 1.1 * d.size / 10


def test_sixteen_bit_draws_and_two_operators_in_one_program():
    """Two rng operators of one program draw from different keys; f16 results stay inside the half-open interval."""
    from metalhlo_b200 import capi

    text = """func.func @main(%a: tensor<f16>, %b: tensor<f16>) -> (tensor<4096xf16>, tensor<4096xf16>) {
  %s = stablehlo.constant dense<[4096]> : tensor<1xi64>
  %0 = stablehlo.rng %a, %b, %s, distribution = UNIFORM : (tensor<f16>, tensor<f16>, tensor<1xi64>) -> tensor<4096xf16>
  %1 = stablehlo.rng %a, %b, %s, distribution = UNIFORM : (tensor<f16>, tensor<f16>, tensor<1xi64>) -> tensor<4096xf16>
  return %0, %1 : tensor<4096xf16>, tensor<4096xf16>
}"""
    c = capi.Client()
    exe = c.compile(text, 3)
    x, y = [o.to_numpy() for o in exe.execute([c.buffer(np.float16(0)), c.buffer(np.float16(1))])]
    assert x.min() >= 0 and x.max() < 1 and y.min() >= 0 and y.max() < 1
    assert not np.array_equal(x, y)
    assert abs(float(x.astype(np.float32).mean()) - 0.5) < 0.03
