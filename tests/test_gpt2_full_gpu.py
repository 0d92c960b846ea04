"""The GPT-2-small forward pass at its real extents — 12 pre-LN layers, d_model 768, 12 heads, MLP 3072 with tanh GELU,
vocabulary 50257, 1024 tokens per sequence, fp32 parameters ~ N(0, 0.02), fp16 compute — through the C API and through
the PJRT plugin, against the numpy oracle (one sequence; the oracle needs about a minute for it) and, at the benchmark's
batch of 32, the fused O3 program against the unfused O0 program on the GPU.

The per-element rule of tests/parity.py is applied to sampled rows of the logits; the whole tensor is held normwise.
"""
import numpy as np
import pytest

from metalhlo_b200 import modules
from oracle import interp
from parity import assert_close, error_report

pytestmark = pytest.mark.gpu

VOCAB, SEQ = 50257, 1024


def gpt2_inputs(params, seed=7):
    rng = np.random.default_rng(seed)
    out = []
    for name, shape, dt in params:
        if dt == "i32":
            out.append(rng.integers(0, VOCAB, size=shape).astype(np.int32))
        elif name.endswith("_g"):
            out.append(np.ones(shape, np.float32))
        elif name.endswith(("ln1_b", "ln2_b", "lnf_b")):
            out.append(np.zeros(shape, np.float32))
        else:
            out.append((0.02 * rng.standard_normal(shape)).astype(np.float32))
    return out


@pytest.fixture(scope="module")
def one_sequence():
    """Module text, inputs and the oracle's fp64 logits for one sequence of 1024 tokens at the full model extents."""
    text, params = modules.gpt2_module(batch=1, seq=SEQ)
    ins = gpt2_inputs(params)
    want = interp.evaluate(text, ins)[0]
    assert want.shape == (1, SEQ, VOCAB)
    return text, params, ins, want


def check_logits(got, want, what):
    got = got.astype(np.float64)
    assert got.shape == want.shape
    assert np.isfinite(got).all(), what
    rel_l2 = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel_l2 < 2e-2, f"{what}: relative L2 error {rel_l2:.3e}"
    # per element on sampled token rows (the whole tensor is 51 M elements): plain |got - want| <= 2e-2 |want| on the
    # elements at or above the mean magnitude, 2e-2 * mean below it
    rows = np.arange(0, SEQ, 37)
    assert_close(got[0, rows], want[0, rows], 2e-2, f"{what}: sampled rows")
    r = error_report(got[0, rows], want[0, rows], 2e-2)
    print(f"{what}: rel L2 {rel_l2:.3e}, worst plain relative error on {r['large']} large sampled elements {r['worst_plain_rel']:.3e}")
    # greedy next-token ids agree wherever the oracle's top-2 margin exceeds the 16-bit resolution
    top2 = np.partition(want[0], -2, axis=-1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 0.05 * np.abs(top2[:, 1]) + 1e-3
    assert clear.sum() > 0
    assert np.array_equal(got[0].argmax(-1)[clear], want[0].argmax(-1)[clear]), what


@pytest.mark.parametrize("level", [3, 0])
def test_one_sequence_through_the_c_api_matches_the_oracle(one_sequence, level):
    from metalhlo_b200 import capi

    text, params, ins, want = one_sequence
    client = capi.Client()
    exe = client.compile(text, level)
    got = exe.execute([client.buffer(a) for a in ins])[0].to_numpy()
    if level == 3:
        fused = [s for s in exe.steps if s.startswith("fused")]
        assert fused.count("fused_scaled_dot_product_attention") == 12
        assert fused.count("fused_matmul_bias_activation") == 48
    check_logits(got, want, f"C API O{level}")


def test_one_sequence_through_the_pjrt_plugin_matches_the_oracle(one_sequence):
    """BufferFromHostBuffer -> Compile -> Execute -> ToHostBuffer through GetPjrtApi, the calls a PJRT host makes
    (Tests/PJRTMetalHLOTests/PJRTPluginTests.swift:160-467 drives the reference's plugin the same way)."""
    from metalhlo_b200 import capi, pjrt

    text, params, ins, want = one_sequence
    host = pjrt.Host()
    assert host.platform_name == "metalhlo"
    exe = host.compile(text)
    outs = exe.execute([host.buffer(a) for a in ins])
    assert len(outs) == 1
    got = outs[0].to_numpy()
    assert got.dtype == np.float16 and got.shape == (1, SEQ, VOCAB)
    check_logits(got, want, "PJRT")
    # the plugin is layered on the C API: same program, same kernels, same bits
    client = capi.Client()
    direct = client.compile(text).execute([client.buffer(a) for a in ins])[0].to_numpy()
    assert np.array_equal(got.view(np.uint16), direct.view(np.uint16))


def test_benchmark_batch_fused_program_against_the_unfused_program():
    """Batch 32 x 1024 tokens: the O3 program (fused attention, norms, GEMM epilogues) against the O0 program (one
    kernel per StableHLO op) on the same device inputs, compared on the device because each result is 3.3 GB."""
    import torch

    from metalhlo_b200 import capi

    text, params = modules.gpt2_module(batch=32, seq=SEQ)
    ins = gpt2_inputs(params)
    client = capi.Client()
    bufs = [client.buffer(a) for a in ins]
    ptrs = [b.device_pointer for b in bufs]
    results = {}
    for level in (3, 0):
        exe = client.compile(text, level)
        out = torch.empty(32, SEQ, VOCAB, dtype=torch.float16, device="cuda")
        exe.execute_on_device(ptrs, [out.data_ptr()], torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        results[level] = out
        del exe
    from metalhlo_b200 import cuda

    assert cuda.device_error() == 0
    fused, plain = results[3], results[0]
    assert bool(torch.isfinite(fused).all()) and bool(torch.isfinite(plain).all())
    num = den = 0.0
    worst = 0.0
    agree = total = 0
    for b in range(32):
        f, p = fused[b].float(), plain[b].float()
        num += float(((f - p) ** 2).sum())
        den += float((p ** 2).sum())
        scale = float(p.abs().mean())
        bound = 2e-2 * torch.clamp(p.abs(), min=scale)
        # both sides are fp16 evaluations of the same graph: each may be off by the 16-bit tolerance, so the difference of
        # the two is held to twice the single-sided bound
        worst = max(worst, float(((f - p).abs() / bound).max()))
        agree += int((f.argmax(-1) == p.argmax(-1)).sum())
        total += SEQ
    rel_l2 = (num / den) ** 0.5
    print(f"O3 vs O0 at batch 32: rel L2 {rel_l2:.3e}, worst error / bound {worst:.3f}, greedy agreement {agree}/{total}")
    assert rel_l2 < 2e-2
    assert worst <= 2.0
    assert agree >= 0.98 * total
