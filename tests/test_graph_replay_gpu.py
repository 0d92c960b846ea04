"""CUDA-graph replay of a compiled program: the second execution on the same stream and buffers records the launch
list, later ones replay it; results follow the buffers' current contents, and other buffers fall back to plain launches."""
import numpy as np
import pytest
import torch

from metalhlo_b200 import capi, cuda, modules
from oracle import interp

pytestmark = pytest.mark.gpu


def reduced_gpt2():
    text, params = modules.gpt2_module(batch=2, seq=128, layers=2, d_model=256, heads=4, vocab=1031, dt="f16")
    rng = np.random.default_rng(4)
    ins = []
    for name, shape, dt in params:
        if dt == "i32":
            ins.append(rng.integers(0, 1031, size=shape).astype(np.int32))
        elif name.endswith("_g"):
            ins.append(np.ones(shape, np.float32))
        else:
            ins.append((0.05 * rng.standard_normal(shape)).astype(np.float32))
    return text, ins


def test_replay_matches_plain_launches_and_follows_new_contents():
    text, ins = reduced_gpt2()
    client = capi.Client()
    exe = client.compile(text, opt_level=3)
    assert len(exe.steps) >= 8
    bufs = [client.buffer(a) for a in ins]
    ptrs = [b.device_pointer for b in bufs]
    out = torch.empty(2, 128, 1031, device="cuda", dtype=torch.float16)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        exe.execute_on_device(ptrs, [out.data_ptr()], stream.cuda_stream)   # plain launches; the combination is remembered
        stream.synchronize()
        first = out.clone()
        assert exe.graph_replays == 0
        out.zero_()
        exe.execute_on_device(ptrs, [out.data_ptr()], stream.cuda_stream)   # recorded, then replayed
        stream.synchronize()
        assert exe.graph_replays == 1
        assert torch.equal(out, first)
        # new token ids in the same buffer: the replay reads the buffer, not a snapshot
        ids = torch.randint(0, 1031, (2, 128), dtype=torch.int32, device="cuda")
        id_index = [i for i, a in enumerate(ins) if a.dtype == np.int32][0]
        cuda.check(cuda.lib.mhlo_cuda_copy(ptrs[id_index], ids.data_ptr(), ids.numel() * 4, stream.cuda_stream))
        exe.execute_on_device(ptrs, [out.data_ptr()], stream.cuda_stream)
        stream.synchronize()
        assert exe.graph_replays == 2
    new_ins = list(ins)
    new_ins[id_index] = ids.cpu().numpy()
    want = interp.evaluate(text, new_ins)[0]
    got = out.double().cpu().numpy()
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 2e-2
    assert not torch.equal(out, first)


def test_default_stream_and_changing_buffers_use_plain_launches():
    text, ins = reduced_gpt2()
    client = capi.Client()
    exe = client.compile(text, opt_level=3)
    bufs = [client.buffer(a) for a in ins]
    ptrs = [b.device_pointer for b in bufs]
    outs = [torch.empty(2, 128, 1031, device="cuda", dtype=torch.float16) for _ in range(6)]
    for o in outs[:2]:
        exe.execute_on_device(ptrs, [o.data_ptr()], None)                   # default stream: never recorded
        exe.execute_on_device(ptrs, [o.data_ptr()], None)
    torch.cuda.synchronize()
    assert exe.graph_replays == 0
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for o in outs:                                                       # six different outputs, each seen once
            exe.execute_on_device(ptrs, [o.data_ptr()], stream.cuda_stream)
        stream.synchronize()
    assert exe.graph_replays == 0
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
