"""Dispatch plans and the communicator of the device runtime (mhlo_cuda_kernel_lookup / plan_create / plan_execute /
tuner_measure / comm_init / all_gather): the surface a host executor binds in place of the reference's pipeline states,
buffer bindings and dispatch configurations (Sources/MetalHLOCore/Compiler/KernelTypes.swift:12-143,
Runtime/IntegratedExecutor.swift:150-270). A plan must give exactly what the same kernels give when called one by one."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import oracle
from parity import assert_close, to_np


def cuda_mod():
    from metalhlo_b200 import cuda

    return cuda


def test_kernel_lookup_names_the_fused_ops_of_the_pass_pipeline():
    cuda = cuda_mod()
    ids = {}
    for name in ("fused_layer_norm", "fused_rms_norm", "fused_softmax", "dot_general", "fused_matmul_bias_activation",
                 "fused_scaled_dot_product_attention", "fused_gelu", "fused_silu"):
        k = C.c_int32()
        assert cuda.lib.mhlo_cuda_kernel_lookup(name.encode(), cuda.BF16, C.byref(k)) == 0, name
        ids[name] = k.value
    assert ids["dot_general"] == ids["fused_matmul_bias_activation"] and len(set(ids.values())) == 7
    k = C.c_int32()
    assert cuda.lib.mhlo_cuda_kernel_lookup(b"fused_ffn", cuda.BF16, C.byref(k)) == 4 and "fused_ffn" in cuda.last_error()
    assert cuda.lib.mhlo_cuda_kernel_lookup(b"fused_softmax", cuda.I32, C.byref(k)) == 4
    assert cuda.lib.mhlo_cuda_kernel_lookup(b"fused_softmax", 99, C.byref(k)) == 10


def test_plans_with_bindings_out_of_range_are_refused_before_anything_is_allocated():
    cuda = cuda_mod()
    good = cuda.plan_op("fused_softmax", cuda.F32, [(cuda.SRC_INPUT, 0, 0), (cuda.SRC_OUTPUT, 0, 0)], [4, 8, 1])
    for bad_args in ([(cuda.SRC_INPUT, 1, 0), (cuda.SRC_OUTPUT, 0, 0)], [(cuda.SRC_INPUT, 0, 0), (cuda.SRC_OUTPUT, 2, 0)],
                     [(cuda.SRC_UNIFIED, 0, 4096), (cuda.SRC_OUTPUT, 0, 0)], [(cuda.SRC_CONSTANT, 0, 0), (cuda.SRC_OUTPUT, 0, 0)],
                     [(7, 0, 0), (cuda.SRC_OUTPUT, 0, 0)], [(cuda.SRC_INPUT, 0, -16), (cuda.SRC_OUTPUT, 0, 0)]):
        op = cuda.plan_op("fused_softmax", cuda.F32, bad_args, [4, 8, 1])
        with pytest.raises(RuntimeError, match="out of range"):
            cuda.Plan([good, op], 1, 1, arena_bytes=4096)
    bad_kernel = cuda.PlanOp()
    bad_kernel.kernel = 42
    with pytest.raises(RuntimeError, match="unknown kernel"):
        cuda.Plan([bad_kernel], 1, 1)


@pytest.mark.gpu
def test_mlp_block_as_a_plan_equals_the_kernels_called_one_by_one():
    """LayerNorm -> x.W1 + b1 with tanh GELU -> .W2 + b2: parameters in the constant pool, intermediates in the arena."""
    cuda = cuda_mod()
    rows, d, hdim = 512, 256, 1024
    g = torch.Generator().manual_seed(0)
    x = torch.randn(rows, d, generator=g).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16)
    beta = (0.1 * torch.randn(d, generator=g)).to(torch.bfloat16)
    w1 = (torch.randn(d, hdim, generator=g) / math.sqrt(d)).to(torch.bfloat16)
    b1 = (0.1 * torch.randn(hdim, generator=g)).to(torch.bfloat16)
    w2 = (torch.randn(hdim, d, generator=g) / math.sqrt(hdim)).to(torch.bfloat16)
    b2 = (0.1 * torch.randn(d, generator=g)).to(torch.bfloat16)
    # constant pool: every parameter at a 256-byte aligned offset
    pool, offsets = bytearray(), {}
    for name, t in (("gamma", gamma), ("beta", beta), ("w1", w1), ("b1", b1), ("w2", w2), ("b2", b2)):
        while len(pool) % 256:
            pool.append(0)
        offsets[name] = len(pool)
        pool += t.view(torch.int16).numpy().tobytes()
    ln_off, h_off = 0, rows * d * 2                     # arena: normalised rows, then the hidden activations
    arena = h_off + rows * hdim * 2
    BF = cuda.BF16
    ops = [
        cuda.plan_op("fused_layer_norm", BF, [(cuda.SRC_INPUT, 0, 0), (cuda.SRC_CONSTANT, 0, offsets["gamma"]), (cuda.SRC_CONSTANT, 0, offsets["beta"]),
                                              (cuda.SRC_UNIFIED, 0, ln_off)], [rows, d], scalars=[1e-5]),
        cuda.plan_op("fused_matmul_bias_activation", BF, [(cuda.SRC_UNIFIED, 0, ln_off), (cuda.SRC_CONSTANT, 0, offsets["w1"]),
                                                          (cuda.SRC_CONSTANT, 0, offsets["b1"]), (cuda.SRC_UNIFIED, 0, h_off)],
                     [1, 1, rows, hdim, d], strides=[0, 0, d, 1, 0, 0, hdim, 1], flags=[cuda.EPILOGUES["gelu_tanh"]]),
        cuda.plan_op("dot_general", BF, [(cuda.SRC_UNIFIED, 0, h_off), (cuda.SRC_CONSTANT, 0, offsets["w2"]), (cuda.SRC_CONSTANT, 0, offsets["b2"]),
                                         (cuda.SRC_OUTPUT, 0, 0)], [1, 1, rows, d, hdim], strides=[0, 0, hdim, 1, 0, 0, d, 1], tuning=[128, 3, 1]),
    ]
    plan = cuda.Plan(ops, 1, 1, arena_bytes=arena, constants=bytes(pool))
    xd = x.cuda()
    y = torch.empty(rows, d, dtype=torch.bfloat16, device="cuda")
    plan.execute([xd], [y])
    torch.cuda.synchronize()
    assert cuda.device_error() == 0
    # the same three kernels, one call each
    n = cuda.layer_norm(xd, gamma.cuda(), beta.cuda(), 1e-5)
    h = cuda.gemm(n, w1.cuda(), bias=b1.cuda(), epilogue="gelu_tanh")
    want_dev = cuda.gemm(h, w2.cuda(), bias=b2.cuda())
    assert torch.equal(y.view(torch.int16), want_dev.view(torch.int16))
    # and against the fp64 oracle on the rounded intermediates
    hn = oracle.layer_norm(x, gamma, beta)
    assert_close(to_np(n), hn, 2e-2, "plan layer_norm")
    hh = oracle.gemm(n.cpu(), w1) + b1.double().numpy()
    hh = 0.5 * hh * (1 + np.tanh(0.7978845608028654 * (hh + 0.044715 * hh ** 3)))
    assert_close(to_np(h), hh, 2e-2, "plan hidden")
    assert_close(to_np(y), oracle.gemm(h.cpu(), w2) + b2.double().numpy(), 2e-2, "plan output")
    # a second execution on the same plan gives the same bits; the measurement step reports a positive median
    y2 = torch.empty_like(y)
    plan.execute([xd], [y2])
    torch.cuda.synchronize()
    assert torch.equal(y2.view(torch.int16), y.view(torch.int16))
    assert 0 < plan.measure([xd], [y2], warmup=2, iterations=5) < 50
    with pytest.raises(RuntimeError, match="takes 1 inputs and 1 outputs"):
        plan.execute([xd, xd], [y])


@pytest.mark.gpu
def test_attention_softmax_and_activation_ops_in_a_plan():
    cuda = cuda_mod()
    b, h, s, d = 2, 3, 256, 64
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(b, h, s, d, generator=g).to(torch.float16) for _ in range(3))
    st = [h * s * d, s * d, d]
    ops = [
        cuda.plan_op("fused_scaled_dot_product_attention", cuda.F16,
                     [(cuda.SRC_INPUT, 0, 0), (cuda.SRC_INPUT, 1, 0), (cuda.SRC_INPUT, 2, 0), (cuda.SRC_NONE, 0, 0), (cuda.SRC_UNIFIED, 0, 0)],
                     [b, h, s, s, d], strides=st * 4, scalars=[0.125], flags=[1], tuning=[2]),
        cuda.plan_op("fused_silu", cuda.F16, [(cuda.SRC_UNIFIED, 0, 0), (cuda.SRC_UNIFIED, 0, q.numel() * 2)], [q.numel()]),
        cuda.plan_op("fused_softmax", cuda.F16, [(cuda.SRC_UNIFIED, 0, q.numel() * 2), (cuda.SRC_OUTPUT, 0, 0)], [b * h * s, d, 1]),
    ]
    plan = cuda.Plan(ops, 3, 1, arena_bytes=2 * q.numel() * 2)
    out = torch.empty_like(q, device="cuda")
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    plan.execute([qd, kd, vd], [out])
    torch.cuda.synchronize()
    assert cuda.device_error() == 0
    a = cuda.attention(qd, kd, vd, 0.125, causal=True)
    assert_close(to_np(a), oracle.attention(q, k, v, 0.125, causal=True), 2e-2, "plan attention", magnitude=oracle.attention(q, k, v.abs(), 0.125, causal=True))
    act = to_np(a)
    act = act / (1 + np.exp(-act))
    act16 = torch.from_numpy(act).to(torch.float16)
    assert_close(to_np(out), oracle.softmax(act16), 2e-2, "plan silu + softmax")


@pytest.mark.gpu
def test_communicator_on_the_visible_devices():
    cuda = cuda_mod()
    n = torch.cuda.device_count()
    comm = C.c_void_p()
    assert cuda.lib.mhlo_cuda_comm_init(n + 1, C.byref(comm)) == 10 and not comm.value
    assert cuda.lib.mhlo_cuda_comm_init(n, C.byref(comm)) == 0
    assert cuda.lib.mhlo_cuda_comm_size(comm) == n
    shard = 1 << 20  # bytes per device
    bufs = []
    for d in range(n):
        t = torch.zeros(n * shard, dtype=torch.uint8, device=f"cuda:{d}")
        t[d * shard:(d + 1) * shard] = torch.randint(0, 255, (shard,), dtype=torch.uint8, generator=torch.Generator().manual_seed(d)).to(t.device)
        bufs.append(t)
    torch.cuda.synchronize()
    ptrs = (C.c_void_p * n)(*[t.data_ptr() for t in bufs])
    assert cuda.lib.mhlo_cuda_all_gather(comm, ptrs, shard) == 0, cuda.last_error()
    want = torch.cat([torch.randint(0, 255, (shard,), dtype=torch.uint8, generator=torch.Generator().manual_seed(d)) for d in range(n)])
    for t in bufs:
        assert torch.equal(t.cpu(), want)
    assert cuda.lib.mhlo_cuda_all_gather(comm, ptrs, 24) == 10  # shards are whole 16-byte words
    assert cuda.lib.mhlo_cuda_comm_destroy(comm) == 0
    torch.cuda.set_device(0)
