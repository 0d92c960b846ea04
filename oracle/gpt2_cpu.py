"""TEST AND BASELINE INFRASTRUCTURE — not part of the product.

fp32 CPU forward pass of the GPT-2-architecture module that metalhlo_b200.modules.gpt2_module prints, composed from
the host kernels of the reference's CPU partition as this directory restates them: matrix products through the host
BLAS sgemm (the reference calls vDSP_mmul, Sources/HeterogeneousFusion/MatmulCPU.swift:29-50), LayerNorm, tanh-GELU and
causal attention through the OpenMP kernels of mhlo_oracle.c (LayerNormCPU / ElementwiseCPU / the tiled attention order,
cited there). It is what bench.py times as the CPU baseline and as its reference arm; tests pin it to the fp64 module
interpreter (oracle/interp.py).

Arguments come in the order of gpt2_module's parameter list: ids, wte, wpe, then per layer ln1_g, ln1_b, w_qkv, b_qkv,
w_o, b_o, ln2_g, ln2_b, w_fc, b_fc, w_proj, b_proj, then lnf_g, lnf_b.
"""
from __future__ import annotations

import math

import numpy as np

import oracle

PER_LAYER = 12


def forward(inputs, heads: int, eps: float = 1e-5) -> np.ndarray:
    """Logits [batch, seq, vocab] in fp32."""
    ids, wte, wpe = inputs[0], inputs[1], inputs[2]
    layers = (len(inputs) - 5) // PER_LAYER
    batch, seq = ids.shape
    d_model = wte.shape[1]
    dh = d_model // heads
    rows = batch * seq
    x = (wte[ids.reshape(-1)] + np.tile(wpe[:seq], (batch, 1))).astype(np.float32)
    h = np.empty_like(x)
    for i in range(layers):
        ln1_g, ln1_b, w_qkv, b_qkv, w_o, b_o, ln2_g, ln2_b, w_fc, b_fc, w_proj, b_proj = inputs[3 + i * PER_LAYER: 3 + (i + 1) * PER_LAYER]
        oracle.cpu_layer_norm_f32(x, ln1_g, ln1_b, h, eps)
        qkv = h @ w_qkv + b_qkv
        q, k, v = (np.ascontiguousarray(qkv[:, j * d_model:(j + 1) * d_model].reshape(batch, seq, heads, dh).transpose(0, 2, 1, 3)).reshape(batch * heads, seq, dh)
                   for j in range(3))
        o = np.empty_like(q)
        oracle.cpu_attention_f32(q, k, v, o, 1.0 / math.sqrt(dh), True)
        attn = np.ascontiguousarray(o.reshape(batch, heads, seq, dh).transpose(0, 2, 1, 3)).reshape(rows, d_model)
        x = x + (attn @ w_o + b_o)
        oracle.cpu_layer_norm_f32(x, ln2_g, ln2_b, h, eps)
        fc = h @ w_fc + b_fc
        act = np.empty_like(fc)
        oracle.cpu_gelu_f32(fc, act)
        x = x + (act @ w_proj + b_proj)
    oracle.cpu_layer_norm_f32(x, inputs[-2], inputs[-1], h, eps)
    return (h @ wte.T).reshape(batch, seq, wte.shape[0])
