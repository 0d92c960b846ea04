// Problem descriptions shared by the contraction dispatcher and the tcgen05 kernels.
#pragma once

#include "common.cuh"

namespace mhlo {

struct GemmProblem {
    const void* a;
    const void* b;
    void* c;
    const void* bias;
    int64_t as[4], bs[4];  // {batch0, batch1, row, col} element strides
    int64_t batch0, batch1, m, n, k;
    int32_t in_dtype, out_dtype, epilogue;
};

struct AttnShape {
    int64_t qs[3], ks[3], vs[3], os[3];  // {batch, head, sequence} element strides; head_dim is contiguous
    int64_t batch, heads, seq_q, seq_k, head_dim;
    float scale;
    int32_t causal;
};

// Tensor-core (tcgen05 + TMA + TMEM) paths; *_supported() says whether the problem meets their layout rules.
bool gemm_tc_supported(const GemmProblem& p);
int gemm_tc_launch(const GemmProblem& p, cudaStream_t stream);
int gemm_device_error();       // synchronises; returns and clears the GEMM kernel's error word (-1: CUDA error)
int attention_device_error();  // same for the attention kernel
bool attention_tc_supported(int dtype, const AttnShape& s, const void* mask);
int attention_tc_launch(int dtype, const void* q, const void* k, const void* v, void* o, const AttnShape& s,
                        cudaStream_t stream);

}  // namespace mhlo
