// Problem descriptions shared by the contraction dispatcher and the tcgen05 kernels.
#pragma once

#include "common.cuh"

namespace mhlo {

struct GemmProblem {
    const void* a;
    const void* b;
    void* c;
    const void* bias;
    const void* residual = nullptr;  // added to the product after the bias: same type, pitch and column offset as C; no activation
    int64_t as[4], bs[4];  // {batch0, batch1, row, col} element strides
    int64_t batch0, batch1, m, n, k;
    int32_t in_dtype, out_dtype, epilogue;
    // Output placement. ldc = elements between rows of C (0: dense, = n); c_col0 = first column this product fills
    // inside a wider matrix; copies[] = further matrices (peers' memory) that receive the same tile stores.
    int64_t ldc = 0, c_col0 = 0;
    void* copies[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    int32_t n_copies = 0;
    int32_t copy_stores = 0;  // how the copies are written: 0 / 1 = 16-byte stores per lane, 2 = bulk tensor stores (one map per copy)
    // Launch knobs of the tensor-core kernel; 0 = chosen by the library. tile_n: 128 or 256 columns per tile; stages: depth
    // of the TMA ring; cta_group: 1 = one CTA per 128-row tile, 2 = a pair of CTAs per 256-row tile.
    int32_t tile_n = 0, stages = 0, cta_group = 0;
};

// A 2-D convolution of dense NHWC input with dense HWIO filters into dense NHWC output, stride 1, one feature group: the
// form the tensor-core kernel reads without a patch matrix.
struct ConvProblem {
    const void* x;
    const void* wgt;
    void* out;
    const void* bias = nullptr;  // one value per output feature, of the output's type
    int32_t dtype, out_dtype, epilogue = 0;
    int64_t images, h, w, channels, kh, kw, features, oh, ow, pad_h, pad_w, dil_h, dil_w;
    int64_t stride_h = 1, stride_w = 1;
};
bool conv_tc_supported(const ConvProblem& c);
int conv_tc_launch(const ConvProblem& c, cudaStream_t stream);

struct AttnShape {
    int64_t qs[3], ks[3], vs[3], os[3];  // {batch, head, sequence} element strides; head_dim is contiguous
    int64_t batch, heads, seq_q, seq_k, head_dim;
    float scale;
    int32_t causal;
    int32_t tile_order = 0;  // tensor-core kernel: 0 = chosen by the library, 1 = long/short pairs per (batch, head), 2 = longest tiles first
};

// Tensor-core (tcgen05 + TMA + TMEM) paths; *_supported() says whether the problem meets their layout rules.
bool gemm_tc_supported(const GemmProblem& p);
int gemm_tc_launch(const GemmProblem& p, cudaStream_t stream);
int gemm_device_error();       // synchronises; returns and clears the GEMM kernel's error word (-1: CUDA error)
int attention_device_error();  // same for the attention kernel
// Stream-ordered copies of the error words into pinned host memory, and host stores into them (clearing, or the test hook).
bool gemm_error_fetch_async(int* pinned_dst, cudaStream_t stream);
bool attention_error_fetch_async(int* pinned_dst, cudaStream_t stream);
bool gemm_error_store(int code);
bool attention_error_store(int code);
bool gemm_wait_expiry_probe(uint64_t limit_ns, cudaStream_t stream);
// One CTA: stores `epoch` into word `rank` of every other rank's flag array, then waits (at most limit_ns) until every word
// of this rank's own array has reached `epoch`; an expired wait records code 95 in the GEMM error word.
bool gemm_peer_barrier_launch(uint64_t* const* flag_arrays, int n_ranks, int rank, uint64_t epoch, uint64_t limit_ns, cudaStream_t stream);
bool attention_tc_supported(int dtype, const AttnShape& s, const void* mask);
int attention_tc_launch(int dtype, const void* q, const void* k, const void* v, void* o, const AttnShape& s,
                        cudaStream_t stream);

}  // namespace mhlo
