/*
 * mhlo_oracle.c — CPU restatement of the reference's fused-op arithmetic. TEST INFRASTRUCTURE ONLY:
 * the checker that the parity tests, the smoke test and the benchmark's CPU-baseline leg call. Nothing in
 * the product (the CUDA library, the C API, the PJRT plugin) links, loads or calls this file.
 *
 * Two families:
 *   oracle_*   fp64 evaluation of the formulas the reference lowers each fused op to. Inputs are fp32
 *              arrays holding the exact values of the (f32/f16/bf16) device inputs; outputs are fp64.
 *   cpu_*_f32  fp32, OpenMP-threaded, same operation order as the reference's CPU partition kernels
 *              (Sources/HeterogeneousFusion/{LayerNorm,Softmax,Elementwise,Matmul}CPU.swift). These are
 *              what the benchmark times as the host-core baseline.
 *
 * Parity pinning: the formulas are checked by tests against the reference's own known-answer tests
 * (Tests/MetalHLOCoreTests/MetalKernelTests.swift:56-102,173-274: softmax rows sum to 1 and match
 * exp/sum on [1,2,3,4]; LayerNorm rows have mean 0 / unit variance; RMSNorm [3,4,0,0] -> [1.2,1.6,0,0];
 * Tests/MetalHLOTests/ActivationOpsTests.swift:137-318 softmax and tanh-GELU host formulas;
 * Tests/MetalHLOTests/OperationTests.swift:327-348 dot [[1,2],[3,4]]x[[5,6],[7,8]]). Fused attention and
 * 16-bit GEMM/norm numerics have no golden vectors in the reference: for those, parity is unpinned by the
 * reference's tests and rests on this fp64 restatement of its lowering.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* Sets the OpenMP team size for the kernels below (launchers such as torchrun export OMP_NUM_THREADS=1). */
ORACLE_API void oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORACLE_API int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---- LayerNorm: FusedLayerNormHandler, Sources/MetalHLOCore/Compiler/CustomCallHandlers.swift:285-342 ----
 * mean over the last axis; variance = mean((x-mean)^2) (biased); y = (x-mean)/sqrt(var+eps)*gamma+beta. */
ORACLE_API void oracle_layer_norm(const float* x, const float* gamma, const float* beta, double* y,
                                  int64_t rows, int64_t hidden, double eps) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * hidden;
        double* yr = y + r * hidden;
        double mean = 0.0;
        for (int64_t j = 0; j < hidden; ++j) mean += (double)xr[j];
        mean /= (double)hidden;
        double var = 0.0;
        for (int64_t j = 0; j < hidden; ++j) {
            double d = (double)xr[j] - mean;
            var += d * d;
        }
        var /= (double)hidden;
        double sd = sqrt(var + eps);
        for (int64_t j = 0; j < hidden; ++j) {
            double g = gamma ? (double)gamma[j] : 1.0;
            double b = beta ? (double)beta[j] : 0.0;
            yr[j] = ((double)xr[j] - mean) / sd * g + b;
        }
    }
}

/* ---- RMSNorm: FusedRMSNormHandler, CustomCallHandlers.swift:349-394 --------------------------------------
 * y = x / sqrt(mean(x^2) + eps) * weight. */
ORACLE_API void oracle_rms_norm(const float* x, const float* gamma, double* y, int64_t rows, int64_t hidden,
                                double eps) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * hidden;
        double* yr = y + r * hidden;
        double ms = 0.0;
        for (int64_t j = 0; j < hidden; ++j) ms += (double)xr[j] * (double)xr[j];
        ms /= (double)hidden;
        double rms = sqrt(ms + eps);
        for (int64_t j = 0; j < hidden; ++j) yr[j] = (double)xr[j] / rms * (gamma ? (double)gamma[j] : 1.0);
    }
}

/* ---- softmax along one axis of [outer, len, inner]: FusedSoftmaxHandler, CustomCallHandlers.swift:644-672;
 * kernel form Sources/MetalHLOCore/Metal/Kernels/SoftmaxKernel.swift:23-167 (max, exp(x-max), sum, divide). */
ORACLE_API void oracle_softmax(const float* x, double* y, int64_t outer, int64_t len, int64_t inner) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < outer * inner; ++r) {
        int64_t base = (r / inner) * len * inner + (r % inner);
        double m = -INFINITY;
        for (int64_t j = 0; j < len; ++j) {
            double v = (double)x[base + j * inner];
            if (v > m) m = v;
        }
        double s = 0.0;
        for (int64_t j = 0; j < len; ++j) {
            double e = exp((double)x[base + j * inner] - m);
            y[base + j * inner] = e;
            s += e;
        }
        for (int64_t j = 0; j < len; ++j) y[base + j * inner] /= s;
    }
}

/* ---- activations: FusedGeluHandler CustomCallHandlers.swift:677-711 (tanh form, constants
 * 0.7978845608028654 and 0.044715; erf form 0.5x(1+erf(x/sqrt2))); SiLU x*sigmoid(x)
 * (Sources/MetalHLOCore/Compiler/CodeGenerator.swift:4875-4896). */
ORACLE_API void oracle_gelu(const float* x, double* y, int64_t n, int approximate) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        double v = (double)x[i];
        if (approximate)
            y[i] = 0.5 * v * (1.0 + tanh(0.7978845608028654 * (v + 0.044715 * v * v * v)));
        else
            y[i] = 0.5 * v * (1.0 + erf(v * 0.70710678118654752440));
    }
}

ORACLE_API void oracle_silu(const float* x, double* y, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        double v = (double)x[i];
        y[i] = v / (1.0 + exp(-v));
    }
}

/* ---- dot_general after layout canonicalisation: C[b,M,N] = sum_k A[b,M,K] * B[b,K,N]
 * (Sources/MetalHLOCore/Compiler/MPSGraphCompiler.swift:814-980 permutes to this form;
 * CodeGenerator.swift:3155-3298). trans_a: A stored [b,K,M]; trans_b: B stored [b,N,K]. */
ORACLE_API void oracle_gemm(const float* a, const float* b, double* c, int64_t batch, int64_t m, int64_t n,
                            int64_t k, int trans_a, int trans_b) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t bi = 0; bi < batch; ++bi) {
        for (int64_t i = 0; i < m; ++i) {
            const float* ab = a + bi * m * k;
            const float* bb = b + bi * k * n;
            double* cr = c + (bi * m + i) * n;
            for (int64_t j = 0; j < n; ++j) cr[j] = 0.0;
            for (int64_t p = 0; p < k; ++p) {
                double av = trans_a ? (double)ab[p * m + i] : (double)ab[i * k + p];
                if (trans_b) {
                    for (int64_t j = 0; j < n; ++j) cr[j] += av * (double)bb[j * k + p];
                } else {
                    const float* br = bb + p * n;
                    for (int64_t j = 0; j < n; ++j) cr[j] += av * (double)br[j];
                }
            }
        }
    }
}

/* ---- scaled dot-product attention: FusedScaledDotProductAttentionHandler.emitManualSDPA,
 * CustomCallHandlers.swift:245-276: scores = Q K^T * scale (+ mask); softmax over keys; out = P V.
 * Q [bh, sq, d], K/V [bh, sk, d] with bh = batch*heads. causal: key j is visible to query i iff
 * j <= i, also when sq != sk (the tiled kernel's `kv_pos > q_pos` cut,
 * Sources/MetalHLOCore/Metal/Kernels/FlashAttentionKernel.swift:545,578). mask (optional) is
 * additive, [sq, sk], shared by all bh. */
ORACLE_API void oracle_attention(const float* q, const float* k, const float* v, const float* mask, double* o,
                                 int64_t bh, int64_t sq, int64_t sk, int64_t d, double scale, int causal) {
#pragma omp parallel
    {
        double* p = (double*)malloc((size_t)sk * sizeof(double));
#pragma omp for collapse(2) schedule(static)
        for (int64_t h = 0; h < bh; ++h) {
            for (int64_t i = 0; i < sq; ++i) {
                const float* qi = q + (h * sq + i) * d;
                int64_t lim = causal ? i + 1 : sk;
                if (lim > sk) lim = sk;
                double m = -INFINITY;
                for (int64_t j = 0; j < lim; ++j) {
                    const float* kj = k + (h * sk + j) * d;
                    double s = 0.0;
                    for (int64_t t = 0; t < d; ++t) s += (double)qi[t] * (double)kj[t];
                    s *= scale;
                    if (mask) s += (double)mask[i * sk + j];
                    p[j] = s;
                    if (s > m) m = s;
                }
                double sum = 0.0;
                for (int64_t j = 0; j < lim; ++j) {
                    p[j] = exp(p[j] - m);
                    sum += p[j];
                }
                double* oi = o + (h * sq + i) * d;
                for (int64_t t = 0; t < d; ++t) oi[t] = 0.0;
                for (int64_t j = 0; j < lim; ++j) {
                    const float* vj = v + (h * sk + j) * d;
                    double w = p[j] / sum;
                    for (int64_t t = 0; t < d; ++t) oi[t] += w * (double)vj[t];
                }
            }
        }
        free(p);
    }
}

/* ======== fp32 host-core baseline, operation order of the reference's CPU partition ====================== */

/* LayerNormCPU.execute, Sources/HeterogeneousFusion/LayerNormCPU.swift:26-63: mean, mean of squares,
 * variance = max(E[x^2] - mean^2, 0), invStd = 1/sqrt(var+eps), then scale by gamma and add beta. */
ORACLE_API void cpu_layer_norm_f32(const float* x, const float* gamma, const float* beta, float* y, int64_t rows,
                                   int64_t hidden, float eps) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * hidden;
        float* yr = y + r * hidden;
        float s = 0.f, q = 0.f;
        for (int64_t j = 0; j < hidden; ++j) {
            s += xr[j];
            q += xr[j] * xr[j];
        }
        float mean = s / (float)hidden;
        float var = q / (float)hidden - mean * mean;
        if (var < 0.f) var = 0.f;
        float inv = 1.0f / sqrtf(var + eps);
        for (int64_t j = 0; j < hidden; ++j) yr[j] = (xr[j] - mean) * inv * gamma[j] + beta[j];
    }
}

/* Same structure without the mean (rms_norm_kernel, Sources/MetalHLOCore/Metal/Kernels/LayerNormKernel.swift:
 * 427-520: sum of squares, rsqrt(mean+eps), times gamma). */
ORACLE_API void cpu_rms_norm_f32(const float* x, const float* gamma, float* y, int64_t rows, int64_t hidden,
                                 float eps) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * hidden;
        float* yr = y + r * hidden;
        float q = 0.f;
        for (int64_t j = 0; j < hidden; ++j) q += xr[j] * xr[j];
        float inv = 1.0f / sqrtf(q / (float)hidden + eps);
        for (int64_t j = 0; j < hidden; ++j) yr[j] = xr[j] * inv * gamma[j];
    }
}

/* SoftmaxCPU.execute, Sources/HeterogeneousFusion/SoftmaxCPU.swift:16-52: max, subtract, exp, sum, scale by
 * 1/sum. */
ORACLE_API void cpu_softmax_f32(const float* x, float* y, int64_t rows, int64_t cols) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        float* yr = y + r * cols;
        float m = xr[0];
        for (int64_t j = 1; j < cols; ++j) m = xr[j] > m ? xr[j] : m;
        float s = 0.f;
        for (int64_t j = 0; j < cols; ++j) {
            yr[j] = expf(xr[j] - m);
            s += yr[j];
        }
        float inv = 1.0f / s;
        for (int64_t j = 0; j < cols; ++j) yr[j] *= inv;
    }
}

/* ElementwiseCPU gelu, Sources/HeterogeneousFusion/ElementwiseCPU.swift:47-55. */
ORACLE_API void cpu_gelu_f32(const float* x, float* y, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float v = x[i];
        float inner = 0.7978845608f * (v + 0.044715f * v * v * v);
        y[i] = 0.5f * v * (1.0f + tanhf(inner));
    }
}

/* MatmulCPU.execute, Sources/HeterogeneousFusion/MatmulCPU.swift:29-50: C = A[M,K] x B[K,N], fp32. The
 * reference calls vDSP_mmul; this is a cache-blocked, threaded triple loop with the same result order per
 * output element up to fp32 reassociation inside a k-panel. */
ORACLE_API void cpu_gemm_f32(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k) {
    const int64_t KB = 256;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; ++i) {
        float* cr = c + i * n;
        for (int64_t j = 0; j < n; ++j) cr[j] = 0.f;
        for (int64_t p0 = 0; p0 < k; p0 += KB) {
            int64_t p1 = p0 + KB < k ? p0 + KB : k;
            for (int64_t p = p0; p < p1; ++p) {
                float av = a[i * k + p];
                const float* br = b + p * n;
                for (int64_t j = 0; j < n; ++j) cr[j] += av * br[j];
            }
        }
    }
}

/* fp32 attention in the tiled kernel's online-softmax order
 * (Sources/MetalHLOCore/Metal/Kernels/FlashAttentionKernel.swift:469-615), one query row at a time. */
ORACLE_API void cpu_attention_f32(const float* q, const float* k, const float* v, float* o, int64_t bh,
                                  int64_t sq, int64_t sk, int64_t d, float scale, int causal) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t h = 0; h < bh; ++h) {
        for (int64_t i = 0; i < sq; ++i) {
            const float* qi = q + (h * sq + i) * d;
            float* oi = o + (h * sq + i) * d;
            float acc[512];
            float m = -INFINITY, l = 0.f;
            for (int64_t t = 0; t < d; ++t) acc[t] = 0.f;
            int64_t lim = causal ? i + 1 : sk;
            if (lim > sk) lim = sk;
            for (int64_t j = 0; j < lim; ++j) {
                const float* kj = k + (h * sk + j) * d;
                const float* vj = v + (h * sk + j) * d;
                float s = 0.f;
                for (int64_t t = 0; t < d; ++t) s += qi[t] * kj[t];
                s *= scale;
                float mn = s > m ? s : m;
                float corr = expf(m - mn);
                float p = expf(s - mn);
                l = l * corr + p;
                for (int64_t t = 0; t < d; ++t) acc[t] = acc[t] * corr + p * vj[t];
                m = mn;
            }
            for (int64_t t = 0; t < d; ++t) oi[t] = lim > 0 ? acc[t] / l : 0.f;
        }
    }
}
