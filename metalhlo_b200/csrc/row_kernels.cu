// LayerNorm, RMSNorm and softmax over the rows of a [rows, hidden] tensor: HBM-bound kernels that read
// every input byte once and write every output byte once.
//
// Layout in HBM: x and y are row-major [rows, hidden]; gamma/beta are [hidden] and stay L2-resident.
// Algorithmic traffic per row: hidden*sizeof(T) read + hidden*sizeof(T) written.
//
// Fast path (row_vec_kernel): one CTA owns one row at a time. Each thread pulls VPT 16-byte vectors with
// streaming loads straight into fp32 registers, the CTA reduces with warp shuffles plus one shared-memory
// hop, and the result leaves with evict-first 16-byte stores. The row never touches shared memory or L1.
// The slow path (row_strided_kernel) takes any hidden size, alignment or inner stride and re-reads the row
// from L2 per pass.
//
// Semantics follow the reference's fused custom-call handlers
// (Sources/MetalHLOCore/Compiler/CustomCallHandlers.swift:285-394 and :644-672): LayerNorm uses the biased
// variance of the centred row, RMSNorm adds eps to the mean square, softmax subtracts the row maximum.
#include "common.cuh"

namespace mhlo {
namespace {

enum RowOp : int { kLayerNorm = 0, kRmsNorm = 1, kSoftmax = 2 };

template <typename T>
__device__ __forceinline__ float row_exp(float x) {
    // 16-bit outputs keep 8 to 11 mantissa bits: the hardware ex2 path is exact enough and keeps the SFU
    // from becoming the limiter. fp32 rows use the accurate expf.
    if constexpr (sizeof(T) == 2) return __expf(x);
    return expf(x);
}

// Register budget: a thread holds VPT*E fp32 values, so wide configurations cap the CTA size.
template <typename T, int VPT>
constexpr int row_vec_max_threads() {
    constexpr int vals = VPT * VecTraits<T>::kElems;
    return vals > 32 ? 256 : (vals > 16 ? 512 : 1024);
}

template <typename T, int VPT, int OP>
__global__ void __launch_bounds__((row_vec_max_threads<T, VPT>())) row_vec_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                                       const T* __restrict__ beta, T* __restrict__ y,
                                                       int64_t rows, int hidden, float eps) {
    using VT = VecTraits<T>;
    constexpr int E = VT::kElems;
    __shared__ float red[2][32];
    const int nvec = hidden / E;
    const float inv_n = 1.0f / static_cast<float>(hidden);
    int ph = 0;  // which half of red[] the next reduction uses; alternating makes one barrier per reduction safe

    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + row * hidden);
        uint4* yr = reinterpret_cast<uint4*>(y + row * hidden);
        float v[VPT][E];
        bool live[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = threadIdx.x + i * blockDim.x;
            live[i] = idx < nvec;
            if (live[i]) {
                VT::unpack(ld_stream16(xr + idx), v[i]);
            } else {
#pragma unroll
                for (int e = 0; e < E; ++e) v[i][e] = (OP == kSoftmax) ? -INFINITY : 0.f;
            }
        }

        if constexpr (OP == kSoftmax) {
            float m = -INFINITY;
#pragma unroll
            for (int i = 0; i < VPT; ++i)
#pragma unroll
                for (int e = 0; e < E; ++e) m = fmaxf(m, v[i][e]);
            m = cta_reduce<MaxOp>(m, red[ph]);
            ph ^= 1;
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < VPT; ++i)
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    v[i][e] = row_exp<T>(v[i][e] - m);  // exp(-inf) = 0 for the padding lanes
                    s += v[i][e];
                }
            s = cta_reduce<SumOp>(s, red[ph]);
            ph ^= 1;
            const float inv = 1.0f / s;
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                if (!live[i]) continue;
#pragma unroll
                for (int e = 0; e < E; ++e) v[i][e] *= inv;
                st_stream16(yr + threadIdx.x + i * blockDim.x, VT::pack(v[i]));
            }
        } else {
            float mean = 0.f;
            if constexpr (OP == kLayerNorm) {
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < VPT; ++i)
#pragma unroll
                    for (int e = 0; e < E; ++e) s += v[i][e];
                mean = cta_reduce<SumOp>(s, red[ph]) * inv_n;
                ph ^= 1;
            }
            float q = 0.f;
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                if (!live[i]) continue;
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const float d = v[i][e] - mean;
                    q += d * d;
                }
            }
            q = cta_reduce<SumOp>(q, red[ph]);
            ph ^= 1;
            const float rstd = 1.0f / sqrtf(q * inv_n + eps);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                if (!live[i]) continue;
                const int idx = threadIdx.x + i * blockDim.x;
                float g[E], b[E];
                if (gamma != nullptr) {
                    VT::unpack(__ldg(reinterpret_cast<const uint4*>(gamma) + idx), g);
                } else {
#pragma unroll
                    for (int e = 0; e < E; ++e) g[e] = 1.f;
                }
                if (OP == kLayerNorm && beta != nullptr) {
                    VT::unpack(__ldg(reinterpret_cast<const uint4*>(beta) + idx), b);
                } else {
#pragma unroll
                    for (int e = 0; e < E; ++e) b[e] = 0.f;
                }
#pragma unroll
                for (int e = 0; e < E; ++e) v[i][e] = (v[i][e] - mean) * rstd * g[e] + b[e];
                st_stream16(yr + idx, VT::pack(v[i]));
            }
        }
    }
}

// Any shape, any alignment: logical row r = (o, i) of a tensor viewed as [outer, len, inner]; element j of
// that row sits at base + j*inner. One CTA per row; each pass re-reads the row (L2 serves the repeats).
template <typename T, int OP>
__global__ void __launch_bounds__(256) row_strided_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                                          const T* __restrict__ beta, T* __restrict__ y,
                                                          int64_t rows, int64_t len, int64_t inner, float eps) {
    using VT = VecTraits<T>;
    __shared__ float red[2][32];
    const float inv_n = 1.0f / static_cast<float>(len);
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const int64_t base = (row / inner) * len * inner + (row % inner);
        const T* xr = x + base;
        T* yr = y + base;
        if constexpr (OP == kSoftmax) {
            float m = -INFINITY;
            for (int64_t j = threadIdx.x; j < len; j += blockDim.x) m = fmaxf(m, VT::to_float(xr[j * inner]));
            m = cta_reduce<MaxOp>(m, red[0]);
            float s = 0.f;
            for (int64_t j = threadIdx.x; j < len; j += blockDim.x)
                s += row_exp<T>(VT::to_float(xr[j * inner]) - m);
            s = cta_reduce<SumOp>(s, red[1]);
            const float inv = 1.0f / s;
            for (int64_t j = threadIdx.x; j < len; j += blockDim.x)
                yr[j * inner] = VT::from_float(row_exp<T>(VT::to_float(xr[j * inner]) - m) * inv);
        } else {
            float mean = 0.f;
            if constexpr (OP == kLayerNorm) {
                float s = 0.f;
                for (int64_t j = threadIdx.x; j < len; j += blockDim.x) s += VT::to_float(xr[j * inner]);
                mean = cta_reduce<SumOp>(s, red[0]) * inv_n;
            }
            float q = 0.f;
            for (int64_t j = threadIdx.x; j < len; j += blockDim.x) {
                const float d = VT::to_float(xr[j * inner]) - mean;
                q += d * d;
            }
            q = cta_reduce<SumOp>(q, red[1]);
            const float rstd = 1.0f / sqrtf(q * inv_n + eps);
            for (int64_t j = threadIdx.x; j < len; j += blockDim.x) {
                const float g = gamma ? VT::to_float(gamma[j]) : 1.f;
                const float b = (OP == kLayerNorm && beta) ? VT::to_float(beta[j]) : 0.f;
                yr[j * inner] = VT::from_float((VT::to_float(xr[j * inner]) - mean) * rstd * g + b);
            }
        }
        __syncthreads();  // red[] is reused by the next row
    }
}

template <typename T, int OP>
int launch_rows(const void* x, const void* gamma, const void* beta, void* y, int64_t outer, int64_t len,
                int64_t inner, float eps, const mhlo_cuda_row_tuning* tuning, cudaStream_t stream,
                const char* what) {
    constexpr int E = VecTraits<T>::kElems;
    const int64_t rows = outer * inner;
    if (rows == 0 || len == 0) return MHLO_CUDA_OK;
    const T* xp = static_cast<const T*>(x);
    const T* gp = static_cast<const T*>(gamma);
    const T* bp = static_cast<const T*>(beta);
    T* yp = static_cast<T*>(y);

    const int64_t nvec = len / E;
    const bool vec_ok = inner == 1 && len % E == 0 && nvec <= 8 * 1024 && aligned16(x) && aligned16(y) &&
                        aligned16(gamma) && aligned16(beta);
    if (!vec_ok) {
        const int grid = static_cast<int>(rows < 148LL * 64 ? rows : 148LL * 64);
        row_strided_kernel<T, OP><<<grid, 256, 0, stream>>>(xp, gp, bp, yp, rows, len, inner, eps);
        MHLO_CUDA_CHECK_LAUNCH(what);
        return MHLO_CUDA_OK;
    }

    int vpt = tuning ? tuning->vecs_per_thread : 0;
    int threads = tuning ? tuning->threads : 0;
    int ctas_per_sm = tuning ? tuning->ctas_per_sm : 0;
    if (vpt == 0) {
        vpt = 1;
        while (vpt < 8 && nvec > 128LL * vpt) vpt *= 2;
        if (sizeof(T) == 2 && vpt > 4 && nvec <= 1024 * 4) vpt = 4;  // keep 16-bit rows at <= 32 fp32 regs
    }
    if (vpt != 1 && vpt != 2 && vpt != 4 && vpt != 8)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: vecs_per_thread must be 1, 2, 4 or 8 (got %d)", what, vpt);
    if (threads == 0 && !(tuning && tuning->vecs_per_thread)) {
        // grow the per-thread share until the CTA fits its register-derived thread limit
        while (vpt < 8 && (nvec + vpt - 1) / vpt > (vpt * E > 32 ? 256 : (vpt * E > 16 ? 512 : 1024))) vpt *= 2;
    }
    if (threads == 0) threads = static_cast<int>(((nvec + vpt - 1) / vpt + 31) / 32 * 32);
    if (threads % 32 != 0 || threads < 32 || threads > 1024)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: threads must be a multiple of 32 in [32,1024] (got %d)",
                    what, threads);
    const int max_threads = vpt * E > 32 ? 256 : (vpt * E > 16 ? 512 : 1024);
    if (threads > max_threads)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: %d threads exceed the %d allowed with %d vectors per thread",
                    what, threads, max_threads, vpt);
    if (static_cast<int64_t>(threads) * vpt < nvec)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: threads*vecs_per_thread=%d does not cover %lld vectors",
                    what, threads * vpt, static_cast<long long>(nvec));
    int64_t grid = rows;
    if (ctas_per_sm > 0 && grid > static_cast<int64_t>(kNumSMs) * ctas_per_sm)
        grid = static_cast<int64_t>(kNumSMs) * ctas_per_sm;
    if (grid > 0x7fffffffLL) grid = 0x7fffffffLL;
    const int h = static_cast<int>(len);
    const int g = static_cast<int>(grid);
    switch (vpt) {
        case 1: row_vec_kernel<T, 1, OP><<<g, threads, 0, stream>>>(xp, gp, bp, yp, rows, h, eps); break;
        case 2: row_vec_kernel<T, 2, OP><<<g, threads, 0, stream>>>(xp, gp, bp, yp, rows, h, eps); break;
        case 4: row_vec_kernel<T, 4, OP><<<g, threads, 0, stream>>>(xp, gp, bp, yp, rows, h, eps); break;
        default: row_vec_kernel<T, 8, OP><<<g, threads, 0, stream>>>(xp, gp, bp, yp, rows, h, eps); break;
    }
    MHLO_CUDA_CHECK_LAUNCH(what);
    return MHLO_CUDA_OK;
}

template <int OP>
int dispatch_rows(int dtype, const void* x, const void* gamma, const void* beta, void* y, int64_t outer,
                  int64_t len, int64_t inner, float eps, const mhlo_cuda_row_tuning* tuning, void* stream,
                  const char* what) {
    if (outer < 0 || len < 0 || inner < 0)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: negative extent", what);
    if (outer * len * inner > 0 && (x == nullptr || y == nullptr))
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: null tensor pointer", what);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case MHLO_DT_F32:
            return launch_rows<float, OP>(x, gamma, beta, y, outer, len, inner, eps, tuning, s, what);
        case MHLO_DT_F16:
            return launch_rows<__half, OP>(x, gamma, beta, y, outer, len, inner, eps, tuning, s, what);
        case MHLO_DT_BF16:
            return launch_rows<__nv_bfloat16, OP>(x, gamma, beta, y, outer, len, inner, eps, tuning, s, what);
        default:
            return fail(MHLO_CUDA_UNSUPPORTED, "%s: dtype %d is not a float type this kernel handles", what,
                        dtype);
    }
}

}  // namespace
}  // namespace mhlo

extern "C" {

int mhlo_cuda_layer_norm(int dtype, const void* x_dev, const void* gamma_dev, const void* beta_dev, void* y_dev,
                         int64_t rows, int64_t hidden, float eps, const mhlo_cuda_row_tuning* tuning,
                         mhlo_cuda_stream_t stream) {
    return mhlo::dispatch_rows<mhlo::kLayerNorm>(dtype, x_dev, gamma_dev, beta_dev, y_dev, rows, hidden, 1, eps,
                                                 tuning, stream, "layer_norm");
}

int mhlo_cuda_rms_norm(int dtype, const void* x_dev, const void* gamma_dev, void* y_dev, int64_t rows,
                       int64_t hidden, float eps, const mhlo_cuda_row_tuning* tuning, mhlo_cuda_stream_t stream) {
    return mhlo::dispatch_rows<mhlo::kRmsNorm>(dtype, x_dev, gamma_dev, nullptr, y_dev, rows, hidden, 1, eps,
                                               tuning, stream, "rms_norm");
}

int mhlo_cuda_softmax(int dtype, const void* x_dev, void* y_dev, int64_t outer, int64_t axis_len, int64_t inner,
                      const mhlo_cuda_row_tuning* tuning, mhlo_cuda_stream_t stream) {
    return mhlo::dispatch_rows<mhlo::kSoftmax>(dtype, x_dev, nullptr, nullptr, y_dev, outer, axis_len, inner, 0.f,
                                               tuning, stream, "softmax");
}

}  // extern "C"
