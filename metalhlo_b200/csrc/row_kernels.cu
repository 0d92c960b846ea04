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

// Packed fp32x2 arithmetic (one issue slot for two lanes of math on sm_100). The row kernels are bound by
// instruction issue before they are bound by HBM, so every per-element operation is done two at a time.
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 splat2(float a) { return make_float2(a, a); }
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// CTA all-reduce with one barrier. `scratch` is 32 floats whose slots at and above the warp count hold the
// identity (written once at kernel start); the caller never reuses a scratch array for two consecutive
// reductions, which is what makes a single __syncthreads() per reduction safe.
template <typename Op>
__device__ __forceinline__ float cta_reduce1(float v, float* scratch, int nwarps) {
    v = warp_reduce<Op>(v);
    if (nwarps == 1) return v;
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    if (nwarps <= 4) {
        const float4 r = *reinterpret_cast<const float4*>(scratch);
        return Op::apply(Op::apply(r.x, r.y), Op::apply(r.z, r.w));
    }
    return warp_reduce<Op>(scratch[threadIdx.x & 31]);
}

// One CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ... Each thread owns VPT 16-byte vectors of the row
// (vector index tid + i*blockDim.x), keeps them as fp32 pairs in registers and has the next row's vectors in
// flight while it works on the current one. gamma/beta are widened to fp32 once per CTA into shared memory,
// laid out in float4 planes so that a warp's reads are contiguous. FULL = every thread slot maps to a real
// vector (no predicates in the loop).
constexpr int kDepth = 2;

//
// ADD (norms only): the row is x + res, rounded to T as a separate add would leave it; that sum is written to sum_out
// (the residual stream a later layer reads) and normalised from registers.
template <typename T, int VPT, int OP, bool FULL, bool ADD>
__global__ void __launch_bounds__((row_vec_max_threads<T, VPT>()))
row_vec_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
               T* __restrict__ y, int64_t rows, int hidden, float eps, const T* __restrict__ res, T* __restrict__ sum_out,
               int64_t res_rows) {  // res has res_rows rows, repeated down the tensor (res_rows = rows: one per row)
    using VT = VecTraits<T>;
    constexpr int E = VT::kElems;
    constexpr int H = E / 2;  // float2 per vector
    constexpr int P = E / 4;  // float4 planes per vector
    extern __shared__ __align__(16) float params[];
    __shared__ __align__(16) float red[2][32];

    const int tid = threadIdx.x;
    const int nthreads = blockDim.x;
    const int nwarps = nthreads >> 5;
    const int nvec = hidden / E;
    const int nslots = nthreads * VPT;
    const float inv_n = 1.0f / static_cast<float>(hidden);
    float4* const gsm = reinterpret_cast<float4*>(params);
    float4* const bsm = gsm + P * nslots;

    bool live[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) live[i] = FULL || (tid + i * nthreads < nvec);

    grid_dependency_wait();  // gamma / beta may be results of the previous kernel too
    grid_dependency_release();

    if (tid < 32) {
        red[0][tid] = (OP == kSoftmax) ? -INFINITY : 0.f;
        red[1][tid] = 0.f;
    }
    if constexpr (OP != kSoftmax) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = tid + i * nthreads;
            if (!live[i]) continue;
            float2 g[H], b[H];
            if (gamma != nullptr) {
                VT::unpack2(__ldg(reinterpret_cast<const uint4*>(gamma) + idx), g);
            } else {
#pragma unroll
                for (int h = 0; h < H; ++h) g[h] = splat2(1.f);
            }
#pragma unroll
            for (int p = 0; p < P; ++p)
                gsm[p * nslots + idx] = make_float4(g[2 * p].x, g[2 * p].y, g[2 * p + 1].x, g[2 * p + 1].y);
            if constexpr (OP == kLayerNorm) {
                if (beta != nullptr) {
                    VT::unpack2(__ldg(reinterpret_cast<const uint4*>(beta) + idx), b);
                } else {
#pragma unroll
                    for (int h = 0; h < H; ++h) b[h] = splat2(0.f);
                }
#pragma unroll
                for (int p = 0; p < P; ++p)
                    bsm[p * nslots + idx] = make_float4(b[2 * p].x, b[2 * p].y, b[2 * p + 1].x, b[2 * p + 1].y);
            }
        }
    }
    __syncthreads();

    // Register ring of kDepth rows: row r + kDepth*gridDim.x is requested as soon as row r has been unpacked,
    // so kDepth rows per CTA are in flight while one is being worked on.
    uint4 raw[kDepth][VPT];
    uint4 raw_res[ADD ? kDepth : 1][ADD ? VPT : 1];
#pragma unroll
    for (int d = 0; d < kDepth; ++d) {
        const int64_t r = blockIdx.x + static_cast<int64_t>(d) * gridDim.x;
        if (r < rows) {
            const uint4* xr = reinterpret_cast<const uint4*>(x + r * hidden);
#pragma unroll
            for (int i = 0; i < VPT; ++i)
                if (live[i]) raw[d][i] = ld_stream16(xr + tid + i * nthreads);
            if constexpr (ADD) {
                const uint4* rr = reinterpret_cast<const uint4*>(res + (r % res_rows) * hidden);
#pragma unroll
                for (int i = 0; i < VPT; ++i)
                    if (live[i]) raw_res[d][i] = ld_stream16(rr + tid + i * nthreads);
            }
        }
    }
    int ph = 0;
    for (int64_t row0 = blockIdx.x; row0 < rows; row0 += static_cast<int64_t>(kDepth) * gridDim.x) {
#pragma unroll
      for (int d = 0; d < kDepth; ++d) {
        const int64_t row = row0 + static_cast<int64_t>(d) * gridDim.x;
        if (row >= rows) break;
        float2 v[VPT][H];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            if (live[i]) {
                VT::unpack2(raw[d][i], v[i]);
                if constexpr (ADD) {
                    float2 rv[H];
                    VT::unpack2(raw_res[d][i], rv);
#pragma unroll
                    for (int h = 0; h < H; ++h) v[i][h] = add2(v[i][h], rv[h]);
                    const uint4 packed = VT::pack2(v[i]);  // the sum as the element type holds it
                    st_stream16(reinterpret_cast<uint4*>(sum_out + row * hidden) + tid + i * nthreads, packed);
                    VT::unpack2(packed, v[i]);
                }
            } else {
#pragma unroll
                for (int h = 0; h < H; ++h) v[i][h] = splat2((OP == kSoftmax) ? -INFINITY : 0.f);
            }
        }
        const int64_t next = row + static_cast<int64_t>(kDepth) * gridDim.x;
        if (next < rows) {
            const uint4* xn = reinterpret_cast<const uint4*>(x + next * hidden);
#pragma unroll
            for (int i = 0; i < VPT; ++i)
                if (live[i]) raw[d][i] = ld_stream16(xn + tid + i * nthreads);
            if constexpr (ADD) {
                const uint4* rn = reinterpret_cast<const uint4*>(res + (next % res_rows) * hidden);
#pragma unroll
                for (int i = 0; i < VPT; ++i)
                    if (live[i]) raw_res[d][i] = ld_stream16(rn + tid + i * nthreads);
            }
        }
        uint4* yr = reinterpret_cast<uint4*>(y + row * hidden);

        if constexpr (OP == kSoftmax) {
            float m = -INFINITY;
#pragma unroll
            for (int i = 0; i < VPT; ++i)
#pragma unroll
                for (int h = 0; h < H; ++h) m = fmaxf(m, fmaxf(v[i][h].x, v[i][h].y));
            m = cta_reduce1<MaxOp>(m, red[0], nwarps);
            float2 s2 = splat2(0.f);
            if constexpr (sizeof(T) == 2) {
                // exp(x - m) = 2^(x*log2(e) - m*log2(e)): one packed FMA and one ex2 per element
                const float2 l2 = splat2(1.4426950408889634f);
                const float2 nb = splat2(-m * 1.4426950408889634f);
#pragma unroll
                for (int i = 0; i < VPT; ++i)
#pragma unroll
                    for (int h = 0; h < H; ++h) {
                        const float2 t = fma2(v[i][h], l2, nb);
                        v[i][h] = make_float2(ex2_approx(t.x), ex2_approx(t.y));
                        s2 = add2(s2, v[i][h]);
                    }
            } else {
#pragma unroll
                for (int i = 0; i < VPT; ++i)
#pragma unroll
                    for (int h = 0; h < H; ++h) {
                        v[i][h] = make_float2(expf(v[i][h].x - m), expf(v[i][h].y - m));
                        s2 = add2(s2, v[i][h]);
                    }
            }
            const float s = cta_reduce1<SumOp>(s2.x + s2.y, red[1], nwarps);
            const float2 inv = splat2(__frcp_rn(s));
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                if (!live[i]) continue;
#pragma unroll
                for (int h = 0; h < H; ++h) v[i][h] = mul2(v[i][h], inv);
                st_stream16(yr + tid + i * nthreads, VT::pack2(v[i]));
            }
        } else {
            float rstd;
            if constexpr (OP == kLayerNorm) {
                float2 s2 = splat2(0.f);
#pragma unroll
                for (int i = 0; i < VPT; ++i)
#pragma unroll
                    for (int h = 0; h < H; ++h) s2 = add2(s2, v[i][h]);
                const float mean = cta_reduce1<SumOp>(s2.x + s2.y, red[0], nwarps) * inv_n;
                const float2 nm = splat2(-mean);
                float2 q2 = splat2(0.f);
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    if (!live[i]) continue;
#pragma unroll
                    for (int h = 0; h < H; ++h) {
                        v[i][h] = add2(v[i][h], nm);
                        q2 = fma2(v[i][h], v[i][h], q2);
                    }
                }
                rstd = rsqrtf(cta_reduce1<SumOp>(q2.x + q2.y, red[1], nwarps) * inv_n + eps);
            } else {
                float2 q2 = splat2(0.f);
#pragma unroll
                for (int i = 0; i < VPT; ++i)
#pragma unroll
                    for (int h = 0; h < H; ++h) q2 = fma2(v[i][h], v[i][h], q2);
                rstd = rsqrtf(cta_reduce1<SumOp>(q2.x + q2.y, red[ph], nwarps) * inv_n + eps);
                ph ^= 1;
            }
            const float2 r2 = splat2(rstd);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                if (!live[i]) continue;
                const int idx = tid + i * nthreads;
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    const float4 g4 = gsm[p * nslots + idx];
                    if constexpr (OP == kLayerNorm) {
                        const float4 b4 = bsm[p * nslots + idx];
                        v[i][2 * p] = fma2(mul2(v[i][2 * p], r2), make_float2(g4.x, g4.y), make_float2(b4.x, b4.y));
                        v[i][2 * p + 1] =
                            fma2(mul2(v[i][2 * p + 1], r2), make_float2(g4.z, g4.w), make_float2(b4.z, b4.w));
                    } else {
                        v[i][2 * p] = mul2(mul2(v[i][2 * p], r2), make_float2(g4.x, g4.y));
                        v[i][2 * p + 1] = mul2(mul2(v[i][2 * p + 1], r2), make_float2(g4.z, g4.w));
                    }
                }
                st_stream16(yr + idx, VT::pack2(v[i]));
            }
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

// out = round(a + b) elementwise: the sum a fused add + norm has to produce when the row kernel's fast path is not
// available (odd lengths, unaligned pointers).
template <typename T>
__global__ void __launch_bounds__(256) add_rows_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t n,
                                                       int64_t b_period) {  // b holds b_period elements, repeated
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += step)
        out[i] = static_cast<T>(static_cast<float>(a[i]) + static_cast<float>(b[i % b_period]));
}

template <typename T, int OP>
int launch_rows(const void* x, const void* gamma, const void* beta, void* y, int64_t outer, int64_t len,
                int64_t inner, float eps, const mhlo_cuda_row_tuning* tuning, cudaStream_t stream,
                const char* what, const void* res = nullptr, void* sum_out = nullptr, int64_t res_rows = 0) {
    constexpr int E = VecTraits<T>::kElems;
    const int64_t rows = outer * inner;
    if (rows == 0 || len == 0) return MHLO_CUDA_OK;
    if (res_rows <= 0) res_rows = rows;
    const T* xp = static_cast<const T*>(x);
    const T* gp = static_cast<const T*>(gamma);
    const T* bp = static_cast<const T*>(beta);
    T* yp = static_cast<T*>(y);

    const int64_t nvec = len / E;
    // Largest row the register-resident kernel covers: 8 vectors per thread at the CTA size that leaves
    // room for 8*E fp32 values per thread.
    const int64_t max_vecs = 8 * (8 * E > 32 ? 256 : 512);
    const bool with_add = res != nullptr;
    const bool vec_ok = inner == 1 && len % E == 0 && nvec <= max_vecs && aligned16(x) && aligned16(y) &&
                        aligned16(gamma) && aligned16(beta) && aligned16(res) && aligned16(sum_out);
    if (!vec_ok) {
        const int grid = static_cast<int>(rows < 148LL * 64 ? rows : 148LL * 64);
        if (with_add) {
            const int64_t n = rows * len;
            add_rows_kernel<T><<<static_cast<int>(n < 148LL * 2048 ? (n + 255) / 256 : 148 * 8), 256, 0, stream>>>(
                xp, static_cast<const T*>(res), static_cast<T*>(sum_out), n, res_rows * len);
            xp = static_cast<const T*>(sum_out);
        }
        row_strided_kernel<T, OP><<<grid, 256, 0, stream>>>(xp, gp, bp, yp, rows, len, inner, eps);
        MHLO_CUDA_CHECK_LAUNCH(what);
        return MHLO_CUDA_OK;
    }

    if (with_add && sizeof(T) == 4 && nvec > 2 * 1024) {
        // an fp32 row too long for two vectors per thread: separate add, then the plain norm on the sum
        const int64_t n = rows * len;
        add_rows_kernel<T><<<static_cast<int>(n < 148LL * 2048 ? (n + 255) / 256 : 148 * 8), 256, 0, stream>>>(
            xp, static_cast<const T*>(res), static_cast<T*>(sum_out), n, res_rows * len);
        MHLO_CUDA_CHECK_LAUNCH(what);
        return launch_rows<T, OP>(sum_out, gamma, beta, y, outer, len, inner, eps, tuning, stream, what);
    }
    int vpt = tuning ? tuning->vecs_per_thread : 0;
    int threads = tuning ? tuning->threads : 0;
    const int ctas_per_sm = tuning ? tuning->ctas_per_sm : 0;
    if (with_add && sizeof(T) == 4 && (vpt == 0 || vpt > 2)) {
        vpt = nvec > 1024 ? 2 : 1;
        threads = 0;
    }
    if (vpt == 0) {
        // 32 fp32 values per thread measured best on B200 (128 threads for a 4096-wide bf16 row); short rows
        // shrink the share so that a CTA still has at least one full warp.
        vpt = 32 / E;
        while (vpt > 1 && nvec < 32LL * vpt) vpt /= 2;
        while (vpt < 8 && (nvec + vpt - 1) / vpt > (vpt * E > 32 ? 256 : (vpt * E > 16 ? 512 : 1024))) vpt *= 2;
        // a CTA of whole warps that covers the row exactly runs without predicates: worth fewer vectors per thread
        // (a 768-wide 16-bit row: 96 threads x 1 vector measured 35 % faster than 64 threads x 2 with a third of them idle)
        if (nvec % (32LL * vpt) != 0)
            for (int v = vpt / 2; v >= 1; v /= 2)
                if (nvec % (32LL * v) == 0 && nvec / v <= (v * E > 32 ? 256 : (v * E > 16 ? 512 : 1024))) { vpt = v; break; }
    }
    if (vpt != 1 && vpt != 2 && vpt != 4 && vpt != 8)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: vecs_per_thread must be 1, 2, 4 or 8 (got %d)", what, vpt);
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
    const bool full = static_cast<int64_t>(threads) * vpt == nvec;
    const size_t smem = (OP == kLayerNorm ? 2 : (OP == kRmsNorm ? 1 : 0)) * sizeof(float) * E * threads * vpt;
    if (smem > 200 * 1024)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: %d threads x %d vectors need %zu bytes of shared memory",
                    what, threads, vpt, smem);

    using Kernel = void (*)(const T*, const T*, const T*, T*, int64_t, int, float, const T*, T*, int64_t);
    Kernel kernel = nullptr;
    // the residual ring doubles the registers held per vector: fp32 rows take it only up to two vectors per thread
#define MHLO_ROW_PICK(V)                                                                                              \
    case V: {                                                                                                         \
        constexpr bool kAddable = OP != kSoftmax && (sizeof(T) == 2 || V <= 2);                                       \
        if (kAddable && with_add)                                                                                     \
            kernel = full ? row_vec_kernel<T, V, OP, true, kAddable> : row_vec_kernel<T, V, OP, false, kAddable>;     \
        else                                                                                                          \
            kernel = full ? row_vec_kernel<T, V, OP, true, false> : row_vec_kernel<T, V, OP, false, false>;           \
        break;                                                                                                        \
    }
    switch (vpt) {
        MHLO_ROW_PICK(1)
        MHLO_ROW_PICK(2)
        MHLO_ROW_PICK(4)
        MHLO_ROW_PICK(8)
    }
#undef MHLO_ROW_PICK
    if (smem + 1024 > 48 * 1024)
        MHLO_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                      MHLO_CUDA_EXECUTION_FAILED);
    int64_t grid = rows;
    if (ctas_per_sm >= 0) {
        int per_sm = ctas_per_sm;
        if (per_sm == 0) {
            MHLO_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem),
                          MHLO_CUDA_NO_DEVICE);
            // more than ~16 resident warps per SM measured slower (the rows in flight stop fitting the DRAM pages
            // the SM has open), so the occupancy bound is capped
            // (measured: 4 CTAs of 128 threads for 8 KB rows, 8 to 16 CTAs of 96 threads for 1.5 KB rows: about 64 KB of
            // rows in flight per SM with the two-row ring)
            const int64_t row_bytes = len * static_cast<int64_t>(sizeof(T));
            int64_t cap = 65536 / (kDepth * (row_bytes > 0 ? row_bytes : 1));
            cap = cap < 4 ? 4 : (cap > 16 ? 16 : cap);
            if (cap * threads > 2048) cap = 2048 / threads;
            if (per_sm > cap) per_sm = static_cast<int>(cap);
            if (per_sm < 1) per_sm = 1;
        }
        if (grid > static_cast<int64_t>(kNumSMs) * per_sm) grid = static_cast<int64_t>(kNumSMs) * per_sm;
    }
    if (grid > 0x7fffffffLL) grid = 0x7fffffffLL;
    const cudaError_t launched = launch_dependent(kernel, dim3(static_cast<unsigned>(grid)), dim3(static_cast<unsigned>(threads)), smem, stream, xp, gp, bp, yp,
                                                  rows, static_cast<int>(len), eps, static_cast<const T*>(res), static_cast<T*>(sum_out), res_rows);
    if (launched != cudaSuccess) return fail(MHLO_CUDA_EXECUTION_FAILED, "launch of %s failed: %s", what, cudaGetErrorString(launched));
    MHLO_CUDA_CHECK_LAUNCH(what);
    return MHLO_CUDA_OK;
}

template <int OP>
int dispatch_rows(int dtype, const void* x, const void* gamma, const void* beta, void* y, int64_t outer,
                  int64_t len, int64_t inner, float eps, const mhlo_cuda_row_tuning* tuning, void* stream,
                  const char* what, const void* res = nullptr, void* sum_out = nullptr, int64_t res_rows = 0) {
    if (res != nullptr && (res_rows < 0 || (res_rows > 0 && (outer * inner) % res_rows != 0)))
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: %lld residual rows do not tile %lld rows", what, (long long)res_rows, (long long)(outer * inner));
    if (outer < 0 || len < 0 || inner < 0)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: negative extent", what);
    if (outer * len * inner > 0 && (x == nullptr || y == nullptr))
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: null tensor pointer", what);
    if ((res == nullptr) != (sum_out == nullptr))
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: the residual operand and the sum output go together", what);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case MHLO_DT_F32:
            return launch_rows<float, OP>(x, gamma, beta, y, outer, len, inner, eps, tuning, s, what, res, sum_out, res_rows);
        case MHLO_DT_F16:
            return launch_rows<__half, OP>(x, gamma, beta, y, outer, len, inner, eps, tuning, s, what, res, sum_out, res_rows);
        case MHLO_DT_BF16:
            return launch_rows<__nv_bfloat16, OP>(x, gamma, beta, y, outer, len, inner, eps, tuning, s, what, res, sum_out, res_rows);
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

int mhlo_cuda_add_layer_norm(int dtype, const void* x_dev, const void* residual_dev, const void* gamma_dev, const void* beta_dev,
                             void* sum_dev, void* y_dev, int64_t rows, int64_t hidden, float eps, const mhlo_cuda_row_tuning* tuning,
                             mhlo_cuda_stream_t stream) {
    if (rows * hidden > 0 && (residual_dev == nullptr || sum_dev == nullptr))
        return mhlo::fail(MHLO_CUDA_INVALID_ARGUMENT, "add_layer_norm: null residual or sum pointer");
    return mhlo::dispatch_rows<mhlo::kLayerNorm>(dtype, x_dev, gamma_dev, beta_dev, y_dev, rows, hidden, 1, eps, tuning, stream,
                                                 "add_layer_norm", residual_dev, sum_dev);
}

int mhlo_cuda_add_layer_norm_rows(int dtype, const void* x_dev, const void* residual_dev, int64_t residual_rows, const void* gamma_dev,
                                  const void* beta_dev, void* sum_dev, void* y_dev, int64_t rows, int64_t hidden, float eps,
                                  const mhlo_cuda_row_tuning* tuning, mhlo_cuda_stream_t stream) {
    if (rows * hidden > 0 && (residual_dev == nullptr || sum_dev == nullptr))
        return mhlo::fail(MHLO_CUDA_INVALID_ARGUMENT, "add_layer_norm: null residual or sum pointer");
    return mhlo::dispatch_rows<mhlo::kLayerNorm>(dtype, x_dev, gamma_dev, beta_dev, y_dev, rows, hidden, 1, eps, tuning, stream,
                                                 "add_layer_norm", residual_dev, sum_dev, residual_rows);
}

int mhlo_cuda_add_rms_norm_rows(int dtype, const void* x_dev, const void* residual_dev, int64_t residual_rows, const void* gamma_dev, void* sum_dev,
                                void* y_dev, int64_t rows, int64_t hidden, float eps, const mhlo_cuda_row_tuning* tuning,
                                mhlo_cuda_stream_t stream) {
    if (rows * hidden > 0 && (residual_dev == nullptr || sum_dev == nullptr))
        return mhlo::fail(MHLO_CUDA_INVALID_ARGUMENT, "add_rms_norm: null residual or sum pointer");
    return mhlo::dispatch_rows<mhlo::kRmsNorm>(dtype, x_dev, gamma_dev, nullptr, y_dev, rows, hidden, 1, eps, tuning, stream,
                                               "add_rms_norm", residual_dev, sum_dev, residual_rows);
}

int mhlo_cuda_add_rms_norm(int dtype, const void* x_dev, const void* residual_dev, const void* gamma_dev, void* sum_dev, void* y_dev,
                           int64_t rows, int64_t hidden, float eps, const mhlo_cuda_row_tuning* tuning, mhlo_cuda_stream_t stream) {
    if (rows * hidden > 0 && (residual_dev == nullptr || sum_dev == nullptr))
        return mhlo::fail(MHLO_CUDA_INVALID_ARGUMENT, "add_rms_norm: null residual or sum pointer");
    return mhlo::dispatch_rows<mhlo::kRmsNorm>(dtype, x_dev, gamma_dev, nullptr, y_dev, rows, hidden, 1, eps, tuning, stream,
                                               "add_rms_norm", residual_dev, sum_dev);
}

int mhlo_cuda_softmax(int dtype, const void* x_dev, void* y_dev, int64_t outer, int64_t axis_len, int64_t inner,
                      const mhlo_cuda_row_tuning* tuning, mhlo_cuda_stream_t stream) {
    return mhlo::dispatch_rows<mhlo::kSoftmax>(dtype, x_dev, nullptr, nullptr, y_dev, outer, axis_len, inner, 0.f,
                                               tuning, stream, "softmax");
}

}  // extern "C"
