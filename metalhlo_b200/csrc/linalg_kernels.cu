// stablehlo.cholesky and stablehlo.triangular_solve: small dense factorisations and solves as jax.numpy.linalg emits them;
// stablehlo.rng_bit_generator: counter-mode Threefry-2x32 (the last section of this file).
// One CTA per matrix (Cholesky) or per block of right-hand sides (triangular solve); fp32 arithmetic for f32 / f16 / bf16
// tensors, fp64 for f64. These are correctness kernels for matrices of up to a few thousand rows, not tuned: the work is
// O(n^3) with one column (or one substitution step) after the other. The reference lowers both through MPSGraph
// (Sources/MetalHLOCore/Compiler/MPSGraphCompiler.swift), a route this backend does not have.
#include "common.cuh"

#include <cuda_bf16.h>
#include <type_traits>
#include <cuda_fp16.h>

namespace mhlo {
namespace {

template <typename T> struct Compute { using type = float; };
template <> struct Compute<double> { using type = double; };

template <typename T> __device__ __forceinline__ typename Compute<T>::type ld(const T* p) { return static_cast<typename Compute<T>::type>(*p); }
template <> __device__ __forceinline__ float ld<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void st(T* p, typename Compute<T>::type v) { *p = static_cast<T>(v); }
template <> __device__ __forceinline__ void st<__half>(__half* p, float v) { *p = __float2half_rn(v); }
template <> __device__ __forceinline__ void st<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// A = L L^T (lower) or U^T U (upper), column by column (left-looking). The factor is written to `out`, the other triangle
// is set to zero. Element (i, j) of the lower factor lives at out[i*n + j]; of the upper factor at out[j*n + i].
template <typename T>
__global__ void cholesky_kernel(const T* __restrict__ a, T* __restrict__ out, int64_t n, int lower) {
    using C = typename Compute<T>::type;
    const T* am = a + static_cast<int64_t>(blockIdx.x) * n * n;
    T* lm = out + static_cast<int64_t>(blockIdx.x) * n * n;
    auto L = [&](int64_t i, int64_t j) -> T* { return lower ? lm + i * n + j : lm + j * n + i; };
    auto A = [&](int64_t i, int64_t j) -> const T* { return lower ? am + i * n + j : am + j * n + i; };
    __shared__ C diag;
    for (int64_t j = 0; j < n; ++j) {
        // every row i >= j: s_i = a_ij - sum_{k<j} L_ik L_jk (the factor's earlier columns are final and visible after the barrier)
        for (int64_t i = j + threadIdx.x; i < n; i += blockDim.x) {
            C s = ld(A(i, j));
            for (int64_t k = 0; k < j; ++k) s -= ld(L(i, k)) * ld(L(j, k));
            if (i == j) {
                s = sqrt(s);  // a matrix that is not positive definite gives NaN from here on, as LAPACK-style kernels do
                diag = s;
            }
            st(L(i, j), s);
        }
        __syncthreads();
        const C d = diag;
        for (int64_t i = j + 1 + threadIdx.x; i < n; i += blockDim.x) st(L(i, j), ld(L(i, j)) / d);
        for (int64_t i = threadIdx.x; i < j; i += blockDim.x) st(L(i, j), C(0));  // the other triangle
        __syncthreads();
    }
}

// Solves T x = b for one right-hand side per thread, T = op(a) read through `at(i, k)`; forward when T is lower
// triangular, backward otherwise. x is accumulated in `out`, whose element (row i of the unknown, this thread's column) is
// at xo(i).
struct SolveParams {
    int64_t m, n;          // a is m x m; there are n right-hand sides
    int32_t left_side, lower, unit_diagonal, transpose_a;
};

template <typename T>
__global__ void triangular_solve_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, SolveParams p) {
    using C = typename Compute<T>::type;
    const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;  // which right-hand side
    if (c >= p.n) return;
    const int64_t batch = blockIdx.y;
    const T* am = a + batch * p.m * p.m;
    const int64_t bsz = p.m * p.n;
    const T* bm = b + batch * bsz;
    T* xm = out + batch * bsz;
    // left side:  op(a) X = B, B is [m, n], column c.     right side: X op(a) = B, B is [n, m], row c: op(a)^T x^T = b^T.
    const bool transposed = (p.transpose_a != 0) != (p.left_side == 0);
    const bool eff_lower = (p.lower != 0) != transposed;
    auto at = [&](int64_t i, int64_t k) -> C { return transposed ? ld(am + k * p.m + i) : ld(am + i * p.m + k); };
    auto idx = [&](int64_t i) -> int64_t { return p.left_side ? i * p.n + c : c * p.m + i; };
    if (eff_lower) {
        for (int64_t i = 0; i < p.m; ++i) {
            C s = ld(bm + idx(i));
            for (int64_t k = 0; k < i; ++k) s -= at(i, k) * ld(xm + idx(k));
            st(xm + idx(i), p.unit_diagonal ? s : s / at(i, i));
        }
    } else {
        for (int64_t i = p.m - 1; i >= 0; --i) {
            C s = ld(bm + idx(i));
            for (int64_t k = i + 1; k < p.m; ++k) s -= at(i, k) * ld(xm + idx(k));
            st(xm + idx(i), p.unit_diagonal ? s : s / at(i, i));
        }
    }
}

template <typename T>
int launch_cholesky(const void* a, void* out, int64_t batch, int64_t n, int lower, cudaStream_t s) {
    cholesky_kernel<T><<<static_cast<unsigned>(batch), 256, 0, s>>>(static_cast<const T*>(a), static_cast<T*>(out), n, lower);
    MHLO_CUDA_CHECK_LAUNCH("cholesky");
    return MHLO_CUDA_OK;
}

template <typename T>
int launch_solve(const void* a, const void* b, void* out, int64_t batch, const SolveParams& p, cudaStream_t s) {
    const dim3 grid(static_cast<unsigned>((p.n + 127) / 128), static_cast<unsigned>(batch));
    triangular_solve_kernel<T><<<grid, 128, 0, s>>>(static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), p);
    MHLO_CUDA_CHECK_LAUNCH("triangular_solve");
    return MHLO_CUDA_OK;
}

}  // namespace
}  // namespace mhlo

using namespace mhlo;

// Threefry-2x32 with 20 rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3"), the generator behind
// jax.random: key (k0, k1), counter (x0, x1) -> two 32-bit words.
__device__ __forceinline__ void threefry2x32(uint32_t k0, uint32_t k1, uint32_t& x0, uint32_t& x1) {
    const uint32_t ks[3] = {k0, k1, k0 ^ k1 ^ 0x1BD11BDAu};
    const int rot[8] = {13, 15, 26, 6, 17, 29, 16, 24};
    x0 += ks[0];
    x1 += ks[1];
#pragma unroll
    for (int g = 0; g < 5; ++g) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            x0 += x1;
            x1 = __funnelshift_l(x1, x1, rot[4 * (g & 1) + r]) ^ x0;
        }
        x0 += ks[(g + 1) % 3];
        x1 += ks[(g + 2) % 3] + static_cast<uint32_t>(g + 1);
    }
}

// One thread per block of two words. Elements of 32 bits or fewer take one word each (its low bits), 64-bit elements both
// words of a block (first word low). state = {key, counter}; the new counter is written by thread 0.
__global__ void rng_bits_kernel(const uint64_t* __restrict__ state, uint64_t* __restrict__ new_state, void* __restrict__ out, int64_t count,
                                int32_t elem_bytes, int64_t blocks) {
    const int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t key = state[0], ctr = state[1];
    if (b == 0) {
        new_state[0] = key;
        new_state[1] = ctr + static_cast<uint64_t>(blocks);
    }
    if (b >= blocks) return;
    const uint64_t c = ctr + static_cast<uint64_t>(b);
    uint32_t x0 = static_cast<uint32_t>(c), x1 = static_cast<uint32_t>(c >> 32);
    threefry2x32(static_cast<uint32_t>(key), static_cast<uint32_t>(key >> 32), x0, x1);
    if (elem_bytes == 8) {
        static_cast<uint64_t*>(out)[b] = static_cast<uint64_t>(x0) | (static_cast<uint64_t>(x1) << 32);
        return;
    }
    const uint32_t w[2] = {x0, x1};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int64_t e = 2 * b + i;
        if (e >= count) break;
        if (elem_bytes == 4) static_cast<uint32_t*>(out)[e] = w[i];
        else if (elem_bytes == 2) static_cast<uint16_t*>(out)[e] = static_cast<uint16_t>(w[i]);
        else static_cast<uint8_t*>(out)[e] = static_cast<uint8_t>(w[i]);
    }
}

// stablehlo.rng: `count` values drawn from the stream of state = {key, counter} (the state stays where it is; a second,
// one-thread kernel advances its counter behind the draw, so that every execution - a graph replay included - continues the
// stream). UNIFORM floats: a + (b - a) * u with u = the word's top 24 bits / 2^24 in [0, 1); UNIFORM integers: a + word mod
// (b - a); NORMAL: Box-Muller on the two words of a pair, a + b * z.
template <typename T>
__global__ void rng_kernel(const uint64_t* __restrict__ state, const T* __restrict__ a_ptr, const T* __restrict__ b_ptr, T* __restrict__ out,
                           int64_t count, int32_t normal) {
    const int64_t blk = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (2 * blk >= count) return;
    const uint64_t key = state[0], c = state[1] + static_cast<uint64_t>(blk);
    uint32_t x0 = static_cast<uint32_t>(c), x1 = static_cast<uint32_t>(c >> 32);
    threefry2x32(static_cast<uint32_t>(key), static_cast<uint32_t>(key >> 32), x0, x1);
    const uint32_t w[2] = {x0, x1};
    if constexpr (std::is_integral<T>::value) {
        const int64_t lo = static_cast<int64_t>(*a_ptr), hi = static_cast<int64_t>(*b_ptr);
        const uint64_t span = hi > lo ? static_cast<uint64_t>(hi - lo) : 1;
#pragma unroll
        for (int i = 0; i < 2; ++i)
            if (2 * blk + i < count) out[2 * blk + i] = static_cast<T>(lo + static_cast<int64_t>((static_cast<uint64_t>(w[i]) | (static_cast<uint64_t>(w[1 - i]) << 32)) % span));
    } else {
        const float a = static_cast<float>(ld(a_ptr)), b = static_cast<float>(ld(b_ptr));
        float v[2];
        if (normal) {
            const float u1 = (static_cast<float>(w[0] >> 8) + 1.0f) * (1.0f / 16777216.0f);  // (0, 1]
            const float u2 = static_cast<float>(w[1] >> 8) * (1.0f / 16777216.0f);
            const float r = sqrtf(-2.0f * logf(u1));
            float sn, cs;
            sincospif(2.0f * u2, &sn, &cs);
            v[0] = a + b * r * cs;
            v[1] = a + b * r * sn;
        } else {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float u = static_cast<float>(w[i] >> 8) * (1.0f / 16777216.0f);
                float x = a + (b - a) * u;
                // rounding (of the product, or of the result to a 16-bit type) may reach the open end of the interval
                T rounded;
                st(&rounded, static_cast<typename Compute<T>::type>(x));
                if (!(static_cast<float>(ld(&rounded)) < b) && b > a) x = a;
                v[i] = x;
            }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
            if (2 * blk + i < count) st(out + 2 * blk + i, v[i]);
    }
}

__global__ void rng_advance_kernel(uint64_t* state, uint64_t blocks) { state[1] += blocks; }

template <typename T>
int launch_rng(uint64_t* state, const void* a, const void* b, void* out, int64_t count, int normal, cudaStream_t s) {
    const int64_t blocks = (count + 1) / 2;
    if (blocks > 0) {
        rng_kernel<T><<<static_cast<unsigned>((blocks + 255) / 256), 256, 0, s>>>(state, static_cast<const T*>(a), static_cast<const T*>(b),
                                                                                 static_cast<T*>(out), count, normal);
        MHLO_CUDA_CHECK_LAUNCH("rng");
    }
    rng_advance_kernel<<<1, 1, 0, s>>>(state, static_cast<uint64_t>(blocks));
    MHLO_CUDA_CHECK_LAUNCH("rng state");
    return MHLO_CUDA_OK;
}

extern "C" {

int mhlo_cuda_rng(int32_t dtype, int32_t distribution, void* state_dev, const void* a_dev, const void* b_dev, void* out_dev, int64_t count,
                  mhlo_cuda_stream_t stream) {
    if (count < 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "rng: negative count");
    if (distribution != 0 && distribution != 1) return fail(MHLO_CUDA_INVALID_ARGUMENT, "rng: distribution %d (0 uniform, 1 normal)", distribution);
    if (!state_dev || !a_dev || !b_dev || (count > 0 && !out_dev)) return fail(MHLO_CUDA_INVALID_ARGUMENT, "rng: null pointer");
    uint64_t* st = static_cast<uint64_t*>(state_dev);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case MHLO_DT_F32: return launch_rng<float>(st, a_dev, b_dev, out_dev, count, distribution, s);
        case MHLO_DT_F64: return launch_rng<double>(st, a_dev, b_dev, out_dev, count, distribution, s);
        case MHLO_DT_F16: return launch_rng<__half>(st, a_dev, b_dev, out_dev, count, distribution, s);
        case MHLO_DT_BF16: return launch_rng<__nv_bfloat16>(st, a_dev, b_dev, out_dev, count, distribution, s);
        default: break;
    }
    if (distribution == 1) return fail(MHLO_CUDA_UNSUPPORTED, "rng: a normal distribution of dtype %d", dtype);
    switch (dtype) {
        case MHLO_DT_I32: return launch_rng<int32_t>(st, a_dev, b_dev, out_dev, count, 0, s);
        case MHLO_DT_I64: return launch_rng<int64_t>(st, a_dev, b_dev, out_dev, count, 0, s);
        case MHLO_DT_UI32: return launch_rng<uint32_t>(st, a_dev, b_dev, out_dev, count, 0, s);
        case MHLO_DT_UI64: return launch_rng<uint64_t>(st, a_dev, b_dev, out_dev, count, 0, s);
        case MHLO_DT_I8: return launch_rng<int8_t>(st, a_dev, b_dev, out_dev, count, 0, s);
        case MHLO_DT_I16: return launch_rng<int16_t>(st, a_dev, b_dev, out_dev, count, 0, s);
        case MHLO_DT_UI8: return launch_rng<uint8_t>(st, a_dev, b_dev, out_dev, count, 0, s);
        case MHLO_DT_UI16: return launch_rng<uint16_t>(st, a_dev, b_dev, out_dev, count, 0, s);
        default: return fail(MHLO_CUDA_UNSUPPORTED, "rng: dtype %d", dtype);
    }
}

int mhlo_cuda_rng_bit_generator(const void* state_dev, void* new_state_dev, void* out_dev, int64_t count, int32_t elem_bytes,
                                mhlo_cuda_stream_t stream) {
    if (count < 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "rng_bit_generator: negative count");
    if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "rng_bit_generator: elements of %d bytes", elem_bytes);
    if (!state_dev || !new_state_dev || (count > 0 && !out_dev)) return fail(MHLO_CUDA_INVALID_ARGUMENT, "rng_bit_generator: null pointer");
    if (state_dev == new_state_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "rng_bit_generator: the new state must not alias the state");
    const int64_t blocks = elem_bytes == 8 ? count : (count + 1) / 2;
    const int64_t threads = blocks > 0 ? blocks : 1;
    const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
    rng_bits_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint64_t*>(state_dev), static_cast<uint64_t*>(new_state_dev),
                                                                         out_dev, count, elem_bytes, blocks);
    MHLO_CUDA_CHECK_LAUNCH("rng_bit_generator");
    return MHLO_CUDA_OK;
}

int mhlo_cuda_cholesky(int32_t dtype, const void* a_dev, void* out_dev, int64_t batch, int64_t n, int32_t lower, mhlo_cuda_stream_t stream) {
    if (batch < 0 || n < 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "cholesky: negative extent");
    if (batch == 0 || n == 0) return MHLO_CUDA_OK;
    if (!a_dev || !out_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "cholesky: null pointer");
    if (a_dev == out_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "cholesky: the factor must not alias the matrix");
    if (batch > 0x7fffffffLL) return fail(MHLO_CUDA_UNSUPPORTED, "cholesky: too many matrices");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case MHLO_DT_F32: return launch_cholesky<float>(a_dev, out_dev, batch, n, lower, s);
        case MHLO_DT_F64: return launch_cholesky<double>(a_dev, out_dev, batch, n, lower, s);
        case MHLO_DT_F16: return launch_cholesky<__half>(a_dev, out_dev, batch, n, lower, s);
        case MHLO_DT_BF16: return launch_cholesky<__nv_bfloat16>(a_dev, out_dev, batch, n, lower, s);
        default: return fail(MHLO_CUDA_UNSUPPORTED, "cholesky: dtype %d", dtype);
    }
}

int mhlo_cuda_triangular_solve(int32_t dtype, const void* a_dev, const void* b_dev, void* out_dev, int64_t batch, int64_t m, int64_t n,
                               int32_t left_side, int32_t lower, int32_t unit_diagonal, int32_t transpose_a, mhlo_cuda_stream_t stream) {
    if (batch < 0 || m < 0 || n < 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "triangular_solve: negative extent");
    if (batch == 0 || m == 0 || n == 0) return MHLO_CUDA_OK;
    if (!a_dev || !b_dev || !out_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "triangular_solve: null pointer");
    if (batch > 65535) return fail(MHLO_CUDA_UNSUPPORTED, "triangular_solve: more than 65535 matrices");
    SolveParams p{m, n, left_side, lower, unit_diagonal, transpose_a};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case MHLO_DT_F32: return launch_solve<float>(a_dev, b_dev, out_dev, batch, p, s);
        case MHLO_DT_F64: return launch_solve<double>(a_dev, b_dev, out_dev, batch, p, s);
        case MHLO_DT_F16: return launch_solve<__half>(a_dev, b_dev, out_dev, batch, p, s);
        case MHLO_DT_BF16: return launch_solve<__nv_bfloat16>(a_dev, b_dev, out_dev, batch, p, s);
        default: return fail(MHLO_CUDA_UNSUPPORTED, "triangular_solve: dtype %d", dtype);
    }
}

}  // extern "C"
