// stablehlo.fft: discrete Fourier transforms along one axis of a tensor of (re, im) pairs, f32 or f64. A transform over
// several axes is one launch per axis. One CTA per line: the line is staged in shared memory, transformed there and
// written back, so a pass may run in place. Lengths that are a power of two take a radix-2 Stockham autosort FFT
// (n/2 butterflies per stage, two buffers, no bit reversal); every other length takes the direct O(n^2) sum with an exact
// twiddle table, which is what the reference runs for every length (one thread per output and a loop over the line with
// cos / sin per term, Sources/MetalHLOCore/Compiler/CodeGenerator.swift:2701-2830). Correctness kernels: lines are as long
// as shared memory holds (8192 points in a power of two, 14 000 otherwise; half of that in f64); longer powers of two go
// pass by pass through global scratch (fft_pass_kernel).
#include "common.cuh"

#include <type_traits>

namespace mhlo {
namespace {

template <typename R> struct PairOf { using type = float2; };
template <> struct PairOf<double> { using type = double2; };

template <typename C> __device__ __forceinline__ C cadd(C a, C b) { return C{a.x + b.x, a.y + b.y}; }
template <typename C> __device__ __forceinline__ C csub(C a, C b) { return C{a.x - b.x, a.y - b.y}; }
template <typename C> __device__ __forceinline__ C cmul(C a, C b) { return C{a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x}; }

enum : int { kForward = 0, kInverse = 1, kRealToComplex = 2, kComplexToReal = 3 };

// Element j of line (o, i) is pair (o * n + j) * inner + i of a complex tensor [outer, n, inner]. The real side of the
// two half transforms is a dense [lines, n] tensor, their complex side [lines, n/2 + 1] pairs (inner = 1 for both).
template <typename R, bool POW2>
__global__ void __launch_bounds__(256) fft_lines_kernel(const R* in, R* out,  // may alias: a pass between complex tensors runs in place
                                                         int64_t lines, int64_t inner, int n, int kind) {
    using C = typename PairOf<R>::type;
    extern __shared__ __align__(16) unsigned char fft_smem[];
    C* a = reinterpret_cast<C*>(fft_smem);
    C* b = a + n;                    // second Stockham buffer (POW2 only)
    C* w = POW2 ? b + n : a + n;     // exp(-+2 pi i k / n): k < n/2 for the FFT, k < n for the direct sum
    const bool inverse = kind == kInverse || kind == kComplexToReal;
    const int half = n / 2 + 1;
    const int tid = threadIdx.x, nt = blockDim.x;
    for (int k = tid; k < (POW2 ? n / 2 : n); k += nt) {
        double s, c;
        sincospi(2.0 * static_cast<double>(k) / static_cast<double>(n), &s, &c);
        w[k] = C{static_cast<R>(c), static_cast<R>(inverse ? s : -s)};
    }
    const R scale = inverse ? R(1) / static_cast<R>(n) : R(1);
    const C* cin = reinterpret_cast<const C*>(in);
    C* cout = reinterpret_cast<C*>(out);
    for (int64_t line = blockIdx.x; line < lines; line += gridDim.x) {
        const int64_t o = line / inner, i = line - o * inner;
        __syncthreads();  // the previous line's result has been read out of `a` / `b`; the table is complete
        if (kind == kRealToComplex) {
            for (int j = tid; j < n; j += nt) a[j] = C{in[line * n + j], R(0)};
        } else if (kind == kComplexToReal) {
            // the missing half of the spectrum is the conjugate mirror of the given one; the imaginary parts of the
            // zero and the Nyquist bin drop out of the real part of the result
            for (int j = tid; j < n; j += nt) {
                if (j < half) {
                    a[j] = cin[line * half + j];
                } else {
                    const C v = cin[line * half + (n - j)];
                    a[j] = C{v.x, -v.y};
                }
            }
        } else {
            for (int j = tid; j < n; j += nt) a[j] = cin[(o * n + j) * inner + i];
        }
        __syncthreads();
        const int wanted = kind == kRealToComplex ? half : n;  // outputs to produce
        if (POW2) {
            C* x = a;
            C* y = b;
            int log_s = 0;
            for (int len = n; len > 1; len >>= 1, ++log_s) {
                const int m = len >> 1, s = 1 << log_s;
                for (int t = tid; t < n / 2; t += nt) {
                    const int p = t >> log_s, q = t & (s - 1);
                    const C u = x[q + s * p], v = x[q + s * (p + m)];
                    y[q + s * (2 * p)] = cadd(u, v);
                    y[q + s * (2 * p + 1)] = cmul(csub(u, v), w[p << log_s]);
                }
                __syncthreads();
                C* swap = x;
                x = y;
                y = swap;
            }
            for (int k = tid; k < wanted; k += nt) {
                const C r = x[k];
                if (kind == kComplexToReal) out[line * n + k] = r.x * scale;
                else if (kind == kRealToComplex) cout[line * half + k] = r;
                else cout[(o * n + k) * inner + i] = C{r.x * scale, r.y * scale};
            }
        } else {
            for (int k = tid; k < wanted; k += nt) {
                C acc = C{R(0), R(0)};
                int idx = 0;  // (j * k) mod n
                for (int j = 0; j < n; ++j) {
                    acc = cadd(acc, cmul(a[j], w[idx]));
                    idx += k;
                    if (idx >= n) idx -= n;
                }
                if (kind == kComplexToReal) out[line * n + k] = acc.x * scale;
                else if (kind == kRealToComplex) cout[line * half + k] = acc;
                else cout[(o * n + k) * inner + i] = C{acc.x * scale, acc.y * scale};
            }
        }
    }
}

// Lines too long for shared memory (powers of two only): the same radix-2 Stockham passes, one launch per pass, between
// two scratch buffers in global memory laid out [line][n]. The first pass reads the operand in its own layout (strided
// complex lines, real lines, or half spectra completed by their conjugate mirror), the last one writes the result's.
template <typename R>
__global__ void __launch_bounds__(256) fft_pass_kernel(const R* src, R* dst, int64_t lines, int64_t inner, int n, int log_s, int kind, int first, int last) {
    using C = typename PairOf<R>::type;
    const bool inverse = kind == kInverse || kind == kComplexToReal;
    const int half = n / 2 + 1;
    const int64_t total = lines * (n / 2);
    const C* csrc = reinterpret_cast<const C*>(src);
    C* cdst = reinterpret_cast<C*>(dst);
    for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < total; g += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t line = g / (n / 2);
        const int t = static_cast<int>(g - line * (n / 2));
        const int64_t o = line / inner, i = line - o * inner;
        const int s = 1 << log_s, m = n >> (log_s + 1);
        const int p = t >> log_s, q = t & (s - 1);
        auto load = [&](int e) -> C {
            if (!first) return csrc[line * n + e];
            if (kind == kRealToComplex) return C{src[line * n + e], R(0)};
            if (kind == kComplexToReal) {
                if (e < half) return csrc[line * half + e];
                const C v = csrc[line * half + (n - e)];
                return C{v.x, -v.y};
            }
            return csrc[(o * n + e) * inner + i];
        };
        const C u = load(q + s * p), v = load(q + s * (p + m));
        double sn, cs;
        sincospi(2.0 * static_cast<double>(static_cast<int64_t>(p) << log_s) / static_cast<double>(n), &sn, &cs);
        const C w = C{static_cast<R>(cs), static_cast<R>(inverse ? sn : -sn)};
        const C r0 = cadd(u, v), r1 = cmul(csub(u, v), w);
        const R scale = inverse ? R(1) / static_cast<R>(n) : R(1);
        auto store = [&](int e, C r) {
            if (!last) { cdst[line * n + e] = r; return; }
            if (kind == kComplexToReal) dst[line * n + e] = r.x * scale;
            else if (kind == kRealToComplex) { if (e < half) cdst[line * half + e] = r; }
            else cdst[(o * n + e) * inner + i] = C{r.x * scale, r.y * scale};
        };
        store(q + s * (2 * p), r0);
        store(q + s * (2 * p + 1), r1);
    }
}

template <typename R>
int launch_fft_passes(int kind, const void* in, void* out, void* scratch, int64_t outer, int64_t n, int64_t inner, cudaStream_t stream) {
    const int64_t lines = outer * inner;
    if (lines == 0) return MHLO_CUDA_OK;
    int stages = 0;
    while ((int64_t{1} << stages) < n) ++stages;
    R* buf[2] = {static_cast<R*>(scratch), static_cast<R*>(scratch) + 2 * lines * n};
    const int64_t total = lines * (n / 2);
    const int64_t grid = (total + 255) / 256 < 148 * 32 ? (total + 255) / 256 : 148 * 32;
    const R* src = static_cast<const R*>(in);
    for (int st = 0; st < stages; ++st) {
        const bool first = st == 0, last = st == stages - 1;
        R* dst = last ? static_cast<R*>(out) : buf[st & 1];
        fft_pass_kernel<R><<<static_cast<unsigned>(grid), 256, 0, stream>>>(src, dst, lines, inner, static_cast<int>(n), st, kind, first, last);
        MHLO_CUDA_CHECK_LAUNCH("fft (pass)");
        src = dst;
    }
    return MHLO_CUDA_OK;
}

// Whether a line of n points fits the one-launch kernel's shared memory.
template <typename R>
bool fft_line_fits(int64_t n) {
    const bool pow2 = (n & (n - 1)) == 0;
    const size_t pair = 2 * sizeof(R);
    const size_t smem = pow2 ? pair * static_cast<size_t>(n) * 2 + pair * static_cast<size_t>(n / 2 ? n / 2 : 1) : pair * static_cast<size_t>(n) * 2;
    return smem <= 227 * 1024;
}

template <typename R>
int launch_fft(int kind, const void* in, void* out, int64_t outer, int64_t n, int64_t inner, cudaStream_t stream) {
    const bool pow2 = (n & (n - 1)) == 0;
    const size_t pair = 2 * sizeof(R);
    const size_t smem = pow2 ? pair * static_cast<size_t>(n) * 2 + pair * static_cast<size_t>(n / 2 ? n / 2 : 1) : pair * static_cast<size_t>(n) * 2;
    if (smem > 227 * 1024)
        return fail(MHLO_CUDA_UNSUPPORTED, "fft: a line of %lld points needs %zu bytes of shared memory (227 KB at most)", (long long)n, smem);
    const int64_t lines = outer * inner;
    if (lines == 0) return MHLO_CUDA_OK;
    auto kernel = pow2 ? fft_lines_kernel<R, true> : fft_lines_kernel<R, false>;
    if (smem > 48 * 1024)
        MHLO_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)), MHLO_CUDA_EXECUTION_FAILED);
    int threads = 32;
    while (threads < 256 && threads < (pow2 ? n / 2 : n)) threads *= 2;
    const int64_t grid = lines < 148 * 16 ? lines : 148 * 16;
    kernel<<<static_cast<unsigned>(grid), threads, smem, stream>>>(static_cast<const R*>(in), static_cast<R*>(out), lines, inner, static_cast<int>(n), kind);
    MHLO_CUDA_CHECK_LAUNCH("fft");
    return MHLO_CUDA_OK;
}

}  // namespace
}  // namespace mhlo

extern "C" int64_t mhlo_cuda_fft_axis_scratch_bytes(int dtype, int64_t outer, int64_t n, int64_t inner) {
    if (dtype != MHLO_DT_F32 && dtype != MHLO_DT_F64) return 0;
    const bool fits = dtype == MHLO_DT_F32 ? mhlo::fft_line_fits<float>(n) : mhlo::fft_line_fits<double>(n);
    if (fits || (n & (n - 1)) != 0 || outer <= 0 || inner <= 0) return 0;
    return 2 * outer * inner * n * 2 * (dtype == MHLO_DT_F32 ? 4 : 8);  // two buffers of [lines][n] pairs
}

extern "C" int mhlo_cuda_fft_axis_long(int dtype, int kind, const void* in_dev, void* out_dev, void* scratch_dev, int64_t outer, int64_t n,
                                       int64_t inner, mhlo_cuda_stream_t stream) {
    const int64_t need = mhlo_cuda_fft_axis_scratch_bytes(dtype, outer, n, inner);
    if (need == 0) return mhlo_cuda_fft_axis(dtype, kind, in_dev, out_dev, outer, n, inner, stream);
    if (kind < 0 || kind > 3) return mhlo::fail(MHLO_CUDA_INVALID_ARGUMENT, "fft: kind %d", kind);
    if (kind >= 2 && inner != 1) return mhlo::fail(MHLO_CUDA_INVALID_ARGUMENT, "fft: the real side of a half transform is the innermost axis (inner = %lld)", (long long)inner);
    if (n > (1 << 24)) return mhlo::fail(MHLO_CUDA_UNSUPPORTED, "fft: lines of %lld points", (long long)n);
    if (in_dev == nullptr || out_dev == nullptr || scratch_dev == nullptr) return mhlo::fail(MHLO_CUDA_INVALID_ARGUMENT, "fft: null pointer (a line of %lld points needs %lld bytes of scratch)", (long long)n, (long long)need);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == MHLO_DT_F32) return mhlo::launch_fft_passes<float>(kind, in_dev, out_dev, scratch_dev, outer, n, inner, s);
    return mhlo::launch_fft_passes<double>(kind, in_dev, out_dev, scratch_dev, outer, n, inner, s);
}

extern "C" int mhlo_cuda_fft_axis(int dtype, int kind, const void* in_dev, void* out_dev, int64_t outer, int64_t n, int64_t inner,
                                  mhlo_cuda_stream_t stream) {
    if (kind < 0 || kind > 3) return mhlo::fail(MHLO_CUDA_INVALID_ARGUMENT, "fft: kind %d (0 forward, 1 inverse, 2 real to complex, 3 complex to real)", kind);
    if (outer < 0 || inner < 0 || n < 1 || n > (1 << 20)) return mhlo::fail(MHLO_CUDA_INVALID_ARGUMENT, "fft: %lld lines of %lld points", (long long)(outer * inner), (long long)n);
    if (kind >= 2 && inner != 1) return mhlo::fail(MHLO_CUDA_INVALID_ARGUMENT, "fft: the real side of a half transform is the innermost axis (inner = %lld)", (long long)inner);
    if (outer * inner > 0 && (in_dev == nullptr || out_dev == nullptr)) return mhlo::fail(MHLO_CUDA_INVALID_ARGUMENT, "fft: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == MHLO_DT_F32) return mhlo::launch_fft<float>(kind, in_dev, out_dev, outer, n, inner, s);
    if (dtype == MHLO_DT_F64) return mhlo::launch_fft<double>(kind, in_dev, out_dev, outer, n, inner, s);
    return mhlo::fail(MHLO_CUDA_UNSUPPORTED, "fft: dtype %d (f32 and f64 parts are supported)", dtype);
}
