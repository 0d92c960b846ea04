// Shared device/host helpers of libmhlo_cuda.so: status plumbing, dtype traits, 128-bit streaming
// loads/stores and warp/CTA reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/mhlo_cuda.h"

namespace mhlo {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

// Records a printf-style message for mhlo_cuda_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
void clear_error();

// Turns a CUDA runtime error into a status code with the failing call recorded.
#define MHLO_CUDA_TRY(expr, code)                                                                \
    do {                                                                                         \
        cudaError_t _e = (expr);                                                                 \
        if (_e != cudaSuccess)                                                                   \
            return ::mhlo::fail((code), "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),  \
                                __FILE__, __LINE__);                                             \
    } while (0)

// Checks the launch that was just enqueued. A missing device or a wrong-arch build shows up here.
#define MHLO_CUDA_CHECK_LAUNCH(what)                                                             \
    do {                                                                                         \
        cudaError_t _e = cudaGetLastError();                                                     \
        if (_e != cudaSuccess) {                                                                 \
            int _c = (_e == cudaErrorNoDevice || _e == cudaErrorInsufficientDriver)              \
                         ? MHLO_CUDA_NO_DEVICE                                                   \
                         : MHLO_CUDA_EXECUTION_FAILED;                                           \
            return ::mhlo::fail(_c, "launch of %s failed: %s", (what), cudaGetErrorString(_e));  \
        }                                                                                        \
    } while (0)

// Division of n < 2^31 by a divisor fixed at launch: one multiply-high and a shift instead of the ~20 instructions of
// a 32-bit division. mul = ceil(2^(31+s) / d) with s = ceil(log2 d) fits 32 bits, and floor(n * mul / 2^(31+s)) equals
// floor(n / d) because the rounding error of mul contributes less than 2^-s <= 1/d.
struct FastDiv {
    uint32_t mul = 0, shift = 0, d = 1;
    FastDiv() = default;
    explicit FastDiv(uint32_t divisor) : d(divisor < 1 ? 1 : divisor) {
        if (d > 1) {
            uint32_t s = 0;
            while ((uint64_t{1} << s) < d) ++s;
            shift = s - 1;
            mul = static_cast<uint32_t>(((uint64_t{1} << (31 + s)) + d - 1) / d);
        }
    }
    __host__ __device__ __forceinline__ uint32_t div(uint32_t n) const {
#ifdef __CUDA_ARCH__
        return d == 1 ? n : (__umulhi(n, mul) >> shift);
#else
        return d == 1 ? n : static_cast<uint32_t>((static_cast<uint64_t>(n) * mul) >> 32) >> shift;
#endif
    }
    __host__ __device__ __forceinline__ void divmod(uint32_t n, uint32_t* q, uint32_t* r) const {
        *q = div(n);
        *r = n - *q * d;
    }
};

// Programmatic dependent launch: a kernel launched through launch_dependent() may start while its predecessor in the
// stream is still running; it must call grid_dependency_wait() before it touches global memory the predecessor writes
// (or reads something the predecessor may still be reading before overwriting it). grid_dependency_release() lets the
// next kernel of the stream begin its own prologue. Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// METALHLO_PDL=0 turns the overlap off (every launch then waits for the previous kernel to finish, as usual).
bool dependent_launch_enabled();

// Launches `kernel`, which calls grid_dependency_wait(), with the programmatic-serialisation attribute when enabled.
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent_launch_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel that runs as thread-block clusters of `cluster_x` CTAs along x (1 = no cluster attribute).
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_x,
                                     Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (dependent_launch_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = static_cast<unsigned>(cluster_x);
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- 16-byte vectors of T <-> fp32 ------------------------------------------------------------------

template <typename T>
struct VecTraits;

template <>
struct VecTraits<float> {
    static constexpr int kElems = 4;
    __device__ __forceinline__ static void unpack(const uint4& v, float* f) {
        f[0] = __uint_as_float(v.x);
        f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z);
        f[3] = __uint_as_float(v.w);
    }
    __device__ __forceinline__ static uint4 pack(const float* f) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                          __float_as_uint(f[3]));
    }
    __device__ __forceinline__ static void unpack2(const uint4& v, float2* f) {
        f[0] = make_float2(__uint_as_float(v.x), __uint_as_float(v.y));
        f[1] = make_float2(__uint_as_float(v.z), __uint_as_float(v.w));
    }
    __device__ __forceinline__ static uint4 pack2(const float2* f) {
        return make_uint4(__float_as_uint(f[0].x), __float_as_uint(f[0].y), __float_as_uint(f[1].x),
                          __float_as_uint(f[1].y));
    }
    __device__ __forceinline__ static float to_float(float x) { return x; }
    __device__ __forceinline__ static float from_float(float x) { return x; }
};

template <>
struct VecTraits<__nv_bfloat16> {
    static constexpr int kElems = 8;
    __device__ __forceinline__ static void unpack(const uint4& v, float* f) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ __forceinline__ static uint4 pack(const float* f) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&p);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ __forceinline__ static void unpack2(const uint4& v, float2* f) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
            f[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
    }
    __device__ __forceinline__ static uint4 pack2(const float2* f) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 p = __float22bfloat162_rn(f[i]);
            w[i] = *reinterpret_cast<uint32_t*>(&p);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ __forceinline__ static float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
    __device__ __forceinline__ static __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};

template <>
struct VecTraits<__half> {
    static constexpr int kElems = 8;
    __device__ __forceinline__ static void unpack(const uint4& v, float* f) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            f[2 * i] = p.x;
            f[2 * i + 1] = p.y;
        }
    }
    __device__ __forceinline__ static uint4 pack(const float* f) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 p = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&p);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ __forceinline__ static void unpack2(const uint4& v, float2* f) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    }
    __device__ __forceinline__ static uint4 pack2(const float2* f) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 p = __float22half2_rn(f[i]);
            w[i] = *reinterpret_cast<uint32_t*>(&p);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ __forceinline__ static float to_float(__half x) { return __half2float(x); }
    __device__ __forceinline__ static __half from_float(float x) { return __float2half_rn(x); }
};

// Streaming 128-bit global access: the row kernels touch every byte once, so they bypass L1 on the way
// in and mark stores evict-first on the way out.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream16(void* p, const uint4& v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}

// ---- reductions --------------------------------------------------------------------------------------

struct SumOp {
    __device__ __forceinline__ static float apply(float a, float b) { return a + b; }
    __device__ __forceinline__ static float identity() { return 0.f; }
};
struct MaxOp {
    __device__ __forceinline__ static float apply(float a, float b) { return fmaxf(a, b); }
    __device__ __forceinline__ static float identity() { return -INFINITY; }
};

template <typename Op>
__device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// All-reduce over the CTA. `scratch` is 32 floats of shared memory that the caller alternates between
// consecutive reductions, so one __syncthreads() per reduction is enough. With a single warp no shared
// memory is touched.
template <typename Op>
__device__ __forceinline__ float cta_reduce(float v, float* scratch) {
    v = warp_reduce<Op>(v);
    const int nwarps = blockDim.x >> 5;
    if (nwarps == 1) return v;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = lane < nwarps ? scratch[lane] : Op::identity();
    return warp_reduce<Op>(r);
}

}  // namespace mhlo
