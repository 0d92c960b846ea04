// Operators either side of the fused hot path that need kernels of their own: reduce_window (pooling, windowed
// sums; a vector kernel for channel-last pooling and a general one), scatter and select_and_scatter (indexed updates
// with atomics) and sort (bitonic networks in shared and global memory). HBM / L2-bound integer and byte work: one
// thread per output element or 16-byte vector, or one CTA per sorted slice; grids sized in multiples of the SM count.
#include <algorithm>
#include <cstring>
#include <type_traits>

#include "common.cuh"

namespace mhlo {
namespace {

int grid_of(int64_t n, int threads) {
    const int64_t blocks = (n + threads - 1) / threads;
    const int64_t cap = static_cast<int64_t>(kNumSMs) * 16;
    return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

// Element type tags -> storage and accumulator types.
template <typename E> struct AccOf { using type = int64_t; };
template <> struct AccOf<float> { using type = float; };
template <> struct AccOf<__half> { using type = float; };
template <> struct AccOf<__nv_bfloat16> { using type = float; };
template <> struct AccOf<double> { using type = double; };
template <> struct AccOf<uint64_t> { using type = uint64_t; };

template <typename E> __device__ __forceinline__ typename AccOf<E>::type widen(E v) { return static_cast<typename AccOf<E>::type>(v); }
template <> __device__ __forceinline__ float widen<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float widen<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename E> __device__ __forceinline__ E narrow(typename AccOf<E>::type v) { return static_cast<E>(v); }
template <> __device__ __forceinline__ __half narrow<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename A>
__device__ __forceinline__ A combine(int op, A a, A b) {
    switch (op) {
        case MHLO_REDUCE_SUM: return a + b;
        case MHLO_REDUCE_PROD: return a * b;
        case MHLO_REDUCE_MAX:
            if constexpr (std::is_floating_point<A>::value) return (a != a || b != b) ? A(NAN) : (a > b ? a : b);
            else return a > b ? a : b;
        case MHLO_REDUCE_MIN:
            if constexpr (std::is_floating_point<A>::value) return (a != a || b != b) ? A(NAN) : (a < b ? a : b);
            else return a < b ? a : b;
        default:
            if constexpr (std::is_floating_point<A>::value) {
                const bool x = a != A(0), y = b != A(0);
                return A(op == MHLO_REDUCE_AND ? (x && y) : op == MHLO_REDUCE_OR ? (x || y) : (x != y));
            } else {
                return op == MHLO_REDUCE_AND ? (a & b) : op == MHLO_REDUCE_OR ? (a | b) : (a ^ b);
            }
    }
}

// Calls f(tag) with a value of the storage type of `dtype`; false for an unknown dtype. I1 is stored as a byte.
template <typename F>
bool with_element_type(int dtype, F&& f) {
    switch (dtype) {
        case MHLO_DT_F32: f(float{}); return true;
        case MHLO_DT_F16: f(__half{}); return true;
        case MHLO_DT_BF16: f(__nv_bfloat16{}); return true;
        case MHLO_DT_F64: f(double{}); return true;
        case MHLO_DT_I1: case MHLO_DT_UI8: f(uint8_t{}); return true;
        case MHLO_DT_I8: f(int8_t{}); return true;
        case MHLO_DT_I16: f(int16_t{}); return true;
        case MHLO_DT_UI16: f(uint16_t{}); return true;
        case MHLO_DT_I32: f(int32_t{}); return true;
        case MHLO_DT_UI32: f(uint32_t{}); return true;
        case MHLO_DT_I64: f(int64_t{}); return true;
        case MHLO_DT_UI64: f(uint64_t{}); return true;
        default: return false;
    }
}

int dtype_bytes(int dtype) {
    int n = 0;
    with_element_type(dtype, [&](auto tag) { n = static_cast<int>(sizeof(tag)); });
    return n;
}

// ---- reduce_window ---------------------------------------------------------------------------------------------------

struct WindowParams {
    mhlo_cuda_window w;
    int64_t in_shape[MHLO_CUDA_MAX_RANK], in_stride[MHLO_CUDA_MAX_RANK], out_shape[MHLO_CUDA_MAX_RANK];
    const void* in;
    const void* init;
    void* out;
    int64_t n_out, window_count;
    int32_t op;
};

template <typename E>
__global__ void __launch_bounds__(256) reduce_window_kernel(const __grid_constant__ WindowParams p) {
    using A = typename AccOf<E>::type;
    const int rank = p.w.rank;
    const A init = widen<E>(*static_cast<const E*>(p.init));
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t o = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; o < p.n_out; o += step) {
        int64_t origin[MHLO_CUDA_MAX_RANK];  // position of window element 0 in the dilated, unpadded operand
        int64_t rem = o;
        for (int d = rank - 1; d >= 0; --d) {
            origin[d] = (rem % p.out_shape[d]) * p.w.stride[d] - p.w.pad_low[d];
            rem /= p.out_shape[d];
        }
        A acc = init;
        int64_t wi[MHLO_CUDA_MAX_RANK];
        for (int d = 0; d < rank; ++d) wi[d] = 0;
        for (int64_t k = 0; k < p.window_count; ++k) {
            int64_t off = 0;
            bool inside = true;
            for (int d = 0; d < rank; ++d) {
                const int64_t pos = origin[d] + wi[d] * p.w.window_dilation[d];
                const int64_t bd = p.w.base_dilation[d];
                const int64_t src = pos / bd;
                inside = inside && pos >= 0 && src < p.in_shape[d] && src * bd == pos;
                off += src * p.in_stride[d];
            }
            const A v = inside ? widen<E>(static_cast<const E*>(p.in)[off]) : init;
            acc = combine<A>(p.op, acc, v);
            for (int d = rank - 1; d >= 0; --d) {  // next window coordinate, row-major
                if (++wi[d] < p.w.size[d]) break;
                wi[d] = 0;
            }
        }
        static_cast<E*>(p.out)[o] = narrow<E>(acc);
    }
}

// Pooling over the leading dimensions of a tensor whose last dimension (channels of NHWC) is contiguous and not
// windowed: one thread per 16-byte vector of channels, 32-bit index arithmetic, fp32 accumulation.
struct WindowVecParams {
    const uint4* in;
    uint4* out;
    uint32_t n_vecs, last_vecs, window_count;
    int32_t rank;  // of the windowed dimensions (the operand's rank - 1)
    uint32_t out_shape[MHLO_CUDA_MAX_RANK], in_shape[MHLO_CUDA_MAX_RANK], size[MHLO_CUDA_MAX_RANK];
    int32_t stride[MHLO_CUDA_MAX_RANK], pad_low[MHLO_CUDA_MAX_RANK], base_dilation[MHLO_CUDA_MAX_RANK], window_dilation[MHLO_CUDA_MAX_RANK];
    int64_t in_stride_vecs[MHLO_CUDA_MAX_RANK];
    const void* init;  // device scalar of the element type
    int32_t op;
};

// RANK > 0: the number of leading dimensions is known at compile time (loops unroll); 0 = read it from the parameters.
// DILATED = false promises base_dilation == 1 everywhere (no divisions in the tap loop).
template <typename T, int RANK, bool DILATED>
__global__ void __launch_bounds__(256) reduce_window_vec_kernel(const __grid_constant__ WindowVecParams p) {
    constexpr int V = VecTraits<T>::kElems;
    const int rank = RANK > 0 ? RANK : p.rank;
    const float init = widen<T>(*static_cast<const T*>(p.init));
    const uint32_t step = gridDim.x * blockDim.x;
    for (uint32_t o = blockIdx.x * blockDim.x + threadIdx.x; o < p.n_vecs; o += step) {
        const uint32_t cv = o % p.last_vecs;
        uint32_t rem = o / p.last_vecs;
        int32_t origin[MHLO_CUDA_MAX_RANK];
#pragma unroll
        for (int d = rank - 1; d >= 0; --d) {
            origin[d] = static_cast<int32_t>(rem % p.out_shape[d]) * p.stride[d] - p.pad_low[d];
            rem /= p.out_shape[d];
        }
        float acc[V];
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = init;
        uint32_t wi[MHLO_CUDA_MAX_RANK];
        for (int d = 0; d < rank; ++d) wi[d] = 0;
        for (uint32_t k = 0; k < p.window_count; ++k) {
            int64_t off = cv;
            bool inside = true;
#pragma unroll
            for (int d = 0; d < rank; ++d) {
                const int32_t pos = origin[d] + static_cast<int32_t>(wi[d]) * p.window_dilation[d];
                const int32_t src = DILATED ? pos / p.base_dilation[d] : pos;
                inside = inside && pos >= 0 && src < static_cast<int32_t>(p.in_shape[d]) && (!DILATED || src * p.base_dilation[d] == pos);
                off += src * p.in_stride_vecs[d];
            }
            float v[V];
            if (inside) {
                VecTraits<T>::unpack(__ldg(p.in + off), v);
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) v[e] = init;
            }
#pragma unroll
            for (int e = 0; e < V; ++e) acc[e] = combine<float>(p.op, acc[e], v[e]);
            for (int d = rank - 1; d >= 0; --d) {
                if (++wi[d] < p.size[d]) break;
                wi[d] = 0;
            }
        }
        p.out[o] = VecTraits<T>::pack(acc);
    }
}

// Accumulator of one 16-byte vector of a pooling window. Sums (and products) run in fp32; maximum and minimum of 16-bit
// types compare the packed pairs directly, which is exact and needs no conversion.
template <typename T, int OP, bool PACKED = (OP == MHLO_REDUCE_MAX || OP == MHLO_REDUCE_MIN) && !std::is_same<T, float>::value>
struct PoolAcc;

template <typename T, int OP>
struct PoolAcc<T, OP, false> {
    static constexpr int V = VecTraits<T>::kElems;
    float acc[V];
    float init;
    __device__ __forceinline__ void start(float i) {
        init = i;
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = i;
    }
    __device__ __forceinline__ void take(const uint4& raw) {
        float v[V];
        VecTraits<T>::unpack(raw, v);
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = combine<float>(OP, acc[e], v[e]);
    }
    __device__ __forceinline__ void take_padding() {
        if (OP == MHLO_REDUCE_MAX || OP == MHLO_REDUCE_MIN) return;  // the accumulator already dominates the init value
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = combine<float>(OP, acc[e], init);
    }
    __device__ __forceinline__ uint4 result() const { return VecTraits<T>::pack(acc); }
};

template <typename T, int OP>
struct PoolAcc<T, OP, true> {
    using T2 = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
    T2 acc[4];
    __device__ __forceinline__ void start(float i) {
        T2 v;
        if constexpr (std::is_same<T, __half>::value) v = __float2half2_rn(i); else v = __float2bfloat162_rn(i);
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = v;
    }
    __device__ __forceinline__ void take(const uint4& raw) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const T2 v = *reinterpret_cast<const T2*>(&w[e]);
            acc[e] = OP == MHLO_REDUCE_MAX ? __hmax2_nan(acc[e], v) : __hmin2_nan(acc[e], v);
        }
    }
    __device__ __forceinline__ void take_padding() {}
    __device__ __forceinline__ uint4 result() const {
        return make_uint4(*reinterpret_cast<const uint32_t*>(&acc[0]), *reinterpret_cast<const uint32_t*>(&acc[1]),
                          *reinterpret_cast<const uint32_t*>(&acc[2]), *reinterpret_cast<const uint32_t*>(&acc[3]));
    }
};

// The common pooling shape: three leading dimensions (batch, rows, columns of NHWC), no base dilation, offsets that fit
// 32 bits. The window is walked by nested loops with running offsets; divisions use precomputed reciprocals.
struct Pool3Params {
    const uint4* in;
    uint4* out;
    const void* init;
    uint32_t n_vecs;
    FastDiv by_last, by_out[3];
    int32_t in_shape[3], size[3], stride[3], pad_low[3], window_dilation[3], in_stride_vecs[3];
};

template <typename T, int OP>
__global__ void __launch_bounds__(256) pool3_vec_kernel(const __grid_constant__ Pool3Params p) {
    const float init = widen<T>(*static_cast<const T*>(p.init));
    const uint32_t step = gridDim.x * blockDim.x;
    for (uint32_t o = blockIdx.x * blockDim.x + threadIdx.x; o < p.n_vecs; o += step) {
        uint32_t rem, cv, o0, o1, o2;
        p.by_last.divmod(o, &rem, &cv);
        p.by_out[2].divmod(rem, &rem, &o2);
        p.by_out[1].divmod(rem, &o0, &o1);
        const int32_t b0 = static_cast<int32_t>(o0) * p.stride[0] - p.pad_low[0];
        const int32_t b1 = static_cast<int32_t>(o1) * p.stride[1] - p.pad_low[1];
        const int32_t b2 = static_cast<int32_t>(o2) * p.stride[2] - p.pad_low[2];
        PoolAcc<T, OP> acc;
        acc.start(init);
        for (int32_t w0 = 0, p0 = b0; w0 < p.size[0]; ++w0, p0 += p.window_dilation[0]) {
            const bool ok0 = static_cast<uint32_t>(p0) < static_cast<uint32_t>(p.in_shape[0]);
            const int32_t off0 = p0 * p.in_stride_vecs[0] + static_cast<int32_t>(cv);
            for (int32_t w1 = 0, p1 = b1; w1 < p.size[1]; ++w1, p1 += p.window_dilation[1]) {
                const bool ok1 = ok0 && static_cast<uint32_t>(p1) < static_cast<uint32_t>(p.in_shape[1]);
                const int32_t off1 = off0 + p1 * p.in_stride_vecs[1];
                for (int32_t w2 = 0, p2 = b2; w2 < p.size[2]; ++w2, p2 += p.window_dilation[2]) {
                    if (ok1 && static_cast<uint32_t>(p2) < static_cast<uint32_t>(p.in_shape[2])) acc.take(__ldg(p.in + off1 + p2 * p.in_stride_vecs[2]));
                    else acc.take_padding();
                }
            }
        }
        p.out[o] = acc.result();
    }
}

// Fills the parameters of pool3_vec_kernel from the vector parameters; false when the shape does not fit it.
bool pool3_params(const WindowVecParams& q, Pool3Params* r) {
    if (q.rank != 3) return false;
    int64_t span = q.last_vecs;
    for (int d = 0; d < 3; ++d) {
        if (q.base_dilation[d] != 1) return false;
        const int64_t st = q.in_stride_vecs[d] < 0 ? -q.in_stride_vecs[d] : q.in_stride_vecs[d];
        span += (static_cast<int64_t>(q.in_shape[d]) + q.size[d] * q.window_dilation[d] + (q.pad_low[d] < 0 ? -q.pad_low[d] : q.pad_low[d])) * st;
    }
    if (span >= (int64_t{1} << 31)) return false;
    *r = Pool3Params{};
    r->in = q.in;
    r->out = q.out;
    r->init = q.init;
    r->n_vecs = q.n_vecs;
    r->by_last = FastDiv(q.last_vecs);
    for (int d = 0; d < 3; ++d) {
        r->by_out[d] = FastDiv(q.out_shape[d]);
        r->in_shape[d] = static_cast<int32_t>(q.in_shape[d]);
        r->size[d] = static_cast<int32_t>(q.size[d]);
        r->stride[d] = q.stride[d];
        r->pad_low[d] = q.pad_low[d];
        r->window_dilation[d] = q.window_dilation[d];
        r->in_stride_vecs[d] = static_cast<int32_t>(q.in_stride_vecs[d]);
    }
    return true;
}

template <typename T>
bool launch_pool3(const Pool3Params& r, int op, int grid, cudaStream_t s) {
    switch (op) {
        case MHLO_REDUCE_SUM: pool3_vec_kernel<T, MHLO_REDUCE_SUM><<<grid, 256, 0, s>>>(r); return true;
        case MHLO_REDUCE_MAX: pool3_vec_kernel<T, MHLO_REDUCE_MAX><<<grid, 256, 0, s>>>(r); return true;
        case MHLO_REDUCE_MIN: pool3_vec_kernel<T, MHLO_REDUCE_MIN><<<grid, 256, 0, s>>>(r); return true;
        default: return false;
    }
}

bool vec_window_params(const WindowParams& p, int dtype, WindowVecParams* q) {
    const int rank = p.w.rank;
    if (rank < 2) return false;
    if (p.op != MHLO_REDUCE_SUM && p.op != MHLO_REDUCE_MAX && p.op != MHLO_REDUCE_MIN && p.op != MHLO_REDUCE_PROD) return false;
    const int64_t V = dtype == MHLO_DT_F32 ? 4 : 8;
    const int L = rank - 1;
    if (p.w.size[L] != 1 || p.w.stride[L] != 1 || p.w.pad_low[L] != 0 || p.w.base_dilation[L] != 1 || p.w.window_dilation[L] != 1) return false;
    if (p.in_stride[L] != 1 || p.in_shape[L] != p.out_shape[L] || p.in_shape[L] % V) return false;
    if (!aligned16(p.in) || !aligned16(p.out) || p.n_out / V >= (int64_t{1} << 31) || p.window_count >= (int64_t{1} << 31)) return false;
    memset(q, 0, sizeof *q);
    for (int d = 0; d < L; ++d) {
        if (p.in_stride[d] % V) return false;
        const int64_t reach = p.out_shape[d] * p.w.stride[d] + p.w.size[d] * p.w.window_dilation[d] + (p.w.pad_low[d] < 0 ? -p.w.pad_low[d] : p.w.pad_low[d]);
        if (reach >= (int64_t{1} << 30) || p.in_shape[d] >= (int64_t{1} << 30)) return false;
        q->out_shape[d] = static_cast<uint32_t>(p.out_shape[d]);
        q->in_shape[d] = static_cast<uint32_t>(p.in_shape[d]);
        q->size[d] = static_cast<uint32_t>(p.w.size[d]);
        q->stride[d] = static_cast<int32_t>(p.w.stride[d]);
        q->pad_low[d] = static_cast<int32_t>(p.w.pad_low[d]);
        q->base_dilation[d] = static_cast<int32_t>(p.w.base_dilation[d]);
        q->window_dilation[d] = static_cast<int32_t>(p.w.window_dilation[d]);
        q->in_stride_vecs[d] = p.in_stride[d] / V;
    }
    q->in = static_cast<const uint4*>(p.in);
    q->out = static_cast<uint4*>(p.out);
    q->n_vecs = static_cast<uint32_t>(p.n_out / V);
    q->last_vecs = static_cast<uint32_t>(p.in_shape[L] / V);
    q->window_count = static_cast<uint32_t>(p.window_count);
    q->rank = L;
    q->init = p.init;
    q->op = p.op;
    return true;
}

// ---- scatter ---------------------------------------------------------------------------------------------------------

struct ScatterParams {
    mhlo_cuda_scatter_dims d;
    int64_t operand_shape[MHLO_CUDA_MAX_RANK], indices_shape[MHLO_CUDA_MAX_RANK], updates_shape[MHLO_CUDA_MAX_RANK];
    void* result;
    const void* indices;
    const void* updates;
    int64_t n;
    int32_t operand_rank, indices_rank, updates_rank, index_dtype, mode;
};

// Atomic read-modify-write of one element of any width through compare-and-swap on the word that holds it.
template <typename E, typename F>
__device__ __forceinline__ void cas_update(E* addr, F f) {
    if constexpr (sizeof(E) == 8) {
        auto* a = reinterpret_cast<unsigned long long*>(addr);
        unsigned long long old = *a, assumed;
        do {
            assumed = old;
            E cur;
            memcpy(&cur, &assumed, 8);
            const E nv = f(cur);
            unsigned long long nb;
            memcpy(&nb, &nv, 8);
            old = atomicCAS(a, assumed, nb);
        } while (old != assumed);
    } else if constexpr (sizeof(E) == 4) {
        auto* a = reinterpret_cast<unsigned int*>(addr);
        unsigned int old = *a, assumed;
        do {
            assumed = old;
            E cur;
            memcpy(&cur, &assumed, 4);
            const E nv = f(cur);
            unsigned int nb;
            memcpy(&nb, &nv, 4);
            old = atomicCAS(a, assumed, nb);
        } while (old != assumed);
    } else {  // 1 or 2 bytes: swap the aligned 32-bit word around the element
        const uintptr_t at = reinterpret_cast<uintptr_t>(addr);
        auto* a = reinterpret_cast<unsigned int*>(at & ~uintptr_t(3));
        const unsigned shift = static_cast<unsigned>(at & 3) * 8;
        const unsigned int mask = (sizeof(E) == 1 ? 0xffu : 0xffffu) << shift;
        unsigned int old = *a, assumed;
        do {
            assumed = old;
            const unsigned int field = (assumed & mask) >> shift;
            E cur;
            memcpy(&cur, &field, sizeof(E));
            const E nv = f(cur);
            unsigned int nb = 0;
            memcpy(&nb, &nv, sizeof(E));
            old = atomicCAS(a, assumed, (assumed & ~mask) | (nb << shift));
        } while (old != assumed);
    }
}

template <typename E>
__device__ __forceinline__ void scatter_apply(E* addr, E upd, int mode) {
    using A = typename AccOf<E>::type;
    if (mode == MHLO_SCATTER_SET) { *addr = upd; return; }
    if (mode == MHLO_SCATTER_ADD) {
        if constexpr (std::is_same<E, float>::value || std::is_same<E, double>::value || std::is_same<E, __half>::value ||
                      std::is_same<E, __nv_bfloat16>::value || std::is_same<E, int32_t>::value || std::is_same<E, uint32_t>::value) {
            atomicAdd(addr, upd);
            return;
        } else if constexpr (sizeof(E) == 8) {  // two's complement: signed and unsigned 64-bit adds are the same bits
            atomicAdd(reinterpret_cast<unsigned long long*>(addr), static_cast<unsigned long long>(upd));
            return;
        }
    }
    const int op = mode == MHLO_SCATTER_ADD ? MHLO_REDUCE_SUM : mode == MHLO_SCATTER_MUL ? MHLO_REDUCE_PROD
                 : mode == MHLO_SCATTER_MAX ? MHLO_REDUCE_MAX : MHLO_REDUCE_MIN;
    const A u = widen<E>(upd);
    cas_update<E>(addr, [&](E cur) { return narrow<E>(combine<A>(op, widen<E>(cur), u)); });
}

// G = 1: one thread per update element. G = 4 (fp32 add only): one thread per four consecutive elements of the updates'
// last dimension, which the caller guarantees to be a window dimension that lands on the operand's last dimension and
// to be a multiple of four long; the four targets are then consecutive and, when 16-byte aligned, take one vector atomic.
template <typename E, int G>
__global__ void __launch_bounds__(256) scatter_kernel(const __grid_constant__ ScatterParams p) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const bool has_ivd = p.d.index_vector_dim < p.indices_rank;
    for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * G; i < p.n; i += step * G) {
        int64_t uidx[MHLO_CUDA_MAX_RANK];
        int64_t rem = i;
        for (int d = p.updates_rank - 1; d >= 0; --d) { uidx[d] = rem % p.updates_shape[d]; rem /= p.updates_shape[d]; }
        // split the update index into scatter coordinates (into scatter_indices) and window coordinates
        int64_t batch[MHLO_CUDA_MAX_RANK], win[MHLO_CUDA_MAX_RANK];
        int nb = 0, nw = 0;
        for (int d = 0; d < p.updates_rank; ++d) {
            bool is_win = false;
            for (int k = 0; k < p.d.n_update_window_dims; ++k) is_win |= p.d.update_window_dims[k] == d;
            if (is_win) win[nw++] = uidx[d]; else batch[nb++] = uidx[d];
        }
        int64_t target[MHLO_CUDA_MAX_RANK];
        for (int d = 0; d < p.operand_rank; ++d) target[d] = 0;
        for (int k = 0; k < p.d.n_scatter_dims_to_operand; ++k) {
            int64_t off = 0, bi = 0;
            for (int d = 0; d < p.indices_rank; ++d) {
                const int64_t c = (has_ivd && d == p.d.index_vector_dim) ? k : batch[bi++];
                off = off * p.indices_shape[d] + c;
            }
            target[p.d.scatter_dims_to_operand_dims[k]] = p.index_dtype == MHLO_DT_I64 ? static_cast<const int64_t*>(p.indices)[off]
                                                        : p.index_dtype == MHLO_DT_UI32 ? static_cast<int64_t>(static_cast<const uint32_t*>(p.indices)[off])
                                                                                        : static_cast<const int32_t*>(p.indices)[off];
        }
        for (int k = 0; k < p.d.n_input_batching; ++k) {
            int sd = p.d.scatter_indices_batching_dims[k];
            if (has_ivd && sd > p.d.index_vector_dim) --sd;
            target[p.d.input_batching_dims[k]] += batch[sd];
        }
        int64_t dst = 0, c_last = 0;
        int wi = 0;
        bool inside = true;  // for G > 1: of every coordinate but the last
        for (int d = 0; d < p.operand_rank; ++d) {
            bool skip = false;
            for (int k = 0; k < p.d.n_inserted_window_dims; ++k) skip |= p.d.inserted_window_dims[k] == d;
            for (int k = 0; k < p.d.n_input_batching; ++k) skip |= p.d.input_batching_dims[k] == d;
            const int64_t c = target[d] + (skip ? 0 : win[wi++]);
            if (G > 1 && d == p.operand_rank - 1) c_last = c;
            else inside = inside && c >= 0 && c < p.operand_shape[d];
            dst = dst * p.operand_shape[d] + c;
        }
        if constexpr (G == 1) {
            if (inside) scatter_apply<E>(static_cast<E*>(p.result) + dst, static_cast<const E*>(p.updates)[i], p.mode);
        } else {
            if (!inside) continue;
            const int64_t extent = p.operand_shape[p.operand_rank - 1];
            E* to = static_cast<E*>(p.result) + dst;
            const E* from = static_cast<const E*>(p.updates) + i;
            if constexpr (std::is_same<E, float>::value && G == 4) {
                if (c_last >= 0 && c_last + 3 < extent && (reinterpret_cast<uintptr_t>(to) & 15u) == 0) {
                    atomicAdd(reinterpret_cast<float4*>(to), *reinterpret_cast<const float4*>(from));
                    continue;
                }
            }
#pragma unroll
            for (int e = 0; e < G; ++e)
                if (c_last + e >= 0 && c_last + e < extent) scatter_apply<E>(to + e, from[e], p.mode);
        }
    }
}

// ---- select_and_scatter -----------------------------------------------------------------------------------------------

struct SelectScatterParams {
    mhlo_cuda_window w;
    int64_t in_shape[MHLO_CUDA_MAX_RANK], in_stride[MHLO_CUDA_MAX_RANK], src_shape[MHLO_CUDA_MAX_RANK];
    const void* in;
    const void* source;
    const void* init;
    void* result;
    int64_t n_src, window_count;
    int32_t cmp, mode;
};

template <typename A>
__device__ __forceinline__ bool select_holds(int cmp, A a, A b) {
    switch (cmp) {
        case MHLO_EW_CMP_GE: return a >= b;
        case MHLO_EW_CMP_GT: return a > b;
        case MHLO_EW_CMP_LE: return a <= b;
        default: return a < b;
    }
}

template <typename E>
__global__ void __launch_bounds__(256) select_and_scatter_kernel(const __grid_constant__ SelectScatterParams p) {
    using A = typename AccOf<E>::type;
    const int rank = p.w.rank;
    const A init = widen<E>(*static_cast<const E*>(p.init));
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t s = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; s < p.n_src; s += step) {
        int64_t origin[MHLO_CUDA_MAX_RANK];
        int64_t rem = s;
        for (int d = rank - 1; d >= 0; --d) {
            origin[d] = (rem % p.src_shape[d]) * p.w.stride[d] - p.w.pad_low[d];
            rem /= p.src_shape[d];
        }
        int64_t wi[MHLO_CUDA_MAX_RANK];
        for (int d = 0; d < rank; ++d) wi[d] = 0;
        A kept = init;
        int64_t kept_at = -1;  // dense offset into the result, -1 = in the padding
        for (int64_t k = 0; k < p.window_count; ++k) {
            int64_t off = 0, dense = 0;
            bool inside = true;
            for (int d = 0; d < rank; ++d) {
                const int64_t pos = origin[d] + wi[d];
                inside = inside && pos >= 0 && pos < p.in_shape[d];
                off += pos * p.in_stride[d];
                dense = dense * p.in_shape[d] + pos;
            }
            const A v = inside ? widen<E>(static_cast<const E*>(p.in)[off]) : init;
            if (k == 0 || !select_holds<A>(p.cmp, kept, v)) {
                kept = v;
                kept_at = inside ? dense : -1;
            }
            for (int d = rank - 1; d >= 0; --d) {
                if (++wi[d] < p.w.size[d]) break;
                wi[d] = 0;
            }
        }
        if (kept_at >= 0) scatter_apply<E>(static_cast<E*>(p.result) + kept_at, static_cast<const E*>(p.source)[s], p.mode);
    }
}

// ---- sort --------------------------------------------------------------------------------------------------------------
// Every key becomes an unsigned 64-bit number whose order is the wanted one (descending = complemented); the pair
// (key, position in the slice) is unique, so a bitonic network over pairs gives the stable order. Slices are padded to
// a power of two with pairs that sort last.

constexpr int kSortChunk = MHLO_CUDA_SORT_SMEM_MAX;  // pairs a CTA holds in shared memory
constexpr int kSortThreads = 1024;

struct SortParams {
    const void* in[MHLO_CUDA_SORT_MAX_OPERANDS];
    void* out[MHLO_CUDA_SORT_MAX_OPERANDS];
    int32_t elem_size[MHLO_CUDA_SORT_MAX_OPERANDS];
    uint64_t* keys;   // global scratch (long slices only)
    uint32_t* order;
    int64_t n, inner, rows, padded;  // slice length, stride of the sorted dimension, number of slices, power of two >= n
    int32_t n_operands, key_dtype, descending;
};

template <typename E>
__device__ __forceinline__ uint64_t order_key(E v) {
    if constexpr (std::is_same<E, double>::value) {
        const uint64_t b = static_cast<uint64_t>(__double_as_longlong(v));
        return b ^ ((b >> 63) ? ~0ull : (1ull << 63));
    } else if constexpr (std::is_same<E, float>::value || std::is_same<E, __half>::value || std::is_same<E, __nv_bfloat16>::value) {
        const uint32_t b = __float_as_uint(widen<E>(v));
        return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
    } else if constexpr (std::is_signed<E>::value) {
        return static_cast<uint64_t>(static_cast<int64_t>(v)) ^ (1ull << 63);
    } else {
        return static_cast<uint64_t>(v);
    }
}

__device__ __forceinline__ uint64_t load_order_key(const void* base, int dtype, int64_t off, int flags) {
    const bool descending = (flags & 1) != 0, zeros_equal = (flags & 2) != 0;
    uint64_t k = 0;
    switch (dtype) {
        case MHLO_DT_F32: k = order_key(static_cast<const float*>(base)[off]); break;
        case MHLO_DT_F16: k = order_key(static_cast<const __half*>(base)[off]); break;
        case MHLO_DT_BF16: k = order_key(static_cast<const __nv_bfloat16*>(base)[off]); break;
        case MHLO_DT_F64: k = order_key(static_cast<const double*>(base)[off]); break;
        case MHLO_DT_I8: k = order_key(static_cast<const int8_t*>(base)[off]); break;
        case MHLO_DT_I16: k = order_key(static_cast<const int16_t*>(base)[off]); break;
        case MHLO_DT_UI16: k = order_key(static_cast<const uint16_t*>(base)[off]); break;
        case MHLO_DT_I32: k = order_key(static_cast<const int32_t*>(base)[off]); break;
        case MHLO_DT_UI32: k = order_key(static_cast<const uint32_t*>(base)[off]); break;
        case MHLO_DT_I64: k = order_key(static_cast<const int64_t*>(base)[off]); break;
        case MHLO_DT_UI64: k = order_key(static_cast<const uint64_t*>(base)[off]); break;
        default: k = order_key(static_cast<const uint8_t*>(base)[off]); break;  // I1, UI8
    }
    // a FLOAT comparison holds -0 and +0 equal (the stable order then keeps them as they came): both take +0's key
    if (zeros_equal) {
        if (dtype == MHLO_DT_F64) { if (k == 0x7fffffffffffffffull) k = 0x8000000000000000ull; }
        else if ((dtype == MHLO_DT_F32 || dtype == MHLO_DT_F16 || dtype == MHLO_DT_BF16) && k == 0x7fffffffull) k = 0x80000000ull;
    }
    return descending ? ~k : k;
}

__device__ __forceinline__ int64_t slice_base(const SortParams& p, int64_t row) { return (row / p.inner) * p.n * p.inner + row % p.inner; }

__device__ __forceinline__ void move_element(const SortParams& p, int j, int64_t dst, int64_t src) {
    switch (p.elem_size[j]) {
        case 1: static_cast<uint8_t*>(p.out[j])[dst] = static_cast<const uint8_t*>(p.in[j])[src]; break;
        case 2: static_cast<uint16_t*>(p.out[j])[dst] = static_cast<const uint16_t*>(p.in[j])[src]; break;
        case 4: static_cast<uint32_t*>(p.out[j])[dst] = static_cast<const uint32_t*>(p.in[j])[src]; break;
        default: static_cast<uint64_t*>(p.out[j])[dst] = static_cast<const uint64_t*>(p.in[j])[src]; break;
    }
}

// Compare-exchange stages j = j_first, j_first/2, .., 1 of merge size k over `count` pairs in shared memory whose
// first pair has position `origin` in its (padded) slice.
__device__ __forceinline__ void bitonic_stages(uint64_t* keys, uint32_t* order, int count, int64_t origin, int64_t k, int j_first) {
    for (int j = j_first; j > 0; j >>= 1) {
        for (int t = threadIdx.x; t < count / 2; t += blockDim.x) {
            const int i = 2 * t - (t & (j - 1));
            const int l = i + j;
            const bool ascending = ((origin + i) & k) == 0;
            const uint64_t ki = keys[i], kl = keys[l];
            const uint32_t oi = order[i], ol = order[l];
            const bool greater = ki > kl || (ki == kl && oi > ol);
            if (greater == ascending) {
                keys[i] = kl; keys[l] = ki;
                order[i] = ol; order[l] = oi;
            }
        }
        __syncthreads();
    }
}

// Keys of at most 32 bits: the pair (key, position) packs into one 64-bit word, key in the upper half, so a
// compare-exchange is one comparison and the network moves 8 bytes per element instead of 12.
__device__ __forceinline__ uint32_t load_order_key32(const void* base, int dtype, int64_t off, int flags) {
    const bool descending = (flags & 1) != 0, zeros_equal = (flags & 2) != 0;
    uint32_t k = 0;
    switch (dtype) {
        case MHLO_DT_F32: k = static_cast<uint32_t>(order_key(static_cast<const float*>(base)[off])); break;
        case MHLO_DT_F16: k = static_cast<uint32_t>(order_key(static_cast<const __half*>(base)[off])); break;
        case MHLO_DT_BF16: k = static_cast<uint32_t>(order_key(static_cast<const __nv_bfloat16*>(base)[off])); break;
        case MHLO_DT_I8: k = static_cast<uint32_t>(static_cast<int32_t>(static_cast<const int8_t*>(base)[off])) ^ 0x80000000u; break;
        case MHLO_DT_I16: k = static_cast<uint32_t>(static_cast<int32_t>(static_cast<const int16_t*>(base)[off])) ^ 0x80000000u; break;
        case MHLO_DT_I32: k = static_cast<uint32_t>(static_cast<const int32_t*>(base)[off]) ^ 0x80000000u; break;
        case MHLO_DT_UI16: k = static_cast<const uint16_t*>(base)[off]; break;
        case MHLO_DT_UI32: k = static_cast<const uint32_t*>(base)[off]; break;
        default: k = static_cast<const uint8_t*>(base)[off]; break;  // I1, UI8
    }
    if (zeros_equal && (dtype == MHLO_DT_F32 || dtype == MHLO_DT_F16 || dtype == MHLO_DT_BF16) && k == 0x7fffffffu) k = 0x80000000u;
    return descending ? ~k : k;
}

__device__ __forceinline__ void bitonic_stages_packed(uint64_t* v, int count, int k, int j_first) {
    for (int j = j_first; j > 0; j >>= 1) {
        for (int t = threadIdx.x; t < count / 2; t += blockDim.x) {
            const int i = 2 * t - (t & (j - 1));
            const int l = i + j;
            const bool ascending = (i & k) == 0;
            const uint64_t a = v[i], b = v[l];
            if ((a > b) == ascending) { v[i] = b; v[l] = a; }
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kSortThreads) sort_slices_packed_kernel(const __grid_constant__ SortParams p) {
    extern __shared__ __align__(16) unsigned char sort_smem[];
    const int padded = static_cast<int>(p.padded);
    uint64_t* v = reinterpret_cast<uint64_t*>(sort_smem);
    for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const int64_t base = slice_base(p, row);
        for (int i = threadIdx.x; i < padded; i += blockDim.x)
            v[i] = i < p.n ? (static_cast<uint64_t>(load_order_key32(p.in[0], p.key_dtype, base + i * p.inner, p.descending)) << 32) | static_cast<uint32_t>(i)
                           : ~0ull;
        __syncthreads();
        for (int k = 2; k <= padded; k <<= 1) bitonic_stages_packed(v, padded, k, k >> 1);
        for (int j = 0; j < p.n_operands; ++j)
            for (int i = threadIdx.x; i < p.n; i += blockDim.x)
                move_element(p, j, base + i * p.inner, base + static_cast<int64_t>(static_cast<uint32_t>(v[i])) * p.inner);
        __syncthreads();
    }
}

// One CTA sorts one slice of at most kSortChunk elements entirely in shared memory and writes every operand permuted.
__global__ void __launch_bounds__(kSortThreads) sort_slices_kernel(const __grid_constant__ SortParams p) {
    extern __shared__ __align__(16) unsigned char sort_smem[];
    const int padded = static_cast<int>(p.padded);
    uint64_t* keys = reinterpret_cast<uint64_t*>(sort_smem);
    uint32_t* order = reinterpret_cast<uint32_t*>(keys + padded);
    for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const int64_t base = slice_base(p, row);
        for (int i = threadIdx.x; i < padded; i += blockDim.x) {
            const bool real = i < p.n;
            keys[i] = real ? load_order_key(p.in[0], p.key_dtype, base + i * p.inner, p.descending) : ~0ull;
            order[i] = real ? static_cast<uint32_t>(i) : 0xffffffffu;
        }
        __syncthreads();
        for (int k = 2; k <= padded; k <<= 1) bitonic_stages(keys, order, padded, 0, k, k >> 1);
        for (int j = 0; j < p.n_operands; ++j)
            for (int i = threadIdx.x; i < p.n; i += blockDim.x) move_element(p, j, base + i * p.inner, base + static_cast<int64_t>(order[i]) * p.inner);
        __syncthreads();
    }
}

// Long slices: pairs live in global scratch, rows * padded of them.
__global__ void __launch_bounds__(256) sort_init_kernel(const __grid_constant__ SortParams p) {
    const int64_t total = p.rows * p.padded;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < total; g += step) {
        const int64_t row = g / p.padded, i = g % p.padded;
        const bool real = i < p.n;
        p.keys[g] = real ? load_order_key(p.in[0], p.key_dtype, slice_base(p, row) + i * p.inner, p.descending) : ~0ull;
        p.order[g] = real ? static_cast<uint32_t>(i) : 0xffffffffu;
    }
}

// A CTA takes chunks of kSortChunk pairs through the stages that stay inside a chunk: the whole network up to merge
// size kSortChunk when k == 0 (first pass), else the stages j < kSortChunk of merge size k.
__global__ void __launch_bounds__(kSortThreads) sort_chunks_kernel(const __grid_constant__ SortParams p, int64_t k) {
    extern __shared__ __align__(16) unsigned char sort_smem[];
    uint64_t* keys = reinterpret_cast<uint64_t*>(sort_smem);
    uint32_t* order = reinterpret_cast<uint32_t*>(keys + kSortChunk);
    const int64_t chunks = p.rows * p.padded / kSortChunk;
    for (int64_t c = blockIdx.x; c < chunks; c += gridDim.x) {
        const int64_t g0 = c * kSortChunk;
        const int64_t origin = g0 % p.padded;
        for (int i = threadIdx.x; i < kSortChunk; i += blockDim.x) { keys[i] = p.keys[g0 + i]; order[i] = p.order[g0 + i]; }
        __syncthreads();
        if (k == 0) {
            for (int kk = 2; kk <= kSortChunk; kk <<= 1) bitonic_stages(keys, order, kSortChunk, origin, kk, kk >> 1);
        } else {
            bitonic_stages(keys, order, kSortChunk, origin, k, kSortChunk >> 1);
        }
        for (int i = threadIdx.x; i < kSortChunk; i += blockDim.x) { p.keys[g0 + i] = keys[i]; p.order[g0 + i] = order[i]; }
        __syncthreads();
    }
}

// One compare-exchange stage (k, j) with j >= kSortChunk over all slices.
__global__ void __launch_bounds__(256) sort_global_stage_kernel(const __grid_constant__ SortParams p, int64_t k, int64_t j) {
    const int64_t half = p.padded / 2, total = p.rows * half;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < total; g += step) {
        const int64_t row = g / half, t = g % half;
        const int64_t i = 2 * t - (t & (j - 1)), l = i + j;
        const bool ascending = (i & k) == 0;
        uint64_t* keys = p.keys + row * p.padded;
        uint32_t* order = p.order + row * p.padded;
        const uint64_t ki = keys[i], kl = keys[l];
        const uint32_t oi = order[i], ol = order[l];
        const bool greater = ki > kl || (ki == kl && oi > ol);
        if (greater == ascending) {
            keys[i] = kl; keys[l] = ki;
            order[i] = ol; order[l] = oi;
        }
    }
}

__global__ void __launch_bounds__(256) sort_apply_kernel(const __grid_constant__ SortParams p) {
    const int64_t total = p.rows * p.n;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < total; g += step) {
        const int64_t row = g / p.n, i = g % p.n;
        const int64_t base = slice_base(p, row);
        const int64_t src = base + static_cast<int64_t>(p.order[row * p.padded + i]) * p.inner;
        for (int j = 0; j < p.n_operands; ++j) move_element(p, j, base + i * p.inner, src);
    }
}

int64_t next_pow2(int64_t n) {
    int64_t p = 1;
    while (p < n) p <<= 1;
    return p;
}

}  // namespace
}  // namespace mhlo

using namespace mhlo;

extern "C" int mhlo_cuda_reduce_window(const mhlo_cuda_view* in, const mhlo_cuda_window* window, int32_t op, const void* init_dev,
                                       void* out_dev, const int64_t* out_shape, mhlo_cuda_stream_t stream) {
    if (!in || !window || !out_shape) return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce_window: null argument");
    if (window->rank != in->rank || in->rank < 0 || in->rank > MHLO_CUDA_MAX_RANK)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce_window: window rank %d for an operand of rank %d", window->rank, in->rank);
    if (op < MHLO_REDUCE_SUM || op > MHLO_REDUCE_XOR) return fail(MHLO_CUDA_UNSUPPORTED, "reduce_window: reducer %d", op);
    WindowParams p;
    memset(&p, 0, sizeof p);
    p.w = *window;
    p.n_out = 1;
    p.window_count = 1;
    for (int d = 0; d < in->rank; ++d) {
        if (window->size[d] < 1 || window->stride[d] < 1 || window->base_dilation[d] < 1 || window->window_dilation[d] < 1)
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce_window: window size, stride and dilations must be positive (dimension %d)", d);
        p.in_shape[d] = in->shape[d];
        p.in_stride[d] = in->stride[d];
        p.out_shape[d] = out_shape[d];
        p.n_out *= out_shape[d];
        p.window_count *= window->size[d];
    }
    if (p.n_out == 0) return MHLO_CUDA_OK;
    if (!in->base || !init_dev || !out_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce_window: null pointer");
    p.in = in->base;
    p.init = init_dev;
    p.out = out_dev;
    p.op = op;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (in->dtype == MHLO_DT_F32 || in->dtype == MHLO_DT_F16 || in->dtype == MHLO_DT_BF16) {
        WindowVecParams q;
        if (vec_window_params(p, in->dtype, &q)) {
            const int vgrid = grid_of(q.n_vecs, 256);
            Pool3Params r;
            if (pool3_params(q, &r)) {
                const bool launched = in->dtype == MHLO_DT_F32 ? launch_pool3<float>(r, p.op, vgrid, s)
                                    : in->dtype == MHLO_DT_F16 ? launch_pool3<__half>(r, p.op, vgrid, s)
                                                               : launch_pool3<__nv_bfloat16>(r, p.op, vgrid, s);
                if (launched) {
                    MHLO_CUDA_CHECK_LAUNCH("reduce_window (pooling)");
                    return MHLO_CUDA_OK;
                }
            }
            bool dilated = false;
            for (int d = 0; d < q.rank; ++d) dilated |= q.base_dilation[d] != 1;
            auto launch = [&](auto tag) {
                using T = decltype(tag);
                if (dilated) reduce_window_vec_kernel<T, 0, true><<<vgrid, 256, 0, s>>>(q);
                else if (q.rank == 3) reduce_window_vec_kernel<T, 3, false><<<vgrid, 256, 0, s>>>(q);
                else if (q.rank == 2) reduce_window_vec_kernel<T, 2, false><<<vgrid, 256, 0, s>>>(q);
                else reduce_window_vec_kernel<T, 0, false><<<vgrid, 256, 0, s>>>(q);
            };
            if (in->dtype == MHLO_DT_F32) launch(float{});
            else if (in->dtype == MHLO_DT_F16) launch(__half{});
            else launch(__nv_bfloat16{});
            MHLO_CUDA_CHECK_LAUNCH("reduce_window (vectors)");
            return MHLO_CUDA_OK;
        }
    }
    const int grid = grid_of(p.n_out, 256);
    if (!with_element_type(in->dtype, [&](auto tag) { reduce_window_kernel<decltype(tag)><<<grid, 256, 0, s>>>(p); }))
        return fail(MHLO_CUDA_UNSUPPORTED, "reduce_window: dtype %d", in->dtype);
    MHLO_CUDA_CHECK_LAUNCH("reduce_window");
    return MHLO_CUDA_OK;
}

extern "C" int mhlo_cuda_scatter(void* result_inout_dev, int32_t dtype, const int64_t* operand_shape, int32_t operand_rank,
                                 const void* indices_dev, int32_t index_dtype, const int64_t* indices_shape, int32_t indices_rank,
                                 const void* updates_dev, const int64_t* updates_shape, int32_t updates_rank,
                                 const mhlo_cuda_scatter_dims* dims, int32_t mode, mhlo_cuda_stream_t stream) {
    if (!dims || operand_rank < 0 || operand_rank > MHLO_CUDA_MAX_RANK || indices_rank < 0 || indices_rank > MHLO_CUDA_MAX_RANK ||
        updates_rank < 0 || updates_rank > MHLO_CUDA_MAX_RANK)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "scatter: bad rank");
    if (index_dtype != MHLO_DT_I32 && index_dtype != MHLO_DT_I64 && index_dtype != MHLO_DT_UI32)
        return fail(MHLO_CUDA_UNSUPPORTED, "scatter: index dtype %d (I32, UI32 or I64 expected)", index_dtype);
    if (mode < MHLO_SCATTER_SET || mode > MHLO_SCATTER_MIN) return fail(MHLO_CUDA_UNSUPPORTED, "scatter: update computation %d", mode);
    if (dims->n_update_window_dims < 0 || dims->n_update_window_dims > updates_rank || dims->n_inserted_window_dims < 0 ||
        dims->n_input_batching < 0 || dims->n_scatter_dims_to_operand < 0 || dims->n_scatter_dims_to_operand > MHLO_CUDA_MAX_RANK ||
        dims->n_inserted_window_dims + dims->n_input_batching + dims->n_update_window_dims != operand_rank)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "scatter: window, inserted and batching dimensions do not cover the operand's rank %d", operand_rank);
    const bool has_ivd = dims->index_vector_dim < indices_rank;
    if (dims->index_vector_dim < 0 || dims->index_vector_dim > indices_rank)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "scatter: index_vector_dim %d for indices of rank %d", dims->index_vector_dim, indices_rank);
    if (updates_rank - dims->n_update_window_dims != indices_rank - (has_ivd ? 1 : 0))
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "scatter: updates have %d scatter dimensions, indices have %d",
                    updates_rank - dims->n_update_window_dims, indices_rank - (has_ivd ? 1 : 0));
    for (int k = 0; k < dims->n_scatter_dims_to_operand; ++k)
        if (dims->scatter_dims_to_operand_dims[k] < 0 || dims->scatter_dims_to_operand_dims[k] >= operand_rank)
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "scatter: scatter_dims_to_operand_dims entry out of range");
    {   // the scatter dimensions of `updates` walk `indices`: their extents must agree, or the index reads would leave it
        int bi = 0;
        for (int d = 0; d < updates_rank; ++d) {
            bool is_win = false;
            for (int k = 0; k < dims->n_update_window_dims; ++k) is_win |= dims->update_window_dims[k] == d;
            if (is_win) continue;
            if (has_ivd && bi == dims->index_vector_dim) ++bi;
            if (bi >= indices_rank || updates_shape[d] != indices_shape[bi])
                return fail(MHLO_CUDA_INVALID_ARGUMENT, "scatter: dimension %d of the updates does not match the scatter indices", d);
            ++bi;
        }
        const int64_t index_len = has_ivd ? indices_shape[dims->index_vector_dim] : 1;
        if (dims->n_scatter_dims_to_operand > index_len)
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "scatter: scatter_dims_to_operand_dims has %d entries, index vectors have %lld",
                        dims->n_scatter_dims_to_operand, static_cast<long long>(index_len));
        for (int k = 0; k < dims->n_input_batching; ++k)
            if (dims->input_batching_dims[k] < 0 || dims->input_batching_dims[k] >= operand_rank || dims->scatter_indices_batching_dims[k] < 0 ||
                dims->scatter_indices_batching_dims[k] >= indices_rank)
                return fail(MHLO_CUDA_INVALID_ARGUMENT, "scatter: batching dimension out of range");
    }
    ScatterParams p;
    memset(&p, 0, sizeof p);
    p.d = *dims;
    p.n = 1;
    for (int d = 0; d < operand_rank; ++d) p.operand_shape[d] = operand_shape[d];
    for (int d = 0; d < indices_rank; ++d) p.indices_shape[d] = indices_shape[d];
    for (int d = 0; d < updates_rank; ++d) { p.updates_shape[d] = updates_shape[d]; p.n *= updates_shape[d]; }
    if (p.n == 0) return MHLO_CUDA_OK;
    if (!result_inout_dev || !indices_dev || !updates_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "scatter: null pointer");
    p.result = result_inout_dev;
    p.indices = indices_dev;
    p.updates = updates_dev;
    p.operand_rank = operand_rank;
    p.indices_rank = indices_rank;
    p.updates_rank = updates_rank;
    p.index_dtype = index_dtype;
    p.mode = mode;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // rows of fp32 added into a table (an embedding gradient): four elements per thread, one vector atomic each
    bool rows_of_four = dtype == MHLO_DT_F32 && mode == MHLO_SCATTER_ADD && updates_rank >= 1 && operand_rank >= 1 &&
                        updates_shape[updates_rank - 1] % 4 == 0 && dims->n_update_window_dims >= 1 &&
                        (reinterpret_cast<uintptr_t>(updates_dev) & 15u) == 0;
    if (rows_of_four) {
        int last_window = -1;
        for (int k = 0; k < dims->n_update_window_dims; ++k) last_window = std::max(last_window, dims->update_window_dims[k]);
        rows_of_four = last_window == updates_rank - 1;  // the updates' last dimension is the last window dimension ...
        for (int k = 0; k < dims->n_inserted_window_dims; ++k) rows_of_four = rows_of_four && dims->inserted_window_dims[k] != operand_rank - 1;
        for (int k = 0; k < dims->n_input_batching; ++k) rows_of_four = rows_of_four && dims->input_batching_dims[k] != operand_rank - 1;  // ... on the operand's last
    }
    if (rows_of_four) {
        scatter_kernel<float, 4><<<grid_of(p.n / 4, 256), 256, 0, s>>>(p);
        MHLO_CUDA_CHECK_LAUNCH("scatter (rows of four)");
        return MHLO_CUDA_OK;
    }
    const int grid = grid_of(p.n, 256);
    if (!with_element_type(dtype, [&](auto tag) { scatter_kernel<decltype(tag), 1><<<grid, 256, 0, s>>>(p); }))
        return fail(MHLO_CUDA_UNSUPPORTED, "scatter: dtype %d", dtype);
    MHLO_CUDA_CHECK_LAUNCH("scatter");
    return MHLO_CUDA_OK;
}

namespace {

// rows, slice length and inner stride of sorting `shape` along `dimension`; false when the arguments are invalid
bool sort_geometry(const int64_t* shape, int32_t rank, int32_t dimension, int64_t* rows, int64_t* n, int64_t* inner) {
    if (!shape || rank < 1 || rank > MHLO_CUDA_MAX_RANK || dimension < 0 || dimension >= rank) return false;
    *rows = 1;
    *inner = 1;
    for (int d = 0; d < rank; ++d) {
        if (shape[d] < 0) return false;
        if (d != dimension) *rows *= shape[d];
        if (d > dimension) *inner *= shape[d];
    }
    *n = shape[dimension];
    return true;
}

}  // namespace

extern "C" int64_t mhlo_cuda_sort_scratch_bytes(const int64_t* shape, int32_t rank, int32_t dimension) {
    int64_t rows, n, inner;
    if (!sort_geometry(shape, rank, dimension, &rows, &n, &inner)) return -1;
    if (n <= MHLO_CUDA_SORT_SMEM_MAX) return 0;
    return rows * next_pow2(n) * static_cast<int64_t>(sizeof(uint64_t) + sizeof(uint32_t));
}

extern "C" int mhlo_cuda_sort(const void* const* operands_dev, void* const* outs_dev, const int32_t* dtypes, int32_t n_operands,
                              const int64_t* shape, int32_t rank, int32_t dimension, int32_t descending, void* scratch_dev,
                              int64_t scratch_bytes, mhlo_cuda_stream_t stream) {
    if (!operands_dev || !outs_dev || !dtypes || n_operands < 1 || n_operands > MHLO_CUDA_SORT_MAX_OPERANDS)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "sort: between 1 and %d operands expected", MHLO_CUDA_SORT_MAX_OPERANDS);
    SortParams p;
    memset(&p, 0, sizeof p);
    if (!sort_geometry(shape, rank, dimension, &p.rows, &p.n, &p.inner))
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "sort: dimension %d of a rank-%d tensor", dimension, rank);
    if (p.n >= (int64_t{1} << 31)) return fail(MHLO_CUDA_UNSUPPORTED, "sort: slices of 2^31 or more elements");
    for (int j = 0; j < n_operands; ++j) {
        p.elem_size[j] = dtype_bytes(dtypes[j]);
        if (p.elem_size[j] == 0) return fail(MHLO_CUDA_UNSUPPORTED, "sort: dtype %d", dtypes[j]);
        if (p.rows * p.n > 0 && (!operands_dev[j] || !outs_dev[j])) return fail(MHLO_CUDA_INVALID_ARGUMENT, "sort: null pointer");
        if (operands_dev[j] == outs_dev[j] && p.rows * p.n > 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "sort: operand %d aliases its output", j);
        p.in[j] = operands_dev[j];
        p.out[j] = outs_dev[j];
    }
    if (p.rows * p.n == 0) return MHLO_CUDA_OK;
    p.n_operands = n_operands;
    p.key_dtype = dtypes[0];
    p.descending = descending & 3;  // bit 0: descending; bit 1: -0 and +0 compare equal (a FLOAT comparison)
    p.padded = next_pow2(p.n);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t pair_bytes = sizeof(uint64_t) + sizeof(uint32_t);
    if (p.n <= kSortChunk) {
        const size_t smem = static_cast<size_t>(p.padded) * pair_bytes;
        MHLO_CUDA_TRY(cudaFuncSetAttribute(sort_slices_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSortChunk * pair_bytes)),
                      MHLO_CUDA_EXECUTION_FAILED);
        int threads = static_cast<int>(p.padded / 2);
        threads = threads < 32 ? 32 : (threads > kSortThreads ? kSortThreads : threads);
        const int grid = static_cast<int>(p.rows < kNumSMs * 8 ? p.rows : kNumSMs * 8);
        if (p.elem_size[0] <= 4) {  // keys of up to 32 bits: packed (key, position) words
            MHLO_CUDA_TRY(cudaFuncSetAttribute(sort_slices_packed_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSortChunk * sizeof(uint64_t))),
                          MHLO_CUDA_EXECUTION_FAILED);
            sort_slices_packed_kernel<<<grid, threads, static_cast<size_t>(p.padded) * sizeof(uint64_t), s>>>(p);
            MHLO_CUDA_CHECK_LAUNCH("sort (shared memory, packed keys)");
            return MHLO_CUDA_OK;
        }
        sort_slices_kernel<<<grid, threads, smem, s>>>(p);
        MHLO_CUDA_CHECK_LAUNCH("sort (shared memory)");
        return MHLO_CUDA_OK;
    }
    const int64_t need = p.rows * p.padded * static_cast<int64_t>(pair_bytes);
    if (!scratch_dev || scratch_bytes < need)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "sort: slices of %lld elements need %lld bytes of scratch, got %lld", static_cast<long long>(p.n),
                    static_cast<long long>(need), static_cast<long long>(scratch_bytes));
    p.keys = static_cast<uint64_t*>(scratch_dev);
    p.order = reinterpret_cast<uint32_t*>(p.keys + p.rows * p.padded);
    MHLO_CUDA_TRY(cudaFuncSetAttribute(sort_chunks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSortChunk * pair_bytes)),
                  MHLO_CUDA_EXECUTION_FAILED);
    const int64_t chunks = p.rows * p.padded / kSortChunk;
    const int chunk_grid = static_cast<int>(chunks < kNumSMs * 2 ? chunks : kNumSMs * 2);
    const size_t chunk_smem = kSortChunk * pair_bytes;
    sort_init_kernel<<<grid_of(p.rows * p.padded, 256), 256, 0, s>>>(p);
    MHLO_CUDA_CHECK_LAUNCH("sort (keys)");
    sort_chunks_kernel<<<chunk_grid, kSortThreads, chunk_smem, s>>>(p, 0);
    MHLO_CUDA_CHECK_LAUNCH("sort (chunks)");
    for (int64_t k = 2 * static_cast<int64_t>(kSortChunk); k <= p.padded; k <<= 1) {
        for (int64_t j = k >> 1; j >= kSortChunk; j >>= 1) {
            sort_global_stage_kernel<<<grid_of(p.rows * p.padded / 2, 256), 256, 0, s>>>(p, k, j);
            MHLO_CUDA_CHECK_LAUNCH("sort (global stage)");
        }
        sort_chunks_kernel<<<chunk_grid, kSortThreads, chunk_smem, s>>>(p, k);
        MHLO_CUDA_CHECK_LAUNCH("sort (chunk merge)");
    }
    sort_apply_kernel<<<grid_of(p.rows * p.n, 256), 256, 0, s>>>(p);
    MHLO_CUDA_CHECK_LAUNCH("sort (apply)");
    return MHLO_CUDA_OK;
}

extern "C" int mhlo_cuda_select_and_scatter(const mhlo_cuda_view* operand, const void* source_dev, const int64_t* source_shape, const void* init_dev,
                                            const mhlo_cuda_window* window, int32_t select_cmp, int32_t scatter_mode, void* result_inout_dev,
                                            mhlo_cuda_stream_t stream) {
    if (!operand || !window || !source_shape) return fail(MHLO_CUDA_INVALID_ARGUMENT, "select_and_scatter: null argument");
    if (window->rank != operand->rank || operand->rank < 0 || operand->rank > MHLO_CUDA_MAX_RANK)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "select_and_scatter: window rank %d for an operand of rank %d", window->rank, operand->rank);
    if (select_cmp != MHLO_EW_CMP_GE && select_cmp != MHLO_EW_CMP_GT && select_cmp != MHLO_EW_CMP_LE && select_cmp != MHLO_EW_CMP_LT)
        return fail(MHLO_CUDA_UNSUPPORTED, "select_and_scatter: select comparison %d", select_cmp);
    if (scatter_mode < MHLO_SCATTER_ADD || scatter_mode > MHLO_SCATTER_MIN)
        return fail(MHLO_CUDA_UNSUPPORTED, "select_and_scatter: scatter computation %d", scatter_mode);
    SelectScatterParams p;
    memset(&p, 0, sizeof p);
    p.w = *window;
    p.n_src = 1;
    p.window_count = 1;
    for (int d = 0; d < operand->rank; ++d) {
        if (window->size[d] < 1 || window->stride[d] < 1) return fail(MHLO_CUDA_INVALID_ARGUMENT, "select_and_scatter: window size and stride must be positive");
        if (window->base_dilation[d] > 1 || window->window_dilation[d] > 1) return fail(MHLO_CUDA_INVALID_ARGUMENT, "select_and_scatter has no dilations");
        p.in_shape[d] = operand->shape[d];
        p.in_stride[d] = operand->stride[d];
        p.src_shape[d] = source_shape[d];
        p.n_src *= source_shape[d];
        p.window_count *= window->size[d];
    }
    if (p.n_src == 0) return MHLO_CUDA_OK;
    if (!operand->base || !source_dev || !init_dev || !result_inout_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "select_and_scatter: null pointer");
    p.in = operand->base;
    p.source = source_dev;
    p.init = init_dev;
    p.result = result_inout_dev;
    p.cmp = select_cmp;
    p.mode = scatter_mode;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int grid = grid_of(p.n_src, 256);
    if (!with_element_type(operand->dtype, [&](auto tag) { select_and_scatter_kernel<decltype(tag)><<<grid, 256, 0, s>>>(p); }))
        return fail(MHLO_CUDA_UNSUPPORTED, "select_and_scatter: dtype %d", operand->dtype);
    MHLO_CUDA_CHECK_LAUNCH("select_and_scatter");
    return MHLO_CUDA_OK;
}
