// Entry points of the contractions: mhlo_cuda_gemm and mhlo_cuda_attention choose between the tcgen05
// tensor-core kernels and the general-layout kernels, and hold the general-layout attention kernel.
#include "common.cuh"
#include <mutex>

#include "contraction.cuh"

namespace mhlo {
namespace {

template <typename T>
__device__ __forceinline__ float ldf(const T* p) { return VecTraits<T>::to_float(*p); }

// General-layout attention: one warp per query row. Keys are taken 32 at a time - lane j scores key j against
// the query held in shared memory, the warp does the online-softmax update with shuffles, then every lane
// accumulates its slice of the head dimension over the 32 weighted value rows. Any dtype, D <= 256, any strides.
template <typename T>
__global__ void __launch_bounds__(128) attention_rows_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                             const T* __restrict__ v, const T* __restrict__ mask,
                                                             T* __restrict__ o, AttnShape s) {
    constexpr int kMaxPerLane = 8;
    __shared__ float qs[4][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 4 + warp;
    const int64_t total = s.batch * s.heads * s.seq_q;
    if (row >= total) return;
    const int64_t i = row % s.seq_q, h = (row / s.seq_q) % s.heads, b = row / (s.seq_q * s.heads);
    const T* qp = q + b * s.qs[0] + h * s.qs[1] + i * s.qs[2];
    const T* kp = k + b * s.ks[0] + h * s.ks[1];
    const T* vp = v + b * s.vs[0] + h * s.vs[1];
    T* op = o + b * s.os[0] + h * s.os[1] + i * s.os[2];
    const int D = static_cast<int>(s.head_dim);
    for (int d = lane; d < D; d += 32) qs[warp][d] = ldf(qp + d) * s.scale;
    __syncwarp();
    float acc[kMaxPerLane];
#pragma unroll
    for (int t = 0; t < kMaxPerLane; ++t) acc[t] = 0.f;
    float m = -INFINITY, l = 0.f;
    int64_t lim = s.causal ? i + 1 : s.seq_k;  // key j is visible to query i iff j <= i
    if (lim > s.seq_k) lim = s.seq_k;
    for (int64_t j0 = 0; j0 < lim; j0 += 32) {
        const int64_t j = j0 + lane;
        float sc = -INFINITY;
        if (j < lim) {
            const T* kr = kp + j * s.ks[2];
            float dot = 0.f;
            for (int d = 0; d < D; ++d) dot += qs[warp][d] * ldf(kr + d);
            sc = dot;
            if (mask != nullptr) sc += ldf(mask + i * s.seq_k + j);
        }
        float cm = sc;
#pragma unroll
        for (int x = 16; x > 0; x >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, x));
        const float mn = fmaxf(m, cm);
        const float corr = (m == -INFINITY) ? 0.f : __expf(m - mn);
        const float p = (sc == -INFINITY || mn == -INFINITY) ? 0.f : __expf(sc - mn);
        float ps = p;
#pragma unroll
        for (int x = 16; x > 0; x >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, x);
        l = l * corr + ps;
        m = mn;
#pragma unroll
        for (int t = 0; t < kMaxPerLane; ++t) acc[t] *= corr;
        const int cnt = static_cast<int>(lim - j0 < 32 ? lim - j0 : 32);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const T* vr = vp + (j0 + jj) * s.vs[2];
#pragma unroll
            for (int t = 0; t < kMaxPerLane; ++t) {
                const int d = lane + 32 * t;
                if (d < D) acc[t] += pj * ldf(vr + d);
            }
        }
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int t = 0; t < kMaxPerLane; ++t) {
        const int d = lane + 32 * t;
        if (d < D) op[d] = VecTraits<T>::from_float(acc[t] * inv);
    }
}

template <typename T>
int launch_attention_rows(const void* q, const void* k, const void* v, const void* mask, void* o, const AttnShape& s,
                          cudaStream_t stream) {
    const int64_t rows = s.batch * s.heads * s.seq_q;
    const int64_t grid = (rows + 3) / 4;
    if (grid > 0x7fffffffLL) return fail(MHLO_CUDA_UNSUPPORTED, "attention: too many query rows");
    attention_rows_kernel<T><<<static_cast<int>(grid), 128, 0, stream>>>(
        static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), static_cast<const T*>(mask),
        static_cast<T*>(o), s);
    MHLO_CUDA_CHECK_LAUNCH("attention");
    return MHLO_CUDA_OK;
}

}  // namespace
}  // namespace mhlo

using namespace mhlo;

extern "C" {

int mhlo_cuda_device_error(int32_t* out_code) {
    if (!out_code) return fail(MHLO_CUDA_INVALID_ARGUMENT, "device_error: null output");
    const int g = gemm_device_error(), a = attention_device_error();
    if (g < 0 || a < 0) return fail(MHLO_CUDA_EXECUTION_FAILED, "device_error: %s", cudaGetErrorString(cudaGetLastError()));
    *out_code = g != 0 ? g : (a != 0 ? 100 + a : 0);
    if (*out_code != 0) return fail(MHLO_CUDA_EXECUTION_FAILED, "a tensor-core kernel gave up on a bounded wait (code %d)", *out_code);
    return MHLO_CUDA_OK;
}

namespace {
// Pinned host landing slots of the error words, one pair per device, allocated on first use and kept until exit.
std::mutex g_slot_mu;
int* g_error_slots[64] = {nullptr};

int* error_slot_for_current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_slot_mu);
    if (!g_error_slots[dev]) {
        void* p = nullptr;
        if (cudaHostAlloc(&p, 2 * sizeof(int), cudaHostAllocDefault) != cudaSuccess) return nullptr;
        g_error_slots[dev] = static_cast<int*>(p);
        g_error_slots[dev][0] = g_error_slots[dev][1] = 0;
    }
    return g_error_slots[dev];
}
}  // namespace

int mhlo_cuda_device_error_fetch(mhlo_cuda_stream_t stream) {
    int* slot = error_slot_for_current_device();
    if (!slot) return fail(MHLO_CUDA_EXECUTION_FAILED, "device_error_fetch: no pinned slot for the current device");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (!gemm_error_fetch_async(slot, s) || !attention_error_fetch_async(slot + 1, s))
        return fail(MHLO_CUDA_EXECUTION_FAILED, "device_error_fetch: %s", cudaGetErrorString(cudaGetLastError()));
    return MHLO_CUDA_OK;
}

int mhlo_cuda_device_error_take(int32_t* out_code) {
    if (!out_code) return fail(MHLO_CUDA_INVALID_ARGUMENT, "device_error_take: null output");
    int* slot = error_slot_for_current_device();
    if (!slot) return fail(MHLO_CUDA_EXECUTION_FAILED, "device_error_take: no pinned slot for the current device");
    const int g = slot[0], a = slot[1];
    *out_code = g != 0 ? g : (a != 0 ? 100 + a : 0);
    if (*out_code == 0) return MHLO_CUDA_OK;
    slot[0] = slot[1] = 0;
    if (g != 0) gemm_error_store(0);
    if (a != 0) attention_error_store(0);
    return fail(MHLO_CUDA_EXECUTION_FAILED, "a tensor-core kernel gave up on a bounded wait (code %d)", *out_code);
}

int mhlo_cuda_debug_store_device_error(int32_t which, int32_t code) {
    const bool ok = which == 0 ? gemm_error_store(code) : attention_error_store(code);
    return ok ? MHLO_CUDA_OK : fail(MHLO_CUDA_EXECUTION_FAILED, "debug_store_device_error: %s", cudaGetErrorString(cudaGetLastError()));
}

int mhlo_cuda_debug_wait_expiry_probe(uint64_t limit_ns, mhlo_cuda_stream_t stream) {
    if (limit_ns > 1000000000ull) return fail(MHLO_CUDA_INVALID_ARGUMENT, "wait_expiry_probe: limit above one second");
    return gemm_wait_expiry_probe(limit_ns, static_cast<cudaStream_t>(stream))
               ? MHLO_CUDA_OK
               : fail(MHLO_CUDA_EXECUTION_FAILED, "wait_expiry_probe: %s", cudaGetErrorString(cudaGetLastError()));
}

int mhlo_cuda_gemm(int32_t in_dtype, int32_t out_dtype, const void* a_dev, const int64_t a_strides[4],
                   const void* b_dev, const int64_t b_strides[4], void* c_dev, int64_t batch0, int64_t batch1,
                   int64_t m, int64_t n, int64_t k, const void* bias_dev, int32_t epilogue,
                   mhlo_cuda_stream_t stream) {
    return mhlo_cuda_gemm_tuned(in_dtype, out_dtype, a_dev, a_strides, b_dev, b_strides, c_dev, batch0, batch1, m, n, k, bias_dev, epilogue,
                                nullptr, stream);
}

int mhlo_cuda_gemm_tuned(int32_t in_dtype, int32_t out_dtype, const void* a_dev, const int64_t a_strides[4],
                         const void* b_dev, const int64_t b_strides[4], void* c_dev, int64_t batch0, int64_t batch1,
                         int64_t m, int64_t n, int64_t k, const void* bias_dev, int32_t epilogue,
                         const mhlo_cuda_gemm_tuning* tuning, mhlo_cuda_stream_t stream) {
    if (tuning) {
        if ((tuning->tile_n != 0 && tuning->tile_n != 128 && tuning->tile_n != 256) || tuning->stages < 0 || tuning->stages > 8 ||
            tuning->stages == 1 || tuning->cta_group < 0 || tuning->cta_group > 2 || (tuning->cta_group == 2 && tuning->tile_n == 128))
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "gemm: tuning {tile_n %d, stages %d, cta_group %d} is not a configuration of the kernel",
                        tuning->tile_n, tuning->stages, tuning->cta_group);
    }
    if (epilogue < MHLO_EPILOGUE_NONE || epilogue > MHLO_EPILOGUE_SIGMOID)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "gemm: unknown epilogue %d", epilogue);
    if (!a_strides || !b_strides) return fail(MHLO_CUDA_INVALID_ARGUMENT, "gemm: null strides");
    GemmProblem p;
    p.a = a_dev; p.b = b_dev; p.c = c_dev; p.bias = bias_dev;
    for (int i = 0; i < 4; ++i) { p.as[i] = a_strides[i]; p.bs[i] = b_strides[i]; }
    p.batch0 = batch0; p.batch1 = batch1; p.m = m; p.n = n; p.k = k;
    p.in_dtype = in_dtype; p.out_dtype = out_dtype; p.epilogue = epilogue;
    if (tuning) { p.tile_n = tuning->tile_n; p.stages = tuning->stages; p.cta_group = tuning->cta_group; }
    if (gemm_tc_supported(p)) return gemm_tc_launch(p, static_cast<cudaStream_t>(stream));
    int st = mhlo_cuda_dot_strided(in_dtype, out_dtype, a_dev, a_strides, b_dev, b_strides, c_dev, batch0, batch1, m, n, k, stream);
    if (st != MHLO_CUDA_OK || (bias_dev == nullptr && epilogue == MHLO_EPILOGUE_NONE)) return st;
    // bias / activation as an in-place elementwise pass over C
    mhlo_cuda_view in[2];
    memset(in, 0, sizeof in);
    const int64_t rows = batch0 * batch1 * m;
    in[0].base = c_dev; in[0].dtype = out_dtype; in[0].rank = 2;
    in[0].shape[0] = rows; in[0].shape[1] = n; in[0].stride[0] = n; in[0].stride[1] = 1;
    in[1] = in[0];
    in[1].base = bias_dev; in[1].stride[0] = 0;
    mhlo_cuda_ew_inst prog[2];
    int ni = 0, n_in = 1, cur = 0;
    if (bias_dev != nullptr) { n_in = 2; prog[ni++] = {MHLO_EW_ADD, 0, 1, 0, 0.0}; cur = n_in; }
    static const int act_op[] = {MHLO_EW_COPY, MHLO_EW_RELU, MHLO_EW_GELU_TANH, MHLO_EW_GELU_ERF, MHLO_EW_SILU, MHLO_EW_TANH, MHLO_EW_LOGISTIC};
    if (epilogue != MHLO_EPILOGUE_NONE) { prog[ni] = {act_op[epilogue], cur, cur, cur, 0.0}; ++ni; }
    const int64_t shape[2] = {rows, n};
    return mhlo_cuda_elementwise(in, n_in, prog, ni, c_dev, out_dtype, shape, 2, stream);
}

int mhlo_cuda_conv2d_nhwc(int32_t dtype, int32_t out_dtype, const void* x_dev, const void* filter_dev, void* out_dev, int64_t images,
                          int64_t in_h, int64_t in_w, int64_t channels, int64_t filter_h, int64_t filter_w, int64_t features, int64_t out_h,
                          int64_t out_w, int64_t pad_top, int64_t pad_left, int64_t dilation_h, int64_t dilation_w, const void* bias_dev,
                          int32_t epilogue, mhlo_cuda_stream_t stream) {
    return mhlo_cuda_conv2d_nhwc_strided(dtype, out_dtype, x_dev, filter_dev, out_dev, images, in_h, in_w, channels, filter_h, filter_w, features,
                                         out_h, out_w, pad_top, pad_left, dilation_h, dilation_w, 1, 1, bias_dev, epilogue, stream);
}

int mhlo_cuda_conv2d_nhwc_strided(int32_t dtype, int32_t out_dtype, const void* x_dev, const void* filter_dev, void* out_dev, int64_t images,
                                  int64_t in_h, int64_t in_w, int64_t channels, int64_t filter_h, int64_t filter_w, int64_t features,
                                  int64_t out_h, int64_t out_w, int64_t pad_top, int64_t pad_left, int64_t dilation_h, int64_t dilation_w,
                                  int64_t stride_h, int64_t stride_w, const void* bias_dev, int32_t epilogue, mhlo_cuda_stream_t stream) {
    if (epilogue < MHLO_EPILOGUE_NONE || epilogue > MHLO_EPILOGUE_SIGMOID)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "conv2d_nhwc: unknown epilogue %d", epilogue);
    if (images < 0 || in_h < 0 || in_w < 0 || channels < 0 || filter_h < 0 || filter_w < 0 || features < 0 || out_h < 0 || out_w < 0)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "conv2d_nhwc: negative extent");
    if (images * out_h * out_w * features == 0) return MHLO_CUDA_OK;
    if (!x_dev || !filter_dev || !out_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "conv2d_nhwc: null pointer");
    ConvProblem c;
    c.x = x_dev; c.wgt = filter_dev; c.out = out_dev; c.bias = bias_dev;
    c.dtype = dtype; c.out_dtype = out_dtype; c.epilogue = epilogue;
    c.images = images; c.h = in_h; c.w = in_w; c.channels = channels; c.kh = filter_h; c.kw = filter_w; c.features = features;
    c.oh = out_h; c.ow = out_w; c.pad_h = pad_top; c.pad_w = pad_left; c.dil_h = dilation_h; c.dil_w = dilation_w;
    c.stride_h = stride_h; c.stride_w = stride_w;
    if (!conv_tc_supported(c))
        return fail(MHLO_CUDA_UNSUPPORTED, "conv2d_nhwc: needs f16 / bf16 tensors, channels in multiples of 64, feature rows on the 16-byte grid, strides of 1 to 8");
    return conv_tc_launch(c, static_cast<cudaStream_t>(stream));
}

int mhlo_cuda_gemm_residual(int32_t in_dtype, int32_t out_dtype, const void* a_dev, const int64_t a_strides[4], const void* b_dev,
                            const int64_t b_strides[4], void* c_dev, int64_t batch0, int64_t batch1, int64_t m, int64_t n, int64_t k,
                            const void* bias_dev, const void* residual_dev, const mhlo_cuda_gemm_tuning* tuning, mhlo_cuda_stream_t stream) {
    if (residual_dev == nullptr)
        return mhlo_cuda_gemm_tuned(in_dtype, out_dtype, a_dev, a_strides, b_dev, b_strides, c_dev, batch0, batch1, m, n, k, bias_dev,
                                    MHLO_EPILOGUE_NONE, tuning, stream);
    if (!a_strides || !b_strides) return fail(MHLO_CUDA_INVALID_ARGUMENT, "gemm_residual: null strides");
    if (tuning && ((tuning->tile_n != 0 && tuning->tile_n != 128 && tuning->tile_n != 256) || tuning->stages < 0 || tuning->stages > 8 ||
                   tuning->stages == 1 || tuning->cta_group < 0 || tuning->cta_group > 2 || (tuning->cta_group == 2 && tuning->tile_n == 128)))
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "gemm_residual: tuning {tile_n %d, stages %d, cta_group %d} is not a configuration of the kernel",
                    tuning->tile_n, tuning->stages, tuning->cta_group);
    GemmProblem p;
    p.a = a_dev; p.b = b_dev; p.c = c_dev; p.bias = bias_dev; p.residual = residual_dev;
    for (int i = 0; i < 4; ++i) { p.as[i] = a_strides[i]; p.bs[i] = b_strides[i]; }
    p.batch0 = batch0; p.batch1 = batch1; p.m = m; p.n = n; p.k = k;
    p.in_dtype = in_dtype; p.out_dtype = out_dtype; p.epilogue = MHLO_EPILOGUE_NONE;
    if (tuning) { p.tile_n = tuning->tile_n; p.stages = tuning->stages; p.cta_group = tuning->cta_group; }
    const int64_t out_es = out_dtype == MHLO_DT_F32 ? 4 : 2;
    // the epilogue reads the residual in 16-byte pieces of a row: rows of C (and of the residual) on the 16-byte grid
    if (gemm_tc_supported(p) && out_dtype != MHLO_DT_F32 && (n * out_es) % 16 == 0 && aligned16(c_dev) && aligned16(residual_dev))
        return gemm_tc_launch(p, static_cast<cudaStream_t>(stream));
    // otherwise the product first, then the sum as an elementwise pass over C
    int st = mhlo_cuda_gemm_tuned(in_dtype, out_dtype, a_dev, a_strides, b_dev, b_strides, c_dev, batch0, batch1, m, n, k, bias_dev,
                                  MHLO_EPILOGUE_NONE, tuning, stream);
    if (st != MHLO_CUDA_OK) return st;
    mhlo_cuda_view in[2];
    memset(in, 0, sizeof in);
    const int64_t rows = batch0 * batch1 * m;
    in[0].base = c_dev; in[0].dtype = out_dtype; in[0].rank = 2;
    in[0].shape[0] = rows; in[0].shape[1] = n; in[0].stride[0] = n; in[0].stride[1] = 1;
    in[1] = in[0];
    in[1].base = residual_dev;
    mhlo_cuda_ew_inst prog[1] = {{MHLO_EW_ADD, 0, 1, 0, 0.0}};
    const int64_t shape[2] = {rows, n};
    return mhlo_cuda_elementwise(in, 2, prog, 1, c_dev, out_dtype, shape, 2, stream);
}

int mhlo_cuda_gemm_all_gather(int32_t in_dtype, int32_t out_dtype, const void* a_dev, const int64_t a_strides[2], const void* b_dev,
                              const int64_t b_strides[2], void* const* c_devs, int32_t n_ranks, int32_t rank, int64_t m, int64_t n_local,
                              int64_t k, const void* bias_dev, int32_t epilogue, mhlo_cuda_stream_t stream) {
    return mhlo_cuda_gemm_all_gather_tuned(in_dtype, out_dtype, a_dev, a_strides, b_dev, b_strides, c_devs, n_ranks, rank, m, n_local, k, bias_dev,
                                           epilogue, nullptr, 0, stream);
}

int mhlo_cuda_peer_barrier(void* const* flag_devs, int32_t n_ranks, int32_t rank, uint64_t epoch, uint64_t limit_ns, mhlo_cuda_stream_t stream) {
    if (!flag_devs) return fail(MHLO_CUDA_INVALID_ARGUMENT, "peer_barrier: null argument");
    if (n_ranks < 1 || n_ranks > 8 || rank < 0 || rank >= n_ranks)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "peer_barrier: rank %d of %d (1 to 8 ranks)", rank, n_ranks);
    if (limit_ns == 0 || limit_ns > 2000000000ull) return fail(MHLO_CUDA_INVALID_ARGUMENT, "peer_barrier: the wait limit is 1 ns to 2 s");
    uint64_t* arrays[8] = {nullptr};
    for (int r = 0; r < n_ranks; ++r) {
        if (flag_devs[r] == nullptr || (reinterpret_cast<uintptr_t>(flag_devs[r]) & 7u) != 0)
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "peer_barrier: flag array %d is null or not 8-byte aligned", r);
        arrays[r] = static_cast<uint64_t*>(flag_devs[r]);
    }
    if (n_ranks == 1) return MHLO_CUDA_OK;
    return gemm_peer_barrier_launch(arrays, n_ranks, rank, epoch, limit_ns, static_cast<cudaStream_t>(stream))
               ? MHLO_CUDA_OK
               : fail(MHLO_CUDA_EXECUTION_FAILED, "peer_barrier: %s", cudaGetErrorString(cudaGetLastError()));
}

int mhlo_cuda_gemm_all_gather_tuned(int32_t in_dtype, int32_t out_dtype, const void* a_dev, const int64_t a_strides[2], const void* b_dev,
                                    const int64_t b_strides[2], void* const* c_devs, int32_t n_ranks, int32_t rank, int64_t m,
                                    int64_t n_local, int64_t k, const void* bias_dev, int32_t epilogue, const mhlo_cuda_gemm_tuning* tuning,
                                    int32_t copy_stores, mhlo_cuda_stream_t stream) {
    if (copy_stores < 0 || copy_stores > 2) return fail(MHLO_CUDA_INVALID_ARGUMENT, "gemm_all_gather: copy_stores %d (0 to 2)", copy_stores);
    if (tuning && ((tuning->tile_n != 0 && tuning->tile_n != 128 && tuning->tile_n != 256) || tuning->stages < 0 || tuning->stages > 8 ||
                   tuning->stages == 1 || tuning->cta_group < 0 || tuning->cta_group > 2 || (tuning->cta_group == 2 && tuning->tile_n == 128)))
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "gemm_all_gather: tuning {tile_n %d, stages %d, cta_group %d} is not a configuration of this product",
                    tuning->tile_n, tuning->stages, tuning->cta_group);
    if (epilogue < MHLO_EPILOGUE_NONE || epilogue > MHLO_EPILOGUE_SIGMOID)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "gemm_all_gather: unknown epilogue %d", epilogue);
    if (!a_strides || !b_strides || !c_devs) return fail(MHLO_CUDA_INVALID_ARGUMENT, "gemm_all_gather: null argument");
    if (n_ranks < 1 || n_ranks > 8 || rank < 0 || rank >= n_ranks)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "gemm_all_gather: rank %d of %d (1 to 8 ranks)", rank, n_ranks);
    if (m < 0 || n_local < 0 || k < 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "gemm_all_gather: negative extent");
    if (m == 0 || n_local == 0) return MHLO_CUDA_OK;
    for (int r = 0; r < n_ranks; ++r)
        if (c_devs[r] == nullptr) return fail(MHLO_CUDA_INVALID_ARGUMENT, "gemm_all_gather: destination %d is null", r);
    GemmProblem p;
    p.a = a_dev; p.b = b_dev; p.c = c_devs[rank]; p.bias = bias_dev;
    p.as[0] = p.as[1] = 0; p.as[2] = a_strides[0]; p.as[3] = a_strides[1];
    p.bs[0] = p.bs[1] = 0; p.bs[2] = b_strides[0]; p.bs[3] = b_strides[1];
    p.batch0 = p.batch1 = 1; p.m = m; p.n = n_local; p.k = k;
    p.in_dtype = in_dtype; p.out_dtype = out_dtype; p.epilogue = epilogue;
    p.ldc = n_local * n_ranks;
    p.c_col0 = n_local * rank;
    p.n_copies = 0;
    // copies in the order rank + 1, rank + 2, ...: in any one moment the ranks' stores go to different peers
    for (int i = 1; i < n_ranks; ++i) p.copies[p.n_copies++] = c_devs[(rank + i) % n_ranks];
    p.copy_stores = copy_stores;
    if (tuning) { p.tile_n = tuning->tile_n; p.stages = tuning->stages; p.cta_group = tuning->cta_group; }
    if (!gemm_tc_supported(p))
        return fail(MHLO_CUDA_UNSUPPORTED, "gemm_all_gather: needs the tensor-core path (bf16 / f16 operands, 16-byte aligned rows, k > 0)");
    return gemm_tc_launch(p, static_cast<cudaStream_t>(stream));
}

int mhlo_cuda_attention(int32_t dtype, const void* q_dev, const int64_t q_strides[3], const void* k_dev,
                        const int64_t k_strides[3], const void* v_dev, const int64_t v_strides[3],
                        const void* mask_dev, void* o_dev, const int64_t o_strides[3], int64_t batch,
                        int64_t heads, int64_t seq_q, int64_t seq_k, int64_t head_dim, float scale,
                        int32_t causal, mhlo_cuda_stream_t stream) {
    return mhlo_cuda_attention_tuned(dtype, q_dev, q_strides, k_dev, k_strides, v_dev, v_strides, mask_dev, o_dev, o_strides, batch, heads, seq_q,
                                     seq_k, head_dim, scale, causal, nullptr, stream);
}

int mhlo_cuda_attention_tuned(int32_t dtype, const void* q_dev, const int64_t q_strides[3], const void* k_dev,
                              const int64_t k_strides[3], const void* v_dev, const int64_t v_strides[3],
                              const void* mask_dev, void* o_dev, const int64_t o_strides[3], int64_t batch,
                              int64_t heads, int64_t seq_q, int64_t seq_k, int64_t head_dim, float scale,
                              int32_t causal, const mhlo_cuda_attention_tuning* tuning, mhlo_cuda_stream_t stream) {
    if (tuning && (tuning->tile_order < 0 || tuning->tile_order > 2))
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "attention: tuning {tile_order %d} is not a configuration of the kernel", tuning->tile_order);
    if (batch < 0 || heads < 0 || seq_q < 0 || seq_k < 0 || head_dim < 0)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "attention: negative extent");
    if (!q_strides || !k_strides || !v_strides || !o_strides) return fail(MHLO_CUDA_INVALID_ARGUMENT, "attention: null strides");
    if (batch * heads * seq_q * head_dim == 0) return MHLO_CUDA_OK;
    if (!q_dev || !o_dev || (seq_k > 0 && (!k_dev || !v_dev))) return fail(MHLO_CUDA_INVALID_ARGUMENT, "attention: null pointer");
    AttnShape s;
    for (int i = 0; i < 3; ++i) { s.qs[i] = q_strides[i]; s.ks[i] = k_strides[i]; s.vs[i] = v_strides[i]; s.os[i] = o_strides[i]; }
    s.batch = batch; s.heads = heads; s.seq_q = seq_q; s.seq_k = seq_k; s.head_dim = head_dim; s.scale = scale; s.causal = causal;
    if (tuning) s.tile_order = tuning->tile_order;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (attention_tc_supported(dtype, s, mask_dev) && aligned16(q_dev) && aligned16(k_dev) && aligned16(v_dev) && aligned16(o_dev))
        return attention_tc_launch(dtype, q_dev, k_dev, v_dev, o_dev, s, st);
    if (head_dim > 256) return fail(MHLO_CUDA_UNSUPPORTED, "attention: head_dim %lld above 256", (long long)head_dim);
    switch (dtype) {
        case MHLO_DT_F32: return launch_attention_rows<float>(q_dev, k_dev, v_dev, mask_dev, o_dev, s, st);
        case MHLO_DT_F16: return launch_attention_rows<__half>(q_dev, k_dev, v_dev, mask_dev, o_dev, s, st);
        case MHLO_DT_BF16: return launch_attention_rows<__nv_bfloat16>(q_dev, k_dev, v_dev, mask_dev, o_dev, s, st);
        default: return fail(MHLO_CUDA_UNSUPPORTED, "attention: dtype %d", dtype);
    }
}

}  // extern "C"
