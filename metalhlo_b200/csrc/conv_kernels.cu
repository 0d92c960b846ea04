// stablehlo.convolution: the direct kernel that honours every attribute, and the patch-matrix (im2col) kernel that
// turns a convolution into a GEMM for the tensor-core path.
#include <cstring>
#include <type_traits>

#include "common.cuh"

namespace mhlo {
namespace {

template <typename E> struct ConvAcc { using type = int64_t; };
template <> struct ConvAcc<float> { using type = float; };
template <> struct ConvAcc<__half> { using type = float; };
template <> struct ConvAcc<__nv_bfloat16> { using type = float; };
template <> struct ConvAcc<double> { using type = double; };

template <typename E> __device__ __forceinline__ typename ConvAcc<E>::type conv_load(const E* p) { return static_cast<typename ConvAcc<E>::type>(*p); }
template <> __device__ __forceinline__ float conv_load<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float conv_load<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename E> __device__ __forceinline__ E conv_store(typename ConvAcc<E>::type v) { return static_cast<E>(v); }
template <> __device__ __forceinline__ __half conv_store<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 conv_store<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

struct ConvParams {
    mhlo_cuda_conv c;
    const void* in;
    const void* kernel;
    void* out;
    int64_t n_out, out_batch, kernel_volume, features_per_group, row_pitch, n_rows;
};

template <typename E>
__global__ void __launch_bounds__(256) conv_direct_kernel(const __grid_constant__ ConvParams p) {
    using A = typename ConvAcc<E>::type;
    const mhlo_cuda_conv& c = p.c;
    const int ns = c.n_spatial;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t out_per_fgroup = c.out_features / c.feature_group_count;
    const int64_t out_per_bgroup = c.out_features / c.batch_group_count;
    for (int64_t o = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; o < p.n_out; o += step) {
        // o = ((b * out_size.. ) * out_features + oc), output feature fastest
        int64_t rem = o;
        const int64_t oc = rem % c.out_features;
        rem /= c.out_features;
        int64_t origin[MHLO_CUDA_CONV_MAX_SPATIAL];
        int64_t out_off = oc * c.out_feature_stride;
        for (int d = ns - 1; d >= 0; --d) {
            const int64_t od = rem % c.out_size[d];
            rem /= c.out_size[d];
            origin[d] = od * c.stride[d] - c.pad_low[d];
            out_off += od * c.out_spatial_stride[d];
        }
        const int64_t b = rem;
        out_off += b * c.out_batch_stride;
        const int64_t in_b = (oc / out_per_bgroup) * p.out_batch + b;
        const int64_t ic0 = (oc / out_per_fgroup) * p.features_per_group;
        const E* in_base = static_cast<const E*>(p.in) + in_b * c.in_batch_stride + ic0 * c.in_feature_stride;
        const E* w_base = static_cast<const E*>(p.kernel) + oc * c.kernel_out_stride;
        A acc = A(0);
        int64_t k[MHLO_CUDA_CONV_MAX_SPATIAL];
        for (int d = 0; d < ns; ++d) k[d] = 0;
        for (int64_t kv = 0; kv < p.kernel_volume; ++kv) {
            int64_t in_off = 0, w_off = 0;
            bool inside = true;
            for (int d = 0; d < ns; ++d) {
                const int64_t pos = origin[d] + k[d] * c.rhs_dilation[d];
                const int64_t src = pos / c.lhs_dilation[d];
                inside = inside && pos >= 0 && src < c.in_size[d] && src * c.lhs_dilation[d] == pos;
                in_off += src * c.in_spatial_stride[d];
                w_off += (c.reverse[d] ? c.kernel_size[d] - 1 - k[d] : k[d]) * c.kernel_spatial_stride[d];
            }
            if (inside)
                for (int64_t ic = 0; ic < p.features_per_group; ++ic)
                    acc += conv_load<E>(in_base + in_off + ic * c.in_feature_stride) * conv_load<E>(w_base + w_off + ic * c.kernel_in_stride);
            for (int d = ns - 1; d >= 0; --d) {
                if (++k[d] < c.kernel_size[d]) break;
                k[d] = 0;
            }
        }
        static_cast<E*>(p.out)[out_off] = conv_store<E>(acc);
    }
}

// cols[g][m][kk]: kk = (kernel spatial.. row-major, feature within group g), zero-filled up to row_pitch.
template <typename E>
__global__ void __launch_bounds__(256) im2col_kernel(const __grid_constant__ ConvParams p) {
    const mhlo_cuda_conv& c = p.c;
    const int ns = c.n_spatial;
    const int64_t total = c.feature_group_count * p.n_rows * p.row_pitch;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t row_len = p.kernel_volume * p.features_per_group;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
        const int64_t kk = i % p.row_pitch;
        int64_t rem = i / p.row_pitch;
        const int64_t m = rem % p.n_rows;
        const int64_t g = rem / p.n_rows;
        E v = E(0);
        if (kk < row_len) {
            const int64_t ic = kk % p.features_per_group;
            int64_t kv = kk / p.features_per_group;
            int64_t mm = m;
            int64_t in_off = (g * p.features_per_group + ic) * c.in_feature_stride;
            bool inside = true;
            for (int d = ns - 1; d >= 0; --d) {
                int64_t kd = kv % c.kernel_size[d];
                kv /= c.kernel_size[d];
                const int64_t od = mm % c.out_size[d];
                mm /= c.out_size[d];
                if (c.reverse[d]) kd = c.kernel_size[d] - 1 - kd;  // the kernel is read unreversed; reverse the taps instead
                const int64_t pos = od * c.stride[d] - c.pad_low[d] + kd * c.rhs_dilation[d];
                const int64_t src = pos / c.lhs_dilation[d];
                inside = inside && pos >= 0 && src < c.in_size[d] && src * c.lhs_dilation[d] == pos;
                in_off += src * c.in_spatial_stride[d];
            }
            in_off += mm * c.in_batch_stride;
            if (inside) v = static_cast<const E*>(p.in)[in_off];
        }
        static_cast<E*>(p.out)[i] = v;
    }
}

// The same patch matrix moved as 16-byte vectors along the feature dimension: one thread per vector of `V` features of
// one tap, 32-bit index arithmetic. Needs unit feature stride, features per group, pitch and all other input strides
// multiples of V, 16-byte aligned bases and fewer than 2^31 vectors.
struct Im2colVecParams {
    const uint4* in;
    uint4* out;
    uint32_t total_vecs, pitch_vecs, row_vecs, cg_vecs, n_rows, groups;
    int32_t ns;
    FastDiv by_pitch, by_rows, by_cg, by_kernel[MHLO_CUDA_CONV_MAX_SPATIAL], by_out[MHLO_CUDA_CONV_MAX_SPATIAL];
    uint32_t kernel_size[MHLO_CUDA_CONV_MAX_SPATIAL], out_size[MHLO_CUDA_CONV_MAX_SPATIAL], in_size[MHLO_CUDA_CONV_MAX_SPATIAL];
    int32_t stride[MHLO_CUDA_CONV_MAX_SPATIAL], pad_low[MHLO_CUDA_CONV_MAX_SPATIAL], lhs_dilation[MHLO_CUDA_CONV_MAX_SPATIAL],
        rhs_dilation[MHLO_CUDA_CONV_MAX_SPATIAL], reverse[MHLO_CUDA_CONV_MAX_SPATIAL];
    int64_t in_batch_vecs, in_spatial_vecs[MHLO_CUDA_CONV_MAX_SPATIAL];  // strides in vectors
};

// NS > 0: the number of spatial dimensions at compile time; DILATED = false promises lhs_dilation == 1 everywhere.
template <int NS, bool DILATED>
__global__ void __launch_bounds__(256) im2col_vec_kernel(const __grid_constant__ Im2colVecParams p) {
    const int ns = NS > 0 ? NS : p.ns;
    const uint32_t step = gridDim.x * blockDim.x;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < p.total_vecs; i += step) {
        uint32_t kvec, rem, m, g;
        p.by_pitch.divmod(i, &rem, &kvec);
        p.by_rows.divmod(rem, &g, &m);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (kvec < p.row_vecs) {
            uint32_t icv, kv;
            p.by_cg.divmod(kvec, &kv, &icv);
            int64_t off = static_cast<int64_t>(g) * p.cg_vecs + icv;
            bool inside = true;
#pragma unroll
            for (int d = ns - 1; d >= 0; --d) {
                uint32_t kd, od;
                p.by_kernel[d].divmod(kv, &kv, &kd);
                p.by_out[d].divmod(m, &m, &od);
                if (p.reverse[d]) kd = p.kernel_size[d] - 1 - kd;
                const int32_t pos = static_cast<int32_t>(od) * p.stride[d] - p.pad_low[d] + static_cast<int32_t>(kd) * p.rhs_dilation[d];
                const int32_t src = DILATED ? pos / p.lhs_dilation[d] : pos;
                inside = inside && pos >= 0 && src < static_cast<int32_t>(p.in_size[d]) && (!DILATED || src * p.lhs_dilation[d] == pos);
                off += src * p.in_spatial_vecs[d];
            }
            off += m * p.in_batch_vecs;
            if (inside) v = __ldg(p.in + off);
        }
        p.out[i] = v;
    }
}

// Fills the vector parameters; false when the layout does not allow the vector path.
bool vec_im2col_params(const ConvParams& p, int elem_bytes, Im2colVecParams* q) {
    const mhlo_cuda_conv& c = p.c;
    const int64_t V = 16 / elem_bytes;
    if (elem_bytes > 16 || 16 % elem_bytes) return false;
    if (c.in_feature_stride != 1 || p.features_per_group % V || p.row_pitch % V || c.in_batch_stride % V) return false;
    if (!aligned16(p.in) || !aligned16(p.out)) return false;
    const int64_t total = c.feature_group_count * p.n_rows * (p.row_pitch / V);
    if (total >= (int64_t{1} << 31) || p.n_rows >= (int64_t{1} << 31)) return false;
    *q = Im2colVecParams{};
    for (int d = 0; d < c.n_spatial; ++d) {
        if (c.in_spatial_stride[d] % V) return false;
        const int64_t reach = c.out_size[d] * c.stride[d] + c.kernel_size[d] * c.rhs_dilation[d] + (c.pad_low[d] < 0 ? -c.pad_low[d] : c.pad_low[d]);
        if (reach >= (int64_t{1} << 30) || c.in_size[d] >= (int64_t{1} << 30)) return false;
        q->kernel_size[d] = static_cast<uint32_t>(c.kernel_size[d]);
        q->out_size[d] = static_cast<uint32_t>(c.out_size[d]);
        q->in_size[d] = static_cast<uint32_t>(c.in_size[d]);
        q->stride[d] = static_cast<int32_t>(c.stride[d]);
        q->pad_low[d] = static_cast<int32_t>(c.pad_low[d]);
        q->lhs_dilation[d] = static_cast<int32_t>(c.lhs_dilation[d]);
        q->rhs_dilation[d] = static_cast<int32_t>(c.rhs_dilation[d]);
        q->reverse[d] = c.reverse[d];
        q->in_spatial_vecs[d] = c.in_spatial_stride[d] / V;
    }
    q->in = static_cast<const uint4*>(p.in);
    q->out = static_cast<uint4*>(p.out);
    q->total_vecs = static_cast<uint32_t>(total);
    q->pitch_vecs = static_cast<uint32_t>(p.row_pitch / V);
    q->row_vecs = static_cast<uint32_t>(p.kernel_volume * p.features_per_group / V);
    q->cg_vecs = static_cast<uint32_t>(p.features_per_group / V);
    q->n_rows = static_cast<uint32_t>(p.n_rows);
    q->groups = static_cast<uint32_t>(c.feature_group_count);
    q->ns = c.n_spatial;
    q->in_batch_vecs = c.in_batch_stride / V;
    q->by_pitch = FastDiv(q->pitch_vecs);
    q->by_rows = FastDiv(q->n_rows);
    q->by_cg = FastDiv(q->cg_vecs);
    for (int d = 0; d < c.n_spatial; ++d) { q->by_kernel[d] = FastDiv(q->kernel_size[d]); q->by_out[d] = FastDiv(q->out_size[d]); }
    return q->row_vecs > 0 && q->cg_vecs > 0;
}

int fill_params(const mhlo_cuda_conv* conv, ConvParams* p, const char* what) {
    if (!conv) return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: null geometry", what);
    if (conv->n_spatial < 0 || conv->n_spatial > MHLO_CUDA_CONV_MAX_SPATIAL)
        return fail(MHLO_CUDA_UNSUPPORTED, "%s: %d spatial dimensions (at most %d)", what, conv->n_spatial, MHLO_CUDA_CONV_MAX_SPATIAL);
    if (conv->feature_group_count < 1 || conv->batch_group_count < 1 || conv->batch < 0 || conv->in_features < 0 || conv->out_features < 0)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: bad feature / batch counts", what);
    if (conv->in_features % conv->feature_group_count || conv->out_features % conv->feature_group_count ||
        conv->out_features % conv->batch_group_count || conv->batch % conv->batch_group_count)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: group counts do not divide the feature / batch sizes", what);
    memset(p, 0, sizeof *p);
    p->c = *conv;
    p->kernel_volume = 1;
    p->n_rows = conv->batch / conv->batch_group_count;
    for (int d = 0; d < conv->n_spatial; ++d) {
        if (conv->stride[d] < 1 || conv->lhs_dilation[d] < 1 || conv->rhs_dilation[d] < 1 || conv->kernel_size[d] < 0 || conv->out_size[d] < 0)
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: strides and dilations must be positive (dimension %d)", what, d);
        p->kernel_volume *= conv->kernel_size[d];
        p->n_rows *= conv->out_size[d];
    }
    p->out_batch = conv->batch / conv->batch_group_count;
    p->features_per_group = conv->in_features / conv->feature_group_count;
    p->n_out = p->n_rows * conv->out_features;
    return MHLO_CUDA_OK;
}

int conv_grid(int64_t n) {
    const int64_t blocks = (n + 255) / 256, cap = static_cast<int64_t>(kNumSMs) * 16;
    return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace
}  // namespace mhlo

using namespace mhlo;

#define MHLO_CONV_DISPATCH(dtype, KERNEL, grid, s, p, what)                                                  \
    switch (dtype) {                                                                                         \
        case MHLO_DT_F32: KERNEL<float><<<grid, 256, 0, s>>>(p); break;                                      \
        case MHLO_DT_F16: KERNEL<__half><<<grid, 256, 0, s>>>(p); break;                                     \
        case MHLO_DT_BF16: KERNEL<__nv_bfloat16><<<grid, 256, 0, s>>>(p); break;                             \
        case MHLO_DT_F64: KERNEL<double><<<grid, 256, 0, s>>>(p); break;                                     \
        case MHLO_DT_I8: KERNEL<int8_t><<<grid, 256, 0, s>>>(p); break;                                      \
        case MHLO_DT_UI8: KERNEL<uint8_t><<<grid, 256, 0, s>>>(p); break;                                    \
        case MHLO_DT_I16: KERNEL<int16_t><<<grid, 256, 0, s>>>(p); break;                                    \
        case MHLO_DT_UI16: KERNEL<uint16_t><<<grid, 256, 0, s>>>(p); break;                                  \
        case MHLO_DT_I32: KERNEL<int32_t><<<grid, 256, 0, s>>>(p); break;                                    \
        case MHLO_DT_UI32: KERNEL<uint32_t><<<grid, 256, 0, s>>>(p); break;                                  \
        case MHLO_DT_I64: KERNEL<int64_t><<<grid, 256, 0, s>>>(p); break;                                    \
        case MHLO_DT_UI64: KERNEL<uint64_t><<<grid, 256, 0, s>>>(p); break;                                  \
        default: return fail(MHLO_CUDA_UNSUPPORTED, "%s: dtype %d", what, dtype);                            \
    }

extern "C" int mhlo_cuda_convolution(int32_t dtype, const void* in_dev, const void* kernel_dev, void* out_dev, const mhlo_cuda_conv* conv,
                                     mhlo_cuda_stream_t stream) {
    ConvParams p;
    if (int st = fill_params(conv, &p, "convolution")) return st;
    if (conv->feature_group_count > 1 && conv->batch_group_count > 1)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "convolution: feature_group_count and batch_group_count cannot both exceed 1");
    if (p.n_out == 0) return MHLO_CUDA_OK;
    if (!in_dev || !kernel_dev || !out_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "convolution: null pointer");
    p.in = in_dev;
    p.kernel = kernel_dev;
    p.out = out_dev;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int grid = conv_grid(p.n_out);
    MHLO_CONV_DISPATCH(dtype, conv_direct_kernel, grid, s, p, "convolution");
    MHLO_CUDA_CHECK_LAUNCH("convolution");
    return MHLO_CUDA_OK;
}

extern "C" int mhlo_cuda_im2col(int32_t dtype, const void* in_dev, void* cols_dev, int64_t row_pitch, const mhlo_cuda_conv* conv,
                                mhlo_cuda_stream_t stream) {
    ConvParams p;
    if (int st = fill_params(conv, &p, "im2col")) return st;
    if (conv->batch_group_count != 1) return fail(MHLO_CUDA_UNSUPPORTED, "im2col: batch_group_count %lld", static_cast<long long>(conv->batch_group_count));
    if (row_pitch < p.kernel_volume * p.features_per_group)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "im2col: row pitch %lld below the patch length %lld", static_cast<long long>(row_pitch),
                    static_cast<long long>(p.kernel_volume * p.features_per_group));
    p.row_pitch = row_pitch;
    const int64_t total = conv->feature_group_count * p.n_rows * row_pitch;
    if (total == 0) return MHLO_CUDA_OK;
    if (!in_dev || !cols_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "im2col: null pointer");
    p.in = in_dev;
    p.out = cols_dev;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int elem_bytes = 0;
    switch (dtype) {
        case MHLO_DT_I1: case MHLO_DT_I8: case MHLO_DT_UI8: elem_bytes = 1; break;
        case MHLO_DT_F16: case MHLO_DT_BF16: case MHLO_DT_I16: case MHLO_DT_UI16: elem_bytes = 2; break;
        case MHLO_DT_F32: case MHLO_DT_I32: case MHLO_DT_UI32: elem_bytes = 4; break;
        case MHLO_DT_F64: case MHLO_DT_I64: case MHLO_DT_UI64: elem_bytes = 8; break;
        default: break;
    }
    Im2colVecParams q;
    if (elem_bytes && vec_im2col_params(p, elem_bytes, &q)) {
        bool dilated = false;
        for (int d = 0; d < q.ns; ++d) dilated |= q.lhs_dilation[d] != 1;
        const int vgrid = conv_grid(q.total_vecs);
        if (dilated) im2col_vec_kernel<0, true><<<vgrid, 256, 0, s>>>(q);
        else if (q.ns == 2) im2col_vec_kernel<2, false><<<vgrid, 256, 0, s>>>(q);
        else im2col_vec_kernel<0, false><<<vgrid, 256, 0, s>>>(q);
        MHLO_CUDA_CHECK_LAUNCH("im2col (vectors)");
        return MHLO_CUDA_OK;
    }
    const int grid = conv_grid(total);
    MHLO_CONV_DISPATCH(dtype, im2col_kernel, grid, s, p, "im2col");
    MHLO_CUDA_CHECK_LAUNCH("im2col");
    return MHLO_CUDA_OK;
}
