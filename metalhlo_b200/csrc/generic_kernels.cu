// Generic tensor kernels over strided views: the elementwise-program interpreter (every unary / binary /
// compare / select / clamp / convert / iota op, data movement expressed as a strided copy, and fused
// elementwise chains), reductions, gather, dynamic slicing and the any-layout dot product. They are the
// non-specialised side of the hot path; the specialised side (row kernels, tensor-core GEMM, attention) lives
// in its own files.
#include <cfloat>

#include <mutex>

#include "common.cuh"

#include <type_traits>

namespace mhlo {
namespace {

// ---- loads / stores in a compute domain ----------------------------------------------------------------------

template <typename C>
__device__ __forceinline__ C load_as(const void* base, int dtype, int64_t off) {
    switch (dtype) {
        case MHLO_DT_F32: return static_cast<C>(static_cast<const float*>(base)[off]);
        case MHLO_DT_F16: return static_cast<C>(__half2float(static_cast<const __half*>(base)[off]));
        case MHLO_DT_BF16: return static_cast<C>(__bfloat162float(static_cast<const __nv_bfloat16*>(base)[off]));
        case MHLO_DT_F64: return static_cast<C>(static_cast<const double*>(base)[off]);
        case MHLO_DT_I1: return static_cast<C>(static_cast<const uint8_t*>(base)[off] != 0);
        case MHLO_DT_I8: return static_cast<C>(static_cast<const int8_t*>(base)[off]);
        case MHLO_DT_UI8: return static_cast<C>(static_cast<const uint8_t*>(base)[off]);
        case MHLO_DT_I16: return static_cast<C>(static_cast<const int16_t*>(base)[off]);
        case MHLO_DT_UI16: return static_cast<C>(static_cast<const uint16_t*>(base)[off]);
        case MHLO_DT_I32: return static_cast<C>(static_cast<const int32_t*>(base)[off]);
        case MHLO_DT_UI32: return static_cast<C>(static_cast<const uint32_t*>(base)[off]);
        case MHLO_DT_I64: return static_cast<C>(static_cast<const int64_t*>(base)[off]);
        default: {  // UI64
            const uint64_t v = static_cast<const uint64_t*>(base)[off];
            if constexpr (sizeof(C) == 8 && !std::is_floating_point<C>::value) return static_cast<C>(v);
            return static_cast<C>(v);
        }
    }
}

// float -> integer follows a C cast (toward zero) that saturates at the ends of the result type and maps NaN to 0, for the
// types narrower than the 64 bits CUDA converts through as well; integer -> narrower integer keeps the low bits.
template <typename C>
__device__ __forceinline__ int64_t to_integer(C v, int64_t lo, int64_t hi) {
    int64_t i = static_cast<int64_t>(v);
    if constexpr (std::is_floating_point<C>::value) i = i < lo ? lo : (i > hi ? hi : i);
    return i;
}

template <typename C>
__device__ __forceinline__ void store_as(void* base, int dtype, int64_t off, C v) {
    if constexpr (std::is_floating_point<C>::value) {
        // NaN -> 0 for every integer type (the hardware conversion gives 0 or the type's minimum depending on the widths)
        if (v != v && dtype != MHLO_DT_F32 && dtype != MHLO_DT_F16 && dtype != MHLO_DT_BF16 && dtype != MHLO_DT_F64 && dtype != MHLO_DT_I1) v = C(0);
    }
    switch (dtype) {
        case MHLO_DT_F32: static_cast<float*>(base)[off] = static_cast<float>(v); break;
        case MHLO_DT_F16: static_cast<__half*>(base)[off] = __float2half_rn(static_cast<float>(v)); break;
        case MHLO_DT_BF16: static_cast<__nv_bfloat16*>(base)[off] = __float2bfloat16_rn(static_cast<float>(v)); break;
        case MHLO_DT_F64: static_cast<double*>(base)[off] = static_cast<double>(v); break;
        case MHLO_DT_I1: static_cast<uint8_t*>(base)[off] = v != C(0) ? 1 : 0; break;
        case MHLO_DT_I8: static_cast<int8_t*>(base)[off] = static_cast<int8_t>(to_integer(v, -128, 127)); break;
        case MHLO_DT_UI8: static_cast<uint8_t*>(base)[off] = static_cast<uint8_t>(to_integer(v, 0, 255)); break;
        case MHLO_DT_I16: static_cast<int16_t*>(base)[off] = static_cast<int16_t>(to_integer(v, -32768, 32767)); break;
        case MHLO_DT_UI16: static_cast<uint16_t*>(base)[off] = static_cast<uint16_t>(to_integer(v, 0, 65535)); break;
        case MHLO_DT_I32: static_cast<int32_t*>(base)[off] = static_cast<int32_t>(v); break;
        case MHLO_DT_UI32: static_cast<uint32_t*>(base)[off] = static_cast<uint32_t>(to_integer(v, 0, 4294967295LL)); break;
        case MHLO_DT_I64: static_cast<int64_t*>(base)[off] = static_cast<int64_t>(v); break;
        default:
            if constexpr (std::is_floating_point<C>::value) static_cast<uint64_t*>(base)[off] = static_cast<uint64_t>(v);  // saturates; negative and NaN -> 0
            else static_cast<uint64_t*>(base)[off] = static_cast<uint64_t>(static_cast<int64_t>(v));
            break;
    }
}

// ---- elementwise program ---------------------------------------------------------------------------------------

struct EwParams {
    mhlo_cuda_view in[MHLO_CUDA_EW_MAX_INPUTS];
    mhlo_cuda_ew_inst prog[MHLO_CUDA_EW_MAX_INSTS];
    int64_t out_shape[MHLO_CUDA_MAX_RANK];
    int64_t n;
    void* out;
    int32_t n_inputs, n_insts, rank, out_dtype;
    int32_t contiguous_mask;  // bit k: input k is dense row-major over the output shape (offset = linear index)
    int32_t unsigned_mode;    // integer domain: treat values as uint64 for div/rem/shift/compare/min/max
    int32_t bool_mode;        // integer domain: NOT is logical (i1)
    int32_t int_bits;         // integer domain: width of the operand type (shifts, popcnt, clz)
    int32_t out_strided;      // store through out_stride instead of the linear index
    int64_t out_stride[MHLO_CUDA_MAX_RANK];
};

// stablehlo.reduce_precision on the bits of a float (8 / 23) or a double (11 / 52): round the mantissa to nearest even at
// `mant` bits, then clamp the exponent range to `expo` bits (overflow -> infinity, underflow -> signed zero).
template <typename U, int kExpBits, int kMantBits>
__device__ __forceinline__ U reduce_precision_bits(U bits, int expo, int mant) {
    const U one = 1;
    const U exp_mask = ((one << kExpBits) - 1) << kMantBits, mant_mask = (one << kMantBits) - 1, sign = bits & (one << (kExpBits + kMantBits));
    const bool is_nan = (bits & exp_mask) == exp_mask && (bits & mant_mask) != 0;
    if (is_nan) return mant > 0 ? bits : (sign | exp_mask);  // a format without mantissa bits has no NaN: it becomes infinity
    if (mant < kMantBits) {
        const U last = one << (kMantBits - mant);
        const U bias = (last >> 1) - 1 + ((bits & last) >> (kMantBits - mant));
        bits = (bits + bias) & ~(last - 1);
    }
    if (expo < kExpBits) {
        const long long full_bias = (1ll << (kExpBits - 1)) - 1, reduced_bias = (1ll << (expo - 1)) - 1;
        const U max_exp = static_cast<U>(full_bias + reduced_bias) << kMantBits, min_exp = static_cast<U>(full_bias - reduced_bias) << kMantBits;
        const U e = bits & exp_mask;
        if (e > max_exp) bits = sign | exp_mask;
        else if (e <= min_exp) bits = sign;
    }
    return bits;
}
__device__ __forceinline__ float reduce_precision_value(float a, int expo, int mant) {
    return __uint_as_float(reduce_precision_bits<uint32_t, 8, 23>(__float_as_uint(a), expo, mant));
}
__device__ __forceinline__ double reduce_precision_value(double a, int expo, int mant) {
    return __longlong_as_double(static_cast<long long>(reduce_precision_bits<unsigned long long, 11, 52>(static_cast<unsigned long long>(__double_as_longlong(a)), expo, mant)));
}

template <typename C>
__device__ __forceinline__ C ew_float_op(int op, C a, C b, C c, double imm) {
    switch (op) {
        case MHLO_EW_COPY: return a;
        case MHLO_EW_IMM: return static_cast<C>(imm);
        case MHLO_EW_ADD: return a + b;
        case MHLO_EW_SUB: return a - b;
        case MHLO_EW_MUL: return a * b;
        case MHLO_EW_DIV: return a / b;
        case MHLO_EW_REM: return fmod(a, b);
        case MHLO_EW_MAX: return (a != a || b != b) ? C(NAN) : (a > b ? a : b);
        case MHLO_EW_MIN: return (a != a || b != b) ? C(NAN) : (a < b ? a : b);
        case MHLO_EW_POW: return pow(a, b);
        case MHLO_EW_ATAN2: return atan2(a, b);
        case MHLO_EW_AND: return C(a != C(0) && b != C(0));
        case MHLO_EW_OR: return C(a != C(0) || b != C(0));
        case MHLO_EW_XOR: return C((a != C(0)) != (b != C(0)));
        case MHLO_EW_NEG: return -a;
        case MHLO_EW_ABS: return fabs(a);
        case MHLO_EW_EXP: return exp(a);
        case MHLO_EW_EXPM1: return expm1(a);
        case MHLO_EW_LOG: return log(a);
        case MHLO_EW_LOG1P: return log1p(a);
        case MHLO_EW_SQRT: return sqrt(a);
        case MHLO_EW_RSQRT: return C(1) / sqrt(a);
        case MHLO_EW_CBRT: return cbrt(a);
        case MHLO_EW_TANH: return tanh(a);
        case MHLO_EW_LOGISTIC: return C(1) / (C(1) + exp(-a));
        case MHLO_EW_SIN: return sin(a);
        case MHLO_EW_COS: return cos(a);
        case MHLO_EW_TAN: return tan(a);
        case MHLO_EW_FLOOR: return floor(a);
        case MHLO_EW_CEIL: return ceil(a);
        case MHLO_EW_ROUND_AFZ: return round(a);
        case MHLO_EW_ROUND_EVEN: return rint(a);
        case MHLO_EW_SIGN: return a != a ? a : C((a > C(0)) - (a < C(0)));
        case MHLO_EW_NOT: return C(a == C(0));
        case MHLO_EW_IS_FINITE: return C(isfinite(a) ? 1 : 0);
        case MHLO_EW_CMP_EQ: return C(a == b);
        case MHLO_EW_CMP_NE: return C(a != b);
        case MHLO_EW_CMP_LT: return C(a < b);
        case MHLO_EW_CMP_LE: return C(a <= b);
        case MHLO_EW_CMP_GT: return C(a > b);
        case MHLO_EW_CMP_GE: return C(a >= b);
        case MHLO_EW_SELECT: return a != C(0) ? b : c;
        case MHLO_EW_CLAMP: {  // minimum(maximum(operand, min), max), each of which hands a NaN on
            if (a != a || b != b || c != c) return C(NAN);
            C lo = b < a ? a : b;
            return lo > c ? c : lo;
        }
        case MHLO_EW_GELU_TANH: {
            const C inner = C(0.7978845608028654) * (a + C(0.044715) * a * a * a);
            return C(0.5) * a * (C(1) + tanh(inner));
        }
        case MHLO_EW_GELU_ERF: return C(0.5) * a * (C(1) + erf(a * C(0.70710678118654752440)));
        case MHLO_EW_SILU: return a / (C(1) + exp(-a));
        case MHLO_EW_RELU: return a > C(0) ? a : (a != a ? a : C(0));
        case MHLO_EW_ROUND_TO: {
            const int dt = static_cast<int>(imm);
            if (dt == MHLO_DT_F16) return C(__half2float(__float2half_rn(static_cast<float>(a))));
            if (dt == MHLO_DT_BF16) return C(__bfloat162float(__float2bfloat16_rn(static_cast<float>(a))));
            if (dt == MHLO_DT_F32) return C(static_cast<float>(a));
            return a;
        }
        case MHLO_EW_ERF: return erf(a);
        case MHLO_EW_REDUCE_PRECISION: return reduce_precision_value(a, static_cast<int>(imm) / 64, static_cast<int>(imm) % 64);
        default: return a;
    }
}

__device__ __forceinline__ int64_t ew_int_op(int op, int64_t a, int64_t b, int64_t c, double imm, bool uns, bool boolean,
                                             int bits) {
    const uint64_t ua = static_cast<uint64_t>(a), ub = static_cast<uint64_t>(b);
    const uint64_t wmask = bits >= 64 ? ~0ull : ((1ull << bits) - 1);  // operand width: shifts and bit counts are per type
    switch (op) {
        case MHLO_EW_COPY: return a;
        case MHLO_EW_IMM: return static_cast<int64_t>(imm);
        case MHLO_EW_ADD: return static_cast<int64_t>(ua + ub);
        case MHLO_EW_SUB: return static_cast<int64_t>(ua - ub);
        case MHLO_EW_MUL: return static_cast<int64_t>(ua * ub);
        case MHLO_EW_DIV: return b == 0 ? -1 : (uns ? static_cast<int64_t>(ua / ub) : (b == -1 ? static_cast<int64_t>(0 - ua) : a / b));
        case MHLO_EW_REM: return b == 0 ? a : (uns ? static_cast<int64_t>(ua % ub) : (b == -1 ? 0 : a % b));
        case MHLO_EW_MAX: return uns ? static_cast<int64_t>(ua > ub ? ua : ub) : (a > b ? a : b);
        case MHLO_EW_MIN: return uns ? static_cast<int64_t>(ua < ub ? ua : ub) : (a < b ? a : b);
        case MHLO_EW_POW: {
            if (b < 0 && !uns) return a == 1 ? 1 : (a == -1 ? ((b & 1) ? -1 : 1) : 0);
            uint64_t r = 1, base = ua, e = ub;
            while (e) { if (e & 1) r *= base; base *= base; e >>= 1; }
            return static_cast<int64_t>(r);
        }
        case MHLO_EW_AND: return a & b;
        case MHLO_EW_OR: return a | b;
        case MHLO_EW_XOR: return a ^ b;
        case MHLO_EW_SHL: return ub >= static_cast<uint64_t>(bits) ? 0 : static_cast<int64_t>(ua << ub);
        case MHLO_EW_SHR_A: return ub >= static_cast<uint64_t>(bits) ? (a < 0 ? -1 : 0) : (a >> ub);
        case MHLO_EW_SHR_L: return ub >= static_cast<uint64_t>(bits) ? 0 : static_cast<int64_t>((ua & wmask) >> ub);
        case MHLO_EW_NEG: return static_cast<int64_t>(0 - ua);
        case MHLO_EW_ABS: return a < 0 ? static_cast<int64_t>(0 - ua) : a;
        case MHLO_EW_SIGN: return (a > 0) - (a < 0);
        case MHLO_EW_NOT: return boolean ? (a == 0) : ~a;
        case MHLO_EW_POPCNT: return __popcll(ua & wmask);
        case MHLO_EW_CLZ: return __clzll(static_cast<int64_t>(ua & wmask)) - (64 - bits);
        case MHLO_EW_CMP_EQ: return a == b;
        case MHLO_EW_CMP_NE: return a != b;
        case MHLO_EW_CMP_LT: return uns ? ua < ub : a < b;
        case MHLO_EW_CMP_LE: return uns ? ua <= ub : a <= b;
        case MHLO_EW_CMP_GT: return uns ? ua > ub : a > b;
        case MHLO_EW_CMP_GE: return uns ? ua >= ub : a >= b;
        case MHLO_EW_SELECT: return a != 0 ? b : c;
        case MHLO_EW_CLAMP: {
            if (uns) { uint64_t lo = ub < ua ? ua : ub; uint64_t uc = static_cast<uint64_t>(c); return static_cast<int64_t>(lo > uc ? uc : lo); }
            int64_t lo = b < a ? a : b; return lo > c ? c : lo;
        }
        case MHLO_EW_RELU: return a > 0 ? a : 0;
        case MHLO_EW_IS_FINITE: return 1;
        default: return a;
    }
}

template <typename C>
__global__ void __launch_bounds__(256) ew_kernel(const __grid_constant__ EwParams p) {
    constexpr int kRegs = MHLO_CUDA_EW_MAX_INPUTS + MHLO_CUDA_EW_MAX_INSTS;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.n; i += step) {
        int64_t idx[MHLO_CUDA_MAX_RANK];
        {
            int64_t rem = i;
#pragma unroll
            for (int d = MHLO_CUDA_MAX_RANK - 1; d >= 0; --d) {
                if (d < p.rank) {
                    const int64_t e = p.out_shape[d];
                    idx[d] = rem % e;
                    rem /= e;
                } else {
                    idx[d] = 0;
                }
            }
        }
        C r[kRegs];
        for (int k = 0; k < p.n_inputs; ++k) {
            int64_t off = i;
            if (!((p.contiguous_mask >> k) & 1)) {
                off = 0;
#pragma unroll
                for (int d = 0; d < MHLO_CUDA_MAX_RANK; ++d)
                    if (d < p.rank) off += idx[d] * p.in[k].stride[d];
            }
            r[k] = load_as<C>(p.in[k].base, p.in[k].dtype, off);
        }
        for (int k = 0; k < p.n_insts; ++k) {
            const mhlo_cuda_ew_inst& in = p.prog[k];
            C res;
            if (in.op == MHLO_EW_IOTA) {
                res = static_cast<C>(idx[static_cast<int>(in.imm)]);
            } else {
                const C a = r[in.a], b = r[in.b], c = r[in.c];
                if constexpr (std::is_floating_point<C>::value) res = ew_float_op<C>(in.op, a, b, c, in.imm);
                else res = ew_int_op(in.op, a, b, c, in.imm, p.unsigned_mode != 0, p.bool_mode != 0, p.int_bits);
            }
            r[p.n_inputs + k] = res;
        }
        int64_t oo = i;
        if (p.out_strided) {
            oo = 0;
#pragma unroll
            for (int d = 0; d < MHLO_CUDA_MAX_RANK; ++d)
                if (d < p.rank) oo += idx[d] * p.out_stride[d];
        }
        store_as<C>(p.out, p.out_dtype, oo, r[p.n_inputs + p.n_insts - 1]);
    }
}

// Fast path of the elementwise program: one instruction, float tensors, every input either dense over the output or
// a single broadcast element. Eight elements per thread through 16-byte accesses; the opcode switch is uniform and
// works on registers, so residual adds, bias-free activations, converts and dense copies run at memory speed.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float* f) {
    if constexpr (sizeof(T) == 4) {
        const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        VecTraits<T>::unpack(v, f);
    }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float* f) {
    if constexpr (sizeof(T) == 4) {
        reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
        reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
    } else {
        *reinterpret_cast<uint4*>(p) = VecTraits<T>::pack(f);
    }
}

struct EwVecParams {
    const void* in[3];
    void* out;
    int64_t n;
    int32_t scalar_mask;  // bit k: input k is one broadcast element
    int32_t n_inputs, op;
    double imm;
    int64_t period[3];    // > 0: input k is dense over its trailing dimensions and repeats every `period` elements
                          // (broadcast over the leading ones: a bias row, a position table); a multiple of 8
};

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) ew_vec_kernel(const EwVecParams p) {
    const int64_t nvec = p.n / 8;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    float sc[3] = {0.f, 0.f, 0.f};
    for (int k = 0; k < p.n_inputs; ++k)
        if ((p.scalar_mask >> k) & 1) sc[k] = VecTraits<TI>::to_float(static_cast<const TI*>(p.in[k])[0]);
    for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += step) {
        float x[3][8], r[8];
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            if (k < p.n_inputs && !((p.scalar_mask >> k) & 1)) {
                const int64_t at = p.period[k] > 0 ? (v * 8) % p.period[k] : v * 8;
                load8(static_cast<const TI*>(p.in[k]) + at, x[k]);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[k][e] = sc[k];
            }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) r[e] = ew_float_op<float>(p.op, x[0][e], x[1][e], x[2][e], p.imm);
        store8(static_cast<TO*>(p.out) + v * 8, r);
    }
    // ragged tail
    if (blockIdx.x == 0 && threadIdx.x < p.n % 8) {
        const int64_t i = nvec * 8 + threadIdx.x;
        float x[3];
        for (int k = 0; k < 3; ++k)
            x[k] = k < p.n_inputs ? (((p.scalar_mask >> k) & 1) ? sc[k]
                                                                : VecTraits<TI>::to_float(static_cast<const TI*>(p.in[k])[p.period[k] > 0 ? i % p.period[k] : i]))
                                  : 0.f;
        static_cast<TO*>(p.out)[i] = VecTraits<TO>::from_float(ew_float_op<float>(p.op, x[0], x[1], x[2], p.imm));
    }
}

template <typename TI>
bool launch_ew_vec_out(int out_dtype, const EwVecParams& p, int grid, cudaStream_t s) {
    switch (out_dtype) {
        case MHLO_DT_F32: ew_vec_kernel<TI, float><<<grid, 256, 0, s>>>(p); return true;
        case MHLO_DT_F16: ew_vec_kernel<TI, __half><<<grid, 256, 0, s>>>(p); return true;
        case MHLO_DT_BF16: ew_vec_kernel<TI, __nv_bfloat16><<<grid, 256, 0, s>>>(p); return true;
        default: return false;
    }
}

// Collapses adjacent dimensions that are mergeable in the output and in every input, drops extent-1 dims.
void collapse_dims(EwParams* p) {
    int64_t shape[MHLO_CUDA_MAX_RANK];
    int64_t strides[MHLO_CUDA_EW_MAX_INPUTS][MHLO_CUDA_MAX_RANK];
    int64_t ostr[MHLO_CUDA_MAX_RANK] = {0};
    int r = 0;
    for (int d = 0; d < p->rank; ++d) {
        if (p->out_shape[d] == 1) continue;
        bool merge = r > 0;
        if (merge)
            for (int k = 0; k < p->n_inputs; ++k)
                if (strides[k][r - 1] != p->in[k].stride[d] * p->out_shape[d]) { merge = false; break; }
        if (merge && p->out_strided && ostr[r - 1] != p->out_stride[d] * p->out_shape[d]) merge = false;
        if (merge) {
            shape[r - 1] *= p->out_shape[d];
            for (int k = 0; k < p->n_inputs; ++k) strides[k][r - 1] = p->in[k].stride[d];
            ostr[r - 1] = p->out_stride[d];
        } else {
            shape[r] = p->out_shape[d];
            for (int k = 0; k < p->n_inputs; ++k) strides[k][r] = p->in[k].stride[d];
            ostr[r] = p->out_stride[d];
            ++r;
        }
    }
    p->rank = r;
    for (int d = 0; d < MHLO_CUDA_MAX_RANK; ++d) p->out_stride[d] = d < r ? ostr[d] : 0;
    for (int d = 0; d < MHLO_CUDA_MAX_RANK; ++d) {
        p->out_shape[d] = d < r ? shape[d] : 1;
        for (int k = 0; k < p->n_inputs; ++k) {
            p->in[k].stride[d] = d < r ? strides[k][d] : 0;
            p->in[k].shape[d] = p->out_shape[d];
        }
    }
    for (int k = 0; k < p->n_inputs; ++k) {
        p->in[k].rank = r;
        bool dense = true;
        int64_t expect = 1;
        for (int d = r - 1; d >= 0; --d) {
            if (p->in[k].stride[d] != expect) { dense = false; break; }
            expect *= p->out_shape[d];
        }
        if (dense) p->contiguous_mask |= 1 << k;
    }
}

// ---- reduce ------------------------------------------------------------------------------------------------------

struct ReduceParams {
    mhlo_cuda_view in;  // kept dims first, reduced dims after
    int64_t n_out, n_red;
    const void* init;
    void* out;
    void* index_out;
    int32_t n_kept, op, index_dtype;
};

template <typename A>
struct Acc {
    A v;
    int64_t idx;
};

template <typename A>
__device__ __forceinline__ Acc<A> red_identity(int op) {
    Acc<A> a;
    a.idx = INT64_MAX;
    if constexpr (std::is_floating_point<A>::value) {
        switch (op) {
            case MHLO_REDUCE_MAX: case MHLO_REDUCE_ARGMAX: a.v = -INFINITY; break;
            case MHLO_REDUCE_MIN: case MHLO_REDUCE_ARGMIN: a.v = INFINITY; break;
            case MHLO_REDUCE_PROD: case MHLO_REDUCE_AND: a.v = 1; break;
            default: a.v = 0;
        }
    } else {
        switch (op) {
            case MHLO_REDUCE_MAX: case MHLO_REDUCE_ARGMAX: a.v = INT64_MIN; break;
            case MHLO_REDUCE_MIN: case MHLO_REDUCE_ARGMIN: a.v = INT64_MAX; break;
            case MHLO_REDUCE_PROD: a.v = 1; break;
            case MHLO_REDUCE_AND: a.v = -1; break;
            default: a.v = 0;
        }
    }
    return a;
}

template <typename A>
__device__ __forceinline__ Acc<A> red_combine(int op, Acc<A> x, Acc<A> y) {
    Acc<A> r = x;
    switch (op) {
        case MHLO_REDUCE_SUM: r.v = x.v + y.v; break;
        case MHLO_REDUCE_PROD: r.v = x.v * y.v; break;
        case MHLO_REDUCE_MAX:
            if constexpr (std::is_floating_point<A>::value) r.v = (x.v != x.v || y.v != y.v) ? A(NAN) : (x.v > y.v ? x.v : y.v);
            else r.v = x.v > y.v ? x.v : y.v;
            break;
        case MHLO_REDUCE_MIN:
            if constexpr (std::is_floating_point<A>::value) r.v = (x.v != x.v || y.v != y.v) ? A(NAN) : (x.v < y.v ? x.v : y.v);
            else r.v = x.v < y.v ? x.v : y.v;
            break;
        case MHLO_REDUCE_AND:
            if constexpr (std::is_floating_point<A>::value) r.v = A(x.v != 0 && y.v != 0); else r.v = x.v & y.v;
            break;
        case MHLO_REDUCE_OR:
            if constexpr (std::is_floating_point<A>::value) r.v = A(x.v != 0 || y.v != 0); else r.v = x.v | y.v;
            break;
        case MHLO_REDUCE_XOR:
            if constexpr (std::is_floating_point<A>::value) r.v = A((x.v != 0) != (y.v != 0)); else r.v = x.v ^ y.v;
            break;
        case MHLO_REDUCE_ARGMAX:
        case MHLO_REDUCE_ARGMIN: {
            const bool mx = op == MHLO_REDUCE_ARGMAX;
            bool take_y;
            bool xn = false, yn = false;
            if constexpr (std::is_floating_point<A>::value) { xn = x.v != x.v; yn = y.v != y.v; }
            if (xn || yn) take_y = yn && (!xn || y.idx < x.idx);
            else if (y.v == x.v) take_y = y.idx < x.idx;
            else take_y = mx ? (y.v > x.v) : (y.v < x.v);
            if (take_y) r = y;
            break;
        }
    }
    return r;
}

template <typename A>
__device__ __forceinline__ Acc<A> red_shfl(Acc<A> a, int o) {
    Acc<A> r;
    r.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    r.idx = __shfl_xor_sync(0xffffffffu, a.idx, o);
    return r;
}

// GROUP threads cooperate on one output element: 1 (thread), 32 (warp) or 256 (whole CTA).
template <typename A, int GROUP>
__global__ void __launch_bounds__(256) reduce_kernel(const __grid_constant__ ReduceParams p) {
    __shared__ Acc<A> sm[8];
    const int groups_per_cta = 256 / GROUP;
    const int g = threadIdx.x / GROUP, t = threadIdx.x % GROUP;
    const int n_red_dims = p.in.rank - p.n_kept;
    for (int64_t o0 = static_cast<int64_t>(blockIdx.x) * groups_per_cta; o0 < p.n_out;
         o0 += static_cast<int64_t>(gridDim.x) * groups_per_cta) {
        const int64_t o = o0 + g;
        const bool valid = o < p.n_out;
        int64_t base = 0;
        if (valid) {
            int64_t rem = o;
            for (int d = p.n_kept - 1; d >= 0; --d) {
                base += (rem % p.in.shape[d]) * p.in.stride[d];
                rem /= p.in.shape[d];
            }
        }
        Acc<A> acc = red_identity<A>(p.op);
        if (valid) {
            for (int64_t r = t; r < p.n_red; r += GROUP) {
                int64_t off = base;
                if (n_red_dims == 1) {
                    off += r * p.in.stride[p.n_kept];
                } else {
                    int64_t rem = r;
                    for (int d = p.in.rank - 1; d >= p.n_kept; --d) {
                        off += (rem % p.in.shape[d]) * p.in.stride[d];
                        rem /= p.in.shape[d];
                    }
                }
                Acc<A> e;
                e.v = load_as<A>(p.in.base, p.in.dtype, off);
                e.idx = r;
                acc = red_combine<A>(p.op, acc, e);
            }
        }
        if (GROUP >= 32) {
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) acc = red_combine<A>(p.op, acc, red_shfl(acc, s));
        }
        if (GROUP == 256) {
            __syncthreads();
            if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
            __syncthreads();
            acc = sm[0];
            for (int w = 1; w < 8; ++w) acc = red_combine<A>(p.op, acc, sm[w]);
        }
        if (valid && t == 0) {
            if (p.init != nullptr && p.op != MHLO_REDUCE_ARGMAX && p.op != MHLO_REDUCE_ARGMIN) {
                Acc<A> e;
                e.v = load_as<A>(p.init, p.in.dtype, 0);
                e.idx = INT64_MAX;
                acc = red_combine<A>(p.op, acc, e);
            }
            store_as<A>(p.out, p.in.dtype, o, acc.v);
            if (p.index_out != nullptr) {
                const int64_t ix = acc.idx == INT64_MAX ? 0 : acc.idx;
                if (p.index_dtype == MHLO_DT_I64) static_cast<int64_t*>(p.index_out)[o] = ix;
                else static_cast<int32_t*>(p.index_out)[o] = static_cast<int32_t>(ix);
            }
        }
    }
}

// ---- split reduce: few outputs, long reductions -------------------------------------------------------------------
// reduce_kernel gives one output element to at most one CTA, so a reduction to a scalar (or a handful of values) would
// run on a single SM. Here every output's reduced range is cut into `splits` segments, one CTA each, whose partial
// accumulators go to scratch memory (partials[o * splits + s]); a second kernel folds the partials, and the init
// value, in a fixed order and writes the result. Scratch = n_out * splits * sizeof(Acc) bytes.

struct SplitPlan {
    int splits;
    int64_t chunk;  // reduced elements per segment (multiple of 256)
    size_t scratch_bytes;
};

// splits == 0: chosen so that n_out * splits is about four CTAs per SM.
inline bool plan_split(int64_t n_out, int64_t n_red, int requested_splits, SplitPlan* plan) {
    if (n_out < 1 || n_out > 65535 || n_red < 1) return false;
    int64_t splits = requested_splits > 0 ? requested_splits : std::max<int64_t>(1, (148 * 4) / n_out);
    splits = std::min<int64_t>(splits, (n_red + 255) / 256);
    int64_t chunk = (n_red + splits - 1) / splits;
    chunk = (chunk + 255) / 256 * 256;
    splits = (n_red + chunk - 1) / chunk;
    plan->splits = static_cast<int>(splits);
    plan->chunk = chunk;
    plan->scratch_bytes = static_cast<size_t>(n_out) * static_cast<size_t>(splits) * sizeof(Acc<int64_t>);
    return true;
}

template <typename A>
__global__ void __launch_bounds__(256) reduce_split_kernel(const __grid_constant__ ReduceParams p, Acc<A>* partials, int splits, int64_t chunk) {
    __shared__ Acc<A> sm[8];
    const int64_t o = blockIdx.y;
    const int s = blockIdx.x;
    const int n_red_dims = p.in.rank - p.n_kept;
    int64_t base = 0, rem_o = o;
    for (int d = p.n_kept - 1; d >= 0; --d) {
        base += (rem_o % p.in.shape[d]) * p.in.stride[d];
        rem_o /= p.in.shape[d];
    }
    const int64_t r_end = min(p.n_red, (static_cast<int64_t>(s) + 1) * chunk);
    Acc<A> acc = red_identity<A>(p.op);
    for (int64_t r = static_cast<int64_t>(s) * chunk + threadIdx.x; r < r_end; r += 256) {
        int64_t off = base;
        if (n_red_dims == 1) {
            off += r * p.in.stride[p.n_kept];
        } else {
            int64_t rem = r;
            for (int d = p.in.rank - 1; d >= p.n_kept; --d) {
                off += (rem % p.in.shape[d]) * p.in.stride[d];
                rem /= p.in.shape[d];
            }
        }
        Acc<A> e;
        e.v = load_as<A>(p.in.base, p.in.dtype, off);
        e.idx = r;
        acc = red_combine<A>(p.op, acc, e);
    }
#pragma unroll
    for (int w = 16; w > 0; w >>= 1) acc = red_combine<A>(p.op, acc, red_shfl(acc, w));
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        acc = sm[0];
        for (int w = 1; w < 8; ++w) acc = red_combine<A>(p.op, acc, sm[w]);
        partials[o * splits + s] = acc;
    }
}

// One warp per output folds that output's partials (lane-strided, then a shuffle tree), then the init value.
template <typename A>
__global__ void __launch_bounds__(32) reduce_finish_kernel(const __grid_constant__ ReduceParams p, const Acc<A>* partials, int splits) {
    const int64_t o = blockIdx.x;
    Acc<A> acc = red_identity<A>(p.op);
    for (int s = threadIdx.x; s < splits; s += 32) acc = red_combine<A>(p.op, acc, partials[o * splits + s]);
#pragma unroll
    for (int w = 16; w > 0; w >>= 1) acc = red_combine<A>(p.op, acc, red_shfl(acc, w));
    if (threadIdx.x != 0) return;
    if (p.init != nullptr && p.op != MHLO_REDUCE_ARGMAX && p.op != MHLO_REDUCE_ARGMIN) {
        Acc<A> e;
        e.v = load_as<A>(p.init, p.in.dtype, 0);
        e.idx = INT64_MAX;
        acc = red_combine<A>(p.op, acc, e);
    }
    store_as<A>(p.out, p.in.dtype, o, acc.v);
    if (p.index_out != nullptr) {
        const int64_t ix = acc.idx == INT64_MAX ? 0 : acc.idx;
        if (p.index_dtype == MHLO_DT_I64) static_cast<int64_t*>(p.index_out)[o] = ix;
        else static_cast<int32_t*>(p.index_out)[o] = static_cast<int32_t>(ix);
    }
}

// ---- row gather: out[i, :] = operand[clamp(index[i]), :] (an embedding lookup) ------------------------------------
// One warp per output row, 16-byte vectors; the start index is clamped into the table like the general kernel does.
template <typename I>
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ table, const I* __restrict__ index, uint4* __restrict__ out,
                                                          int64_t n_rows, int64_t table_rows, int vecs_per_row) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); r < n_rows; r += warps) {
        int64_t src = static_cast<int64_t>(index[r]);
        src = src < 0 ? 0 : (src > table_rows - 1 ? table_rows - 1 : src);
        const uint4* from = table + src * vecs_per_row;
        uint4* to = out + r * vecs_per_row;
        for (int v = lane; v < vecs_per_row; v += 32) to[v] = __ldg(from + v);
    }
}

// ---- gather --------------------------------------------------------------------------------------------------------

struct GatherParams {
    mhlo_cuda_gather_dims d;
    int64_t operand_shape[MHLO_CUDA_MAX_RANK], indices_shape[MHLO_CUDA_MAX_RANK], out_shape[MHLO_CUDA_MAX_RANK];
    const void* operand;
    const void* indices;
    void* out;
    int64_t n;
    int32_t operand_rank, indices_rank, out_rank, elem_size, index_dtype;
};

template <typename E>
__global__ void __launch_bounds__(256) gather_kernel(const __grid_constant__ GatherParams p) {
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.n; i += step) {
        int64_t oidx[MHLO_CUDA_MAX_RANK];
        int64_t rem = i;
        for (int d = p.out_rank - 1; d >= 0; --d) { oidx[d] = rem % p.out_shape[d]; rem /= p.out_shape[d]; }
        // split the output index into batch coordinates (into start_indices) and offset coordinates
        int64_t batch[MHLO_CUDA_MAX_RANK], offs[MHLO_CUDA_MAX_RANK];
        int nb = 0, no = 0;
        for (int d = 0; d < p.out_rank; ++d) {
            bool is_off = false;
            for (int k = 0; k < p.d.n_offset_dims; ++k) is_off |= p.d.offset_dims[k] == d;
            if (is_off) offs[no++] = oidx[d]; else batch[nb++] = oidx[d];
        }
        // start index vector: indices[batch with index_vector_dim spliced in]
        int64_t start[MHLO_CUDA_MAX_RANK];
        for (int d = 0; d < p.operand_rank; ++d) start[d] = 0;
        const bool has_ivd = p.d.index_vector_dim < p.indices_rank;
        for (int k = 0; k < p.d.n_start_index_map; ++k) {
            int64_t off = 0, bi = 0;
            for (int d = 0; d < p.indices_rank; ++d) {
                int64_t c;
                if (has_ivd && d == p.d.index_vector_dim) c = k; else c = batch[bi++];
                off = off * p.indices_shape[d] + c;
            }
            const int64_t v = p.index_dtype == MHLO_DT_I64 ? static_cast<const int64_t*>(p.indices)[off]
                                                           : static_cast<const int32_t*>(p.indices)[off];
            const int od = p.d.start_index_map[k];
            const int64_t hi = p.operand_shape[od] - p.d.slice_sizes[od];
            start[od] = v < 0 ? 0 : (v > hi ? hi : v);
        }
        // batching dims: operand_batching_dims[k] takes the batch coordinate of start_indices_batching_dims[k]
        for (int k = 0; k < p.d.n_operand_batching; ++k) {
            int sd = p.d.start_indices_batching_dims[k];
            if (has_ivd && sd > p.d.index_vector_dim) --sd;
            start[p.d.operand_batching_dims[k]] = batch[sd];
        }
        // offset coordinates fill the operand dims that are neither collapsed nor batching
        int64_t src = 0;
        int oi = 0;
        for (int d = 0; d < p.operand_rank; ++d) {
            bool skip = false;
            for (int k = 0; k < p.d.n_collapsed; ++k) skip |= p.d.collapsed_slice_dims[k] == d;
            for (int k = 0; k < p.d.n_operand_batching; ++k) skip |= p.d.operand_batching_dims[k] == d;
            const int64_t c = start[d] + (skip ? 0 : offs[oi++]);
            src = src * p.operand_shape[d] + c;
        }
        static_cast<E*>(p.out)[i] = static_cast<const E*>(p.operand)[src];
    }
}

// ---- dynamic slice / update ---------------------------------------------------------------------------------------

struct DynSliceParams {
    int64_t operand_shape[MHLO_CUDA_MAX_RANK], window_shape[MHLO_CUDA_MAX_RANK];
    const void* index_ptrs[MHLO_CUDA_MAX_RANK];
    const void* src;
    void* dst;
    int64_t n;
    int32_t rank, index_dtype, update;  // update = 1: window is written into dst (operand); 0: read from src
};

template <typename E>
__global__ void __launch_bounds__(256) dyn_slice_kernel(const __grid_constant__ DynSliceParams p) {
    int64_t start[MHLO_CUDA_MAX_RANK];
    for (int d = 0; d < p.rank; ++d) {
        const int64_t v = p.index_dtype == MHLO_DT_I64 ? *static_cast<const int64_t*>(p.index_ptrs[d])
                                                       : *static_cast<const int32_t*>(p.index_ptrs[d]);
        const int64_t hi = p.operand_shape[d] - p.window_shape[d];
        start[d] = v < 0 ? 0 : (v > hi ? hi : v);
    }
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.n; i += step) {
        int64_t rem = i, off = 0, mul = 1;
        for (int d = p.rank - 1; d >= 0; --d) {
            off += (start[d] + rem % p.window_shape[d]) * mul;
            rem /= p.window_shape[d];
            mul *= p.operand_shape[d];
        }
        if (p.update) static_cast<E*>(p.dst)[off] = static_cast<const E*>(p.src)[i];
        else static_cast<E*>(p.dst)[i] = static_cast<const E*>(p.src)[off];
    }
}

// ---- any-layout dot ------------------------------------------------------------------------------------------------

struct DotParams {
    const void* a;
    const void* b;
    void* c;
    int64_t as[4], bs[4];
    int64_t batch1, m, n, k;
    int32_t in_dtype, out_dtype;
};

// 64x64 output tile per CTA, 16-deep k panels staged in shared memory in the accumulate type, 4x4 outputs per
// thread. Strides are arbitrary, so the global reads are plain element loads; this kernel is the layout-general
// and strict-precision path, not the fast one.
template <typename A>
__global__ void __launch_bounds__(256) dot_strided_kernel(const __grid_constant__ DotParams p) {
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ A sa[BK][BM + 1];
    __shared__ A sb[BK][BN + 1];
    const int64_t bz = blockIdx.z;
    const int64_t b0 = bz / p.batch1, b1 = bz % p.batch1;
    const int64_t a_base = b0 * p.as[0] + b1 * p.as[1];
    const int64_t b_base = b0 * p.bs[0] + b1 * p.bs[1];
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM, n0 = static_cast<int64_t>(blockIdx.x) * BN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    A acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = A(0);
    for (int64_t k0 = 0; k0 < p.k; k0 += BK) {
        for (int e = threadIdx.x; e < BM * BK; e += 256) {
            // A tile: pick the faster-varying coordinate by stride so that unit-stride reads coalesce
            int mi, ki;
            if (p.as[3] == 1) { ki = e % BK; mi = e / BK; } else { mi = e % BM; ki = e / BM; }
            const int64_t gm = m0 + mi, gk = k0 + ki;
            sa[ki][mi] = (gm < p.m && gk < p.k) ? load_as<A>(p.a, p.in_dtype, a_base + gm * p.as[2] + gk * p.as[3]) : A(0);
        }
        for (int e = threadIdx.x; e < BN * BK; e += 256) {
            int ni, ki;
            if (p.bs[2] == 1) { ki = e % BK; ni = e / BK; } else { ni = e % BN; ki = e / BN; }
            const int64_t gn = n0 + ni, gk = k0 + ki;
            sb[ki][ni] = (gn < p.n && gk < p.k) ? load_as<A>(p.b, p.in_dtype, b_base + gk * p.bs[2] + gn * p.bs[3]) : A(0);
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            A av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
        }
        __syncthreads();
    }
    const int64_t c_base = bz * p.m * p.n;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
            if (gm < p.m && gn < p.n) store_as<A>(p.c, p.out_dtype, c_base + gm * p.n + gn, acc[i][j]);
        }
}

int grid_for(int64_t n, int threads) {
    int64_t g = (n + threads - 1) / threads;
    const int64_t cap = static_cast<int64_t>(kNumSMs) * 32;
    return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

bool is_float_dt(int dt) { return dt == MHLO_DT_F16 || dt == MHLO_DT_F32 || dt == MHLO_DT_F64 || dt == MHLO_DT_BF16; }

}  // namespace
}  // namespace mhlo

using namespace mhlo;

// ---- batched dtype conversion ---------------------------------------------------------------------------------------

constexpr int kConvertJobsPerLaunch = 96;
constexpr int kConvertTile = 4096;  // elements per CTA: 256 threads x 16

struct ConvertTable {
    const void* src[kConvertJobsPerLaunch];
    void* dst[kConvertJobsPerLaunch];
    int64_t count[kConvertJobsPerLaunch];
    int32_t first_tile[kConvertJobsPerLaunch + 1];  // tiles of job j are [first_tile[j], first_tile[j+1])
    int8_t src_dtype[kConvertJobsPerLaunch], dst_dtype[kConvertJobsPerLaunch];
    int8_t vector_ok[kConvertJobsPerLaunch];  // both pointers 16-byte aligned
    int32_t n_jobs;
};

template <typename TI, typename TO>
__device__ __forceinline__ void convert_tile(const TI* __restrict__ src, TO* __restrict__ dst, int64_t begin, int64_t end, bool vector_ok) {
    // 16 consecutive elements per thread when the tile is full and aligned, element-wise otherwise
    if (vector_ok && end - begin == kConvertTile) {
        const int64_t i = begin + static_cast<int64_t>(threadIdx.x) * 16;
        float v[16];
        if constexpr (sizeof(TI) == 4) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 f = __ldcs(reinterpret_cast<const float4*>(src + i) + q);
                v[4 * q] = f.x; v[4 * q + 1] = f.y; v[4 * q + 2] = f.z; v[4 * q + 3] = f.w;
            }
        } else {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const uint4 u = __ldcs(reinterpret_cast<const uint4*>(src + i) + q);
                const TI* h = reinterpret_cast<const TI*>(&u);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[8 * q + e] = static_cast<float>(h[e]);
            }
        }
        if constexpr (sizeof(TO) == 4) {
#pragma unroll
            for (int q = 0; q < 4; ++q) reinterpret_cast<float4*>(dst + i)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        } else {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                uint4 u;
                TO* h = reinterpret_cast<TO*>(&u);
#pragma unroll
                for (int e = 0; e < 8; ++e) h[e] = static_cast<TO>(v[8 * q + e]);
                reinterpret_cast<uint4*>(dst + i)[q] = u;
            }
        }
        return;
    }
    for (int64_t i = begin + threadIdx.x; i < end; i += 256) dst[i] = static_cast<TO>(static_cast<float>(src[i]));
}

__global__ void __launch_bounds__(256) convert_many_kernel(const __grid_constant__ ConvertTable t) {
    const int tile = blockIdx.x;
    int lo = 0, hi = t.n_jobs - 1;  // last job whose first tile is <= tile
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (t.first_tile[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    const int j = lo;
    const int64_t begin = static_cast<int64_t>(tile - t.first_tile[j]) * kConvertTile;
    const int64_t end = min(t.count[j], begin + kConvertTile);
    const bool vec = t.vector_ok[j] != 0;
    const int sd = t.src_dtype[j], dd = t.dst_dtype[j];
#define MHLO_CONVERT_CASE(SD, TI, DD, TO) \
    if (sd == SD && dd == DD) return convert_tile<TI, TO>(static_cast<const TI*>(t.src[j]), static_cast<TO*>(t.dst[j]), begin, end, vec)
    MHLO_CONVERT_CASE(MHLO_DT_F32, float, MHLO_DT_F16, __half);
    MHLO_CONVERT_CASE(MHLO_DT_F32, float, MHLO_DT_BF16, __nv_bfloat16);
    MHLO_CONVERT_CASE(MHLO_DT_F16, __half, MHLO_DT_F32, float);
    MHLO_CONVERT_CASE(MHLO_DT_BF16, __nv_bfloat16, MHLO_DT_F32, float);
    MHLO_CONVERT_CASE(MHLO_DT_F32, float, MHLO_DT_F32, float);
    MHLO_CONVERT_CASE(MHLO_DT_F16, __half, MHLO_DT_F16, __half);
    MHLO_CONVERT_CASE(MHLO_DT_BF16, __nv_bfloat16, MHLO_DT_BF16, __nv_bfloat16);
#undef MHLO_CONVERT_CASE
}

extern "C" {

static int elementwise_impl(const mhlo_cuda_view* inputs, int32_t n_inputs, const mhlo_cuda_ew_inst* prog,
                            int32_t n_insts, void* out_dev, int32_t out_dtype, const int64_t* out_shape,
                            int32_t out_rank, const int64_t* out_strides, mhlo_cuda_stream_t stream) {
    if (n_inputs < 0 || n_inputs > MHLO_CUDA_EW_MAX_INPUTS || n_insts < 1 || n_insts > MHLO_CUDA_EW_MAX_INSTS)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "elementwise: %d inputs / %d instructions outside the limits (%d / %d)",
                    n_inputs, n_insts, MHLO_CUDA_EW_MAX_INPUTS, MHLO_CUDA_EW_MAX_INSTS);
    if (out_rank < 0 || out_rank > MHLO_CUDA_MAX_RANK)
        return fail(MHLO_CUDA_UNSUPPORTED, "elementwise: rank %d above %d", out_rank, MHLO_CUDA_MAX_RANK);
    if (mhlo_cuda_dtype_size(out_dtype) == 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "elementwise: bad output dtype %d", out_dtype);
    EwParams p;
    memset(&p, 0, sizeof p);
    p.n = 1;
    p.rank = out_rank;
    for (int d = 0; d < out_rank; ++d) {
        if (out_shape[d] < 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "elementwise: negative extent");
        p.out_shape[d] = out_shape[d];
        p.n *= out_shape[d];
    }
    if (p.n == 0) return MHLO_CUDA_OK;
    if (out_dev == nullptr) return fail(MHLO_CUDA_INVALID_ARGUMENT, "elementwise: null output");
    bool any_f64 = out_dtype == MHLO_DT_F64, any_float = is_float_dt(out_dtype), any_u64 = out_dtype == MHLO_DT_UI64;
    bool all_bool = out_dtype == MHLO_DT_I1;
    for (int k = 0; k < n_inputs; ++k) {
        if (inputs[k].rank != out_rank)
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "elementwise: input %d has rank %d, output has %d", k, inputs[k].rank, out_rank);
        if (inputs[k].base == nullptr) return fail(MHLO_CUDA_INVALID_ARGUMENT, "elementwise: input %d is null", k);
        if (mhlo_cuda_dtype_size(inputs[k].dtype) == 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "elementwise: bad dtype");
        p.in[k] = inputs[k];
        any_f64 |= inputs[k].dtype == MHLO_DT_F64;
        any_float |= is_float_dt(inputs[k].dtype);
        any_u64 |= inputs[k].dtype == MHLO_DT_UI64;
        all_bool &= inputs[k].dtype == MHLO_DT_I1;
    }
    for (int k = 0; k < n_insts; ++k) {
        const mhlo_cuda_ew_inst& in = prog[k];
        const int limit = n_inputs + k;
        if (in.op < 0 || in.op >= MHLO_EW_OP_COUNT) return fail(MHLO_CUDA_INVALID_ARGUMENT, "elementwise: bad opcode %d", in.op);
        if (in.op == MHLO_EW_IOTA && (in.imm < 0 || in.imm >= out_rank))
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "elementwise: iota dimension out of range");
        const bool nullary = in.op == MHLO_EW_IMM || in.op == MHLO_EW_IOTA;
        if (!nullary && (in.a < 0 || in.a >= limit || in.b < 0 || in.b >= (limit > 0 ? limit : 1) || in.c < 0 || in.c >= (limit > 0 ? limit : 1)))
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "elementwise: instruction %d reads a register that is not defined yet", k);
        p.prog[k] = in;
        if (nullary) { p.prog[k].a = p.prog[k].b = p.prog[k].c = 0; }
    }
    p.n_inputs = n_inputs;
    p.n_insts = n_insts;
    p.out = out_dev;
    p.out_dtype = out_dtype;
    p.unsigned_mode = any_u64;
    p.int_bits = static_cast<int>(8 * mhlo_cuda_dtype_size(n_inputs > 0 ? inputs[0].dtype : out_dtype));
    p.bool_mode = all_bool;
    if (out_strides != nullptr) {
        p.out_strided = 1;
        for (int d = 0; d < out_rank; ++d) p.out_stride[d] = out_strides[d];
    }
    // IOTA addresses output dimensions by their original number: keep the shape as is when a program uses it
    bool uses_iota = false;
    for (int k = 0; k < n_insts; ++k) uses_iota |= prog[k].op == MHLO_EW_IOTA;
    if (!uses_iota) collapse_dims(&p);
    else
        for (int k = 0; k < n_inputs; ++k) {
            bool dense = true;
            int64_t expect = 1;
            for (int d = out_rank - 1; d >= 0; --d) {
                if (p.out_shape[d] != 1 && p.in[k].stride[d] != expect) { dense = false; break; }
                expect *= p.out_shape[d];
            }
            if (dense) p.contiguous_mask |= 1 << k;
        }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // fast path: one non-iota instruction over dense / scalar float inputs of one dtype
    if (n_insts == 1 && !uses_iota && out_strides == nullptr && !any_f64 && n_inputs >= 1 && n_inputs <= 3 &&
        (out_dtype == MHLO_DT_F32 || out_dtype == MHLO_DT_F16 || out_dtype == MHLO_DT_BF16) && aligned16(out_dev)) {
        const int in_dt = inputs[0].dtype;
        bool ok = in_dt == MHLO_DT_F32 || in_dt == MHLO_DT_F16 || in_dt == MHLO_DT_BF16;
        EwVecParams vp;
        memset(&vp, 0, sizeof vp);
        for (int k = 0; k < n_inputs && ok; ++k) {
            bool scalar = true;
            for (int d = 0; d < p.rank; ++d) scalar &= p.in[k].stride[d] == 0;
            const bool dense = (p.contiguous_mask >> k) & 1;
            // broadcast over leading dimensions, dense over the rest: the input repeats with a fixed period
            int64_t period = 0;
            if (!scalar && !dense) {
                int q = 0;
                while (q < p.rank && p.in[k].stride[q] == 0) ++q;
                int64_t expect = 1;
                bool tail_dense = q > 0 && q < p.rank;
                for (int d = p.rank - 1; d >= q && tail_dense; --d) {
                    tail_dense = p.out_shape[d] == 1 || p.in[k].stride[d] == expect;
                    expect *= p.out_shape[d];
                }
                if (tail_dense && expect % 8 == 0) period = expect;
            }
            vp.period[k] = period;
            ok = p.in[k].dtype == in_dt && (scalar || ((dense || period > 0) && aligned16(p.in[k].base)));
            if (scalar && !(dense && p.n == 1)) vp.scalar_mask |= 1 << k;
            vp.in[k] = p.in[k].base;
        }
        // instruction operands must name the inputs in order (a = 0, b = 1, c = 2), which is how single ops are built
        ok = ok && prog[0].a == 0 && (n_inputs < 2 || prog[0].b == 1) && (n_inputs < 3 || prog[0].c == 2);
        if (ok) {
            vp.out = out_dev; vp.n = p.n; vp.n_inputs = n_inputs; vp.op = prog[0].op; vp.imm = prog[0].imm;
            const int vgrid = grid_for((p.n + 7) / 8, 256);
            bool launched = false;
            if (in_dt == MHLO_DT_F32) launched = launch_ew_vec_out<float>(out_dtype, vp, vgrid, s);
            else if (in_dt == MHLO_DT_F16) launched = launch_ew_vec_out<__half>(out_dtype, vp, vgrid, s);
            else launched = launch_ew_vec_out<__nv_bfloat16>(out_dtype, vp, vgrid, s);
            if (launched) {
                MHLO_CUDA_CHECK_LAUNCH("elementwise_vec");
                return MHLO_CUDA_OK;
            }
        }
    }
    const int grid = grid_for(p.n, 256);
    if (any_f64) ew_kernel<double><<<grid, 256, 0, s>>>(p);
    else if (any_float) ew_kernel<float><<<grid, 256, 0, s>>>(p);
    else ew_kernel<int64_t><<<grid, 256, 0, s>>>(p);
    MHLO_CUDA_CHECK_LAUNCH("elementwise");
    return MHLO_CUDA_OK;
}

int mhlo_cuda_elementwise(const mhlo_cuda_view* inputs, int32_t n_inputs, const mhlo_cuda_ew_inst* prog,
                          int32_t n_insts, void* out_dev, int32_t out_dtype, const int64_t* out_shape,
                          int32_t out_rank, mhlo_cuda_stream_t stream) {
    return elementwise_impl(inputs, n_inputs, prog, n_insts, out_dev, out_dtype, out_shape, out_rank, nullptr, stream);
}

int mhlo_cuda_elementwise_to_view(const mhlo_cuda_view* inputs, int32_t n_inputs, const mhlo_cuda_ew_inst* prog,
                                  int32_t n_insts, const mhlo_cuda_view* out, mhlo_cuda_stream_t stream) {
    if (!out || out->rank < 0 || out->rank > MHLO_CUDA_MAX_RANK)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "elementwise_to_view: bad destination view");
    return elementwise_impl(inputs, n_inputs, prog, n_insts, const_cast<void*>(out->base), out->dtype, out->shape,
                            out->rank, out->stride, stream);
}

namespace {
// Enqueues both kernels of a split reduce over `scratch` (plan.scratch_bytes, no initial contents required).
inline int launch_split_reduce(const ReduceParams& p, const SplitPlan& plan, void* scratch, cudaStream_t s) {
    const dim3 grid(static_cast<unsigned>(plan.splits), static_cast<unsigned>(p.n_out));
    const int dt = p.in.dtype;
#define MHLO_SPLIT_LAUNCH(A)                                                                                         \
    do {                                                                                                             \
        reduce_split_kernel<A><<<grid, 256, 0, s>>>(p, static_cast<Acc<A>*>(scratch), plan.splits, plan.chunk);       \
        reduce_finish_kernel<A><<<static_cast<unsigned>(p.n_out), 32, 0, s>>>(p, static_cast<const Acc<A>*>(scratch), plan.splits); \
    } while (0)
    if (dt == MHLO_DT_F64) MHLO_SPLIT_LAUNCH(double);
    else if (is_float_dt(dt)) MHLO_SPLIT_LAUNCH(float);
    else if (mhlo_cuda_dtype_size(dt) != 0) MHLO_SPLIT_LAUNCH(int64_t);
    else return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce: bad dtype %d", dt);
#undef MHLO_SPLIT_LAUNCH
    MHLO_CUDA_CHECK_LAUNCH("reduce (split)");
    return MHLO_CUDA_OK;
}

// The split path pays off when the single-stage kernel would leave most SMs idle on a long reduction.
inline bool wants_split(int64_t n_out, int64_t n_red) { return n_out <= 148 && n_red >= (1 << 16) && n_out * 1024 <= n_red; }

}  // namespace

int mhlo_cuda_reduce(const mhlo_cuda_view* in, int32_t n_kept, int32_t op, const void* init_dev, void* out_dev,
                     void* index_out_dev, int32_t index_dtype, mhlo_cuda_stream_t stream) {
    if (!in || in->rank < 0 || in->rank > MHLO_CUDA_MAX_RANK || n_kept < 0 || n_kept > in->rank)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce: bad view or kept-dimension count");
    if (op < MHLO_REDUCE_SUM || op > MHLO_REDUCE_ARGMIN) return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce: bad op %d", op);
    const bool arg = op == MHLO_REDUCE_ARGMAX || op == MHLO_REDUCE_ARGMIN;
    if (arg && (index_out_dev == nullptr || (index_dtype != MHLO_DT_I32 && index_dtype != MHLO_DT_I64)))
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce: argmax/argmin need an I32 or I64 index output");
    ReduceParams p;
    memset(&p, 0, sizeof p);
    p.in = *in;
    p.n_kept = n_kept;
    p.op = op;
    p.init = init_dev;
    p.out = out_dev;
    p.index_out = arg ? index_out_dev : nullptr;
    p.index_dtype = index_dtype;
    p.n_out = 1;
    p.n_red = 1;
    for (int d = 0; d < in->rank; ++d) {
        if (in->shape[d] < 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce: negative extent");
        (d < n_kept ? p.n_out : p.n_red) *= in->shape[d];
    }
    if (p.n_out == 0) return MHLO_CUDA_OK;
    if (out_dev == nullptr || (in->base == nullptr && p.n_red > 0))
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int dt = in->dtype;
    SplitPlan plan;
    if (wants_split(p.n_out, p.n_red) && plan_split(p.n_out, p.n_red, 0, &plan) && plan.splits > 1) {
        // partial accumulators live in stream-ordered scratch: allocated, used and released on `stream`
        void* scratch = nullptr;
        MHLO_CUDA_TRY(cudaMallocAsync(&scratch, plan.scratch_bytes, s), MHLO_CUDA_BUFFER_FAILED);
        const int st = launch_split_reduce(p, plan, scratch, s);
        MHLO_CUDA_TRY(cudaFreeAsync(scratch, s), MHLO_CUDA_EXECUTION_FAILED);
        return st;
    }
#define MHLO_RED_LAUNCH(A)                                                                                   \
    do {                                                                                                     \
        if (p.n_red >= 2048 && p.n_out < 148 * 16)                                                           \
            reduce_kernel<A, 256><<<static_cast<int>(p.n_out < 148 * 32 ? p.n_out : 148 * 32), 256, 0, s>>>(p); \
        else if (p.n_red >= 64)                                                                              \
            reduce_kernel<A, 32><<<grid_for(p.n_out, 8), 256, 0, s>>>(p);                                    \
        else                                                                                                 \
            reduce_kernel<A, 1><<<grid_for(p.n_out, 256), 256, 0, s>>>(p);                                   \
    } while (0)
    if (dt == MHLO_DT_F64) MHLO_RED_LAUNCH(double);
    else if (is_float_dt(dt)) MHLO_RED_LAUNCH(float);
    else if (mhlo_cuda_dtype_size(dt) != 0) MHLO_RED_LAUNCH(int64_t);
    else return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce: bad dtype %d", dt);
#undef MHLO_RED_LAUNCH
    MHLO_CUDA_CHECK_LAUNCH("reduce");
    return MHLO_CUDA_OK;
}

int mhlo_cuda_convert_many(const mhlo_cuda_convert_job* jobs, int32_t n_jobs, mhlo_cuda_stream_t stream) {
    if (n_jobs < 0 || (n_jobs > 0 && jobs == nullptr)) return fail(MHLO_CUDA_INVALID_ARGUMENT, "convert_many: bad job list");
    auto ok_dtype = [](int d) { return d == MHLO_DT_F32 || d == MHLO_DT_F16 || d == MHLO_DT_BF16; };
    for (int32_t j = 0; j < n_jobs; ++j) {
        const mhlo_cuda_convert_job& job = jobs[j];
        if (job.count < 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "convert_many: job %d has a negative count", j);
        if (job.count > 0 && (job.src == nullptr || job.dst == nullptr)) return fail(MHLO_CUDA_INVALID_ARGUMENT, "convert_many: job %d has a null pointer", j);
        const bool pair_ok = ok_dtype(job.src_dtype) && ok_dtype(job.dst_dtype) &&
                             (job.src_dtype == job.dst_dtype || job.src_dtype == MHLO_DT_F32 || job.dst_dtype == MHLO_DT_F32);
        if (!pair_ok) return fail(MHLO_CUDA_UNSUPPORTED, "convert_many: job %d converts dtype %d to %d", j, job.src_dtype, job.dst_dtype);
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int32_t j = 0;
    while (j < n_jobs) {
        ConvertTable t;
        memset(&t, 0, sizeof t);
        int64_t tiles = 0;
        int n = 0;
        for (; j < n_jobs && n < kConvertJobsPerLaunch; ++j) {
            const mhlo_cuda_convert_job& job = jobs[j];
            if (job.count == 0) continue;
            const int64_t job_tiles = (job.count + kConvertTile - 1) / kConvertTile;
            if (tiles + job_tiles > 0x7fffffff) {
                if (n == 0) return fail(MHLO_CUDA_UNSUPPORTED, "convert_many: job %d is too large for one launch", j);
                break;
            }
            t.src[n] = job.src;
            t.dst[n] = job.dst;
            t.count[n] = job.count;
            t.src_dtype[n] = static_cast<int8_t>(job.src_dtype);
            t.dst_dtype[n] = static_cast<int8_t>(job.dst_dtype);
            t.vector_ok[n] = aligned16(job.src) && aligned16(job.dst);
            t.first_tile[n] = static_cast<int32_t>(tiles);
            tiles += job_tiles;
            ++n;
        }
        if (n == 0) continue;
        t.first_tile[n] = static_cast<int32_t>(tiles);
        t.n_jobs = n;
        convert_many_kernel<<<static_cast<unsigned>(tiles), 256, 0, s>>>(t);
        MHLO_CUDA_CHECK_LAUNCH("convert_many");
    }
    return MHLO_CUDA_OK;
}

// ---- split reduce on scratch that is part of the library image -----------------------------------------------------
// Some hosts must not trigger a device allocation while they run: a serving loop that has handed every free byte
// of HBM to its own pool and treats any further allocation as a fault, or code that is already between
// cudaStreamBeginCapture and EndCapture on a stream whose device has no memory pool configured. For them the
// partial accumulators of the split reduce live in a fixed array inside this module instead of coming from the
// stream-ordered allocator. The price: one array per device, so two calls that overlap in time on the same device
// (different streams, or different threads) overwrite each other's partials.
constexpr size_t kStaticScratchBytes = 64 * 1024;
static __device__ __align__(256) unsigned char g_reduce_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_scratch_mu;
void* g_static_scratch_ptr[kMaxDevices] = {};

// Address of the current device's copy of the array; looked up once per device, with that device current.
int static_scratch_for_current_device(void** out) {
    int dev = 0;
    MHLO_CUDA_TRY(cudaGetDevice(&dev), MHLO_CUDA_NO_DEVICE);
    if (dev < 0 || dev >= kMaxDevices) return fail(MHLO_CUDA_UNSUPPORTED, "reduce_static_scratch: device ordinal %d is beyond %d", dev, kMaxDevices);
    std::lock_guard<std::mutex> lock(g_static_scratch_mu);
    if (g_static_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        MHLO_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_reduce_static_scratch), MHLO_CUDA_EXECUTION_FAILED);
        if (ptr == nullptr) return fail(MHLO_CUDA_EXECUTION_FAILED, "reduce_static_scratch: the scratch symbol has no address on device %d", dev);
        g_static_scratch_ptr[dev] = ptr;
    }
    *out = g_static_scratch_ptr[dev];
    return MHLO_CUDA_OK;
}
}  // namespace

int mhlo_cuda_reduce_static_scratch(const mhlo_cuda_view* in, int32_t n_kept, int32_t op, const void* init_dev, void* out_dev,
                                    void* index_out_dev, int32_t index_dtype, int32_t splits, mhlo_cuda_stream_t stream) {
    if (!in || in->rank < 0 || in->rank > MHLO_CUDA_MAX_RANK || n_kept < 0 || n_kept > in->rank)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce_static_scratch: bad view or kept-dimension count");
    if (op < MHLO_REDUCE_SUM || op > MHLO_REDUCE_ARGMIN) return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce_static_scratch: bad op %d", op);
    if (splits < 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce_static_scratch: negative split count");
    const bool arg = op == MHLO_REDUCE_ARGMAX || op == MHLO_REDUCE_ARGMIN;
    if (arg && (index_out_dev == nullptr || (index_dtype != MHLO_DT_I32 && index_dtype != MHLO_DT_I64)))
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce_static_scratch: argmax/argmin need an I32 or I64 index output");
    if (mhlo_cuda_dtype_size(in->dtype) == 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce_static_scratch: bad dtype %d", in->dtype);
    ReduceParams p;
    memset(&p, 0, sizeof p);
    p.in = *in;
    p.n_kept = n_kept;
    p.op = op;
    p.init = init_dev;
    p.out = out_dev;
    p.index_out = arg ? index_out_dev : nullptr;
    p.index_dtype = index_dtype;
    p.n_out = 1;
    p.n_red = 1;
    for (int d = 0; d < in->rank; ++d) {
        if (in->shape[d] < 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce_static_scratch: negative extent");
        (d < n_kept ? p.n_out : p.n_red) *= in->shape[d];
    }
    if (p.n_out == 0) return MHLO_CUDA_OK;
    if (p.n_red == 0) return fail(MHLO_CUDA_UNSUPPORTED, "reduce_static_scratch: empty reduced range; use mhlo_cuda_reduce");
    if (out_dev == nullptr || in->base == nullptr) return fail(MHLO_CUDA_INVALID_ARGUMENT, "reduce_static_scratch: null pointer");
    SplitPlan plan;
    if (!plan_split(p.n_out, p.n_red, splits, &plan))
        return fail(MHLO_CUDA_UNSUPPORTED, "reduce_static_scratch: %lld outputs are more than the 65535 this entry point takes", static_cast<long long>(p.n_out));
    if (plan.scratch_bytes > kStaticScratchBytes)
        return fail(MHLO_CUDA_UNSUPPORTED,
                    "reduce_static_scratch: %lld outputs x %d segments need %zu bytes of partial accumulators, the built-in scratch holds %zu; "
                    "ask for fewer segments or use mhlo_cuda_reduce",
                    static_cast<long long>(p.n_out), plan.splits, plan.scratch_bytes, kStaticScratchBytes);
    void* scratch = nullptr;
    const int st = static_scratch_for_current_device(&scratch);
    if (st != MHLO_CUDA_OK) return st;
    // nothing in the scratch has to start at zero: the first kernel writes every partial the second one reads
    return launch_split_reduce(p, plan, scratch, static_cast<cudaStream_t>(stream));
}

int mhlo_cuda_gather(const void* operand_dev, int32_t elem_size, const int64_t* operand_shape, int32_t operand_rank,
                     const void* indices_dev, int32_t index_dtype, const int64_t* indices_shape,
                     int32_t indices_rank, const mhlo_cuda_gather_dims* dims, void* out_dev,
                     const int64_t* out_shape, int32_t out_rank, mhlo_cuda_stream_t stream) {
    if (!dims || operand_rank < 0 || operand_rank > MHLO_CUDA_MAX_RANK || indices_rank < 0 ||
        indices_rank > MHLO_CUDA_MAX_RANK || out_rank < 0 || out_rank > MHLO_CUDA_MAX_RANK)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "gather: bad rank");
    if (index_dtype != MHLO_DT_I32 && index_dtype != MHLO_DT_I64 && index_dtype != MHLO_DT_UI32)
        return fail(MHLO_CUDA_UNSUPPORTED, "gather: index dtype %d (I32, UI32 or I64 expected)", index_dtype);
    if (dims->n_offset_dims > MHLO_CUDA_MAX_RANK || dims->n_collapsed > MHLO_CUDA_MAX_RANK ||
        dims->n_operand_batching > MHLO_CUDA_MAX_RANK || dims->n_start_index_map > MHLO_CUDA_MAX_RANK)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "gather: dimension-number list too long");
    {   // the dimension numbers must account for every output and operand dimension, or the kernel would index outside
        const bool has_ivd = dims->index_vector_dim < indices_rank;
        if (dims->index_vector_dim < 0 || dims->index_vector_dim > indices_rank)
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "gather: index_vector_dim %d for indices of rank %d", dims->index_vector_dim, indices_rank);
        if (dims->n_offset_dims + dims->n_collapsed + dims->n_operand_batching != operand_rank)
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "gather: offset, collapsed and batching dimensions do not cover the operand's rank %d", operand_rank);
        if (out_rank != dims->n_offset_dims + indices_rank - (has_ivd ? 1 : 0))
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "gather: result rank %d does not match %d offset + %d batch dimensions", out_rank,
                        dims->n_offset_dims, indices_rank - (has_ivd ? 1 : 0));
        const int64_t index_len = has_ivd ? indices_shape[dims->index_vector_dim] : 1;
        if (dims->n_start_index_map > index_len)
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "gather: start_index_map has %d entries, index vectors have %lld", dims->n_start_index_map,
                        static_cast<long long>(index_len));
        for (int k = 0; k < dims->n_offset_dims; ++k)
            if (dims->offset_dims[k] < 0 || dims->offset_dims[k] >= out_rank)
                return fail(MHLO_CUDA_INVALID_ARGUMENT, "gather: offset_dims entry out of range");
        int oi = 0;  // the offset dimensions of the result walk the slice: their extents must be the slice sizes
        for (int d = 0; d < operand_rank; ++d) {
            bool skip = false;
            for (int k = 0; k < dims->n_collapsed; ++k) skip |= dims->collapsed_slice_dims[k] == d;
            for (int k = 0; k < dims->n_operand_batching; ++k) skip |= dims->operand_batching_dims[k] == d;
            if (skip) continue;
            if (oi >= dims->n_offset_dims || out_shape[dims->offset_dims[oi]] != dims->slice_sizes[d])
                return fail(MHLO_CUDA_INVALID_ARGUMENT, "gather: the result's offset dimensions do not match slice_sizes (operand dimension %d)", d);
            ++oi;
        }
        int bi = 0;  // the batch dimensions of the result walk `indices`: their extents must agree
        for (int d = 0; d < out_rank; ++d) {
            bool is_off = false;
            for (int k = 0; k < dims->n_offset_dims; ++k) is_off |= dims->offset_dims[k] == d;
            if (is_off) continue;
            if (has_ivd && bi == dims->index_vector_dim) ++bi;
            if (bi >= indices_rank || out_shape[d] != indices_shape[bi])
                return fail(MHLO_CUDA_INVALID_ARGUMENT, "gather: dimension %d of the result does not match the start indices", d);
            ++bi;
        }
    }
    GatherParams p;
    memset(&p, 0, sizeof p);
    p.d = *dims;
    p.n = 1;
    for (int d = 0; d < operand_rank; ++d) {
        p.operand_shape[d] = operand_shape[d];
        if (dims->slice_sizes[d] < 0 || dims->slice_sizes[d] > operand_shape[d])
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "gather: slice size %lld exceeds operand extent %lld",
                        (long long)dims->slice_sizes[d], (long long)operand_shape[d]);
    }
    for (int d = 0; d < indices_rank; ++d) p.indices_shape[d] = indices_shape[d];
    for (int d = 0; d < out_rank; ++d) { p.out_shape[d] = out_shape[d]; p.n *= out_shape[d]; }
    for (int k = 0; k < dims->n_start_index_map; ++k)
        if (dims->start_index_map[k] < 0 || dims->start_index_map[k] >= operand_rank)
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "gather: start_index_map entry out of range");
    if (p.n == 0) return MHLO_CUDA_OK;
    if (!operand_dev || !indices_dev || !out_dev) return fail(MHLO_CUDA_INVALID_ARGUMENT, "gather: null pointer");
    p.operand = operand_dev; p.indices = indices_dev; p.out = out_dev;
    p.operand_rank = operand_rank; p.indices_rank = indices_rank; p.out_rank = out_rank;
    p.elem_size = elem_size; p.index_dtype = index_dtype == MHLO_DT_UI32 ? MHLO_DT_I32 : index_dtype;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Embedding-style lookup: whole rows of a [rows, ...] table selected by one index each.
    {
        bool rows_only = operand_rank >= 2 && dims->n_collapsed == 1 && dims->collapsed_slice_dims[0] == 0 && dims->n_start_index_map == 1 &&
                         dims->start_index_map[0] == 0 && dims->n_operand_batching == 0 && dims->slice_sizes[0] == 1 &&
                         dims->n_offset_dims == operand_rank - 1 && out_rank >= operand_rank - 1;
        int64_t row_elems = 1;
        for (int d = 1; rows_only && d < operand_rank; ++d) {
            rows_only = dims->slice_sizes[d] == operand_shape[d] && dims->offset_dims[d - 1] == out_rank - (operand_rank - 1) + (d - 1);
            row_elems *= operand_shape[d];
        }
        rows_only = rows_only && (dims->index_vector_dim == indices_rank ||
                                  (dims->index_vector_dim == indices_rank - 1 && indices_rank >= 1 && indices_shape[indices_rank - 1] == 1));
        const int64_t row_bytes = row_elems * elem_size;
        if (rows_only && row_bytes > 0 && row_bytes % 16 == 0 && row_bytes / 16 <= 0x7fffffff && aligned16(operand_dev) && aligned16(out_dev)) {
            const int64_t n_rows = p.n / row_elems;
            const int vecs = static_cast<int>(row_bytes / 16);
            const int grid_rows = static_cast<int>(std::min<int64_t>((n_rows + 7) / 8, 148 * 16));
            if (p.index_dtype == MHLO_DT_I64)
                gather_rows_kernel<int64_t><<<grid_rows, 256, 0, s>>>(static_cast<const uint4*>(operand_dev), static_cast<const int64_t*>(indices_dev),
                                                                     static_cast<uint4*>(out_dev), n_rows, operand_shape[0], vecs);
            else if (index_dtype == MHLO_DT_UI32)
                gather_rows_kernel<uint32_t><<<grid_rows, 256, 0, s>>>(static_cast<const uint4*>(operand_dev), static_cast<const uint32_t*>(indices_dev),
                                                                      static_cast<uint4*>(out_dev), n_rows, operand_shape[0], vecs);
            else
                gather_rows_kernel<int32_t><<<grid_rows, 256, 0, s>>>(static_cast<const uint4*>(operand_dev), static_cast<const int32_t*>(indices_dev),
                                                                     static_cast<uint4*>(out_dev), n_rows, operand_shape[0], vecs);
            MHLO_CUDA_CHECK_LAUNCH("gather (rows)");
            return MHLO_CUDA_OK;
        }
    }
    const int grid = grid_for(p.n, 256);
    switch (elem_size) {
        case 1: gather_kernel<uint8_t><<<grid, 256, 0, s>>>(p); break;
        case 2: gather_kernel<uint16_t><<<grid, 256, 0, s>>>(p); break;
        case 4: gather_kernel<uint32_t><<<grid, 256, 0, s>>>(p); break;
        case 8: gather_kernel<uint64_t><<<grid, 256, 0, s>>>(p); break;
        default: return fail(MHLO_CUDA_INVALID_ARGUMENT, "gather: element size %d", elem_size);
    }
    MHLO_CUDA_CHECK_LAUNCH("gather");
    return MHLO_CUDA_OK;
}

static int dyn_slice_common(const void* src, void* dst, int32_t elem_size, const int64_t* operand_shape, int32_t rank,
                            const int64_t* window_shape, const void* const* index_devs, int32_t index_dtype, int update,
                            mhlo_cuda_stream_t stream, const char* what) {
    if (rank < 0 || rank > MHLO_CUDA_MAX_RANK) return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: bad rank", what);
    if (index_dtype != MHLO_DT_I32 && index_dtype != MHLO_DT_I64) return fail(MHLO_CUDA_UNSUPPORTED, "%s: index dtype %d", what, index_dtype);
    DynSliceParams p;
    memset(&p, 0, sizeof p);
    p.n = 1;
    for (int d = 0; d < rank; ++d) {
        if (window_shape[d] < 0 || window_shape[d] > operand_shape[d])
            return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: window extent %lld exceeds operand extent %lld", what,
                        (long long)window_shape[d], (long long)operand_shape[d]);
        if (!index_devs[d]) return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: null start index", what);
        p.operand_shape[d] = operand_shape[d];
        p.window_shape[d] = window_shape[d];
        p.index_ptrs[d] = index_devs[d];
        p.n *= window_shape[d];
    }
    if (p.n == 0) return MHLO_CUDA_OK;
    if (!src || !dst) return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: null pointer", what);
    p.src = src; p.dst = dst; p.rank = rank; p.index_dtype = index_dtype; p.update = update;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int grid = grid_for(p.n, 256);
    switch (elem_size) {
        case 1: dyn_slice_kernel<uint8_t><<<grid, 256, 0, s>>>(p); break;
        case 2: dyn_slice_kernel<uint16_t><<<grid, 256, 0, s>>>(p); break;
        case 4: dyn_slice_kernel<uint32_t><<<grid, 256, 0, s>>>(p); break;
        case 8: dyn_slice_kernel<uint64_t><<<grid, 256, 0, s>>>(p); break;
        default: return fail(MHLO_CUDA_INVALID_ARGUMENT, "%s: element size %d", what, elem_size);
    }
    MHLO_CUDA_CHECK_LAUNCH(what);
    return MHLO_CUDA_OK;
}

int mhlo_cuda_dynamic_slice(const void* operand_dev, int32_t elem_size, const int64_t* operand_shape, int32_t rank,
                            const void* const* index_devs, int32_t index_dtype, const int64_t* slice_sizes,
                            void* out_dev, mhlo_cuda_stream_t stream) {
    return dyn_slice_common(operand_dev, out_dev, elem_size, operand_shape, rank, slice_sizes, index_devs, index_dtype, 0,
                            stream, "dynamic_slice");
}

int mhlo_cuda_dynamic_update_slice(void* operand_inout_dev, int32_t elem_size, const int64_t* operand_shape,
                                   int32_t rank, const void* update_dev, const int64_t* update_shape,
                                   const void* const* index_devs, int32_t index_dtype, mhlo_cuda_stream_t stream) {
    return dyn_slice_common(update_dev, operand_inout_dev, elem_size, operand_shape, rank, update_shape, index_devs,
                            index_dtype, 1, stream, "dynamic_update_slice");
}

int mhlo_cuda_dot_strided(int32_t in_dtype, int32_t out_dtype, const void* a_dev, const int64_t a_strides[4],
                          const void* b_dev, const int64_t b_strides[4], void* c_dev, int64_t batch0,
                          int64_t batch1, int64_t m, int64_t n, int64_t k, mhlo_cuda_stream_t stream) {
    if (batch0 < 0 || batch1 < 0 || m < 0 || n < 0 || k < 0) return fail(MHLO_CUDA_INVALID_ARGUMENT, "dot: negative extent");
    if (mhlo_cuda_dtype_size(in_dtype) == 0 || mhlo_cuda_dtype_size(out_dtype) == 0)
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "dot: bad dtype");
    if (batch0 * batch1 * m * n == 0) return MHLO_CUDA_OK;
    if (!c_dev || (k > 0 && (!a_dev || !b_dev))) return fail(MHLO_CUDA_INVALID_ARGUMENT, "dot: null pointer");
    if (batch0 * batch1 > 65535) return fail(MHLO_CUDA_UNSUPPORTED, "dot: more than 65535 batch entries");
    DotParams p;
    p.a = a_dev; p.b = b_dev; p.c = c_dev;
    for (int i = 0; i < 4; ++i) { p.as[i] = a_strides[i]; p.bs[i] = b_strides[i]; }
    p.batch1 = batch1; p.m = m; p.n = n; p.k = k; p.in_dtype = in_dtype; p.out_dtype = out_dtype;
    dim3 grid(static_cast<unsigned>((n + 63) / 64), static_cast<unsigned>((m + 63) / 64), static_cast<unsigned>(batch0 * batch1));
    if (grid.y > 65535) return fail(MHLO_CUDA_UNSUPPORTED, "dot: M too large for the general-layout kernel");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (in_dtype == MHLO_DT_F64) dot_strided_kernel<double><<<grid, 256, 0, s>>>(p);
    else if (is_float_dt(in_dtype)) dot_strided_kernel<float><<<grid, 256, 0, s>>>(p);
    else dot_strided_kernel<int64_t><<<grid, 256, 0, s>>>(p);
    MHLO_CUDA_CHECK_LAUNCH("dot_strided");
    return MHLO_CUDA_OK;
}

}  // extern "C"
