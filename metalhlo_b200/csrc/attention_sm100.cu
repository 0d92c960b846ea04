// Fused flash attention on tcgen05: O = softmax(scale * Q K^T [causal]) V for bf16 / f16, head_dim 64 or 128, fp32
// softmax statistics and fp32 accumulation in TMEM. The S^2 score matrix never reaches HBM.
//
// One CTA owns 256 query rows of one (batch, head) as two halves of 128 rows and walks the keys in blocks of 64:
//   warp 0 (one lane)   TMA producer: Q once (both halves), then K_j and V_j tiles through 3-stage rings
//   warp 1 (one lane)   MMA issuer, software-pipelined over the two halves:
//                         S_h(j+1) = Q_h K_{j+1}^T   (tcgen05.mma M128 N64, K-major operands, into TMEM columns S_h)
//                         O_h     += P_h(j) V_j      (M128 N=D, P from shared memory, V N-major, accumulates in TMEM)
//                       so the tensor pipe works on one half while the other half's softmax runs
//   warps 2-5 / 6-9     softmax warpgroups for half 0 / 1; a thread owns one query row: tcgen05.ld of its 64 scores,
//                       running maximum, exp2, row sum, P packed to 16 bit and written to shared memory in the
//                       128-byte-swizzled K-major layout the PV MMA reads. The maximum used in the exponent is only
//                       advanced when it grew by more than 2^8 ("lazy rescale"): only then is O rescaled in TMEM
//                       (tcgen05.ld, multiply, tcgen05.st).
// Causal masking skips key blocks right of the diagonal and masks inside diagonal blocks; ragged sequence ends are
// zero-filled by TMA and masked to -inf. Every mbarrier wait is bounded.
//
// Algorithmic work: 4*B*H*Sq*Sk*D FLOP (half of that, plus the diagonal, when causal); HBM bytes: Q, K, V read once
// per CTA column (K/V re-reads across query blocks are served by L2), O written once.
#include <algorithm>
#include <string>

#include "contraction.cuh"
#include "tc_ptx.cuh"

namespace mhlo {
namespace {

constexpr int kBlockM = 128;     // query rows per half
constexpr int kHalves = 2;
constexpr int kBlockN = 64;      // keys per step
constexpr int kKvStages = 3;
constexpr int kAttnThreads = 32 * (2 + 4 * kHalves);
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;  // in log2 units: exponentials stay below 2^8 between rescales

__device__ int g_attn_error = 0;

struct AttnParams {
    void* o;
    int64_t os[3];  // output element strides {batch, head, sequence}
    int32_t seq_q, seq_k, heads, batch;
    float scale_log2;  // scale * log2(e)
    int32_t causal;
    int32_t is_bf16;
    int32_t debug;
};

template <int D>
struct AttnSmem {
    static constexpr int kQBytes = kHalves * kBlockM * D * 2;
    static constexpr int kKBytes = kBlockN * D * 2;  // one stage
    static constexpr int kVBytes = kBlockN * D * 2;
    static constexpr int kPBytes = kBlockM * kBlockN * 2;  // per half
    static constexpr int kQOff = 0;
    static constexpr int kKOff = kQOff + kQBytes;
    static constexpr int kVOff = kKOff + kKvStages * kKBytes;
    static constexpr int kPOff = kVOff + kKvStages * kVBytes;
    static constexpr int kBarOff = kPOff + 2 * kHalves * kPBytes;  // two P buffers per half
    static constexpr int kTotal = kBarOff + 256 + 1024;
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack16(float a, float b, bool bf16) {
    if (bf16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}


template <int D>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const __grid_constant__ AttnParams p) {
    using L = AttnSmem<D>;
    constexpr int kPanels = D / 64;            // 64-element (128-byte) panels along the head dimension
    constexpr uint32_t kTmemCols = 512;        // S: 4 x 64 columns (two buffers per half), O: 2 x D columns
    constexpr uint32_t kSCol = 0, kOCol = 4 * kBlockN;  // S: [half][2 buffers] x 64 columns, then O: [half] x D
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
    uint64_t* q_full = bars;                       // 1
    uint64_t* k_full = q_full + 1;                 // kKvStages
    uint64_t* k_empty = k_full + kKvStages;
    uint64_t* v_full = k_empty + kKvStages;
    uint64_t* v_empty = v_full + kKvStages;
    uint64_t* s_full = v_empty + kKvStages;        // [half][buffer]
    uint64_t* p_full = s_full + 2 * kHalves;       // [half][buffer]
    uint64_t* pv_done = p_full + 2 * kHalves;      // [half][buffer]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2 * kHalves);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mblk = gridDim.x - 1 - blockIdx.x;  // heavy (late, for causal) query blocks first
    const int head = blockIdx.y, bat = blockIdx.z;
    const int m0 = mblk * kHalves * kBlockM;
    const int causal_off = p.seq_k - p.seq_q;
    // keys this CTA visits: all, or up to the last key its last query row may see
    int kv_len = p.seq_k;
    if (p.causal) kv_len = min(p.seq_k, max(0, min(m0 + kHalves * kBlockM, p.seq_q) + causal_off));
    const int nblk = (kv_len + kBlockN - 1) / kBlockN;

    if (warp == 0 && lane == 0) {
        prefetch_tmap(&map_q);
        prefetch_tmap(&map_k);
        prefetch_tmap(&map_v);
        mbar_init(q_full, 1);
        for (int s = 0; s < kKvStages; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int h = 0; h < kHalves; ++h) { mbar_init(&s_full[2 * h], 1); mbar_init(&s_full[2 * h + 1], 1);
            for (int b = 0; b < 2; ++b) { mbar_init(&p_full[2 * h + b], 4); mbar_init(&pv_done[2 * h + b], 1); } }
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0 && nblk > 0) {
            mbar_expect_tx(q_full, L::kQBytes);
            for (int h = 0; h < kHalves; ++h)
                for (int pn = 0; pn < kPanels; ++pn)
                    tma_load_4d(smem + L::kQOff + (h * kPanels + pn) * kBlockM * 128, &map_q, q_full, pn * 64, m0 + h * kBlockM, head, bat);
            int stage = 0;
            uint32_t phase = 0;
            for (int j = 0; j < nblk; ++j) {
                if (!mbar_wait(&k_empty[stage], phase ^ 1)) { atomicExch(&g_attn_error, 1); break; }
                mbar_expect_tx(&k_full[stage], L::kKBytes);
                for (int pn = 0; pn < kPanels; ++pn)
                    tma_load_4d(smem + L::kKOff + stage * L::kKBytes + pn * kBlockN * 128, &map_k, &k_full[stage], pn * 64, j * kBlockN, head, bat);
                if (!mbar_wait(&v_empty[stage], phase ^ 1)) { atomicExch(&g_attn_error, 2); break; }
                mbar_expect_tx(&v_full[stage], L::kVBytes);
                for (int pn = 0; pn < kPanels; ++pn)
                    tma_load_4d(smem + L::kVOff + stage * L::kVBytes + pn * kBlockN * 128, &map_v, &v_full[stage], pn * 64, j * kBlockN, head, bat);
                if (++stage == kKvStages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the whole warp walks the schedule (uniform control flow keeps descriptors in
        // uniform registers); one elected lane issues the tcgen05 instructions ----------------
        if (nblk > 0) {
            const uint32_t fmt = p.is_bf16 ? 1u : 0u;
            // S = Q K^T: both operands K-major, N = 64. O += P V: P K-major, V N-major (head dim contiguous), N = D.
            const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(kBlockN >> 3) << 17) | (static_cast<uint32_t>(kBlockM >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | (static_cast<uint32_t>(D >> 3) << 17) | (static_cast<uint32_t>(kBlockM >> 4) << 24);
            const uint32_t q_addr = smem_u32(smem + L::kQOff), k_addr = smem_u32(smem + L::kKOff), v_addr = smem_u32(smem + L::kVOff),
                           p_addr = smem_u32(smem + L::kPOff);
            bool ok = mbar_wait(q_full, 0);
            if (!ok) atomicExch(&g_attn_error, 3);
            auto issue_s = [&](int h, int stage, int buf) {
                const uint32_t qa = q_addr + h * kPanels * kBlockM * 128, ka = k_addr + stage * L::kKBytes;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint64_t da = make_smem_desc(qa + (kk / 4) * kBlockM * 128 + (kk % 4) * 32, 16, 1024);
                    const uint64_t db = make_smem_desc(ka + (kk / 4) * kBlockN * 128 + (kk % 4) * 32, 16, 1024);
                    if (elect_one()) umma_f16(tmem_base + kSCol + (2 * h + buf) * kBlockN, da, db, idesc_s, kk != 0 ? 1u : 0u);
                }
                if (elect_one()) umma_commit(&s_full[2 * h + buf]);
                __syncwarp();
            };
            auto issue_pv = [&](int h, int stage, int buf, bool accumulate) {
                const uint32_t pa = p_addr + (2 * h + buf) * L::kPBytes, va = v_addr + stage * L::kVBytes;
#pragma unroll
                for (int kk = 0; kk < kBlockN / 16; ++kk) {
                    const uint64_t da = make_smem_desc(pa + kk * 32, 16, 1024);
                    const uint64_t db = make_smem_desc(va + kk * 16 * 128, kBlockN * 128, 1024);
                    if (elect_one()) umma_f16(tmem_base + kOCol + h * D, da, db, idesc_o, (accumulate || kk != 0) ? 1u : 0u);
                }
                if (elect_one()) umma_commit(&pv_done[2 * h + buf]);
                __syncwarp();
            };
            // Scores run two key blocks ahead of the softmax (two S buffers per half): S_h(j+2) is issued as soon as the
            // softmax has consumed S_h(j), so a warpgroup never waits for the tensor pipe.
            auto kstage = [](int j) { return j % kKvStages; };
            auto kphase = [](int j) { return static_cast<uint32_t>((j / kKvStages) & 1); };
            for (int j = 0; j < 2 && j < nblk && ok; ++j) {
                if (!mbar_wait(&k_full[kstage(j)], kphase(j))) { ok = false; atomicExch(&g_attn_error, 4); break; }
                tc_fence_after();
                issue_s(0, kstage(j), j & 1);
                issue_s(1, kstage(j), j & 1);
                { if (elect_one()) umma_commit(&k_empty[kstage(j)]); __syncwarp(); }
            }
            for (int j = 0; j < nblk && ok; ++j) {
                for (int h = 0; h < kHalves && ok; ++h) {
                    if (!mbar_wait(&p_full[2 * h + (j & 1)], (j >> 1) & 1)) { ok = false; atomicExch(&g_attn_error, 5); break; }
                    if (h == 0 && !mbar_wait(&v_full[kstage(j)], kphase(j))) { ok = false; atomicExch(&g_attn_error, 7); break; }
                    tc_fence_after();
                    issue_pv(h, kstage(j), j & 1, j > 0);
                    if (h == kHalves - 1) { if (elect_one()) umma_commit(&v_empty[kstage(j)]); __syncwarp(); }
                    if (j + 2 < nblk) {
                        if (h == 0 && !mbar_wait(&k_full[kstage(j + 2)], kphase(j + 2))) { ok = false; atomicExch(&g_attn_error, 6); break; }
                        tc_fence_after();
                        issue_s(h, kstage(j + 2), j & 1);
                        if (h == kHalves - 1) { if (elect_one()) umma_commit(&k_empty[kstage(j + 2)]); __syncwarp(); }
                    }
                }
            }
        }
    } else {
// ---------------- softmax warpgroups ----------------
        const int h = (warp - 2) >> 2;       // which half of the query block
        const int quarter = warp & 3;        // TMEM lanes this warp may touch
        const int r = quarter * 32 + lane;   // row inside the half
        const int qi = m0 + h * kBlockM + r; // query index
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t s_taddr0 = tmem_base + lane_base + kSCol + 2 * h * kBlockN;
        const uint32_t o_taddr = tmem_base + lane_base + kOCol + h * D;
        uint8_t* p_row0 = smem + L::kPOff + 2 * h * L::kPBytes + r * 128;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < nblk; ++j) {
            if (!mbar_wait(&s_full[2 * h + (j & 1)], (j >> 1) & 1)) { ok = false; atomicExch(&g_attn_error, 8); break; }
            const uint32_t s_taddr = s_taddr0 + (j & 1) * kBlockN;
            tc_fence_after();
            uint32_t sr[kBlockN];
            if (p.debug != 2) {
            tmem_ld32(s_taddr, sr);
            tmem_ld32(s_taddr + 32, sr + 32);
            tmem_ld_wait();
            } else {
#pragma unroll
                for (int c = 0; c < kBlockN; ++c) sr[c] = 0;
            }
            const int key0 = j * kBlockN;
            const int last_visible = p.causal ? min(p.seq_k - 1, qi + causal_off) : p.seq_k - 1;
            if (key0 + kBlockN - 1 > last_visible) {  // diagonal or ragged block: mask the invisible keys
#pragma unroll
                for (int c = 0; c < kBlockN; ++c)
                    if (key0 + c > last_visible) sr[c] = 0xff800000u;  // -inf
            }
            // row maximum of the raw scores with four independent chains (scale > 0, so it commutes with max)
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < kBlockN; c += 4) {
#pragma unroll
                for (int u = 0; u < 4; ++u) mx4[u] = fmaxf(mx4[u], __uint_as_float(sr[c + u]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
            // advance the reference maximum only when it would otherwise let exponentials exceed 2^threshold
            const bool grow = mx > m_ref + kRescaleThreshold;
            float alpha = 1.f;
            if (grow) {
                alpha = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - mx);
                m_ref = mx;
                l *= alpha;
            }
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            // p = 2^(s * scale*log2e - m): one packed FMA per two scores, then ex2
            const float2 c2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(-m_use, -m_use);
            uint32_t packed[kBlockN / 2];
            float2 rs2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int c = 0; c < kBlockN; c += 2) {
                const float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[c]), __uint_as_float(sr[c + 1])), c2, nm2);
                const float2 e = p.debug == 1 ? x : make_float2(fast_exp2(x.x), fast_exp2(x.y));
                rs2[(c >> 1) & 1] = __fadd2_rn(rs2[(c >> 1) & 1], e);
                packed[c / 2] = pack16(e.x, e.y, p.is_bf16 != 0);
            }
            l += (rs2[0].x + rs2[0].y) + (rs2[1].x + rs2[1].y);
            // The accumulator may only be rescaled once every PV product issued so far has completed (rare path).
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                if (!mbar_wait(&pv_done[2 * h + ((j - 1) & 1)], ((j - 1) >> 1) & 1)) { ok = false; atomicExch(&g_attn_error, 9); break; }
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t orow[32];
                    tmem_ld32(o_taddr + c0, orow);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) orow[c] = __float_as_uint(__uint_as_float(orow[c]) * alpha);
                    tmem_st32(o_taddr + c0, orow);
                }
                tmem_st_wait();
            }
            // P buffer (j & 1) is free once the PV product of block j-2 has read it
            if (j >= 2) {
                if (!mbar_wait(&pv_done[2 * h + (j & 1)], ((j - 2) >> 1) & 1)) { ok = false; atomicExch(&g_attn_error, 11); break; }
            }
            uint8_t* p_row = p_row0 + (j & 1) * L::kPBytes;
            // row r of the K-major, 128-byte-swizzled P tile: 16-byte chunk c lands at chunk (c ^ (r & 7))
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(p_row + ((c ^ (r & 7)) << 4)) =
                    make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[2 * h + (j & 1)]);
        }
        // ---- write O / l ----
        if (ok && nblk > 0) {
            if (!mbar_wait(&pv_done[2 * h + ((nblk - 1) & 1)], ((nblk - 1) >> 1) & 1)) { ok = false; atomicExch(&g_attn_error, 10); }
            tc_fence_after();
        }
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        uint8_t* orow_ptr = static_cast<uint8_t*>(p.o) + (static_cast<int64_t>(bat) * p.os[0] + static_cast<int64_t>(head) * p.os[1] +
                                                         static_cast<int64_t>(qi) * p.os[2]) * 2;
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t orow[32];
            if (ok && nblk > 0) {
                tmem_ld32(o_taddr + c0, orow);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int c = 0; c < 32; ++c) orow[c] = 0u;
            }
            if (qi < p.seq_q) {
#pragma unroll
                for (int c = 0; c < 32; c += 8) {
                    uint4 w;
                    w.x = pack16(__uint_as_float(orow[c]) * inv, __uint_as_float(orow[c + 1]) * inv, p.is_bf16 != 0);
                    w.y = pack16(__uint_as_float(orow[c + 2]) * inv, __uint_as_float(orow[c + 3]) * inv, p.is_bf16 != 0);
                    w.z = pack16(__uint_as_float(orow[c + 4]) * inv, __uint_as_float(orow[c + 5]) * inv, p.is_bf16 != 0);
                    w.w = pack16(__uint_as_float(orow[c + 6]) * inv, __uint_as_float(orow[c + 7]) * inv, p.is_bf16 != 0);
                    *reinterpret_cast<uint4*>(orow_ptr + (c0 + c) * 2) = w;
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}


using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [B, H, S, D] operand (D contiguous) as the 4-D map {D, S, H, B}; one box = 64 head-dim elements x `rows` positions.
bool qkv_map(CUtensorMap* map, const void* base, int64_t d, int64_t s, int64_t h, int64_t b, const int64_t strides[3], uint32_t rows,
             std::string* why) {
    static EncodeFn encode = nullptr;
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || fn == nullptr) {
            *why = "cuTensorMapEncodeTiled is not available from this driver";
            return false;
        }
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const cuuint64_t gdim[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(s), static_cast<cuuint64_t>(h), static_cast<cuuint64_t>(b)};
    const int64_t span = std::max<int64_t>(16, (d * 2 + 15) / 16 * 16);
    cuuint64_t gstr[3];
    const int64_t ext[3] = {s, h, b};
    for (int i = 0; i < 3; ++i) {
        int64_t bytes = strides[2 - i] * 2;  // strides come as {batch, head, sequence}
        if (ext[i] == 1 || bytes == 0) bytes = span;
        gstr[i] = static_cast<cuuint64_t>(bytes);
    }
    const cuuint32_t box[4] = {64, rows, 1, 1}, es[4] = {1, 1, 1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), gdim, gstr, box, es,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        *why = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(r));
        return false;
    }
    return true;
}

template <int D>
int launch_attention(int dtype, const void* q, const void* k, const void* v, void* o, const AttnShape& s, cudaStream_t stream) {
    using L = AttnSmem<D>;
    CUtensorMap mq, mk, mv;
    std::string why;
    if (!qkv_map(&mq, q, D, s.seq_q, s.heads, s.batch, s.qs, kBlockM, &why) || !qkv_map(&mk, k, D, s.seq_k, s.heads, s.batch, s.ks, kBlockN, &why) ||
        !qkv_map(&mv, v, D, s.seq_k, s.heads, s.batch, s.vs, kBlockN, &why))
        return fail(MHLO_CUDA_EXECUTION_FAILED, "attention: tensor map: %s", why.c_str());
    AttnParams p;
    p.o = o;
    for (int i = 0; i < 3; ++i) p.os[i] = s.os[i];
    p.seq_q = static_cast<int>(s.seq_q); p.seq_k = static_cast<int>(s.seq_k);
    p.heads = static_cast<int>(s.heads); p.batch = static_cast<int>(s.batch);
    p.scale_log2 = s.scale * kLog2e;
    p.causal = s.causal;
    p.is_bf16 = dtype == MHLO_DT_BF16;
    p.debug = getenv("MHLO_ATTN_DEBUG") ? atoi(getenv("MHLO_ATTN_DEBUG")) : 0;
    auto kernel = attention_tcgen05_kernel<D>;
    static bool attr_set = false;
    if (!attr_set) {
        MHLO_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal), MHLO_CUDA_EXECUTION_FAILED);
        attr_set = true;
    }
    dim3 grid(static_cast<unsigned>((s.seq_q + kHalves * kBlockM - 1) / (kHalves * kBlockM)), static_cast<unsigned>(s.heads),
              static_cast<unsigned>(s.batch));
    kernel<<<grid, kAttnThreads, L::kTotal, stream>>>(mq, mk, mv, p);
    MHLO_CUDA_CHECK_LAUNCH("attention_tcgen05");
    return MHLO_CUDA_OK;
}

bool stride16(int64_t elems) { return elems > 0 && (elems * 2) % 16 == 0; }

}  // namespace

int attention_device_error() {
    int v = 0, zero = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, g_attn_error, sizeof v) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_attn_error, &zero, sizeof zero);
    return v;
}

bool attention_tc_supported(int dtype, const AttnShape& s, const void* mask) {
    if (dtype != MHLO_DT_BF16 && dtype != MHLO_DT_F16) return false;
    if (mask != nullptr) return false;
    if (!(s.scale > 0.f)) return false;  // the kernel takes the row maximum before scaling
    if (s.head_dim != 64 && s.head_dim != 128) return false;
    if (s.seq_q < 1 || s.seq_k < 1 || s.heads < 1 || s.batch < 1 || s.heads > 65535 || s.batch > 65535) return false;
    if (s.seq_q > 0x3fffffff || s.seq_k > 0x3fffffff) return false;
    if (s.seq_q * s.seq_k < 64 * 64) return false;  // tiny problems: the row kernel has less fixed cost
    auto ok3 = [&](const int64_t* st, int64_t seq) {
        return (seq == 1 || stride16(st[2])) && (s.heads == 1 || stride16(st[1])) && (s.batch == 1 || stride16(st[0]));
    };
    return ok3(s.qs, s.seq_q) && ok3(s.ks, s.seq_k) && ok3(s.vs, s.seq_k) && ok3(s.os, s.seq_q);
}

int attention_tc_launch(int dtype, const void* q, const void* k, const void* v, void* o, const AttnShape& s, cudaStream_t stream) {
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o))
        return fail(MHLO_CUDA_INVALID_ARGUMENT, "attention: tensor-core path needs 16-byte aligned tensors");
    if (s.head_dim == 128) return launch_attention<128>(dtype, q, k, v, o, s, stream);
    return launch_attention<64>(dtype, q, k, v, o, s, stream);
}

}  // namespace mhlo
