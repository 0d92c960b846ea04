// Fused flash attention on tcgen05: O = softmax(scale * Q K^T [causal]) V for bf16 / f16, head_dim 64 or 128, fp32
// softmax statistics and fp32 accumulation in TMEM. The S^2 score matrix never reaches HBM.
//
// One CTA owns 256 query rows of one (batch, head) as two halves of 128 rows and walks the keys in blocks of 128:
//   warp 0 (one lane)   TMA producer: Q once (both halves), then K_j and V_j tiles through 2-stage rings
//   warp 1              MMA issuer (warp-uniform loop, one elected lane issues), ping-ponging the two halves:
//                         S_h(j+1) = Q_h K_{j+1}^T   (tcgen05.mma M128 N128, both operands K-major in shared memory)
//                         O_h     += P_h(j) V_j      (P read from tensor memory, V N-major in shared memory, N = D)
//                       so the tensor pipe works on one half while the other half's softmax runs
//   warps 2-5 / 6-9     softmax warpgroups for half 0 / 1; a thread owns one query row: two passes of tcgen05.ld over
//                       its 128 scores (row maximum, then exp2 and row sum), probabilities packed to 16 bit and
//                       written with tcgen05.st over the score columns they came from - P never touches shared
//                       memory. The maximum used in the exponent only advances when it grew by more than 2^8
//                       ("lazy rescale"); only then is O rescaled in TMEM (tcgen05.ld, multiply, tcgen05.st).
// TMEM: S_h/P_h 2 x 128 columns, O_h 2 x D columns (all 512 at D = 128). Shared memory at D = 128: Q 64 KiB,
// K 2 x 32 KiB, V 2 x 32 KiB.
// Causal masking skips key blocks right of the diagonal and masks inside diagonal blocks; ragged sequence ends are
// zero-filled by TMA and masked to -inf. Every mbarrier wait is bounded.
//
// Algorithmic work: 4*B*H*Sq*Sk*D FLOP (half of that, plus the diagonal, when causal); HBM bytes: Q, K, V read once
// per CTA column (K/V re-reads across query blocks are served by L2), O written once.
#include <atomic>
#include <algorithm>
#include <string>

#include "contraction.cuh"
#include "tc_ptx.cuh"

namespace mhlo {
namespace {

constexpr int kBlockM = 128;     // query rows per half
constexpr int kHalves = 2;
constexpr int kBlockN = 128;     // keys per step
constexpr int kKvStages = 2;
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
    int32_t by_length;  // tile order: 0 = long/short pairs per (batch, head); 1 = longest tiles first, dealt out in a snake
};

template <int D>
struct AttnSmem {
    static constexpr int kQBytes = kHalves * kBlockM * D * 2;
    static constexpr int kKBytes = kBlockN * D * 2;  // one stage
    static constexpr int kVBytes = kBlockN * D * 2;
    static constexpr int kQOff = 0;
    static constexpr int kKOff = kQOff + kQBytes;
    static constexpr int kVOff = kKOff + kKvStages * kKBytes;
    static constexpr int kBarOff = kVOff + kKvStages * kVBytes;
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

__device__ __forceinline__ uint32_t scale16x2(uint32_t v, float a, bool bf16) {
    if (bf16) {
        __nv_bfloat162 h = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&v), __float2bfloat162_rn(a));
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __half2 h = __hmul2(*reinterpret_cast<__half2*>(&v), __float2half2_rn(a));
    return *reinterpret_cast<uint32_t*>(&h);
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (the probabilities) is read from tensor memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Exponentials of one row's 128 scores: p = 2^(s * scale*log2e - m), packed to 16 bit and written over the score
// columns they came from (keys [c, c+64) become 32 packed columns at c/2); returns the row's sum of p.
// kMask: the block crosses the causal diagonal or the end of the keys; scores right of last_visible become -inf.
// kCheck: m is a reference maximum carried over from earlier key blocks rather than this block's own. The
// probabilities are then held back until the whole warp has seen sums below 2^15, which bounds every p below the
// largest f16 / bf16 value; otherwise nothing is written, *stored is false and the caller redoes the block with its
// true maximum (the scores are still intact).
constexpr float kCarryLimit = 32768.f;
// p_taddr: where the packed probabilities go (s_taddr itself when they overwrite the scores). s_read: when not null, the
// barrier this warp arrives on once its last score has left tensor memory (the next block's scores may then replace them).
template <bool kMask, bool kCheck>
__device__ __forceinline__ float softmax_exp(uint32_t s_taddr, float scale_log2, float m_use, int key0, int last_visible, bool is_bf16,
                                             bool* stored, uint32_t p_taddr, uint64_t* s_read = nullptr) {
    const float2 c2 = make_float2(scale_log2, scale_log2), nm2 = make_float2(-m_use, -m_use);
    float2 rs2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
    uint32_t packed[kBlockN / 64][32];
#pragma unroll
    for (int ci = 0; ci < kBlockN / 64; ++ci) {
        uint32_t sr[64];
        tmem_ld32(s_taddr + ci * 64, sr);
        tmem_ld32(s_taddr + ci * 64 + 32, sr + 32);
        tmem_ld_wait();
        if (!kCheck && ci == kBlockN / 64 - 1 && s_read != nullptr) {
            tc_fence_before();
            __syncwarp();
            if ((threadIdx.x & 31) == 0) mbar_arrive(s_read);
        }
        if (kMask) {
#pragma unroll
            for (int c = 0; c < 64; ++c)
                if (key0 + ci * 64 + c > last_visible) sr[c] = 0xff800000u;  // -inf
        }
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[c]), __uint_as_float(sr[c + 1])), c2, nm2);
            const float2 e = make_float2(fast_exp2(x.x), fast_exp2(x.y));
            rs2[(c >> 1) & 1] = __fadd2_rn(rs2[(c >> 1) & 1], e);
            packed[ci][c / 2] = pack16(e.x, e.y, is_bf16);
        }
        if (!kCheck) tmem_st32(p_taddr + ci * 32, packed[ci]);  // in place: those score columns have been consumed already
    }
    const float rs = (rs2[0].x + rs2[0].y) + (rs2[1].x + rs2[1].y);
    if (kCheck) {
        const bool safe = !__any_sync(0xffffffffu, !(rs < kCarryLimit));
        if (safe) {
#pragma unroll
            for (int ci = 0; ci < kBlockN / 64; ++ci) tmem_st32(p_taddr + ci * 32, packed[ci]);
        }
        *stored = safe;
    }
    return rs;
}

// One unit of work: 256 query rows of one (batch, head).
struct Tile {
    int bat, head, m0;
    int nblk;   // key blocks this tile visits (0: no key is visible to any of its rows)
    int nblk0;  // key blocks its first half (rows m0 .. m0 + 127) takes part in: under a causal mask the tile's last block
                // lies wholly right of that half's diagonal, and the half skips it
};

// The tiles of one CTA. Tiles are numbered g = (batch*heads + head) * n_m + s, where position s inside a (batch, head)
// alternates long and short query blocks (last, first, second-to-last, second, ...), so that under a causal mask two
// consecutive tiles always add up to the same number of key blocks. A CTA takes pairs 2u, 2u+1 for
// u = blockIdx.x, blockIdx.x + gridDim.x, ...: CTAs running at the same time work on neighbouring (batch, head)
// and share their K and V through L2.
struct TileWalk {
    int n_m, total, u, e, step, cta;
    __device__ TileWalk(const AttnParams& p, int first, int stride)
        : n_m((p.seq_q + kHalves * kBlockM - 1) / (kHalves * kBlockM)), u(first), e(0), step(stride), cta(first) {
        total = n_m * p.heads * p.batch;
        if (p.by_length) u = 0;  // u counts the passes over the CTAs
    }
    __device__ bool next(const AttnParams& p, Tile* t) {
        int hb, mblk;
        if (p.by_length) {
            // Tiles sorted by length (all (batch, head) pairs of the last query block, then of the one before, ...), dealt
            // to the CTAs forwards on even passes and backwards on odd ones: the CTA that got the longest tile of a pass
            // gets the shortest of the next. Used when all keys and values fit L2, where the order costs no re-reads from HBM.
            const int j = u * step + ((u & 1) ? step - 1 - cta : cta);
            if (j >= total) return false;
            const int hbs = p.heads * p.batch;
            const int rank = j / hbs;
            hb = j - rank * hbs;
            mblk = n_m - 1 - rank;
            ++u;
        } else {
            const int g = 2 * u + e;
            if (g >= total) return false;
            hb = g / n_m;
            const int s = g - hb * n_m;
            mblk = (s & 1) ? (s >> 1) : n_m - 1 - (s >> 1);
            if (++e == 2) { e = 0; u += step; }
        }
        t->bat = hb / p.heads;
        t->head = hb - t->bat * p.heads;
        t->m0 = mblk * kHalves * kBlockM;
        int kv_len = p.seq_k;  // keys this tile visits: all, or up to the last key its last query row may see
        if (p.causal) kv_len = min(p.seq_k, min(t->m0 + kHalves * kBlockM, p.seq_q));  // key j is visible to query i iff j <= i
        t->nblk = (kv_len + kBlockN - 1) / kBlockN;
        t->nblk0 = p.causal ? min(t->nblk, t->m0 / kBlockN + 1) : t->nblk;
        return true;
    }
    // Next tile that has at least one key block (the producer and the MMA issuer skip the others).
    __device__ bool next_nonempty(const AttnParams& p, Tile* t) {
        while (next(p, t))
            if (t->nblk > 0) return true;
        return false;
    }
};

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const __grid_constant__ AttnParams p) {
    using L = AttnSmem<D>;
    constexpr int kPanels = D / 64;       // 64-element (128-byte) panels along the head dimension
    constexpr uint32_t kTmemCols = 512;   // S_h: 128 columns per half (P overwrites them in place), O_h: D columns per half
    constexpr uint32_t kSCol = 0, kOCol = kHalves * kBlockN;
    // At head dim 64 the 512 columns also hold the probabilities beside the scores (64 packed columns per half). The
    // scores of key block j + 1 are then issued as soon as the softmax warps have read those of block j out of tensor
    // memory, instead of after P.V of block j: Q.K^T and P.V run under the exponentials and the softmax warps go from
    // one block to the next without waiting for the tensor pipe. At head dim 128 there is no room: P overwrites S.
    constexpr bool kEarly = kHalves * (kBlockN + D + kBlockN / 2) <= 512;
    constexpr uint32_t kPCol = kEarly ? kOCol + kHalves * D : kSCol;
    constexpr uint32_t kPStride = kEarly ? kBlockN / 2 : kBlockN;  // columns between the two halves' probabilities
    constexpr int kQHalfBytes = kBlockM * D * 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
    uint64_t* q_full = bars;                 // per half: the tile's query rows are in shared memory
    uint64_t* q_empty = q_full + kHalves;    // per half: the tile's last S product has read them
    uint64_t* k_full = q_empty + kHalves;
    uint64_t* k_empty = k_full + kKvStages;
    uint64_t* v_full = k_empty + kKvStages;
    uint64_t* v_empty = v_full + kKvStages;
    uint64_t* s_full = v_empty + kKvStages;  // per half: scores of the current key block are in TMEM
    uint64_t* p_full = s_full + kHalves;     // per half: probabilities written (and O rescaled if needed)
    uint64_t* pv_done = p_full + kHalves;    // per half: every PV product issued so far has completed
    uint64_t* s_free = pv_done + kHalves;    // per half (kEarly): the softmax warps have read the scores out of TMEM
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + kHalves);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (warp == 0 && lane == 0) {
        prefetch_tmap(&map_q);
        prefetch_tmap(&map_k);
        prefetch_tmap(&map_v);
        for (int s = 0; s < kKvStages; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int h = 0; h < kHalves; ++h) {
            mbar_init(&q_full[h], 1); mbar_init(&q_empty[h], 1);
            mbar_init(&s_full[h], 1); mbar_init(&p_full[h], 4); mbar_init(&pv_done[h], 1); mbar_init(&s_free[h], 4);
        }
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
    TileWalk walk(p, static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x));
    // the set-up above touched only shared memory and TMEM: it may overlap the previous kernel's tail
    grid_dependency_wait();
    grid_dependency_release();

    if (warp == 0) {
        // ---------------- producer: runs ahead of the other warps as far as the rings allow, across tile boundaries
        if (lane == 0) {
            Tile t;
            int stage = 0;
            uint32_t phase = 0, qn = 0;  // qn: tiles loaded so far (parity of the q barriers)
            bool ok = true;
            while (ok && walk.next_nonempty(p, &t)) {
                for (int h = 0; h < kHalves && ok; ++h) {
                    if (!mbar_wait(&q_empty[h], (qn & 1) ^ 1)) { atomicExch(&g_attn_error, 11); ok = false; break; }
                    mbar_expect_tx(&q_full[h], kQHalfBytes);
                    for (int pn = 0; pn < kPanels; ++pn)
                        tma_load_4d(smem + L::kQOff + (h * kPanels + pn) * kBlockM * 128, &map_q, &q_full[h], pn * 64, t.m0 + h * kBlockM, t.head, t.bat);
                }
                for (int j = 0; j < t.nblk && ok; ++j) {
                    if (!mbar_wait(&k_empty[stage], phase ^ 1)) { atomicExch(&g_attn_error, 1); ok = false; break; }
                    mbar_expect_tx(&k_full[stage], L::kKBytes);
                    for (int pn = 0; pn < kPanels; ++pn)
                        tma_load_4d(smem + L::kKOff + stage * L::kKBytes + pn * kBlockN * 128, &map_k, &k_full[stage], pn * 64, j * kBlockN, t.head, t.bat);
                    if (!mbar_wait(&v_empty[stage], phase ^ 1)) { atomicExch(&g_attn_error, 2); ok = false; break; }
                    mbar_expect_tx(&v_full[stage], L::kVBytes);
                    for (int pn = 0; pn < kPanels; ++pn)
                        tma_load_4d(smem + L::kVOff + stage * L::kVBytes + pn * kBlockN * 128, &map_v, &v_full[stage], pn * 64, j * kBlockN, t.head, t.bat);
                    if (++stage == kKvStages) { stage = 0; phase ^= 1; }
                }
                ++qn;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the whole warp walks the schedule (uniform control flow keeps descriptors in
        // uniform registers); one elected lane issues the tcgen05 instructions ----------------
        const uint32_t fmt = p.is_bf16 ? 1u : 0u;
        // S = Q K^T: both operands K-major from shared memory, N = 128 keys.
        // O += P V: P from tensor memory (K-major), V from shared memory N-major (head dim contiguous), N = D.
        const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(kBlockN >> 3) << 17) | (static_cast<uint32_t>(kBlockM >> 4) << 24);
        const uint32_t idesc_o = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | (static_cast<uint32_t>(D >> 3) << 17) | (static_cast<uint32_t>(kBlockM >> 4) << 24);
        const uint32_t q_addr = smem_u32(smem + L::kQOff), k_addr = smem_u32(smem + L::kKOff), v_addr = smem_u32(smem + L::kVOff);
        auto issue_s = [&](int h, int stage) {
            const uint32_t qa = q_addr + h * kPanels * kBlockM * 128, ka = k_addr + stage * L::kKBytes;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const uint64_t da = make_smem_desc(qa + (kk / 4) * kBlockM * 128 + (kk % 4) * 32, 16, 1024);
                const uint64_t db = make_smem_desc(ka + (kk / 4) * kBlockN * 128 + (kk % 4) * 32, 16, 1024);
                if (elect_one()) umma_f16(tmem_base + kSCol + h * kBlockN, da, db, idesc_s, kk != 0 ? 1u : 0u);
            }
            if (elect_one()) umma_commit(&s_full[h]);
            __syncwarp();
        };
        auto issue_pv = [&](int h, int stage, bool accumulate) {
            const uint32_t va = v_addr + stage * L::kVBytes;
#pragma unroll
            for (int kk = 0; kk < kBlockN / 16; ++kk) {
                // 16 keys of P = 8 packed 32-bit columns; 16 keys of V = 16 rows of 128 bytes in every head-dim panel
                const uint64_t db = make_smem_desc(va + kk * 16 * 128, kBlockN * 128, 1024);
                if (elect_one()) umma_f16_ts(tmem_base + kOCol + h * D, tmem_base + kPCol + h * kPStride + kk * 8, db, idesc_o, (accumulate || kk != 0) ? 1u : 0u);
            }
            if (elect_one()) umma_commit(&pv_done[h]);
            __syncwarp();
        };
        auto commit_to = [&](uint64_t* bar) {
            if (elect_one()) umma_commit(bar);
            __syncwarp();
        };
        Tile cur, nxt;
        bool has_cur = walk.next_nonempty(p, &cur);
        int stage = 0;
        uint32_t phase = 0, qn = 0;   // qn: tiles so far
        uint32_t it_h[kHalves] = {0, 0};  // key blocks each half has gone through (parity of its per-block barriers)
        uint32_t s_count[kHalves] = {1, 1};  // S products issued per half, the first tile's first ones included (kEarly)
        bool ok = true;
        if (has_cur) {
            // first scores of the first tile
            if (!mbar_wait(&q_full[0], 0) || !mbar_wait(&q_full[1], 0)) { ok = false; atomicExch(&g_attn_error, 3); }
            if (ok && !mbar_wait(&k_full[0], 0)) { ok = false; atomicExch(&g_attn_error, 4); }
            if (ok) {
                tc_fence_after();
                issue_s(0, 0);
                if (cur.nblk0 == 1) commit_to(&q_empty[0]);
                issue_s(1, 0);
                if (cur.nblk == 1) commit_to(&q_empty[1]);
                commit_to(&k_empty[0]);
            }
        }
        // Tensor-pipe order per key block j: PV_0(j), S_0(next), PV_1(j), S_1(next), where "next" is block j+1 of this
        // tile or block 0 of the CTA's next tile. The pipe executes one thread's MMAs in order, so S_h(next) overwrites
        // the S/P columns only after PV_h(j) has read the probabilities from them.
        while (has_cur && ok) {
            const bool has_nxt = walk.next_nonempty(p, &nxt);
            for (int j = 0; j < cur.nblk && ok; ++j) {
                const int nstage = stage + 1 == kKvStages ? 0 : stage + 1;
                const uint32_t nphase = stage + 1 == kKvStages ? phase ^ 1 : phase;
                const bool last = j + 1 == cur.nblk;
                const bool more = !last || has_nxt;
                if (!mbar_wait(&v_full[stage], phase)) { ok = false; atomicExch(&g_attn_error, 7); break; }
                if constexpr (kEarly) {
                    // Tensor-pipe order per key block j: S_0(next), S_1(next), PV_0(j), PV_1(j). S_h(next) goes out when
                    // half h has read its scores of block j (s_free, about half way through its exponentials), PV_h(j)
                    // when it has written the probabilities: both S products are under way before either half finishes.
                    if (more) {
                        for (int h = 0; h < kHalves && ok; ++h) {
                            const int nb = h == 0 ? cur.nblk0 : cur.nblk;
                            if (last && !mbar_wait(&q_full[h], (qn + 1) & 1)) { ok = false; atomicExch(&g_attn_error, 12); break; }
                            if (h == 0 && !mbar_wait(&k_full[nstage], nphase)) { ok = false; atomicExch(&g_attn_error, 6); break; }
                            if (last || j + 1 < nb) {
                                // one s_free arrival per S issued: the one before this one has been read
                                if (!mbar_wait(&s_free[h], (s_count[h] - 1) & 1)) { ok = false; atomicExch(&g_attn_error, 13); break; }
                                tc_fence_after();
                                issue_s(h, nstage);
                                ++s_count[h];
                                const int nb_of_s = last ? (h == 0 ? nxt.nblk0 : nxt.nblk) : nb;
                                if (last ? nb_of_s == 1 : j + 2 == nb_of_s) commit_to(&q_empty[h]);
                            }
                            if (h == kHalves - 1) commit_to(&k_empty[nstage]);
                        }
                    }
                    for (int h = 0; h < kHalves && ok; ++h) {
                        const int nb = h == 0 ? cur.nblk0 : cur.nblk;
                        if (j < nb) {
                            if (!mbar_wait(&p_full[h], it_h[h] & 1)) { ok = false; atomicExch(&g_attn_error, 5); break; }
                            tc_fence_after();
                            issue_pv(h, stage, j > 0);
                            ++it_h[h];
                        }
                        if (h == kHalves - 1) commit_to(&v_empty[stage]);
                    }
                    stage = nstage;
                    phase = nphase;
                    continue;
                }
                for (int h = 0; h < kHalves && ok; ++h) {
                    const int nb = h == 0 ? cur.nblk0 : cur.nblk;  // blocks this half takes part in
                    if (j < nb) {
                        if (!mbar_wait(&p_full[h], it_h[h] & 1)) { ok = false; atomicExch(&g_attn_error, 5); break; }
                        tc_fence_after();
                        issue_pv(h, stage, j > 0);
                        ++it_h[h];
                    }
                    if (h == kHalves - 1) commit_to(&v_empty[stage]);
                    if (more) {
                        if (last && !mbar_wait(&q_full[h], (qn + 1) & 1)) { ok = false; atomicExch(&g_attn_error, 12); break; }
                        if (h == 0 && !mbar_wait(&k_full[nstage], nphase)) { ok = false; atomicExch(&g_attn_error, 6); break; }
                        // the next scores of this half: block j + 1 of this tile when the half takes part in it, block 0 of
                        // the next tile after this tile's last block
                        if (last || j + 1 < nb) {
                            tc_fence_after();
                            issue_s(h, nstage);
                            const int nb_of_s = last ? (h == 0 ? nxt.nblk0 : nxt.nblk) : nb;
                            if (last ? nb_of_s == 1 : j + 2 == nb_of_s) commit_to(&q_empty[h]);  // that was the tile's last S of this half
                        }
                        if (h == kHalves - 1) commit_to(&k_empty[nstage]);
                    }
                }
                stage = nstage;
                phase = nphase;
            }
            cur = nxt;
            has_cur = has_nxt;
            ++qn;
        }
    } else {
        // ---------------- softmax warpgroups ----------------
        const int h = (warp - 2) >> 2;       // which half of the query block
        const int quarter = warp & 3;        // TMEM lanes this warp may touch
        const int r = quarter * 32 + lane;   // row inside the half
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t s_taddr = tmem_base + lane_base + kSCol + h * kBlockN;
        const uint32_t o_taddr = tmem_base + lane_base + kOCol + h * D;
        const uint32_t p_taddr = tmem_base + lane_base + kPCol + h * kPStride;
        Tile t;
        uint32_t it = 0;  // key blocks so far on this CTA (parity of the per-block barriers)
        bool ok = true;
        while (walk.next(p, &t)) {
            const int qi = t.m0 + h * kBlockM + r;  // query index
            const int last_visible = p.causal ? min(p.seq_k - 1, qi) : p.seq_k - 1;
            float m_ref = -INFINITY, l = 0.f;
            const int nb = h == 0 ? t.nblk0 : t.nblk;  // under a causal mask the first half has nothing to see in the last block
            for (int j = 0; j < nb && ok; ++j, ++it) {
                if (!mbar_wait(&s_full[h], it & 1)) { ok = false; atomicExch(&g_attn_error, 8); break; }
                tc_fence_after();
                const int key0 = j * kBlockN;
                const bool need_mask = key0 + kBlockN - 1 > last_visible;  // diagonal or ragged block
                // one decision per warp: tcgen05.ld / st are warp-wide instructions and must not sit in divergent code
                const bool mask_block = __any_sync(0xffffffffu, need_mask);
                // ---- after a tile's first block: one pass, exponentials against the reference maximum carried over from
                // the earlier blocks; it fails (rarely) when a row's scores have grown by more than 2^15
                bool done = false;
                if constexpr (kEarly) {
                    // One pass in two chunks of 64 keys, first blocks included (their reference maximum starts at -inf
                    // and moves to the first chunk's own). After the second chunk's loads the scores are out of tensor
                    // memory and the next block's may replace them. Each chunk looks at its own maximum first: when that
                    // would push an exponential past 2^threshold (the first chunk of a tile; rare afterwards), the
                    // reference maximum moves there and what has been accumulated so far - l, O, the block's first
                    // chunk of probabilities - is scaled down.
                    const float2 c2 = make_float2(p.scale_log2, p.scale_log2);
                    float2 rs2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
                    bool pv_waited = it == 0;  // P.V of the block before this one: it reads P and writes O
#pragma unroll 1
                    for (int ci = 0; ci < kBlockN / 64; ++ci) {
                        uint32_t sr[64];
                        tmem_ld32(s_taddr + ci * 64, sr);
                        tmem_ld32(s_taddr + ci * 64 + 32, sr + 32);
                        tmem_ld_wait();
                        if (ci == kBlockN / 64 - 1) {
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&s_free[h]);
                        }
                        if (mask_block) {
#pragma unroll
                            for (int c = 0; c < 64; ++c)
                                if (key0 + ci * 64 + c > last_visible) sr[c] = 0xff800000u;  // -inf
                        }
                        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                        for (int c = 0; c < 64; c += 4) {
                            mx0 = fmax3(mx0, __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]));
                            mx1 = fmax3(mx1, __uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3]));
                        }
                        const float mx = fmaxf(mx0, mx1) * p.scale_log2;
                        const bool grow = mx > m_ref + kRescaleThreshold;
                        if (__any_sync(0xffffffffu, grow)) {
                            float alpha = 1.f;
                            if (grow) {
                                alpha = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - mx);
                                m_ref = mx;
                                l *= alpha;
                            }
                            rs2[0].x *= alpha; rs2[0].y *= alpha; rs2[1].x *= alpha; rs2[1].y *= alpha;
                            if (j > 0 || ci > 0) {
                                if (!pv_waited) {
                                    if (!mbar_wait(&pv_done[h], (it - 1) & 1)) { ok = false; atomicExch(&g_attn_error, 14); }
                                    tc_fence_after();
                                    pv_waited = true;
                                }
                                // O of the earlier blocks (j > 0), then the probabilities of this block's first chunk (ci > 0)
#pragma unroll 1
                                for (int c0 = j > 0 ? 0 : D; c0 < D + (ci > 0 ? 32 : 0); c0 += 32) {
                                    const uint32_t at = c0 < D ? o_taddr + c0 : p_taddr;
                                    uint32_t row[32];
                                    if (c0 >= D) tmem_st_wait();  // this thread's own store of that chunk
                                    tmem_ld32(at, row);
                                    tmem_ld_wait();
                                    if (c0 < D) {
#pragma unroll
                                        for (int c = 0; c < 32; ++c) row[c] = __float_as_uint(__uint_as_float(row[c]) * alpha);
                                    } else {
#pragma unroll
                                        for (int c = 0; c < 32; ++c) row[c] = scale16x2(row[c], alpha, p.is_bf16 != 0);
                                    }
                                    tmem_st32(at, row);
                                }
                            }
                        }
                        const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
                        const float2 nm2 = make_float2(-m_use, -m_use);
                        uint32_t packed[32];
#pragma unroll
                        for (int c = 0; c < 64; c += 2) {
                            const float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[c]), __uint_as_float(sr[c + 1])), c2, nm2);
                            const float2 e = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                            rs2[(c >> 1) & 1] = __fadd2_rn(rs2[(c >> 1) & 1], e);
                            packed[c / 2] = pack16(e.x, e.y, p.is_bf16 != 0);
                        }
                        if (!pv_waited) {  // the probabilities of the block before this one have been read by its P.V
                            if (!mbar_wait(&pv_done[h], (it - 1) & 1)) { ok = false; atomicExch(&g_attn_error, 15); }
                            tc_fence_after();
                            pv_waited = true;
                        }
                        tmem_st32(p_taddr + ci * 32, packed);
                    }
                    l += (rs2[0].x + rs2[0].y) + (rs2[1].x + rs2[1].y);
                    done = true;
                } else if (j > 0) {
                    const float m_carry = m_ref == -INFINITY ? 0.f : m_ref;
                    const float rs = mask_block ? softmax_exp<true, true>(s_taddr, p.scale_log2, m_carry, key0, last_visible, p.is_bf16 != 0, &done, p_taddr)
                                                : softmax_exp<false, true>(s_taddr, p.scale_log2, m_carry, key0, last_visible, p.is_bf16 != 0, &done, p_taddr);
                    if (done) l += rs;
                }
                if (!kEarly && !done) {
                    // ---- pass 1: row maximum of the raw scores (scale > 0, so scaling commutes with max) ----
                    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                    for (int c0 = 0; c0 < kBlockN; c0 += 64) {
                        uint32_t sr[64];
                        tmem_ld32(s_taddr + c0, sr);
                        tmem_ld32(s_taddr + c0 + 32, sr + 32);
                        tmem_ld_wait();
                        if (need_mask) {
#pragma unroll
                            for (int c = 0; c < 64; ++c)
                                if (key0 + c0 + c > last_visible) sr[c] = 0xff800000u;  // -inf
                        }
#pragma unroll
                        for (int c = 0; c < 64; c += 4) {
                            mx0 = fmax3(mx0, __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]));
                            mx1 = fmax3(mx1, __uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3]));
                        }
                    }
                    const float mx = fmaxf(mx0, mx1) * p.scale_log2;
                    // advance the reference maximum only when it would otherwise let exponentials exceed 2^threshold
                    const bool grow = mx > m_ref + kRescaleThreshold;
                    float alpha = 1.f;
                    if (grow) {
                        alpha = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - mx);
                        m_ref = mx;
                        l *= alpha;
                    }
                    // every PV product issued so far completed before these scores were signalled, so O may be rescaled here
                    if (j > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll 1
                        for (int c0 = 0; c0 < D; c0 += 32) {
                            uint32_t orow[32];
                            tmem_ld32(o_taddr + c0, orow);
                            tmem_ld_wait();
#pragma unroll
                            for (int c = 0; c < 32; ++c) orow[c] = __float_as_uint(__uint_as_float(orow[c]) * alpha);
                            tmem_st32(o_taddr + c0, orow);
                        }
                    }
                    // ---- pass 2: p = 2^(s * scale*log2e - m), packed to 16 bit and written over the scores ----
                    const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
                    uint64_t* s_read = kEarly ? &s_free[h] : nullptr;
                    l += mask_block ? softmax_exp<true, false>(s_taddr, p.scale_log2, m_use, key0, last_visible, p.is_bf16 != 0, nullptr, p_taddr, s_read)
                                    : softmax_exp<false, false>(s_taddr, p.scale_log2, m_use, key0, last_visible, p.is_bf16 != 0, nullptr, p_taddr, s_read);
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_full[h]);
            }
            if (!ok) break;
            // ---- write O / l. The next tile's first PV product for this half is issued only after this warp has
            // arrived on p_full again, which comes after the loads below, so O may be read here without another barrier.
            if (t.nblk > 0) {
                if (!mbar_wait(&pv_done[h], (it - 1) & 1)) { ok = false; atomicExch(&g_attn_error, 10); break; }
                tc_fence_after();
            }
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            uint8_t* orow_ptr = static_cast<uint8_t*>(p.o) + (static_cast<int64_t>(t.bat) * p.os[0] + static_cast<int64_t>(t.head) * p.os[1] +
                                                             static_cast<int64_t>(qi) * p.os[2]) * 2;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t orow[32];
                if (t.nblk > 0) {
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
    auto kernel = attention_tcgen05_kernel<D>;
    // the attribute belongs to the (kernel, device) pair: one flag per device ordinal
    static std::atomic<bool> attr_set[64];
    int attr_dev = 0;
    MHLO_CUDA_TRY(cudaGetDevice(&attr_dev), MHLO_CUDA_EXECUTION_FAILED);
    if (attr_dev < 0 || attr_dev >= 64 || !attr_set[attr_dev].load(std::memory_order_acquire)) {
        MHLO_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal), MHLO_CUDA_EXECUTION_FAILED);
        if (attr_dev >= 0 && attr_dev < 64) attr_set[attr_dev].store(true, std::memory_order_release);
    }
    // persistent grid: one CTA per SM, each walking its share of the (batch, head, query block) tiles in pairs
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        MHLO_CUDA_TRY(cudaGetDevice(&dev), MHLO_CUDA_EXECUTION_FAILED);
        MHLO_CUDA_TRY(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev), MHLO_CUDA_EXECUTION_FAILED);
    }
    const int64_t tiles = (s.seq_q + kHalves * kBlockM - 1) / (kHalves * kBlockM) * s.heads * s.batch;
    // causal tiles differ in length: when K and V of all heads stay in L2 anyway, order them by length (see TileWalk)
    const int64_t kv_bytes = 2 * s.batch * s.heads * s.seq_k * static_cast<int64_t>(D) * 2;
    // METALHLO_ATTN_BY_LENGTH: 0 = never, 2 = for every causal call (measurements), otherwise by the size of K and V
    static const int by_length_mode = [] { const char* v = getenv("METALHLO_ATTN_BY_LENGTH"); return v ? atoi(v) : 1; }();
    static int64_t l2_bytes = 0;
    if (l2_bytes == 0) {
        int dev = 0, v = 0;
        MHLO_CUDA_TRY(cudaGetDevice(&dev), MHLO_CUDA_EXECUTION_FAILED);
        MHLO_CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, dev), MHLO_CUDA_EXECUTION_FAILED);
        l2_bytes = v > 0 ? v : 1;
    }
    // measured on B200 (126 MB of L2): 98 MB and 100 MB of K + V gain 10-20 %, 268 MB is neutral, 537 MB loses 15 %
    const bool fits = by_length_mode == 2 || kv_bytes <= l2_bytes / 100 * 85;
    // without a mask all tiles are equally long; dealing them one by one still evens out the last pass
    p.by_length = (by_length_mode != 0 && fits && tiles < (int64_t{1} << 30)) ? 1 : 0;
    if (s.tile_order == 1) p.by_length = 0;
    else if (s.tile_order == 2 && tiles < (int64_t{1} << 30)) p.by_length = 1;
    const unsigned grid = static_cast<unsigned>(p.by_length ? std::min<int64_t>(tiles, sm_count) : std::min<int64_t>((tiles + 1) / 2, sm_count));
    const cudaError_t launched = launch_dependent(kernel, dim3(grid), dim3(kAttnThreads), L::kTotal, stream, mq, mk, mv, p);
    if (launched != cudaSuccess) return fail(MHLO_CUDA_EXECUTION_FAILED, "launch of attention_tcgen05 failed: %s", cudaGetErrorString(launched));
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

bool attention_error_fetch_async(int* pinned_dst, cudaStream_t stream) {
    return cudaMemcpyFromSymbolAsync(pinned_dst, g_attn_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream) == cudaSuccess;
}

bool attention_error_store(int code) { return cudaMemcpyToSymbol(g_attn_error, &code, sizeof code) == cudaSuccess; }

bool attention_tc_supported(int dtype, const AttnShape& s, const void* mask) {
    if (dtype != MHLO_DT_BF16 && dtype != MHLO_DT_F16) return false;
    if (mask != nullptr) return false;
    if (!(s.scale > 0.f)) return false;  // the kernel takes the row maximum before scaling
    if (s.head_dim != 64 && s.head_dim != 128) return false;
    if (s.seq_q < 1 || s.seq_k < 1 || s.heads < 1 || s.batch < 1 || s.heads > 65535 || s.batch > 65535) return false;
    if (s.seq_q > 0x3fffffff || s.seq_k > 0x3fffffff) return false;
    if ((s.seq_q + kHalves * kBlockM - 1) / (kHalves * kBlockM) * s.heads * s.batch > 0x3fffffff) return false;  // tile index is an int
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
