// dot_general on the 5th-generation tensor cores: a persistent, warp-specialised tcgen05 GEMM.
//
//   C[b, m, n] = act( sum_k A[b, m, k] * B[b, k, n] + bias[n] ),  A/B bf16 or f16, fp32 accumulation in TMEM.
//
// One CTA per SM walks output tiles of 128 x BN (BN = 256 or 128). Per tile the K loop advances in 64-element
// panels through a ring of shared-memory stages:
//   warp 0 (one lane)  producer: TMA (cp.async.bulk.tensor, 128-byte swizzle, zero fill out of bounds) of the
//                      A and B panels into the next free stage, completion on the stage's "full" mbarrier
//   warp 1 (one lane)  MMA issuer: four tcgen05.mma.cta_group::1.kind::f16 (K = 16 each) per stage from
//                      shared-memory descriptors into one of two TMEM accumulator buffers; tcgen05.commit hands
//                      the stage back to the producer and, after the last panel, the accumulator to the epilogue
//   warps 2-9          epilogue: tcgen05.ld of the accumulator (each warp 32 TMEM lanes = 32 rows, half the columns),
//                      bias + activation in fp32, conversion, 16-byte stores; the other accumulator buffer is
//                      being filled by the MMA warp meanwhile
// Operand layouts: A may be K-major ([m][k], k contiguous) or M-major ([k][m]); B K-major ([n][k]) or N-major
// ([k][n]) - the instruction descriptor carries the majors, so transposed operands are read in place. Up to two
// batch dimensions ride along as TMA coordinates. Every mbarrier wait is bounded: on expiry the kernel records an
// error word and drains, it never spins forever.
//
// HBM traffic per tile pass: A and B panels are re-read from L2 across tiles; the tile order walks 16 row-tiles
// per column band so that the 148 concurrently resident tiles share operands in L2. Algorithmic bytes:
// (M*K + K*N) * 2 read + M*N * sizeof(out) written per batch entry.
#include <atomic>
#include <cuda.h>

#include <algorithm>
#include <string>

#include "contraction.cuh"
#include "tc_ptx.cuh"

namespace mhlo {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // one 128-byte swizzle row of 16-bit elements
constexpr int UMMA_K = 16;
constexpr int kEpilogueWarps = 8;  // two per TMEM lane quarter, each taking half of the tile's columns
constexpr int kGemmThreads = 32 * (2 + kEpilogueWarps);

__device__ int g_gemm_error = 0;

template <int ACT>
__device__ __forceinline__ float epilogue_act(float v) {
    if constexpr (ACT == MHLO_EPILOGUE_RELU) return fmaxf(v, 0.f);
    if constexpr (ACT == MHLO_EPILOGUE_GELU_TANH) {
        const float inner = 0.7978845608028654f * v * fmaf(0.044715f * v, v, 1.0f);
        float t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(inner));  // 2^-11 relative error: below the 16-bit output resolution
        const float hv = 0.5f * v;
        return fmaf(hv, t, hv);
    }
    if constexpr (ACT == MHLO_EPILOGUE_GELU_ERF) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
    if constexpr (ACT == MHLO_EPILOGUE_SILU) return v / (1.0f + __expf(-v));
    if constexpr (ACT == MHLO_EPILOGUE_TANH) return tanhf(v);
    if constexpr (ACT == MHLO_EPILOGUE_SIGMOID) return 1.0f / (1.0f + __expf(-v));
    return v;
}

// GELU (tanh form) on two f16 values at once: five half2 operations and one tanh.approx.f16x2 for the pair, where the fp32
// form spends five fp32 operations and one tanh.approx per value. The argument is the f16-rounded pre-activation; the
// arithmetic error (about 1.5e-3 relative) is that of the same chain evaluated op by op on f16 tensors.
__device__ __forceinline__ uint32_t gelu_tanh_f16x2(uint32_t xbits) {
    const __half2 x = *reinterpret_cast<const __half2*>(&xbits);
    const __half2 c0 = __float2half2_rn(0.7978845608028654f), c1 = __float2half2_rn(0.7978845608028654f * 0.044715f);
    const __half2 inner = __hmul2(x, __hfma2(__hmul2(x, x), c1, c0));
    uint32_t t;
    asm("tanh.approx.f16x2 %0, %1;" : "=r"(t) : "r"(*reinterpret_cast<const uint32_t*>(&inner)));
    const __half2 hx = __hmul2(x, __float2half2_rn(0.5f));
    const __half2 y = __hfma2(hx, *reinterpret_cast<const __half2*>(&t), hx);
    return *reinterpret_cast<const uint32_t*>(&y);
}

struct GemmParams {
    void* c;
    const void* bias;
    const void* residual;  // a matrix of C's type, pitch and column offset that is added to the product (after bias), or null
    int64_t m, n, k;
    int64_t batch0, batch1;
    int32_t tiles_m, tiles_n;
    int64_t num_tiles;
    int32_t a_mn_major, b_mn_major;  // 0 = K-major, 1 = M/N-major
    int32_t in_bf16;                 // operand format: 1 = bf16, 0 = f16
    int32_t out_dtype;               // MHLO_DT_BF16 / F16 / F32
    int32_t epilogue;
    int32_t c_vec_ok;                // rows of C start 16-byte aligned: vector stores allowed
    int64_t ldc, c_col0;             // row pitch of C in elements; first column of this product inside the wider matrix
    void* copies[7];                 // further destinations of every tile store (the same matrix in peers' memory)
    int32_t n_copies;
    int32_t c_tma;                   // C has a tensor map: the epilogue stores its staged boxes with bulk tensor copies
    int32_t stages;                  // depth of the TMA ring in use (<= the kernel's STAGES)
    // MODE 3 (convolution without a patch matrix): a row tile is an 8 x 16 patch of output positions of one image
    // (batch index = image, tiles_m = patches per image); k-block kb = (filter tap, 64 input channels)
    int32_t conv_tiles_x, conv_kw, conv_cblocks, conv_pad_h, conv_pad_w, conv_dil_h, conv_dil_w, conv_oh, conv_stride_h, conv_stride_w;
};

// Tensor maps of the further copies of C (GemmParams::copies, in the same order), used when the copies are written with
// bulk tensor stores.
template <bool PEER>
struct PeerMaps {
    CUtensorMap m[7];
};
template <>
struct PeerMaps<false> {};  // kernels that never store into copies carry no maps in their parameters

// CTAS = 2: a pair of CTAs shares one (2 * BM) x BN tile; each stages its own BM rows of A and BN / 2 rows of B.
template <int BN, int STAGES, int CTAS = 1>
struct SmemLayout {
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN / CTAS * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarrierBytes = 256;
    static constexpr int kStagingBytes = kEpilogueWarps * 4096;  // one 32-row x 128-byte tile per epilogue warp
    static constexpr int kBiasBytes = kEpilogueWarps * 128;      // 32 fp32 bias values per epilogue warp
    static constexpr int kStagingOff = STAGES * kStageBytes;
    static constexpr int kBiasOff = kStagingOff + kStagingBytes;
    static constexpr int kBarrierOff = kBiasOff + kBiasBytes;
    static constexpr int kTotal = kBarrierOff + kBarrierBytes + 1024;  // + slack for 1024-byte alignment
};

// Tile order: bands of 16 row-tiles; inside a band the column index is the slow one.
__device__ __forceinline__ void tile_coords(int64_t tile, const GemmParams& p, int* bz, int* tm, int* tn) {
    const int64_t per_batch = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
    *bz = static_cast<int>(tile / per_batch);
    int64_t t = tile % per_batch;
    constexpr int kBand = 16;
    const int64_t band_tiles = static_cast<int64_t>(kBand) * p.tiles_n;
    const int band = static_cast<int>(t / band_tiles);
    const int rows_in_band = min(kBand, p.tiles_m - band * kBand);
    t -= band * band_tiles;
    *tm = band * kBand + static_cast<int>(t % rows_in_band);
    *tn = static_cast<int>(t / rows_in_band);
}

// MODE: 0 = the plain product, 1 = with the tensor maps of further copies of C (bulk stores into peers), 2 = with a residual
// matrix added in the epilogue, 3 = a 2-D convolution read straight from its NHWC input: the A tile of k-block (tap, 64
// channels) is the 8 x 16 patch of input pixels that tap sees, one bulk tensor load whose out-of-image pixels arrive as
// zeros (the padding), and the result tile goes back as boxes of the NHWC output. The variants are separate instantiations
// so that the plain product carries neither the maps in its parameters nor the residual's registers.
template <int BN, int STAGES, int ACT, int CTAS, int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)  // ten warps are allocated as twelve: 168 registers per thread is the ceiling
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_c, const __grid_constant__ GemmParams p,
                    const __grid_constant__ PeerMaps<MODE == 1> peer_maps) {
    using L = SmemLayout<BN, STAGES, CTAS>;
    constexpr bool PEER = MODE == 1, RES = MODE == 2;
    constexpr bool kPair = CTAS == 2;
    constexpr int BNL = BN / CTAS;  // rows of B (columns of the tile) this CTA stages
    const uint32_t cta_rank = kPair ? cluster_cta_rank() : 0u;
    const bool leader = cta_rank == 0;
    // the walker of output tiles is the CTA, or the pair: p.tiles_m counts (CTAS * BM)-row tiles
    const int64_t walker = kPair ? blockIdx.x >> 1 : blockIdx.x, walkers = kPair ? gridDim.x >> 1 : gridDim.x;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarrierOff);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tmem_full = empty_bar + STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = static_cast<int>((p.k + BK - 1) / BK);
    constexpr uint32_t kTmemCols = 2 * BN;

    if (warp == 0 && lane == 0) {
        prefetch_tmap(&map_a);
        prefetch_tmap(&map_b);
        if (p.c_tma) {
            prefetch_tmap(&map_c);
            if constexpr (PEER)
                for (int d = 0; d < p.n_copies; ++d) prefetch_tmap(&peer_maps.m[d]);
        }
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], kEpilogueWarps * CTAS); }
        fence_barrier_init();
    }
    if (warp == 1) {
        if constexpr (kPair) {  // one warp of each CTA of the pair: the columns are taken in both CTAs' TMEM
            tmem_alloc_pair(tmem_slot, kTmemCols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, kTmemCols);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (kPair) {  // both CTAs' barriers exist before either signals the other's
        cluster_arrive();
        cluster_wait();
    }
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // everything above touched only this CTA's shared memory and TMEM: it may overlap the previous kernel's tail
    grid_dependency_wait();
    grid_dependency_release();

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t tile = walker; tile < p.num_tiles && ok; tile += walkers) {
                int bz, tm, tn;
                tile_coords(tile, p, &bz, &tm, &tn);
                const int b0 = bz / static_cast<int>(p.batch1), b1 = bz % static_cast<int>(p.batch1);
                const int row_a = (tm * CTAS + static_cast<int>(cta_rank)) * BM;    // first row of A this CTA stages
                const int row_b = tn * BN + static_cast<int>(cta_rank) * BNL;       // first row of B (column of the tile)
                for (int kb = 0; kb < k_blocks; ++kb) {
                    const bool freed = kPair ? mbar_wait_pair(&empty_bar[stage], phase ^ 1) : mbar_wait(&empty_bar[stage], phase ^ 1);
                    if (!freed) { ok = false; atomicExch(&g_gemm_error, 1); break; }
                    uint8_t* sa = smem + stage * L::kStageBytes;
                    uint8_t* sb = sa + L::kABytes;
                    // Pair: the bytes of both CTAs are counted on the leader's barrier, which alone is armed (by the leader)
                    uint32_t full_addr = 0;
                    if constexpr (kPair) {
                        full_addr = map_to_cta(smem_u32(&full_bar[stage]), 0);
                        if (leader) mbar_expect_tx(&full_bar[stage], CTAS * L::kStageBytes);
                    } else {
                        mbar_expect_tx(&full_bar[stage], L::kStageBytes);
                    }
                    auto load = [&](uint8_t* dst, const CUtensorMap* map, int c0, int c1) {
                        if constexpr (kPair) tma_load_4d_pair(dst, map, full_addr, c0, c1, b1, b0);
                        else if constexpr (MODE == 3) tma_load_4d(dst, map, &full_bar[stage], c0, c1, 0, 0);  // the filter matrix has no batch
                        else tma_load_4d(dst, map, &full_bar[stage], c0, c1, b1, b0);
                    };
                    if constexpr (MODE == 3) {
                        const int ty = tm / p.conv_tiles_x, tx = tm - ty * p.conv_tiles_x;
                        const int tap = kb / p.conv_cblocks, cb = kb - tap * p.conv_cblocks;
                        const int dy = tap / p.conv_kw, dx = tap - dy * p.conv_kw;
                        // {channel, x, y, image}: pixels outside the image (the padding) are filled with zeros by the copy
                        // (a strided convolution reads every conv_stride-th pixel: the tensor map's traversal strides)
                        tma_load_4d(sa, &map_a, &full_bar[stage], cb * 64, tx * 16 * p.conv_stride_w + dx * p.conv_dil_w - p.conv_pad_w,
                                    ty * 8 * p.conv_stride_h + dy * p.conv_dil_h - p.conv_pad_h, bz);
                    } else if (!p.a_mn_major) {
                        load(sa, &map_a, kb * BK, row_a);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j) load(sa + j * 64 * BK * 2, &map_a, row_a + j * 64, kb * BK);
                    }
                    if (!p.b_mn_major) {
                        load(sb, &map_b, kb * BK, row_b);
                    } else {
#pragma unroll
                        for (int j = 0; j < BNL / 64; ++j) load(sb + j * 64 * BK * 2, &map_b, row_b + j * 64, kb * BK);
                    }
                    if (++stage == p.stages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the whole warp runs the loop so that descriptors stay in uniform registers;
        // one elected lane issues the tcgen05 instructions. In a pair only the leader CTA issues: its MMAs write the
        // accumulator halves in both CTAs' TMEM and its commits arrive on both CTAs' barriers ----------------
        if (leader) {
            // instruction descriptor: D = f32, A/B = bf16 or f16, majors, N >> 3, M >> 4
            const uint32_t fmt = p.in_bf16 ? 1u : 0u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(p.a_mn_major) << 15) |
                                   (static_cast<uint32_t>(p.b_mn_major) << 16) | (static_cast<uint32_t>(BN >> 3) << 17) |
                                   (static_cast<uint32_t>((BM * CTAS) >> 4) << 24);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            auto commit = [&](uint64_t* bar) {  // arrival on `bar` of this CTA and, in a pair, of the other CTA too
                if constexpr (kPair) {
                    umma_commit_pair(map_to_cta(smem_u32(bar), 0));
                    umma_commit_pair(map_to_cta(smem_u32(bar), 1));
                } else {
                    umma_commit(bar);
                }
            };
            for (int64_t tile = walker; tile < p.num_tiles && ok; tile += walkers) {
                const bool drained = kPair ? mbar_wait_pair(&tmem_empty[acc], acc_phase ^ 1) : mbar_wait(&tmem_empty[acc], acc_phase ^ 1);
                if (!drained) { atomicExch(&g_gemm_error, 2); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase)) { ok = false; atomicExch(&g_gemm_error, 3); break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
                    const uint32_t sb = sa + L::kABytes;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // K-major: 8-row groups are 1024 B apart, a K step of 16 elements is 32 B along the swizzled row.
                        // M/N-major: 64-element blocks are one 8 KiB box apart (LBO), 8-row K groups 1024 B (SBO), a K
                        // step is 16 rows = 2048 B.
                        const uint64_t da = p.a_mn_major ? make_smem_desc(sa + k * UMMA_K * 128, 64 * BK * 2, 1024)
                                                         : make_smem_desc(sa + k * UMMA_K * 2, 16, 1024);
                        const uint64_t db = p.b_mn_major ? make_smem_desc(sb + k * UMMA_K * 128, 64 * BK * 2, 1024)
                                                         : make_smem_desc(sb + k * UMMA_K * 2, 16, 1024);
                        if (elect_one()) {
                            if constexpr (kPair) umma_f16_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                            else umma_f16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                        }
                    }
                    if (elect_one()) commit(&empty_bar[stage]);  // stage is free once these MMAs have read it
                    __syncwarp();
                    if (++stage == p.stages) { stage = 0; phase ^= 1; }
                }
                if (elect_one()) commit(&tmem_full[acc]);  // accumulator complete
                __syncwarp();
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ---------------- epilogue (warps 2..9) ----------------
        const int quarter = warp & 3;  // TMEM lanes this warp may read: 32*quarter .. +31
        const int col_begin = ((warp - 2) >> 2) * (BN / 2), col_end = col_begin + BN / 2;
        int acc = 0;
        uint32_t acc_phase = 0;
        const size_t out_es = p.out_dtype == MHLO_DT_F32 ? 4 : 2;
        for (int64_t tile = walker; tile < p.num_tiles; tile += walkers) {
            int bz, tm, tn;
            tile_coords(tile, p, &bz, &tm, &tn);
            // The residual (16-bit results only): this thread's row of the warp's BN/2 columns, at most 256 bytes, asked for
            // before the wait for the accumulator so that the loads run under the tile's MMAs. Pieces beyond the last
            // column (n is a multiple of the 16-byte piece here) stay zero.
            constexpr bool use_res = RES;
            uint4 res_tile[16];
            if (use_res) {
                const int64_t rrow = (static_cast<int64_t>(tm) * CTAS + cta_rank) * BM + quarter * 32 + lane;
                const int64_t rcol = static_cast<int64_t>(tn) * BN + col_begin;
                const uint8_t* rp = static_cast<const uint8_t*>(p.residual) + static_cast<int64_t>(bz) * p.m * p.ldc * 2 + (rrow * p.ldc + p.c_col0 + rcol) * 2;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    res_tile[j] = make_uint4(0u, 0u, 0u, 0u);
                    if (j * 8 < BN / 2 && rrow < p.m && rcol + j * 8 < p.n) res_tile[j] = __ldg(reinterpret_cast<const uint4*>(rp) + j);
                }
            }
            const bool filled = kPair ? mbar_wait_pair(&tmem_full[acc], acc_phase) : mbar_wait(&tmem_full[acc], acc_phase);
            if (!filled) { atomicExch(&g_gemm_error, 4); break; }
            tc_fence_after();
            // Each warp turns its 32 rows x (BN/2) columns into output in chunks of 128 bytes per row: the thread that owns
            // a row (TMEM lane) writes its 128 bytes into a swizzled shared-memory tile, then the warp reads the tile back
            // row-wise so that every global store instruction covers whole rows (coalesced), whatever the row pitch of C.
            const int64_t row0 = (static_cast<int64_t>(tm) * CTAS + cta_rank) * BM + quarter * 32;
            const int chunk_cols = p.out_dtype == MHLO_DT_F32 ? 32 : 64;
            uint8_t* stage_tile = smem + L::kStagingOff + (warp - 2) * 4096;
            const int64_t batch_off = static_cast<int64_t>(bz) * p.m * p.ldc * out_es;
            uint8_t* cbase = static_cast<uint8_t*>(p.c) + batch_off;
            // bias of this warp's BN/2 columns: lane l holds columns l, 32 + l, ... (one global load per column per tile). For
            // every group of 32 columns the lanes put their value into the warp's 128 bytes of shared memory and each thread
            // reads all 32 back with broadcast loads: eight 16-byte loads per group instead of 32 shuffles.
            constexpr int kBiasPerLane = BN / 2 / 32;
            float breg[kBiasPerLane];
            const bool has_bias = p.bias != nullptr;
            float* bias_tile = reinterpret_cast<float*>(smem + L::kBiasOff) + (warp - 2) * 32;
#pragma unroll
            for (int q = 0; q < kBiasPerLane; ++q) {
                const int64_t col = static_cast<int64_t>(tn) * BN + col_begin + q * 32 + lane;
                float bv = 0.f;
                if (has_bias && col < p.n) {
                    if (p.out_dtype == MHLO_DT_F32) bv = static_cast<const float*>(p.bias)[col];
                    else if (p.out_dtype == MHLO_DT_BF16) bv = __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col]);
                    else bv = __half2float(static_cast<const __half*>(p.bias)[col]);
                }
                breg[q] = bv;
            }
#pragma unroll 1
            for (int c0 = col_begin; c0 < col_end; c0 += chunk_cols) {
                const int64_t col0 = static_cast<int64_t>(tn) * BN + c0;
                uint4 out16[8];
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN + c0);
                // this chunk's share of the residual pieces fetched at the start of the tile
                uint4 res[8];
                if (use_res) {
                    const bool second = c0 != col_begin;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        res[j].x = second ? res_tile[8 + j].x : res_tile[j].x; res[j].y = second ? res_tile[8 + j].y : res_tile[j].y;
                        res[j].z = second ? res_tile[8 + j].z : res_tile[j].z; res[j].w = second ? res_tile[8 + j].w : res_tile[j].w;
                    }
                }
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (half * 32 >= chunk_cols) break;
                    // 32 accumulator columns at a time: a 64-column load measured no faster and costs 32 more live registers,
                    // which the 168 available here do not have
                    uint32_t r[32];
                    tmem_ld32(taddr + half * 32, r);
                    tmem_ld_wait();
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    if (has_bias) {
                        const int group = (c0 - col_begin) / 32 + half;  // which 32 columns of the warp's range
                        float mine = breg[0];
#pragma unroll
                        for (int q = 1; q < kBiasPerLane; ++q) mine = group == q ? breg[q] : mine;
                        bias_tile[lane] = mine;
                        __syncwarp();
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float4 b4 = reinterpret_cast<const float4*>(bias_tile)[j];  // the same address in every lane
                            v[4 * j] += b4.x; v[4 * j + 1] += b4.y; v[4 * j + 2] += b4.z; v[4 * j + 3] += b4.w;
                        }
                        __syncwarp();  // every lane has read the group before the next one is written
                    }
                    if (use_res) {  // 16-bit results without activation (the launcher sends every other product elsewhere)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint4 q4 = res[half * 4 + j];
                            const uint32_t w4[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                float lo, hi;
                                if (p.out_dtype == MHLO_DT_BF16) {
                                    lo = __uint_as_float(w4[q] << 16);
                                    hi = __uint_as_float(w4[q] & 0xffff0000u);
                                } else {
                                    const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&w4[q]));
                                    lo = f2.x; hi = f2.y;
                                }
                                v[8 * j + 2 * q] += lo;
                                v[8 * j + 2 * q + 1] += hi;
                            }
                        }
                    }
                    // f16 results take the tanh-form GELU in packed f16 arithmetic after the conversion below
                    constexpr bool kPackedGelu = ACT == MHLO_EPILOGUE_GELU_TANH;
                    if (ACT != MHLO_EPILOGUE_NONE && !(kPackedGelu && p.out_dtype == MHLO_DT_F16)) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = epilogue_act<ACT>(v[j]);
                    }
                    if (p.out_dtype == MHLO_DT_F32) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            out16[j] = make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]), __float_as_uint(v[4 * j + 2]), __float_as_uint(v[4 * j + 3]));
                    } else if (p.out_dtype == MHLO_DT_BF16) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t w[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                __nv_bfloat162 hh = __floats2bfloat162_rn(v[8 * j + 2 * q], v[8 * j + 2 * q + 1]);
                                w[q] = *reinterpret_cast<uint32_t*>(&hh);
                            }
                            out16[half * 4 + j] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t w[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                __half2 hh = __floats2half2_rn(v[8 * j + 2 * q], v[8 * j + 2 * q + 1]);
                                w[q] = *reinterpret_cast<uint32_t*>(&hh);
                                if constexpr (kPackedGelu) w[q] = gelu_tanh_f16x2(w[q]);
                            }
                            out16[half * 4 + j] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
                if (p.c_tma) {
                    if (lane == 0) tma_store_wait_read();  // the previous chunk's bulk store has read the staging tile
                }
                __syncwarp();  // the previous chunk's read-back is finished
#pragma unroll
                for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(stage_tile + lane * 128 + ((c ^ (lane & 7)) << 4)) = out16[c];
                const int64_t cols_left = p.n - col0;  // columns of this chunk that exist
                if (p.c_tma) {
                    // the staging tile is exactly a 128-byte-swizzled box of 32 rows: one bulk tensor store writes it, clipped
                    // at the edges of C by the hardware
                    fence_proxy_async();
                    __syncwarp();
                    if constexpr (MODE == 3) {
                        // the warp's 32 rows are two rows of 16 output pixels: one box {columns, 16, 2} of the NHWC result,
                        // clipped at the image's edges by the copy
                        const int ty = tm / p.conv_tiles_x, tx = tm - ty * p.conv_tiles_x;
                        if (lane == 0 && cols_left > 0 && ty * 8 + quarter * 2 < p.conv_oh) {  // no store starts outside the image
                            tma_store_4d(&map_c, stage_tile, static_cast<int>(col0), tx * 16, ty * 8 + quarter * 2, bz);
                            tma_store_commit();
                        }
                        continue;
                    }
                    if (lane == 0 && cols_left > 0 && row0 < p.m) {
                        const int b1 = static_cast<int>(bz % p.batch1), b0 = static_cast<int>(bz / p.batch1);
                        tma_store_4d(&map_c, stage_tile, static_cast<int>(col0), static_cast<int>(row0), b1, b0);
                        // the same box into every other copy of C: bulk stores over NVLink, in the same group
                        if constexpr (PEER)
                            for (int d = 0; d < p.n_copies; ++d)
                                tma_store_4d(&peer_maps.m[d], stage_tile, static_cast<int>(col0), static_cast<int>(row0), b1, b0);
                        tma_store_commit();
                    }
                    continue;
                }
                __syncwarp();
                if (cols_left <= 0) continue;
                if (p.c_vec_ok && cols_left >= chunk_cols) {
                    // 8 lanes cover one row's 128 bytes, four rows per instruction
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int rr = it * 4 + (lane >> 3), c = lane & 7;
                        if (row0 + rr < p.m) {
                            const uint4 val = *reinterpret_cast<const uint4*>(stage_tile + rr * 128 + ((c ^ (rr & 7)) << 4));
                            const int64_t at = ((row0 + rr) * p.ldc + p.c_col0 + col0) * out_es + c * 16;
                            *reinterpret_cast<uint4*>(cbase + at) = val;
                            // the same 16 bytes into every other copy of C (peer GPUs' memory, plain stores over NVLink)
                            for (int d = 0; d < p.n_copies; ++d)
                                *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.copies[d]) + batch_off + at) = val;
                        }
                    }
                } else if (cols_left >= chunk_cols && p.n_copies == 0) {
                    // Rows of C that do not start on 16-byte boundaries (a row pitch such as 50257 f16): every row's 128
                    // bytes are still written mostly with 16-byte stores. With a = (address of the row's chunk) mod 16, the
                    // aligned 16-byte pieces of global memory inside the chunk hold staged bytes [16 g - a, 16 g - a + 16),
                    // g = 1..7: the tail of staged piece g - 1 and the head of piece g. Rows eight apart share a (eight
                    // pitches are a multiple of 16 bytes), so one instruction serves rows j, j + 8, j + 16, j + 24 with 8
                    // lanes each: a is uniform over the warp, the two staged pieces come in with 16-byte loads and one
                    // funnel shift per word realigns them. The (16 - a) head bytes and a tail bytes of a row, 16 bytes
                    // together, go out one element per lane.
                    const int edge_elems = 16 / static_cast<int>(out_es);
#pragma unroll 1
                    for (int j = 0; j < 8; ++j) {
                        const int rr = j + 8 * (lane >> 3), c = lane & 7;
                        uint8_t* dst = cbase + ((row0 + rr) * p.ldc + p.c_col0 + col0) * out_es;
                        const int a = static_cast<int>(reinterpret_cast<uintptr_t>(dst) & 15);  // the same in every lane
                        if (row0 + rr >= p.m) continue;
                        const uint8_t* srow = stage_tile + rr * 128;
                        auto staged_piece = [&](int g) { return *reinterpret_cast<const uint4*>(srow + ((g ^ (rr & 7)) << 4)); };
                        if (a == 0) {
                            *reinterpret_cast<uint4*>(dst + c * 16) = staged_piece(c);
                            continue;
                        }
                        if (c < 7) {
                            const uint4 lo = staged_piece(c), hi = staged_piece(c + 1);
                            const int s = 16 - a;  // first byte of the aligned piece inside lo:hi
                            uint32_t x0, x1, x2, x3, x4;
                            switch (s >> 2) {
                                case 0: x0 = lo.x; x1 = lo.y; x2 = lo.z; x3 = lo.w; x4 = hi.x; break;
                                case 1: x0 = lo.y; x1 = lo.z; x2 = lo.w; x3 = hi.x; x4 = hi.y; break;
                                case 2: x0 = lo.z; x1 = lo.w; x2 = hi.x; x3 = hi.y; x4 = hi.z; break;
                                default: x0 = lo.w; x1 = hi.x; x2 = hi.y; x3 = hi.z; x4 = hi.w; break;
                            }
                            uint4 v;
                            if (s & 2) {
                                v.x = __funnelshift_r(x0, x1, 16); v.y = __funnelshift_r(x1, x2, 16);
                                v.z = __funnelshift_r(x2, x3, 16); v.w = __funnelshift_r(x3, x4, 16);
                            } else {
                                v = make_uint4(x0, x1, x2, x3);
                            }
                            *reinterpret_cast<uint4*>(dst + 16 * (c + 1) - a) = v;
                        }
                        if (c < edge_elems) {
                            auto staged_word = [&](int wi) {  // 32-bit word wi of the row, through the tile's swizzle
                                return *reinterpret_cast<const uint32_t*>(srow + ((((wi >> 2) ^ (rr & 7)) << 4) | ((wi & 3) << 2)));
                            };
                            const int head = (16 - a) / static_cast<int>(out_es);             // elements before the first aligned piece
                            const int e = c < head ? c : 128 / static_cast<int>(out_es) - (edge_elems - head) + (c - head);
                            if (out_es == 2) {
                                const uint32_t word = staged_word(e >> 1);
                                reinterpret_cast<uint16_t*>(dst)[e] = static_cast<uint16_t>((e & 1) ? word >> 16 : word & 0xffffu);
                            } else {
                                reinterpret_cast<uint32_t*>(dst)[e] = staged_word(e);
                            }
                        }
                    }
                } else {
                    // ragged edge (or copies in peers' memory behind an unaligned pitch): one row per instruction, 4 bytes per lane
                    const int per_lane = out_es == 4 ? 1 : 2;  // elements in a lane's 4 bytes
                    for (int rr = 0; rr < 32 && row0 + rr < p.m; ++rr) {
                        const uint32_t word = *reinterpret_cast<const uint32_t*>(stage_tile + rr * 128 + (((lane >> 2) ^ (rr & 7)) << 4) + (lane & 3) * 4);
                        const int64_t at = ((row0 + rr) * p.ldc + p.c_col0 + col0) * out_es;
                        const int e0 = lane * per_lane;
                        for (int d = -1; d < p.n_copies; ++d) {
                            uint8_t* dst = (d < 0 ? cbase : static_cast<uint8_t*>(p.copies[d]) + batch_off) + at;
                            if (out_es == 4) {
                                if (e0 < cols_left) reinterpret_cast<uint32_t*>(dst)[e0] = word;
                            } else {
                                if (e0 < cols_left) reinterpret_cast<uint16_t*>(dst)[e0] = static_cast<uint16_t>(word & 0xffffu);
                                if (e0 + 1 < cols_left) reinterpret_cast<uint16_t*>(dst)[e0 + 1] = static_cast<uint16_t>(word >> 16);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {  // the accumulator buffer goes back to the MMA issuer (the leader's, in a pair)
                if (leader) mbar_arrive(&tmem_empty[acc]);
                else mbar_arrive_remote(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
            }
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
        if (p.c_tma && lane == 0) tma_store_wait_all();  // shared memory stays allocated until the last box has been read
    }

    tc_fence_before();
    __syncthreads();
    if constexpr (kPair) {  // neither CTA leaves, or gives up its TMEM, while the other may still address it
        cluster_arrive();
        cluster_wait();
    }
    if (warp == 1) {
        tc_fence_after();
        if constexpr (kPair) tmem_dealloc_pair(tmem_base, kTmemCols);
        else tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- host side ---------------------------------------------------------------------------------------------------------

bool encode_map(CUtensorMap* map, const void* base, const int64_t dims[4], const int64_t strides_bytes[3], const uint32_t box[4],
                std::string* why) {
    cuuint64_t gdim[4];
    cuuint64_t gstr[3];
    cuuint32_t bx[4], es[4] = {1, 1, 1, 1};
    for (int i = 0; i < 4; ++i) { gdim[i] = static_cast<cuuint64_t>(dims[i]); bx[i] = box[i]; }
    for (int i = 0; i < 3; ++i) gstr[i] = static_cast<cuuint64_t>(strides_bytes[i]);
    // The driver entry point is looked up at run time so that the library loads on machines without libcuda
    // (the host-side compiler and the ABI tests run there).
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
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
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), gdim, gstr, bx, es,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        *why = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(r));
        return false;
    }
    return true;
}

// Operand as a 4-D tensor map {inner, outer, batch1, batch0}. `inner_is_k`: the contiguous dimension is K.
bool operand_map(CUtensorMap* map, const void* base, int64_t inner, int64_t outer, int64_t outer_stride, int64_t b1, int64_t b1_stride,
                 int64_t b0, int64_t b0_stride, uint32_t box_inner, uint32_t box_outer, std::string* why) {
    const int64_t dims[4] = {inner, outer, b1, b0};
    // a dimension of extent 1 still needs a legal stride (non-zero multiple of 16)
    const int64_t span = std::max<int64_t>(16, ((outer > 1 ? outer_stride * outer : inner) * 2 + 15) / 16 * 16);
    int64_t s1 = outer_stride * 2, s2 = b1_stride * 2, s3 = b0_stride * 2;
    if (outer == 1 || s1 == 0) s1 = span;
    if (b1 == 1 || s2 == 0) s2 = span;
    if (b0 == 1 || s3 == 0) s3 = span;
    const int64_t strides[3] = {s1, s2, s3};
    const uint32_t box[4] = {box_inner, box_outer, 1, 1};
    return encode_map(map, base, dims, strides, box, why);
}

bool stride_ok(int64_t elems) { return elems > 0 && (elems * 2) % 16 == 0; }

// C [batch0, batch1, m, n] with row pitch ldc as a 4-D map {n, m, batch1, batch0}; one box = 128 bytes x 32 rows, the
// staging tile of one epilogue warp.
bool output_map(CUtensorMap* map, void* base, int out_dtype, int64_t n, int64_t m, int64_t ldc, int64_t b1, int64_t b0, std::string* why) {
    const int64_t es = out_dtype == MHLO_DT_F32 ? 4 : 2;
    cuuint64_t gdim[4] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(m), static_cast<cuuint64_t>(b1), static_cast<cuuint64_t>(b0)};
    cuuint64_t gstr[3] = {static_cast<cuuint64_t>(ldc * es), static_cast<cuuint64_t>(m * ldc * es), static_cast<cuuint64_t>(b1 * m * ldc * es)};
    cuuint32_t box[4] = {static_cast<cuuint32_t>(128 / es), 32, 1, 1}, estr[4] = {1, 1, 1, 1};
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
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
    const CUtensorMapDataType dt = out_dtype == MHLO_DT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : (out_dtype == MHLO_DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
    const CUresult r = encode(map, dt, 4, base, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        *why = "cuTensorMapEncodeTiled (output) failed with CUresult " + std::to_string(static_cast<int>(r));
        return false;
    }
    return true;
}

}  // namespace

bool gemm_tc_supported(const GemmProblem& p) {
    const bool f16 = p.in_dtype == MHLO_DT_F16, bf16 = p.in_dtype == MHLO_DT_BF16;
    if (!f16 && !bf16) return false;
    if (p.out_dtype != p.in_dtype && p.out_dtype != MHLO_DT_F32) return false;
    if (p.m <= 0 || p.n <= 0 || p.k <= 0 || p.batch0 <= 0 || p.batch1 <= 0) return false;
    if (p.m * p.n < 64 * 64) return false;  // tiny products: the general kernel has less fixed cost
    if (!aligned16(p.a) || !aligned16(p.b)) return false;
    // one of (row, col) strides must be 1; the other, and the batch strides, 16-byte multiples
    const bool a_k = p.as[3] == 1 || p.k == 1, a_m = p.as[2] == 1 || p.m == 1;
    const bool b_n = p.bs[3] == 1 || p.n == 1, b_k = p.bs[2] == 1 || p.k == 1;
    if (!(a_k || a_m) || !(b_n || b_k)) return false;
    auto batch_ok = [&](const int64_t* s) {
        return (p.batch0 == 1 || stride_ok(s[0])) && (p.batch1 == 1 || stride_ok(s[1]));
    };
    if (!batch_ok(p.as) || !batch_ok(p.bs)) return false;
    if (a_k ? !(p.m == 1 || stride_ok(p.as[2])) : !(p.k == 1 || stride_ok(p.as[3]))) return false;
    if (b_k ? !(p.n == 1 || stride_ok(p.bs[3])) : !(p.k == 1 || stride_ok(p.bs[2]))) return false;
    if (p.batch0 * p.batch1 > 0x7fffffffLL || p.m > 0x7fffffffLL || p.n > 0x7fffffffLL || p.k > 0x7fffffffLL) return false;
    return true;
}

template <int BN, int STAGES, int ACT, int CTAS, int MODE = 0>
static int launch_gemm_act(const GemmProblem& pr, cudaStream_t stream) {
    constexpr bool PEER = MODE == 1;
    using L = SmemLayout<BN, STAGES, CTAS>;
    const bool a_k = pr.as[3] == 1 || pr.k == 1;
    const bool b_k = pr.bs[2] == 1 || pr.k == 1;  // K-major B = [n][k] with k contiguous
    CUtensorMap map_a, map_b;
    std::string why;
    bool ok;
    if (a_k) ok = operand_map(&map_a, pr.a, pr.k, pr.m, pr.as[2], pr.batch1, pr.as[1], pr.batch0, pr.as[0], BK, BM, &why);
    else ok = operand_map(&map_a, pr.a, pr.m, pr.k, pr.as[3], pr.batch1, pr.as[1], pr.batch0, pr.as[0], 64, BK, &why);
    if (!ok) return fail(MHLO_CUDA_EXECUTION_FAILED, "gemm: tensor map for A: %s", why.c_str());
    if (b_k) ok = operand_map(&map_b, pr.b, pr.k, pr.n, pr.bs[3], pr.batch1, pr.bs[1], pr.batch0, pr.bs[0], BK, BN / CTAS, &why);
    else ok = operand_map(&map_b, pr.b, pr.n, pr.k, pr.bs[2], pr.batch1, pr.bs[1], pr.batch0, pr.bs[0], 64, BK, &why);
    if (!ok) return fail(MHLO_CUDA_EXECUTION_FAILED, "gemm: tensor map for B: %s", why.c_str());

    GemmParams p;
    p.c = pr.c;
    p.bias = pr.bias;
    p.residual = pr.residual;
    p.m = pr.m; p.n = pr.n; p.k = pr.k;
    p.batch0 = pr.batch0; p.batch1 = pr.batch1;
    p.tiles_m = static_cast<int>((pr.m + BM * CTAS - 1) / (BM * CTAS));
    p.stages = pr.stages >= 2 && pr.stages <= STAGES ? pr.stages : STAGES;
    p.tiles_n = static_cast<int>((pr.n + BN - 1) / BN);
    p.num_tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n * pr.batch0 * pr.batch1;
    p.a_mn_major = a_k ? 0 : 1;
    p.b_mn_major = b_k ? 0 : 1;
    p.in_bf16 = pr.in_dtype == MHLO_DT_BF16;
    p.out_dtype = pr.out_dtype;
    p.epilogue = pr.epilogue;
    const size_t out_es = pr.out_dtype == MHLO_DT_F32 ? 4 : 2;
    p.ldc = pr.ldc > 0 ? pr.ldc : pr.n;
    p.c_col0 = pr.c_col0;
    p.n_copies = pr.n_copies;
    bool aligned = aligned16(pr.c) && (p.ldc * out_es) % 16 == 0 && (p.c_col0 * out_es) % 16 == 0;
    for (int d = 0; d < 7; ++d) {
        p.copies[d] = d < pr.n_copies ? pr.copies[d] : nullptr;
        if (d < pr.n_copies) aligned = aligned && aligned16(pr.copies[d]);
    }
    p.c_vec_ok = aligned;
    // Bulk tensor stores need 16-byte aligned rows and a 16-byte aligned base. The map of a column block inside a wider
    // matrix starts at the block's first column and is n columns wide. Copies in peers' memory are written with bulk
    // stores too (one more map per copy) when the problem asks for it; otherwise they keep the per-lane stores.
    CUtensorMap map_c;
    memset(&map_c, 0, sizeof map_c);
    PeerMaps<PEER> peer_maps;
    memset(&peer_maps, 0, sizeof peer_maps);
    p.c_tma = 0;
    static const bool tma_store_enabled = [] {
        const char* v = getenv("METALHLO_GEMM_TMA_STORE");
        return !(v && v[0] == '0');  // METALHLO_GEMM_TMA_STORE=0 keeps the per-lane stores
    }();
    const bool copies_by_tma = pr.n_copies == 0 || (PEER && pr.copy_stores == 2);
    if (tma_store_enabled && aligned && copies_by_tma && pr.m * p.ldc * static_cast<int64_t>(out_es) % 16 == 0) {
        const size_t col_off = static_cast<size_t>(p.c_col0) * out_es;
        if (!output_map(&map_c, static_cast<uint8_t*>(pr.c) + col_off, pr.out_dtype, pr.n, pr.m, p.ldc, pr.batch1, pr.batch0, &why))
            return fail(MHLO_CUDA_EXECUTION_FAILED, "gemm: tensor map for C: %s", why.c_str());
        if constexpr (PEER)
            for (int d = 0; d < pr.n_copies; ++d)
                if (!output_map(&peer_maps.m[d], static_cast<uint8_t*>(pr.copies[d]) + col_off, pr.out_dtype, pr.n, pr.m, p.ldc, pr.batch1, pr.batch0, &why))
                return fail(MHLO_CUDA_EXECUTION_FAILED, "gemm: tensor map for copy %d of C: %s", d, why.c_str());
        p.c_tma = 1;
    }

    auto kernel = gemm_tcgen05_kernel<BN, STAGES, ACT, CTAS, MODE>;
    // the attribute belongs to the (kernel, device) pair: one flag per device ordinal
    static std::atomic<bool> attr_set[64];
    int attr_dev = 0;
    MHLO_CUDA_TRY(cudaGetDevice(&attr_dev), MHLO_CUDA_EXECUTION_FAILED);
    if (attr_dev < 0 || attr_dev >= 64 || !attr_set[attr_dev].load(std::memory_order_acquire)) {
        MHLO_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal), MHLO_CUDA_EXECUTION_FAILED);
        if (attr_dev >= 0 && attr_dev < 64) attr_set[attr_dev].store(true, std::memory_order_release);
    }
    int walkers = kNumSMs;
    if (CTAS == 2) {
        // pairs that can be resident at once (a pair sits inside one GPC; not every SM need have a partner free)
        static std::atomic<int> resident_pairs[64];
        int pairs = attr_dev >= 0 && attr_dev < 64 ? resident_pairs[attr_dev].load(std::memory_order_acquire) : 0;
        if (pairs == 0) {
            cudaLaunchConfig_t q = {};
            q.gridDim = dim3(kNumSMs);
            q.blockDim = dim3(kGemmThreads);
            q.dynamicSmemBytes = L::kTotal;
            cudaLaunchAttribute qa[1];
            qa[0].id = cudaLaunchAttributeClusterDimension;
            qa[0].val.clusterDim.x = 2;
            qa[0].val.clusterDim.y = 1;
            qa[0].val.clusterDim.z = 1;
            q.attrs = qa;
            q.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&pairs, kernel, &q) != cudaSuccess || pairs < 1) { cudaGetLastError(); pairs = kNumSMs / 2; }
            pairs = std::min(pairs, kNumSMs / 2);
            if (attr_dev >= 0 && attr_dev < 64) resident_pairs[attr_dev].store(pairs, std::memory_order_release);
        }
        walkers = pairs;
    }
    const int grid = CTAS * static_cast<int>(std::min<int64_t>(p.num_tiles, walkers));
    const cudaError_t launched = launch_dependent_cluster(kernel, dim3(grid), dim3(kGemmThreads), L::kTotal, stream, CTAS, map_a, map_b, map_c, p, peer_maps);
    if (launched != cudaSuccess) return fail(MHLO_CUDA_EXECUTION_FAILED, "launch of gemm_tcgen05 failed: %s", cudaGetErrorString(launched));
    MHLO_CUDA_CHECK_LAUNCH("gemm_tcgen05");
    return MHLO_CUDA_OK;
}

template <int BN, int STAGES, int CTAS = 1>
static int launch_gemm(const GemmProblem& p, cudaStream_t stream) {
    // bulk stores into the copies: the instantiation that carries the copies' tensor maps exists for products without
    // an activation; with one, the copies keep the lane stores
    if (p.n_copies > 0 && p.copy_stores == 2 && p.epilogue == MHLO_EPILOGUE_NONE && p.residual == nullptr)
        return launch_gemm_act<BN, STAGES, MHLO_EPILOGUE_NONE, CTAS, 1>(p, stream);
    if (p.residual != nullptr) {
        if (p.epilogue != MHLO_EPILOGUE_NONE || p.out_dtype == MHLO_DT_F32 || p.n_copies > 0)
            return fail(MHLO_CUDA_UNSUPPORTED, "gemm: a residual goes with a 16-bit result, no activation and no further copies of C");
        return launch_gemm_act<BN, STAGES, MHLO_EPILOGUE_NONE, CTAS, 2>(p, stream);
    }
    switch (p.epilogue) {
        case MHLO_EPILOGUE_RELU: return launch_gemm_act<BN, STAGES, MHLO_EPILOGUE_RELU, CTAS>(p, stream);
        case MHLO_EPILOGUE_GELU_TANH: return launch_gemm_act<BN, STAGES, MHLO_EPILOGUE_GELU_TANH, CTAS>(p, stream);
        case MHLO_EPILOGUE_GELU_ERF: return launch_gemm_act<BN, STAGES, MHLO_EPILOGUE_GELU_ERF, CTAS>(p, stream);
        case MHLO_EPILOGUE_SILU: return launch_gemm_act<BN, STAGES, MHLO_EPILOGUE_SILU, CTAS>(p, stream);
        case MHLO_EPILOGUE_TANH: return launch_gemm_act<BN, STAGES, MHLO_EPILOGUE_TANH, CTAS>(p, stream);
        case MHLO_EPILOGUE_SIGMOID: return launch_gemm_act<BN, STAGES, MHLO_EPILOGUE_SIGMOID, CTAS>(p, stream);
        default: return launch_gemm_act<BN, STAGES, MHLO_EPILOGUE_NONE, CTAS>(p, stream);
    }
}

// ---- convolution without a patch matrix (MODE 3) ----

// step_w / step_h: the box takes every step-th pixel (16 x box_h of them), for the input of a strided convolution.
bool conv_map(CUtensorMap* map, const void* base, int64_t elem_bytes, int64_t inner, int64_t w, int64_t h, int64_t n, uint32_t box_inner,
              uint32_t box_h, bool is_f32, std::string* why, uint32_t step_w = 1, uint32_t step_h = 1) {
    cuuint64_t gdim[4] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(w), static_cast<cuuint64_t>(h), static_cast<cuuint64_t>(n)};
    cuuint64_t gstr[3] = {static_cast<cuuint64_t>(inner * elem_bytes), static_cast<cuuint64_t>(w * inner * elem_bytes),
                          static_cast<cuuint64_t>(h * w * inner * elem_bytes)};
    // with a traversal stride s a box extent of (k - 1) s + 1 elements delivers k of them
    cuuint32_t box[4] = {box_inner, 15 * step_w + 1, (box_h - 1) * step_h + 1, 1}, estr[4] = {1, step_w, step_h, 1};
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
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
    const CUresult r = encode(map, is_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), gdim, gstr,
                              box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        *why = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(r));
        return false;
    }
    return true;
}

bool conv_tc_supported(const ConvProblem& c) {
    const bool f16 = c.dtype == MHLO_DT_F16, bf16 = c.dtype == MHLO_DT_BF16;
    if (!f16 && !bf16) return false;
    if (c.out_dtype != c.dtype && c.out_dtype != MHLO_DT_F32) return false;
    if (c.images <= 0 || c.h <= 0 || c.w <= 0 || c.channels <= 0 || c.kh <= 0 || c.kw <= 0 || c.features <= 0 || c.oh <= 0 || c.ow <= 0) return false;
    if (c.channels % 64 != 0) return false;  // a k-block is one tap x 64 channels
    const int64_t out_es = c.out_dtype == MHLO_DT_F32 ? 4 : 2;
    if ((c.features * 2) % 16 != 0 || (c.features * out_es) % 16 != 0) return false;
    if (!aligned16(c.x) || !aligned16(c.wgt) || !aligned16(c.out)) return false;
    if (c.dil_h < 1 || c.dil_w < 1 || c.pad_h < 0 || c.pad_w < 0) return false;
    if (c.stride_h < 1 || c.stride_w < 1 || c.stride_h > 8 || c.stride_w > 8) return false;  // traversal strides of a tensor map
    // the window arithmetic of a stride-1 convolution must give the declared result
    if (c.oh > c.h + 2 * 0x3fff || c.images > 0x7fffffff) return false;
    return true;
}

template <int ACT>
static int launch_conv_act(const ConvProblem& c, cudaStream_t stream) {
    constexpr int BN = 128, STAGES = 6;
    using L = SmemLayout<BN, STAGES, 1>;
    std::string why;
    CUtensorMap map_a, map_b, map_c;
    if (!conv_map(&map_a, c.x, 2, c.channels, c.w, c.h, c.images, 64, 8, false, &why, static_cast<uint32_t>(c.stride_w), static_cast<uint32_t>(c.stride_h)))
        return fail(MHLO_CUDA_EXECUTION_FAILED, "convolution: tensor map for the input: %s", why.c_str());
    const int64_t kc = c.kh * c.kw * c.channels;
    if (!operand_map(&map_b, c.wgt, c.features, kc, c.features, 1, 0, 1, 0, 64, BK, &why))
        return fail(MHLO_CUDA_EXECUTION_FAILED, "convolution: tensor map for the filter: %s", why.c_str());
    const bool f32_out = c.out_dtype == MHLO_DT_F32;
    if (!conv_map(&map_c, c.out, f32_out ? 4 : 2, c.features, c.ow, c.oh, c.images, f32_out ? 32 : 64, 2, f32_out, &why))
        return fail(MHLO_CUDA_EXECUTION_FAILED, "convolution: tensor map for the result: %s", why.c_str());
    GemmParams p;
    memset(&p, 0, sizeof p);
    p.c = c.out;
    p.bias = c.bias;
    const int tiles_x = static_cast<int>((c.ow + 15) / 16), tiles_y = static_cast<int>((c.oh + 7) / 8);
    p.tiles_m = tiles_x * tiles_y;
    p.m = static_cast<int64_t>(p.tiles_m) * BM;  // every row of a tile "exists": the copies clip at the image's edges
    p.n = c.features;
    p.k = kc;
    p.batch0 = 1;
    p.batch1 = c.images;
    p.stages = STAGES;
    p.tiles_n = static_cast<int>((c.features + BN - 1) / BN);
    p.num_tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n * c.images;
    p.a_mn_major = 0;
    p.b_mn_major = 1;  // the filter matrix [taps x channels, features] has the features contiguous
    p.in_bf16 = c.dtype == MHLO_DT_BF16;
    p.out_dtype = c.out_dtype;
    p.epilogue = c.epilogue;
    p.ldc = c.features;
    p.c_vec_ok = 1;
    p.c_tma = 1;
    p.conv_tiles_x = tiles_x;
    p.conv_kw = static_cast<int32_t>(c.kw);
    p.conv_cblocks = static_cast<int32_t>(c.channels / 64);
    p.conv_pad_h = static_cast<int32_t>(c.pad_h);
    p.conv_pad_w = static_cast<int32_t>(c.pad_w);
    p.conv_dil_h = static_cast<int32_t>(c.dil_h);
    p.conv_dil_w = static_cast<int32_t>(c.dil_w);
    p.conv_oh = static_cast<int32_t>(c.oh);
    p.conv_stride_h = static_cast<int32_t>(c.stride_h);
    p.conv_stride_w = static_cast<int32_t>(c.stride_w);
    auto kernel = gemm_tcgen05_kernel<BN, STAGES, ACT, 1, 3>;
    static std::atomic<bool> attr_set[64];
    int attr_dev = 0;
    MHLO_CUDA_TRY(cudaGetDevice(&attr_dev), MHLO_CUDA_EXECUTION_FAILED);
    if (attr_dev < 0 || attr_dev >= 64 || !attr_set[attr_dev].load(std::memory_order_acquire)) {
        MHLO_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal), MHLO_CUDA_EXECUTION_FAILED);
        if (attr_dev >= 0 && attr_dev < 64) attr_set[attr_dev].store(true, std::memory_order_release);
    }
    const int grid = static_cast<int>(std::min<int64_t>(p.num_tiles, kNumSMs));
    PeerMaps<false> none;
    const cudaError_t launched = launch_dependent_cluster(kernel, dim3(grid), dim3(kGemmThreads), L::kTotal, stream, 1, map_a, map_b, map_c, p, none);
    if (launched != cudaSuccess) return fail(MHLO_CUDA_EXECUTION_FAILED, "launch of the convolution failed: %s", cudaGetErrorString(launched));
    MHLO_CUDA_CHECK_LAUNCH("convolution (tcgen05)");
    return MHLO_CUDA_OK;
}

int conv_tc_launch(const ConvProblem& c, cudaStream_t stream) {
    switch (c.epilogue) {
        case MHLO_EPILOGUE_RELU: return launch_conv_act<MHLO_EPILOGUE_RELU>(c, stream);
        case MHLO_EPILOGUE_GELU_TANH: return launch_conv_act<MHLO_EPILOGUE_GELU_TANH>(c, stream);
        case MHLO_EPILOGUE_GELU_ERF: return launch_conv_act<MHLO_EPILOGUE_GELU_ERF>(c, stream);
        case MHLO_EPILOGUE_SILU: return launch_conv_act<MHLO_EPILOGUE_SILU>(c, stream);
        case MHLO_EPILOGUE_TANH: return launch_conv_act<MHLO_EPILOGUE_TANH>(c, stream);
        case MHLO_EPILOGUE_SIGMOID: return launch_conv_act<MHLO_EPILOGUE_SIGMOID>(c, stream);
        default: return launch_conv_act<MHLO_EPILOGUE_NONE>(c, stream);
    }
}

int gemm_tc_launch(const GemmProblem& p, cudaStream_t stream) {
    // 128 x 256 tiles run the tensor pipe at its full rate; a 128 x 128 tile takes about 0.6 of the time of a wide one
    // (measured: 0.33 us against 0.27 us per 64-deep step at half the work), so narrow tiles only pay when they save
    // whole waves over the SMs.
    // explicit knobs first (the tuner's records and the tests): 0 leaves a knob to the heuristic below
    static const int pair_env = [] {
        const char* v = getenv("METALHLO_GEMM_PAIR");  // 0 = never a CTA pair, 1 = a pair wherever the tile allows
        return v && (v[0] == '0' || v[0] == '1') ? v[0] - '0' : -1;
    }();
    int cta_group = p.cta_group;
    if (cta_group == 0 && pair_env >= 0 && p.n_copies == 0) cta_group = pair_env + 1;
    if (cta_group == 2) return launch_gemm<256, 6, 2>(p, stream);
    if (p.tile_n == 256) return launch_gemm<256, 4>(p, stream);
    if (p.tile_n == 128) return launch_gemm<128, 6>(p, stream);
    if (p.n <= 128) return launch_gemm<128, 6>(p, stream);
    // A pair of CTAs per 256 x 256 tile halves the shared-memory traffic of B per SM and measured 5-10 % faster than one
    // CTA per 128 x 256 tile wherever there are enough tiles to occupy most of the 74 pairs (8192^3: 1481 against 1314 TFLOP/s,
    // [32768,768].[768,3072]: 1124 against 1032); below that the narrower one-CTA tiles spread better over the SMs.
    // Products with a short K are bound by their epilogue and by HBM (the batched [2048,128].[128,2048] product ran at
    // 3.5 TB/s in pairs against 4.9 TB/s alone): a pair has to wait for both CTAs' epilogues before it reuses an accumulator.
    // Rows of C off the 16-byte grid (a pitch such as 50257 f16) are written by the lanes, not by bulk stores: that epilogue
    // is the longer one, and a pair would wait for both of its CTAs (logits [32768,768].[768,50257]: 2.64 ms alone, 2.79 ms in pairs).
    const int64_t out_es = p.out_dtype == MHLO_DT_F32 ? 4 : 2;
    const bool rows_on_grid = ((p.ldc > 0 ? p.ldc : p.n) * out_es) % 16 == 0 && (p.c_col0 * out_es) % 16 == 0 && aligned16(p.c);
    // (products that also store into peers' copies included: four ranks, 8192^3 split by columns: 0.295 ms in pairs, 0.320 ms alone)
    if (cta_group == 0 && p.m > BM && p.k >= 8 * BK && rows_on_grid) {
        const int64_t pair_tiles = (p.m + 2 * BM - 1) / (2 * BM) * ((p.n + 255) / 256) * p.batch0 * p.batch1;
        if (pair_tiles >= 40) return launch_gemm<256, 6, 2>(p, stream);  // (48 pairs on [4096,3072].[3072,768]: 23.7 us against 25.3 us alone)
    }
    const int64_t rows = (p.m + BM - 1) / BM * p.batch0 * p.batch1;
    const int64_t tiles_256 = rows * ((p.n + 255) / 256), tiles_128 = rows * ((p.n + 127) / 128);
    const int64_t waves_256 = (tiles_256 + kNumSMs - 1) / kNumSMs, waves_128 = (tiles_128 + kNumSMs - 1) / kNumSMs;
    if (waves_256 * 100 <= waves_128 * 61) return launch_gemm<256, 4>(p, stream);
    return launch_gemm<128, 6>(p, stream);
}

int gemm_device_error() {
    int v = 0, zero = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof v) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof zero);
    return v;
}

bool gemm_error_fetch_async(int* pinned_dst, cudaStream_t stream) {
    return cudaMemcpyFromSymbolAsync(pinned_dst, g_gemm_error, sizeof(int), 0, cudaMemcpyDeviceToHost, stream) == cudaSuccess;
}

bool gemm_error_store(int code) { return cudaMemcpyToSymbol(g_gemm_error, &code, sizeof code) == cudaSuccess; }

namespace {
// One CTA that waits on an mbarrier nobody arrives at, for at most `limit_ns`, and then records code 90 the way the
// contraction kernels record an expired wait. The wait ends by itself: nothing here can spin for longer than the limit.
__global__ void wait_expiry_probe_kernel(uint64_t limit_ns) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_barrier_init();
        const uint32_t addr = smem_u32(&bar);
        const uint64_t start = global_timer_ns();
        bool done = false;
        while (!done && global_timer_ns() - start <= limit_ns) {
            uint32_t ok;
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                "selp.b32 %0, 1, 0, p;\n\t}"
                : "=r"(ok)
                : "r"(addr), "r"(0u)
                : "memory");
            done = ok != 0;
        }
        if (!done) atomicExch(&g_gemm_error, 90);
    }
}

struct PeerFlags {
    uint64_t* arrays[8];  // arrays[r] = rank r's flag words (8 of them), in r's memory
};

// Completion barrier of an exchange whose stores went straight into the peers' memory. It runs in stream order after the
// kernel that stored, so those stores are complete on this GPU's side; thread r publishes the epoch to rank r with a
// system-scope release and then waits, with a time limit, for rank r's word in this rank's own array. Epochs only grow,
// so a word that already holds a later epoch satisfies an earlier wait.
__global__ void peer_barrier_kernel(const __grid_constant__ PeerFlags f, int n_ranks, int rank, uint64_t epoch, uint64_t limit_ns) {
    const int r = threadIdx.x;
    if (r >= n_ranks || r == rank) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(f.arrays[r] + rank), "l"(epoch) : "memory");
    const uint64_t* mine = f.arrays[rank] + r;
    const uint64_t start = global_timer_ns();
    for (;;) {
        uint64_t seen;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(mine) : "memory");
        if (seen >= epoch) break;
        if (global_timer_ns() - start > limit_ns) {
            atomicExch(&g_gemm_error, 95);
            break;
        }
    }
}
}  // namespace

bool gemm_peer_barrier_launch(uint64_t* const* flag_arrays, int n_ranks, int rank, uint64_t epoch, uint64_t limit_ns, cudaStream_t stream) {
    PeerFlags f;
    for (int r = 0; r < 8; ++r) f.arrays[r] = r < n_ranks ? flag_arrays[r] : nullptr;
    peer_barrier_kernel<<<1, 32, 0, stream>>>(f, n_ranks, rank, epoch, limit_ns);
    return cudaGetLastError() == cudaSuccess;
}

bool gemm_wait_expiry_probe(uint64_t limit_ns, cudaStream_t stream) {
    wait_expiry_probe_kernel<<<1, 32, 0, stream>>>(limit_ns);
    return cudaGetLastError() == cudaSuccess;
}

}  // namespace mhlo
