// Warp-specialised, persistent tcgen05 GEMM for sm_100a.
//
//   D[M x N] (fp32, TMEM) = A[M x K] * B[K x N]      fp16 operands, 128B-swizzled shared memory
//
// One CTA per SM. Warp 0 feeds operands with TMA (plain per-CTA loads, no multicast), warp 1
// issues tcgen05.mma from one thread and owns TMEM, warps 2-9 drain the accumulator
// (tcgen05.ld -> registers -> fused epilogue -> global), and, for the embedding layers, warps 10-17
// synthesise the one-hot operand directly in shared memory from the 80-byte puzzle states, so the
// one-hot matrix never exists in HBM.
//
// Operand forms
//   A  K-major  : global [M][K] (K contiguous), one TMA box 64(K) x 128(M) per stage
//   A  MN-major : global [K][M] (M contiguous), two TMA boxes 64(M) x 64(K) per stage
//   B  K-major  : global [N][K] (K contiguous), one TMA box 64(K) x BN(N)
//   B  MN-major : global [K][N] (N contiguous), ceil(BN/64) TMA boxes 64(N) x 64(K)
//   B  one-hot  : K-major rows of 128 bytes written by the synth warps; only the (at most a few)
//                 non-zero halfs of a row are set before the MMA and cleared after it.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>

#include "ptx_sm100.cuh"

namespace mgt {

enum class BSource : int { kTmaK = 0, kTmaMN = 1, kOneHotFwd = 2, kOneHotGrad = 3 };

enum class Epi : int {
    kBiasReluF16 = 0,      // out_f16 = relu(acc + bias)
    kBiasReluF32F16,       // out_f32 = out_f16 = relu(acc + bias)
    kBiasResReluF32F16,    // v = relu(add + (acc + bias)); out_f32 = v (may alias add); out_f16 = v
    kMaskF16,              // out_f16 = acc * [mask > 0]
    kAddMaskF32F16,        // v = (acc + add) * [mask > 0]; out_f32 = v (may alias add); out_f16 = v
    kPartialF32,           // partial[split][m][n] = acc
    kEmbGrad,              // out_f32[n][m] (+)= acc               (D is the transposed gradient)
    kBiasF32,              // out_f32 = acc + bias                 (a pre-activation kept in fp32: input of batch normalisation)
    kEmbFwdRows,           // out_f16[m][n] = relu(acc), bits[m][n / 32] bit (n % 32) = [acc > 0]   (the activation kept as D lies: one row
                           // per output column of the layer; the sign words are the ReLU mask the backward pass needs)
    kMaskRowsumF16,        // out_f16[m][n] = acc * [bit n of bits[m]]; rowsum[(n tile, warp of the quadrant)][m] = sum over the warp's columns
};

struct GemmArgs {
    uint32_t M, N, K;
    uint32_t m_tiles, n_tiles, splits, k_chunks;
    uint32_t groups;         // number of stacked problems (grouped form), else 1
    const float* bias;
    float* out_f32;
    uint32_t ld_f32;
    __half* out_f16;
    uint32_t ld_f16;
    const float* add_f32;
    uint32_t ld_add;
    const __half* mask;
    uint32_t ld_mask;
    float* partial;
    // Optional fp32 column sums of the values the kMaskF16 / kAddMaskF32F16 epilogues produce
    // (bias gradients): row (blockIdx.x * 8 + epilogue warp) of colsum[gridDim.x * 8][N] accumulates
    // what that warp handled. The buffer must be zero before the launch.
    float* colsum;
    // kMaskRowsumF16: fp32 row sums of the masked values, one partial row of M floats per (N tile, warp of a lane quadrant):
    // rowsum[(n_tile * EPI_WARPS / 4 + w)][m]; every slot of a launch is written (no zeroing needed)
    float* rowsum;
    // kEmbFwdRows writes, kMaskRowsumF16 reads: one 32-bit word per row and 32 columns, ld_bits words per row
    uint32_t* bits;
    uint32_t ld_bits;
    // one-hot operand synthesis
    const uint8_t* states;   // [samples][80]
    uint32_t state_len;      // positions per state
    uint32_t value_pad;      // classes per position
    uint32_t samples;
    uint32_t in_rows;        // state_len * value_pad; row `in_rows` is the all-ones (bias) row
    uint32_t bf16;           // operands and 16-bit outputs are bfloat16 instead of fp16
    int* status;             // device status word, 0 = ok
};

// BSTAT_: "B-stationary" - for short reductions (K <= 64*SB_) the whole B operand of the CTA's N tile is loaded
// once and stays in shared memory while the CTA streams its M tiles (all units of a CTA then share the N tile).
// GROUPED_: one launch computes args.groups independent products of the same shape; operand g is slice g
// (third coordinate) of the 3-D tensors behind the two descriptors, result g goes to its own partial planes.
template <int BN_, int NACC_, bool A_MN_, BSource BSRC_, Epi EPI_, int SA_, int SB_, bool BSTAT_ = false, bool GROUPED_ = false, int EPI_WARPS_ = 8>
struct GemmCfg {
    static constexpr bool BSTAT = BSTAT_;
    static constexpr bool GROUPED = GROUPED_;
    static constexpr int BM = 128;
    static constexpr int BK = 64;
    static constexpr int BN = BN_;
    static constexpr int NACC = NACC_;
    static constexpr bool A_MN = A_MN_;
    static constexpr BSource BSRC = BSRC_;
    static constexpr Epi EPI = EPI_;
    static constexpr int SA = SA_;
    static constexpr int SB = SB_;
    static constexpr bool kOneHot = (BSRC_ == BSource::kOneHotFwd || BSRC_ == BSource::kOneHotGrad);
    static constexpr bool B_MN = (BSRC_ == BSource::kTmaMN);
    static constexpr int N_GROUPS = (BN_ + 63) / 64;
    static constexpr int A_STAGE_BYTES = BM * 128;
    static constexpr int B_ACC_BYTES = B_MN ? N_GROUPS * 8192 : BN_ * 128;
    static constexpr int B_STAGE_BYTES = NACC_ * B_ACC_BYTES;
    static constexpr int ACC_BUFS = 2 / NACC_;
    static constexpr int ACC_COLS = 256;  // TMEM columns reserved per accumulator
    static constexpr int EPI_WARPS = EPI_WARPS_;        // a multiple of four: EPI_WARPS/4 warps share a TMEM lane quadrant
    static constexpr int EPI_STRIDE = EPI_WARPS_ / 4;  // ... and take every EPI_STRIDE-th 32-column chunk
    static constexpr int SYNTH_WARPS = 8;
    static constexpr int FIRST_SYNTH_THREAD = 64 + 32 * EPI_WARPS;
    static constexpr int THREADS = FIRST_SYNTH_THREAD + (kOneHot ? 32 * SYNTH_WARPS : 0);
    static constexpr int EPI_TILE_PITCH = 36;
    // per epilogue warp: a padded 32x32 fp32 tile, 32 words of ReLU-mask bits and four rows of column-sum accumulators
    // (the embedding epilogues write transposed and need no staging)
    static constexpr int EPI_WARP_BYTES = (kOneHot || EPI_ == Epi::kMaskRowsumF16) ? 0 : (32 * EPI_TILE_PITCH * 4 + 128 + 4 * 32 * 4);
    static constexpr int EPI_STAGE_BYTES = EPI_WARPS * EPI_WARP_BYTES;
    static constexpr int SMEM_BYTES = 1024 + SA_ * A_STAGE_BYTES + SB_ * B_STAGE_BYTES + 256 + EPI_STAGE_BYTES;
    static_assert(BN_ % 16 == 0 && BN_ >= 16 && BN_ <= 256, "UMMA N");
    static_assert(BN_ % 32 == 0, "epilogue drains 32 columns at a time");
    static_assert(NACC_ == 1 || NACC_ == 2, "one or two accumulators");
    static_assert(EPI_WARPS_ == 8 || EPI_WARPS_ == 16, "epilogue warps");
    static_assert(!kOneHot || EPI_WARPS_ == 8, "the synthesis warps follow eight epilogue warps");
    static_assert(B_ACC_BYTES % 1024 == 0, "swizzle atoms must stay 1024-byte aligned");
    static_assert(!kOneHot || (SB_ >= 2 && SB_ <= 4), "one-hot ring depth");
    static_assert(!GROUPED_ || (EPI_ == Epi::kPartialF32 && A_MN_ && BSRC_ == BSource::kTmaMN && !BSTAT_), "grouped form: split-K weight gradients");
    static_assert(!BSTAT_ || (!kOneHot && NACC_ == 1), "B-stationary applies to TMA-fed single-accumulator tiles");
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

namespace detail {

__device__ __forceinline__ void store_f16x32(__half* dst, const float (&v)[32], uint32_t valid, bool vec_ok, bool bf16) {
    if (valid == 32 && vec_ok) {
        uint4* p = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = ptx::pack_operand_pair(v[q * 8 + 0], v[q * 8 + 1], bf16);
            u.y = ptx::pack_operand_pair(v[q * 8 + 2], v[q * 8 + 3], bf16);
            u.z = ptx::pack_operand_pair(v[q * 8 + 4], v[q * 8 + 5], bf16);
            u.w = ptx::pack_operand_pair(v[q * 8 + 6], v[q * 8 + 7], bf16);
            p[q] = u;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (static_cast<uint32_t>(j) < valid) reinterpret_cast<uint16_t*>(dst)[j] = ptx::to_operand(v[j], bf16);
    }
}

__device__ __forceinline__ void store_f32x32(float* dst, const float (&v)[32], uint32_t valid, bool vec_ok) {
    if (valid == 32 && vec_ok) {
        float4* p = reinterpret_cast<float4*>(dst);
#pragma unroll
        for (int q = 0; q < 8; ++q) p[q] = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (static_cast<uint32_t>(j) < valid) dst[j] = v[j];
    }
}

__device__ __forceinline__ void load_f32x32(const float* src, float (&v)[32], uint32_t valid, bool vec_ok) {
    if (valid == 32 && vec_ok) {
        const float4* p = reinterpret_cast<const float4*>(src);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 f = p[q];
            v[q * 4] = f.x;
            v[q * 4 + 1] = f.y;
            v[q * 4 + 2] = f.z;
            v[q * 4 + 3] = f.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = static_cast<uint32_t>(j) < valid ? src[j] : 0.0f;
    }
}

// positive-mask from fp16 activations: m[j] = src[j] > 0
__device__ __forceinline__ uint32_t load_mask32(const __half* src, uint32_t valid, bool vec_ok) {
    uint32_t bits = 0;
    if (valid == 32 && vec_ok) {
        const uint4* p = reinterpret_cast<const uint4*>(src);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 u = p[q];
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                // a positive non-zero half has sign 0 and a non-zero magnitude
                const uint32_t lo = w[e] & 0xFFFFU, hi = w[e] >> 16;
                if (lo != 0U && (lo & 0x8000U) == 0U) bits |= 1U << (q * 8 + e * 2);
                if (hi != 0U && (hi & 0x8000U) == 0U) bits |= 1U << (q * 8 + e * 2 + 1);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (static_cast<uint32_t>(j) < valid) {
                // positive in either 16-bit format: sign clear, magnitude non-zero
                const uint16_t h = reinterpret_cast<const uint16_t*>(src)[j];
                if (h != 0U && h < 0x8000U) bits |= 1U << j;
            }
    }
    return bits;
}

}  // namespace detail

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const GemmArgs args) {
    using namespace ptx;
    constexpr int BM = Cfg::BM, BN = Cfg::BN, NACC = Cfg::NACC, SA = Cfg::SA, SB = Cfg::SB;
    constexpr int ACC_BUFS = Cfg::ACC_BUFS;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = ((raw_addr + 1023U) & ~1023U) - raw_addr;
    uint8_t* smem = smem_raw + pad;
    uint8_t* a_ring = smem;
    uint8_t* b_ring = smem + SA * Cfg::A_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(b_ring + SB * Cfg::B_STAGE_BYTES);
    uint64_t* full_a = bars;
    uint64_t* empty_a = full_a + SA;
    uint64_t* full_b = empty_a + SA;
    uint64_t* empty_b = full_b + SB;
    uint64_t* acc_full = empty_b + SB;
    uint64_t* acc_empty = acc_full + ACC_BUFS;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + ACC_BUFS);
    volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_holder + 1);
    float* epi_stage = reinterpret_cast<float*>(b_ring + SB * Cfg::B_STAGE_BYTES + 256);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31U;
    const uint32_t units_per_group = args.m_tiles * args.n_tiles * args.splits;
    const uint32_t total_units = units_per_group * (Cfg::GROUPED ? args.groups : 1U);

    if (threadIdx.x == 0) {
        for (int s = 0; s < SA; ++s) {
            mbar_init(&full_a[s], 1);
            mbar_init(&empty_a[s], 1);
        }
        for (int s = 0; s < SB; ++s) {
            mbar_init(&full_b[s], Cfg::kOneHot ? Cfg::SYNTH_WARPS : 1);
            mbar_init(&empty_b[s], 1);
        }
        for (int s = 0; s < ACC_BUFS; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 32 * Cfg::EPI_WARPS);
        }
        *cta_abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&tma_a);
        if (!Cfg::kOneHot) prefetch_tensormap(&tma_b);
    }
    if (Cfg::kOneHot) {
        // the one-hot ring starts as all zeros; afterwards only single halfs are set and cleared
        uint4* z = reinterpret_cast<uint4*>(b_ring);
        for (uint32_t i = threadIdx.x; i < SB * Cfg::B_STAGE_BYTES / 16; i += Cfg::THREADS) z[i] = make_uint4(0, 0, 0, 0);
        fence_proxy_async_smem();
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    // unit -> (m tile, n tile, split): splits of one tile are neighbours for TMA-fed GEMMs; for the
    // embedding layers units that share the A stream (same m tile and split) are neighbours.
    auto group_of = [&](uint32_t unit) { return Cfg::GROUPED ? unit / units_per_group : 0U; };
    auto decode = [&](uint32_t unit, uint32_t& mt, uint32_t& nt, uint32_t& sp) {
        if (Cfg::GROUPED) unit %= units_per_group;
        if (Cfg::kOneHot) {
            nt = unit % args.n_tiles;
            const uint32_t rest = unit / args.n_tiles;
            sp = rest % args.splits;
            mt = rest / args.splits;
        } else {
            sp = unit % args.splits;
            const uint32_t rest = unit / args.splits;
            nt = rest % args.n_tiles;
            mt = rest / args.n_tiles;
        }
    };
    auto chunk_begin = [&](uint32_t sp) { return static_cast<uint32_t>((static_cast<uint64_t>(sp) * args.k_chunks) / args.splits); };

    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
                uint32_t mt, nt, sp;
                decode(unit, mt, nt, sp);
                const uint32_t c0 = chunk_begin(sp), c1 = chunk_begin(sp + 1);
                for (uint32_t c = c0; c < c1; ++c, ++it) {
                    const uint32_t sa = it % SA, pa = (it / SA) & 1U;
                    if (!mbar_wait_spin(&empty_a[sa], pa ^ 1U, cta_abort, kAbortProducerWait)) { ok = false; break; }
                    uint8_t* a_dst = a_ring + sa * Cfg::A_STAGE_BYTES;
                    mbar_arrive_expect_tx(&full_a[sa], Cfg::A_STAGE_BYTES);
                    if (Cfg::GROUPED) {
                        const int32_t g = static_cast<int32_t>(group_of(unit));
                        tma_load_3d(a_dst, &tma_a, static_cast<int32_t>(mt * BM), static_cast<int32_t>(c * 64), g, &full_a[sa]);
                        tma_load_3d(a_dst + 8192, &tma_a, static_cast<int32_t>(mt * BM + 64), static_cast<int32_t>(c * 64), g, &full_a[sa]);
                    } else if (Cfg::A_MN) {
                        tma_load_2d(a_dst, &tma_a, static_cast<int32_t>(mt * BM), static_cast<int32_t>(c * 64), &full_a[sa]);
                        tma_load_2d(a_dst + 8192, &tma_a, static_cast<int32_t>(mt * BM + 64), static_cast<int32_t>(c * 64), &full_a[sa]);
                    } else {
                        tma_load_2d(a_dst, &tma_a, static_cast<int32_t>(c * 64), static_cast<int32_t>(mt * BM), &full_a[sa]);
                    }
                    if (!Cfg::kOneHot && (!Cfg::BSTAT || unit == blockIdx.x)) {
                        // B-stationary: chunk c of B lives in stage c for the whole kernel, loaded with the first unit
                        const uint32_t sb = Cfg::BSTAT ? (c - c0) : it % SB, pb = Cfg::BSTAT ? 0U : (it / SB) & 1U;
                        if (!Cfg::BSTAT && !mbar_wait_spin(&empty_b[sb], pb ^ 1U, cta_abort, kAbortProducerWait)) { ok = false; break; }
                        uint8_t* b_dst = b_ring + sb * Cfg::B_STAGE_BYTES;
                        mbar_arrive_expect_tx(&full_b[sb], Cfg::B_STAGE_BYTES);
#pragma unroll
                        for (int acc = 0; acc < NACC; ++acc) {
                            const uint32_t n0 = (nt * NACC + acc) * BN;
                            if (Cfg::GROUPED) {
                                const int32_t z = static_cast<int32_t>(group_of(unit));
#pragma unroll
                                for (int g = 0; g < Cfg::N_GROUPS; ++g)
                                    tma_load_3d(b_dst + acc * Cfg::B_ACC_BYTES + g * 8192, &tma_b, static_cast<int32_t>(n0 + g * 64),
                                                static_cast<int32_t>(c * 64), z, &full_b[sb]);
                            } else if (Cfg::B_MN) {
#pragma unroll
                                for (int g = 0; g < Cfg::N_GROUPS; ++g)
                                    tma_load_2d(b_dst + acc * Cfg::B_ACC_BYTES + g * 8192, &tma_b, static_cast<int32_t>(n0 + g * 64),
                                                static_cast<int32_t>(c * 64), &full_b[sb]);
                            } else {
                                tma_load_2d(b_dst + acc * Cfg::B_ACC_BYTES, &tma_b, static_cast<int32_t>(c * 64), static_cast<int32_t>(n0), &full_b[sb]);
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------- UMMA issuer --------------------------------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc_f16(BM, BN, Cfg::A_MN, Cfg::B_MN, args.bf16 != 0U);
            uint32_t it = 0, unit_iter = 0;
            bool ok = true;
            for (uint32_t unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++unit_iter) {
                uint32_t mt, nt, sp;
                decode(unit, mt, nt, sp);
                const uint32_t c0 = chunk_begin(sp), c1 = chunk_begin(sp + 1);
                const uint32_t ab = unit_iter % ACC_BUFS, aph = (unit_iter / ACC_BUFS) & 1U;
                if (!mbar_wait_spin(&acc_empty[ab], aph ^ 1U, cta_abort, kAbortMmaWait)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_base = tmem_base + ab * (NACC * Cfg::ACC_COLS);
                for (uint32_t c = c0; c < c1; ++c, ++it) {
                    const uint32_t sa = it % SA, pa = (it / SA) & 1U;
                    const uint32_t sb = Cfg::BSTAT ? (c - c0) : it % SB, pb = Cfg::BSTAT ? 0U : (it / SB) & 1U;
                    // (the issuing thread polls its barriers: waking from a suspended wait costs more than the hand-over itself)
                    if (!mbar_wait_spin(&full_a[sa], pa, cta_abort, kAbortMmaWait)) { ok = false; break; }
                    if (!Cfg::BSTAT || unit == blockIdx.x) {
                        if (!mbar_wait_spin(&full_b[sb], pb, cta_abort, kAbortMmaWait)) { ok = false; break; }
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(a_ring + sa * Cfg::A_STAGE_BYTES);
                    const uint32_t b_addr = smem_u32(b_ring + sb * Cfg::B_STAGE_BYTES);
                    const uint32_t k_left = args.K - c * 64U;
                    const uint32_t ksteps = k_left >= 64U ? 4U : (k_left + 15U) / 16U;
                    // Descriptors of the chunk's first K step; a later step only moves the start address (bits [0,14) in
                    // units of 16 bytes, no carry: shared-memory addresses are below 2^18). One thread issues everything,
                    // so the fewer dependent instructions stand between two MMAs the better: the full chunk is unrolled.
                    constexpr uint64_t kStepA = Cfg::A_MN ? 2048U / 16U : 32U / 16U, kStepB = Cfg::B_MN ? 2048U / 16U : 32U / 16U;
                    const uint64_t a_desc0 = Cfg::A_MN ? make_smem_desc(a_addr, 8192U, 1024U) : make_smem_desc(a_addr, 16U, 1024U);
                    const uint32_t first = c > c0 ? 1U : 0U;
                    if (ksteps == 4U) {
#pragma unroll
                        for (int acc = 0; acc < NACC; ++acc) {
                            const uint64_t b_desc0 = Cfg::B_MN ? make_smem_desc(b_addr + acc * Cfg::B_ACC_BYTES, 8192U, 1024U)
                                                               : make_smem_desc(b_addr + acc * Cfg::B_ACC_BYTES, 16U, 1024U);
#pragma unroll
                            for (uint32_t kk = 0; kk < 4U; ++kk)
                                umma_f16(d_base + acc * Cfg::ACC_COLS, a_desc0 + kk * kStepA, b_desc0 + kk * kStepB, idesc, kk == 0U ? first : 1U);
                        }
                    } else {
#pragma unroll
                        for (int acc = 0; acc < NACC; ++acc) {
                            const uint64_t b_desc0 = Cfg::B_MN ? make_smem_desc(b_addr + acc * Cfg::B_ACC_BYTES, 8192U, 1024U)
                                                               : make_smem_desc(b_addr + acc * Cfg::B_ACC_BYTES, 16U, 1024U);
                            for (uint32_t kk = 0; kk < ksteps; ++kk)
                                umma_f16(d_base + acc * Cfg::ACC_COLS, a_desc0 + kk * kStepA, b_desc0 + kk * kStepB, idesc, kk == 0U ? first : 1U);
                        }
                    }
                    umma_commit(&empty_a[sa]);
                    if (!Cfg::BSTAT) umma_commit(&empty_b[sb]);
                }
                if (ok) umma_commit(&acc_full[ab]);
            }
        }
        __syncwarp();
    } else if (warp < 2U + Cfg::EPI_WARPS) {
        // ------------------------------- epilogue -----------------------------------------
        // Eight warps: TMEM lanes [32*quad, 32*quad+32) can only be read by warps with warp%4 == quad, so two
        // warps share a quadrant and take alternate 32-column chunks.
        const uint32_t ew = warp - 2U;
        const uint32_t quad = warp & 3U;
        const uint32_t chunk_parity = ew >> 2;
        uint32_t unit_iter = 0;
        bool ok = true;
        if constexpr (Cfg::kOneHot) {
            // Embedding layers. Forward: the activation is kept the way D lies ([hd1][samples]), a lane writes the 32
            // columns of its row. Gradient: D is the transposed table gradient, a TMEM lane (row of D) is a column of the
            // row-major table and the 32 lanes of a warp write consecutive addresses.
            for (uint32_t unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++unit_iter) {
                uint32_t mt, nt, sp;
                decode(unit, mt, nt, sp);
                const uint32_t ab = unit_iter % ACC_BUFS, aph = (unit_iter / ACC_BUFS) & 1U;
                if (!__all_sync(0xFFFFFFFFU, mbar_wait(&acc_full[ab], aph, cta_abort, kAbortEpilogueWait))) { ok = false; break; }
                tc_fence_after();
                const uint32_t m = mt * BM + quad * 32U + lane;
                const bool m_ok = m < args.M;
#pragma unroll 1
                for (int acc = 0; acc < NACC; ++acc) {
#pragma unroll 1
                    for (int cc = static_cast<int>(chunk_parity); cc < BN / 32; cc += Cfg::EPI_STRIDE) {
                        const uint32_t n0 = (nt * NACC + acc) * BN + cc * 32;
                        if (n0 >= args.N) continue;
                        uint32_t r[32];
                        tmem_ld_32x32(tmem_base + ((quad * 32U) << 16) + ab * (NACC * Cfg::ACC_COLS) + acc * Cfg::ACC_COLS + cc * 32, r);
                        tmem_ld_wait();
                        const uint32_t valid = min(32U, args.N - n0);
                        if constexpr (Cfg::EPI == Epi::kEmbFwdRows) {
                            // a lane owns 32 consecutive columns of its row: 64 bytes, four 16-byte stores
                            if (m_ok) {
                                uint16_t* dst = reinterpret_cast<uint16_t*>(args.out_f16) + static_cast<uint64_t>(m) * args.ld_f16 + n0;
                                if (args.bits != nullptr) {
                                    uint32_t word = 0;
#pragma unroll
                                    for (int j = 0; j < 32; ++j) word |= (static_cast<uint32_t>(j) < valid && __uint_as_float(r[j]) > 0.0f) ? (1U << j) : 0U;
                                    args.bits[static_cast<uint64_t>(m) * args.ld_bits + (n0 >> 5)] = word;
                                }
                                if (valid == 32U && (args.ld_f16 & 7U) == 0U) {
#pragma unroll
                                    for (int q = 0; q < 4; ++q) {
                                        uint4 u;
                                        u.x = pack_operand_pair(fmaxf(__uint_as_float(r[8 * q + 0]), 0.0f), fmaxf(__uint_as_float(r[8 * q + 1]), 0.0f), args.bf16 != 0U);
                                        u.y = pack_operand_pair(fmaxf(__uint_as_float(r[8 * q + 2]), 0.0f), fmaxf(__uint_as_float(r[8 * q + 3]), 0.0f), args.bf16 != 0U);
                                        u.z = pack_operand_pair(fmaxf(__uint_as_float(r[8 * q + 4]), 0.0f), fmaxf(__uint_as_float(r[8 * q + 5]), 0.0f), args.bf16 != 0U);
                                        u.w = pack_operand_pair(fmaxf(__uint_as_float(r[8 * q + 6]), 0.0f), fmaxf(__uint_as_float(r[8 * q + 7]), 0.0f), args.bf16 != 0U);
                                        reinterpret_cast<uint4*>(dst)[q] = u;
                                    }
                                } else {
#pragma unroll
                                    for (int j = 0; j < 32; ++j)
                                        if (static_cast<uint32_t>(j) < valid) dst[j] = to_operand(fmaxf(__uint_as_float(r[j]), 0.0f), args.bf16 != 0U);
                                }
                            }
                        } else if (m_ok) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (static_cast<uint32_t>(j) < valid) {
                                    const float x = __uint_as_float(r[j]);
                                    float* dst = args.out_f32 + static_cast<uint64_t>(n0 + j) * args.ld_f32 + m;
                                    if (args.splits > 1U) atomicAdd(dst, x); else *dst = x;
                                }
                            }
                        }
                    }
                }
                tc_fence_before();
                mbar_arrive(&acc_empty[ab]);
            }
        } else if constexpr (Cfg::EPI == Epi::kMaskRowsumF16) {
            // D and the output have a row per TMEM lane and the warp's 32 columns side by side in that row: 64 bytes per lane,
            // written as four 16-byte vectors straight from registers; the mask of a chunk is one word per lane; the row
            // sum is a sum over the lane's own registers. (Full 32-byte sectors; whole rows per warp are not needed.)
            const bool vec_ok = (args.ld_f16 & 7U) == 0U;
            constexpr int CPW = (BN / 32 + Cfg::EPI_STRIDE - 1) / Cfg::EPI_STRIDE;  // chunks of a unit per warp
            // the mask words of a unit do not depend on its MMAs: those of the NEXT unit are requested while this one is drained
            auto request = [&](uint32_t unit, uint32_t (&words)[CPW]) {
                uint32_t mt, nt, sp;
                decode(unit, mt, nt, sp);
                const uint32_t m = mt * BM + quad * 32U + lane;
#pragma unroll
                for (int ci = 0; ci < CPW; ++ci) {
                    const uint32_t n0 = nt * BN + (chunk_parity + ci * Cfg::EPI_STRIDE) * 32U;
                    words[ci] = (unit < total_units && m < args.M && n0 < args.N) ? __ldg(args.bits + static_cast<uint64_t>(m) * args.ld_bits + (n0 >> 5)) : 0U;
                }
            };
            uint32_t mw_next[CPW];
            request(blockIdx.x, mw_next);
            for (uint32_t unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++unit_iter) {
                uint32_t mt, nt, sp;
                decode(unit, mt, nt, sp);
                const uint32_t ab = unit_iter % ACC_BUFS, aph = (unit_iter / ACC_BUFS) & 1U;
                const uint32_t m = mt * BM + quad * 32U + lane;
                const bool m_ok = m < args.M;
                uint32_t mw[CPW];
#pragma unroll
                for (int ci = 0; ci < CPW; ++ci) mw[ci] = mw_next[ci];
                request(unit + gridDim.x, mw_next);
                if (!__all_sync(0xFFFFFFFFU, mbar_wait(&acc_full[ab], aph, cta_abort, kAbortEpilogueWait))) { ok = false; break; }
                tc_fence_after();
                float row_sum = 0.0f;
#pragma unroll
                for (int ci = 0; ci < CPW; ++ci) {
                    const uint32_t cc = chunk_parity + ci * Cfg::EPI_STRIDE;
                    const uint32_t n0 = nt * BN + cc * 32U;
                    if (cc >= static_cast<uint32_t>(BN / 32) || n0 >= args.N) continue;  // (warp-uniform)
                    const uint32_t valid = min(32U, args.N - n0);
                    const bool vec = valid == 32U && vec_ok;
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((quad * 32U) << 16) + ab * Cfg::ACC_COLS + cc * 32, r);
                    tmem_ld_wait();
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = ((mw[ci] >> j) & 1U) ? __uint_as_float(r[j]) : 0.0f;
#pragma unroll
                    for (int j = 0; j < 32; ++j) row_sum += v[j];  // (columns past N were masked with zeros above)
                    if (m_ok) {
                        uint16_t* dst = reinterpret_cast<uint16_t*>(args.out_f16) + static_cast<uint64_t>(m) * args.ld_f16 + n0;
                        if (vec) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint4 u;
                                u.x = pack_operand_pair(v[8 * q + 0], v[8 * q + 1], args.bf16 != 0U);
                                u.y = pack_operand_pair(v[8 * q + 2], v[8 * q + 3], args.bf16 != 0U);
                                u.z = pack_operand_pair(v[8 * q + 4], v[8 * q + 5], args.bf16 != 0U);
                                u.w = pack_operand_pair(v[8 * q + 6], v[8 * q + 7], args.bf16 != 0U);
                                reinterpret_cast<uint4*>(dst)[q] = u;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (static_cast<uint32_t>(j) < valid) dst[j] = to_operand(v[j], args.bf16 != 0U);
                        }
                    }
                }
                if (args.rowsum != nullptr && m_ok) args.rowsum[(static_cast<uint64_t>(nt) * Cfg::EPI_STRIDE + chunk_parity) * args.M + m] = row_sum;
                tc_fence_before();
                mbar_arrive(&acc_empty[ab]);
            }
        } else {
            // Row-major tensors: a TMEM lane holds one row, but global memory wants a warp on whole rows. Each warp
            // stages operands and results through its own padded 32x32 fp32 tile in shared memory, so that every
            // global access is a full 64/128-byte row segment: 16-byte vectors, four (fp32) or eight (fp16) rows per
            // instruction. The global operands of a chunk (residual/skip values, ReLU mask source, bias) are
            // requested one chunk ahead - for the first chunk of a tile before the tile's MMAs have even finished -
            // so their latency is off the critical path. Ragged shapes take a scalar form without prefetch.
            constexpr bool kPlainF32 = Cfg::EPI == Epi::kBiasF32;  // fp32 out only: no ReLU, no 16-bit copy
            constexpr bool kHasBias = Cfg::EPI == Epi::kBiasReluF16 || Cfg::EPI == Epi::kBiasReluF32F16 || Cfg::EPI == Epi::kBiasResReluF32F16 || kPlainF32;
            constexpr bool kHasAdd = Cfg::EPI == Epi::kBiasResReluF32F16 || Cfg::EPI == Epi::kAddMaskF32F16;
            constexpr bool kHasMask = Cfg::EPI == Epi::kMaskF16 || Cfg::EPI == Epi::kAddMaskF32F16;
            constexpr bool kOutF32 = Cfg::EPI == Epi::kBiasReluF32F16 || Cfg::EPI == Epi::kBiasResReluF32F16 || Cfg::EPI == Epi::kAddMaskF32F16 || kPlainF32;
            constexpr bool kPartial = Cfg::EPI == Epi::kPartialF32;
            constexpr uint32_t TP = Cfg::EPI_TILE_PITCH;  // floats per staged row (16-byte aligned, bank-friendly)
            float* tile = epi_stage + ew * (Cfg::EPI_WARP_BYTES / 4);
            uint32_t* mask_words = reinterpret_cast<uint32_t*>(tile + 32 * TP);
            // B-stationary kernels keep one N tile per CTA, so a warp meets the same (at most four) column chunks in every
            // unit: their column sums are accumulated here and written once at the end instead of a global
            // read-modify-write per chunk
            float* col_acc = reinterpret_cast<float*>(mask_words + 32);
            constexpr bool kColsumLocal = Cfg::BSTAT && kHasMask && BN / (32 * Cfg::EPI_STRIDE) <= 4;
            if (kColsumLocal) {
#pragma unroll
                for (int i = 0; i < 4; ++i) col_acc[i * 32 + lane] = 0.0f;
                __syncwarp();
            }
            const uint32_t r4 = lane >> 3, c4 = (lane & 7U) * 4U;  // fp32 vectors: 4 rows x 8 lanes
            const uint32_t r8 = lane >> 2, c8 = (lane & 3U) * 8U;  // fp16 vectors: 8 rows x 4 lanes
            const bool ld_vec = (!kHasAdd || (args.ld_add & 3U) == 0U) && (!kHasMask || (args.ld_mask & 7U) == 0U) &&
                                (!kOutF32 || (args.ld_f32 & 3U) == 0U) && (kPartial ? (args.N & 3U) == 0U : (kPlainF32 || (args.ld_f16 & 7U) == 0U));
            struct Operands {
                float4 add[kHasAdd ? 8 : 1];
                uint4 mask[kHasMask ? 4 : 1];
                float bias;
            };
            // requests the global operands of chunk n0 of the tile whose first row is m_base (vector form only)
            auto request = [&](Operands& o, uint32_t m_base, uint32_t rows_ok, uint32_t n0) {
                if (n0 + 32U > args.N || !ld_vec) return;
                if constexpr (kHasBias) o.bias = __ldg(args.bias + n0 + lane);
                if constexpr (kHasAdd) {
#pragma unroll
                    for (uint32_t i = 0; i < 8U; ++i) {
                        const uint32_t rr = r4 + 4U * i;
                        o.add[i] = rr < rows_ok ? *reinterpret_cast<const float4*>(args.add_f32 + static_cast<uint64_t>(m_base + rr) * args.ld_add + n0 + c4)
                                                : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
                if constexpr (kHasMask) {
#pragma unroll
                    for (uint32_t i = 0; i < 4U; ++i) {
                        const uint32_t rr = r8 + 8U * i;
                        o.mask[i] = rr < rows_ok ? *reinterpret_cast<const uint4*>(args.mask + static_cast<uint64_t>(m_base + rr) * args.ld_mask + n0 + c8)
                                                 : make_uint4(0, 0, 0, 0);
                    }
                }
            };
            for (uint32_t unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++unit_iter) {
                uint32_t mt, nt, sp;
                decode(unit, mt, nt, sp);
                const uint32_t ab = unit_iter % ACC_BUFS, aph = (unit_iter / ACC_BUFS) & 1U;
                const uint32_t m_base = mt * BM + quad * 32U;
                const uint32_t rows_ok = m_base < args.M ? min(32U, args.M - m_base) : 0U;
                Operands next{};
                request(next, m_base, rows_ok, nt * BN + chunk_parity * 32U);
                // the TMEM loads below are warp-collective, so the whole warp takes the same way out
                if (!__all_sync(0xFFFFFFFFU, mbar_wait(&acc_full[ab], aph, cta_abort, kAbortEpilogueWait))) { ok = false; break; }
                tc_fence_after();
#pragma unroll 1
                for (int cc = static_cast<int>(chunk_parity); cc < BN / 32; cc += Cfg::EPI_STRIDE) {
                    const uint32_t n0 = nt * BN + cc * 32;
                    if (n0 >= args.N) break;
                    const Operands cur = next;
                    if (cc + Cfg::EPI_STRIDE < BN / 32) request(next, m_base, rows_ok, n0 + 32U * Cfg::EPI_STRIDE);
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((quad * 32U) << 16) + ab * Cfg::ACC_COLS + cc * 32, r);
                    tmem_ld_wait();
                    const uint32_t valid = min(32U, args.N - n0);
                    const bool vec = valid == 32U && ld_vec;
                    const bool col_ok = lane < valid;
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    if constexpr (kHasBias) {
                        const float bias_l = vec ? cur.bias : (col_ok ? __ldg(args.bias + n0 + lane) : 0.0f);
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] += __shfl_sync(0xFFFFFFFFU, bias_l, j);
                    }
                    if constexpr (kHasAdd) {
                        if (vec) {
#pragma unroll
                            for (uint32_t i = 0; i < 8U; ++i) *reinterpret_cast<float4*>(tile + (r4 + 4U * i) * TP + c4) = cur.add[i];
                        } else {
                            for (uint32_t rr = 0; rr < 32U; ++rr)
                                tile[rr * TP + lane] = (rr < rows_ok && col_ok) ? args.add_f32[static_cast<uint64_t>(m_base + rr) * args.ld_add + n0 + lane] : 0.0f;
                        }
                        __syncwarp();
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const float4 x = *reinterpret_cast<const float4*>(tile + lane * TP + q * 4);
                            v[q * 4] = x.x + v[q * 4];
                            v[q * 4 + 1] = x.y + v[q * 4 + 1];
                            v[q * 4 + 2] = x.z + v[q * 4 + 2];
                            v[q * 4 + 3] = x.w + v[q * 4 + 3];
                        }
                        __syncwarp();
                    }
                    if constexpr (kHasMask) {
                        uint32_t bits = 0;
                        if (vec) {
                            uint8_t* mask_bytes = reinterpret_cast<uint8_t*>(mask_words);
#pragma unroll
                            for (uint32_t i = 0; i < 4U; ++i) {
                                const uint32_t w4[4] = {cur.mask[i].x, cur.mask[i].y, cur.mask[i].z, cur.mask[i].w};
                                uint32_t byte = 0;
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    // a positive non-zero half: sign clear, magnitude non-zero
                                    const uint32_t lo = w4[e] & 0xFFFFU, hi = w4[e] >> 16;
                                    byte |= (lo != 0U && lo < 0x8000U) ? (1U << (2 * e)) : 0U;
                                    byte |= (hi != 0U && hi < 0x8000U) ? (1U << (2 * e + 1)) : 0U;
                                }
                                mask_bytes[(r8 + 8U * i) * 4U + (lane & 3U)] = static_cast<uint8_t>(byte);
                            }
                            __syncwarp();
                            bits = mask_words[lane];
                            __syncwarp();
                        } else {
                            for (uint32_t rr = 0; rr < 32U; ++rr) {
                                const uint16_t mh = (rr < rows_ok && col_ok) ? reinterpret_cast<const uint16_t*>(args.mask)[static_cast<uint64_t>(m_base + rr) * args.ld_mask + n0 + lane] : 0U;
                                const bool positive = mh != 0U && mh < 0x8000U;
                                const uint32_t row_bits = __ballot_sync(0xFFFFFFFFU, positive);
                                if (lane == rr) bits = row_bits;
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = ((bits >> j) & 1U) ? v[j] : 0.0f;
                    } else if constexpr (!kPartial && !kPlainF32) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
                    }
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        *reinterpret_cast<float4*>(tile + lane * TP + q * 4) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
                    __syncwarp();
                    if constexpr (kPartial || kOutF32) {
                        float* base = kPartial ? args.partial + ((static_cast<uint64_t>(group_of(unit)) * args.splits + sp) * args.M + m_base) * args.N + n0
                                               : args.out_f32 + static_cast<uint64_t>(m_base) * args.ld_f32 + n0;
                        const uint64_t ld = kPartial ? args.N : args.ld_f32;
                        if (vec) {
#pragma unroll
                            for (uint32_t i = 0; i < 8U; ++i) {
                                const uint32_t rr = r4 + 4U * i;
                                if (rr < rows_ok) *reinterpret_cast<float4*>(base + rr * ld + c4) = *reinterpret_cast<const float4*>(tile + rr * TP + c4);
                            }
                        } else {
                            for (uint32_t rr = 0; rr < rows_ok; ++rr)
                                if (col_ok) base[rr * ld + lane] = tile[rr * TP + lane];
                        }
                    }
                    if constexpr (!kPartial && !kPlainF32) {
                        if (vec) {
#pragma unroll
                            for (uint32_t i = 0; i < 4U; ++i) {
                                const uint32_t rr = r8 + 8U * i;
                                if (rr < rows_ok) {
                                    const float4 x0 = *reinterpret_cast<const float4*>(tile + rr * TP + c8);
                                    const float4 x1 = *reinterpret_cast<const float4*>(tile + rr * TP + c8 + 4U);
                                    const bool bf = args.bf16 != 0U;
                                    uint4 u;
                                    u.x = pack_operand_pair(x0.x, x0.y, bf);
                                    u.y = pack_operand_pair(x0.z, x0.w, bf);
                                    u.z = pack_operand_pair(x1.x, x1.y, bf);
                                    u.w = pack_operand_pair(x1.z, x1.w, bf);
                                    *reinterpret_cast<uint4*>(args.out_f16 + static_cast<uint64_t>(m_base + rr) * args.ld_f16 + n0 + c8) = u;
                                }
                            }
                        } else {
                            for (uint32_t rr = 0; rr < rows_ok; ++rr)
                                if (col_ok) reinterpret_cast<uint16_t*>(args.out_f16)[static_cast<uint64_t>(m_base + rr) * args.ld_f16 + n0 + lane] = to_operand(tile[rr * TP + lane], args.bf16 != 0U);
                        }
                    }
                    if constexpr (kHasMask) {
                        if (args.colsum != nullptr) {
                            float total = 0.0f;  // column `lane` of the staged tile, rows in order
#pragma unroll 8
                            for (uint32_t rr = 0; rr < 32U; ++rr) total += rr < rows_ok ? tile[rr * TP + lane] : 0.0f;
                            if (kColsumLocal) {
                                col_acc[(cc / Cfg::EPI_STRIDE) * 32 + lane] += total;  // this lane is the only user of the slot
                            } else if (col_ok) {
                                float* dst = args.colsum + (static_cast<uint64_t>(blockIdx.x) * Cfg::EPI_WARPS + ew) * args.N + n0 + lane;
                                *dst += total;  // this warp is the only writer of its row
                            }
                        }
                    }
                    __syncwarp();
                }
                tc_fence_before();
                mbar_arrive(&acc_empty[ab]);
            }
            if (kColsumLocal && args.colsum != nullptr && blockIdx.x < total_units) {
                const uint32_t nt = blockIdx.x % args.n_tiles;  // the N tile of every unit of this CTA
                for (int cc = static_cast<int>(chunk_parity); cc < BN / 32; cc += Cfg::EPI_STRIDE) {
                    const uint32_t n = nt * BN + cc * 32 + lane;
                    if (n < args.N) args.colsum[(static_cast<uint64_t>(blockIdx.x) * Cfg::EPI_WARPS + ew) * args.N + n] = col_acc[(cc / Cfg::EPI_STRIDE) * 32 + lane];
                }
            }
        }
    } else {
        // ------------------------------- one-hot synthesis --------------------------------
        if constexpr (Cfg::kOneHot) {
            // Every non-zero place of the operand is owned by one warp (set and later cleared by it),
            // so the synth warps never wait for one another: each warp polls the stage barrier itself
            // and arrives once when its share is in place.
            const uint32_t t = threadIdx.x - Cfg::FIRST_SYNTH_THREAD;  // 0 .. 32*SYNTH_WARPS-1
            constexpr uint32_t NT = 32U * Cfg::SYNTH_WARPS;
            const uint32_t V = args.value_pad, L = args.state_len, IN = args.in_rows;
            constexpr uint32_t ROWS = NACC * BN;  // rows of the synthesised operand per stage
            const uint16_t one = operand_one(args.bf16 != 0U);  // 1.0 in the operand format
            auto place = [&](uint8_t* buf, uint32_t n, uint32_t k) -> uint16_t* {
                uint8_t* row = buf + (n / BN) * Cfg::B_ACC_BYTES + (n % BN) * 128U;
                return reinterpret_cast<uint16_t*>(row + ((((k >> 3) ^ (n & 7U)) << 4) | ((k & 7U) << 1)));
            };
            // writes `value` (fp16 1.0 or 0) at the non-zero places of item (nt, c) in stage buffer `buf`
            auto apply = [&](uint8_t* buf, uint32_t nt, uint32_t c, uint16_t value) {
                if constexpr (Cfg::BSRC == BSource::kOneHotFwd) {
                    // rows = samples (thread-owned), K = input rows [64c, 64c+64)
                    const uint32_t k0 = c * 64U;
                    const uint32_t p_lo = k0 / V;
                    const uint32_t p_hi = min((k0 + 63U) / V, L - 1U);
                    const uint32_t kb = IN - k0;  // the all-ones column that multiplies the bias row
#pragma unroll
                    for (uint32_t i = 0; i < (ROWS + NT - 1U) / NT; ++i) {
                        const uint32_t n = t + i * NT;
                        const uint32_t sample = nt * ROWS + n;
                        if (sample < args.samples && n < ROWS) {
                            const uint8_t* st = args.states + static_cast<uint64_t>(sample) * 80U;
                            for (uint32_t p = p_lo; p <= p_hi && p < L; ++p) {
                                const uint32_t k = p * V + __ldg(st + p) - k0;
                                if (k < 64U) *place(buf, n, k) = value;
                            }
                            if (kb < 64U) *place(buf, n, kb) = value;
                        }
                    }
                } else {
                    // rows = input rows [r0, r0+ROWS), K = samples [64c, 64c+64); the four threads that
                    // share a sample sit in one warp and split its positions
                    const uint32_t r0 = nt * ROWS;
                    const uint32_t k = t >> 2;
                    const uint32_t sample = c * 64U + k;
                    if (sample < args.samples) {
                        const uint8_t* st = args.states + static_cast<uint64_t>(sample) * 80U;
                        const uint32_t p_lo = r0 / V;
                        const uint32_t p_hi = min((r0 + ROWS - 1U) / V, L - 1U);
                        for (uint32_t p = p_lo + (t & 3U); p <= p_hi && p < L; p += 4U) {
                            const uint32_t n = p * V + __ldg(st + p) - r0;
                            if (n < ROWS) *place(buf, n, k) = value;
                        }
                        const uint32_t nb = IN - r0;  // optional all-ones row (bias gradient)
                        if ((t & 3U) == 0U && nb < ROWS) *place(buf, nb, k) = value;
                    }
                }
            };
            static_assert(Cfg::BSRC != BSource::kOneHotGrad || NT == 256U, "64 samples x 4 threads");
            // One stage hand-over: wait until the MMAs that read stage `sb` are done (warp-uniform).
            auto acquire = [&](uint32_t it) -> bool {
                return __all_sync(0xFFFFFFFFU, mbar_wait_spin(&empty_b[it % SB], ((it / SB) & 1U) ^ 1U, cta_abort, kAbortSynthWait));
            };
            auto publish = [&](uint32_t it) {
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_b[it % SB]);
            };
            bool fast = false;
            if constexpr (Cfg::BSRC == BSource::kOneHotFwd) {
                // ---- forward, pipelined form: a row's ones sit at k_p = p*V + s[p], increasing in p, and the chunks of
                // a unit are visited in increasing k, so each row keeps a cursor. With V >= 64 a 64-wide chunk holds at
                // most two of a row's ones (plus the all-ones column that multiplies the bias row, in the last chunk).
                // Everything that needs arithmetic or a load - the places of the NEXT item - is worked out while the
                // MMAs of the current items run; between "stage released" and "stage published" the warp only stores:
                // zeros at the places it remembers from two items ago, ones at the new places.
                fast = args.splits == 1U && V >= 64U;
                if (fast) {
                    constexpr uint32_t RPT = (ROWS + NT - 1U) / NT;
                    constexpr uint32_t kNone = 0xFFFFFFFFU;
                    struct Cursor { uint32_t p, s0, s1; };
                    Cursor cur[RPT];
                    uint32_t next[RPT][3], hist[SB][RPT][3];  // hist[0]: what this thread set in the stage that comes round now
#pragma unroll
                    for (uint32_t i = 0; i < RPT; ++i)
#pragma unroll
                        for (uint32_t j = 0; j < 3U; ++j)
#pragma unroll
                            for (int q = 0; q < SB; ++q) hist[q][i][j] = kNone;
                    auto offset_of = [&](uint32_t n, uint32_t k) -> uint32_t {
                        return (n / BN) * Cfg::B_ACC_BYTES + (n % BN) * 128U + ((((k >> 3) ^ (n & 7U)) << 4) | ((k & 7U) << 1));
                    };
                    // places of item (nt, c) -> next[][]; advances the cursors (rewound at the first chunk of a unit)
                    auto prepare = [&](uint32_t nt, uint32_t c) {
                        const uint32_t k0 = c * 64U;
                        const uint32_t kb = IN - k0;
#pragma unroll
                        for (uint32_t i = 0; i < RPT; ++i) {
                            const uint32_t n = t + i * NT, sample = nt * ROWS + n;
                            const bool active = sample < args.samples && n < ROWS;
                            const uint8_t* st = args.states + static_cast<uint64_t>(sample) * 80U;
                            Cursor& q = cur[i];
                            if (c == 0U) {
                                q.p = active ? 0U : L;
                                q.s0 = active ? __ldg(st) : 0U;
                                q.s1 = (active && L > 1U) ? __ldg(st + 1) : 0U;
                            }
#pragma unroll
                            for (uint32_t j = 0; j < 2U; ++j) {
                                const uint32_t k = q.p * V + q.s0 - k0;  // never below the chunk: earlier chunks consumed those
                                const bool hit = q.p < L && k < 64U;
                                next[i][j] = hit ? offset_of(n, k) : kNone;
                                if (hit) {
                                    ++q.p;
                                    q.s0 = q.s1;
                                    q.s1 = (q.p + 1U < L) ? __ldg(st + q.p + 1U) : 0U;
                                }
                            }
                            next[i][2] = (kb < 64U && active) ? offset_of(n, kb) : kNone;
                        }
                    };
                    uint32_t unit = blockIdx.x, mt, nt, sp;
                    bool have = unit < total_units && args.k_chunks > 0U;
                    uint32_t c = 0;
                    if (have) {
                        decode(unit, mt, nt, sp);
                        prepare(nt, 0);
                    }
                    uint32_t it = 0;
                    while (have) {
                        uint32_t unit2 = unit, nt2 = nt, c2 = c + 1U;
                        bool have2 = true;
                        if (c2 >= args.k_chunks) {
                            unit2 += gridDim.x;
                            c2 = 0;
                            have2 = unit2 < total_units;
                            if (have2) {
                                uint32_t mt2, sp2;
                                decode(unit2, mt2, nt2, sp2);
                            }
                        }
                        if (!acquire(it)) break;
                        uint8_t* buf = b_ring + (it % SB) * Cfg::B_STAGE_BYTES;
#pragma unroll
                        for (uint32_t i = 0; i < RPT; ++i)
#pragma unroll
                            for (uint32_t j = 0; j < 3U; ++j) {
                                const uint32_t old = hist[0][i][j];
                                if (old != kNone) *reinterpret_cast<uint16_t*>(buf + old) = 0;
                            }
#pragma unroll
                        for (uint32_t i = 0; i < RPT; ++i)
#pragma unroll
                            for (uint32_t j = 0; j < 3U; ++j) {
                                const uint32_t off = next[i][j];
                                if (off != kNone) *reinterpret_cast<uint16_t*>(buf + off) = one;
#pragma unroll
                                for (int q = 0; q + 1 < SB; ++q) hist[q][i][j] = hist[q + 1][i][j];
                                hist[SB - 1][i][j] = off;
                            }
                        publish(it);
                        if (have2) prepare(nt2, c2);
                        unit = unit2; nt = nt2; c = c2; have = have2;
                        ++it;
                    }
                }
            } else {
                // ---- gradient, pipelined form: thread (sample k = t/4, quarter q = t%4) owns up to three of
                // the tile's positions of its sample. The state bytes of the NEXT item are fetched while the
                // current one is published; what was set in a stage is remembered and cleared from registers.
                const uint32_t max_positions = (ROWS + V - 1U) / V + 1U;
                fast = max_positions <= 12U;
                if (fast) {
                    constexpr uint32_t kNone = 0xFFFFFFFFU;
                    const uint32_t k = t >> 2, q = t & 3U;
                    uint32_t cur[3];
                    uint32_t hist[SB][4];  // hist[0]: what this thread set in the stage that comes round now
#pragma unroll
                    for (int q2 = 0; q2 < SB; ++q2)
#pragma unroll
                        for (int j = 0; j < 4; ++j) hist[q2][j] = kNone;
                    auto fetch = [&](uint32_t nt, uint32_t c) {
                        const uint32_t sample = c * 64U + k, r0 = nt * ROWS;
                        const uint32_t p_lo = r0 / V, p_hi = min((r0 + ROWS - 1U) / V, L - 1U);
                        const uint8_t* st = args.states + static_cast<uint64_t>(sample) * 80U;
#pragma unroll
                        for (uint32_t j = 0; j < 3U; ++j) {
                            const uint32_t p = p_lo + q + 4U * j;
                            cur[j] = (sample < args.samples && p <= p_hi && p < L) ? __ldg(st + p) : kNone;
                        }
                    };
                    auto offset_of = [&](uint32_t n) -> uint32_t {
                        return (n / BN) * Cfg::B_ACC_BYTES + (n % BN) * 128U + ((((k >> 3) ^ (n & 7U)) << 4) | ((k & 7U) << 1));
                    };
                    uint32_t unit = blockIdx.x, mt, nt, sp;
                    decode(unit, mt, nt, sp);
                    uint32_t c = chunk_begin(sp), c_end = chunk_begin(sp + 1);
                    bool have = unit < total_units && c < c_end;
                    if (have) fetch(nt, c);
                    uint32_t it = 0;
                    while (have) {
                        // coordinates of the item after this one
                        uint32_t unit2 = unit, nt2 = nt, c2 = c + 1U, c_end2 = c_end;
                        bool have2 = true;
                        if (c2 >= c_end2) {
                            unit2 += gridDim.x;
                            have2 = unit2 < total_units;
                            if (have2) {
                                uint32_t mt2, sp2;
                                decode(unit2, mt2, nt2, sp2);
                                c2 = chunk_begin(sp2);
                                c_end2 = chunk_begin(sp2 + 1);
                                have2 = c2 < c_end2;
                            }
                        }
                        if (!acquire(it)) break;
                        uint8_t* buf = b_ring + (it % SB) * Cfg::B_STAGE_BYTES;
#pragma unroll
                        for (uint32_t j = 0; j < 4U; ++j) {
                            const uint32_t off = hist[0][j];
                            if (off != kNone) *reinterpret_cast<uint16_t*>(buf + off) = 0;
                        }
                        __syncwarp();  // a place cleared by one lane may be set by another lane of this warp
                        const uint32_t r0 = nt * ROWS, p_lo = r0 / V;
                        uint32_t offs[4];
#pragma unroll
                        for (uint32_t j = 0; j < 3U; ++j) {
                            const uint32_t n = (p_lo + q + 4U * j) * V + cur[j] - r0;
                            offs[j] = (cur[j] != kNone && n < ROWS) ? offset_of(n) : kNone;
                        }
                        const uint32_t nb = IN - r0;  // optional all-ones row
                        offs[3] = (q == 0U && nb < ROWS && c * 64U + k < args.samples) ? offset_of(nb) : kNone;
#pragma unroll
                        for (uint32_t j = 0; j < 4U; ++j) {
                            if (offs[j] != kNone) *reinterpret_cast<uint16_t*>(buf + offs[j]) = one;
#pragma unroll
                            for (int q2 = 0; q2 + 1 < SB; ++q2) hist[q2][j] = hist[q2 + 1][j];
                            hist[SB - 1][j] = offs[j];
                        }
                        if (have2) fetch(nt2, c2);
                        publish(it);
                        unit = unit2; nt = nt2; c = c2; c_end = c_end2; have = have2;
                        ++it;
                    }
                }
            }
            if (!fast) {
                // generic form (any class count, any split): recompute the places of an item from the states
                uint32_t it = 0;
                uint32_t h_nt[SB] = {}, h_c[SB] = {};  // the last SB items, oldest first: [0] is what the stage coming round now holds
                bool ok = true;
                for (uint32_t unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
                    uint32_t mt, nt, sp;
                    decode(unit, mt, nt, sp);
                    const uint32_t c0 = chunk_begin(sp), c1 = chunk_begin(sp + 1);
                    for (uint32_t c = c0; c < c1; ++c, ++it) {
                        if (!acquire(it)) { ok = false; break; }
                        uint8_t* buf = b_ring + (it % SB) * Cfg::B_STAGE_BYTES;
                        if (it >= static_cast<uint32_t>(SB)) apply(buf, h_nt[0], h_c[0], 0);
                        __syncwarp();  // a place cleared by one lane may be set by another lane of this warp
                        apply(buf, nt, c, one);
#pragma unroll
                        for (int q2 = 0; q2 + 1 < SB; ++q2) { h_nt[q2] = h_nt[q2 + 1]; h_c[q2] = h_c[q2 + 1]; }
                        h_nt[SB - 1] = nt; h_c[SB - 1] = c;
                        publish(it);
                    }
                }
            }
        }
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*cta_abort != 0) {
        // give copies that are still in flight time to land before the CTA's memory is released
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        if (threadIdx.x == 0 && args.status != nullptr) atomicCAS(args.status, 0, *cta_abort);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace mgt
