// The residual tower as ONE kernel per direction (sm_100a, tcgen05 + TMEM).
//
// A CTA owns 128 samples and carries them through all R residual blocks without going back to HBM for the
// running state: the fp32 state S[128 x H] lives in TMEM columns [256, 256+H), the temporary product D in
// columns [0, H), and the two fp16 MMA operands (S rounded, T rounded) in 128B-swizzled shared memory where
// the epilogue warps write them for the next MMA. HBM sees only what the other kernels need afterwards: the
// fp16 tapes (activations for the weight-gradient GEMMs, dz tensors), ReLU sign bits and bias-gradient sums.
//
//   forward, block k :  D = Sh * W1_k            T = relu(D + b1_k)          -> tape_t[k],   bits_t[k]
//                       S += Th * W2_k           S = relu(S + b2_k)          -> tape_s[k+1], bits_s[k+1]
//   backward, block k:  D = Sh * W2_k^T          T = D * [r1_k > 0]          -> tape_t[k],   colsum[k]
//   (k = R-1 .. 0)      S += Th * W1_k^T         S = S * [x_k > 0]           -> tape_s[k],   colsum[R+k]
//
// (mlp_backward.cu:1280-1330 is the reference's forward loop over the blocks, 1367-1413 its backward loop; the
// rounding points - fp16 operands, fp32 accumulation, fp32 skip path - are the same.)
//
// Warp 0 streams the weights with TMA (3-stage ring, one 64-deep K chunk per stage), warp 1 issues the MMAs,
// warps 2-9 are the epilogue: two warps per TMEM lane quadrant taking alternate 32-column chunks. The MMA of
// the next layer starts on K chunk c as soon as the epilogue has written columns [64c, 64c+64) of its operand.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>

#include "ptx_sm100.cuh"

namespace mgt {

struct ChainArgs {
    uint32_t samples, H, R, tiles;
    float* state_f32;          // forward: x entering the tower (read) and leaving it (written); backward: dL/dz entering it (read)
    uint32_t ld_f32;
    const float* bias;         // forward: bias of layer l (fc1 of block k: l = 2k, fc2: l = 2k+1) at bias + l * bias_stride
    uint64_t bias_stride;
    __half* tape_s;            // entry e at tape_s + e * tape_s_stride, row pitch ld_s (halfs)
    uint64_t tape_s_stride;
    uint32_t ld_s;
    __half* tape_t;
    uint64_t tape_t_stride;
    uint32_t ld_t;
    uint32_t* bits_s;          // ReLU sign bits, entry e at bits_s + e * bits_stride, 8 words per row (tiles*128 rows)
    uint32_t* bits_t;
    uint64_t bits_stride;
    float* colsum;             // backward: slot j at colsum + j * colsum_stride, [tiles*4][H] partial column sums
    uint64_t colsum_stride;
    uint32_t bf16;             // operands and tapes are bfloat16 instead of fp16
    int* status;
};

struct ChainCfg {
    static constexpr int EPI_WARPS = 16;            // a multiple of four: EPI_WARPS/4 warps share a TMEM lane quadrant
    static constexpr int THREADS = 64 + 32 * EPI_WARPS;
    static constexpr int SW = 3;                    // weight ring stages
    static constexpr int ACT_BYTES = 4 * 16384;     // one operand: up to four 64-column panels of 128 rows x 128 bytes
    static constexpr int W_STAGE_BYTES = 32768;
    static constexpr int SMEM_BYTES = 1024 + 2 * ACT_BYTES + SW * W_STAGE_BYTES + 256 + 1024;  // + barriers + bias slices
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

namespace detail {

// Sum over the 32 lanes of a warp of each of 32 per-lane values: afterwards lane L holds the sum of v[L] over
// all lanes (a fixed tree, so the result does not depend on timing). Destroys v.
__device__ __forceinline__ float warp_column_sums(float (&v)[32], uint32_t lane) {
#pragma unroll
    for (int w = 16; w >= 1; w >>= 1) {
        const bool hi = (lane & static_cast<uint32_t>(w)) != 0U;
#pragma unroll
        for (int j = 0; j < w; ++j) {
            const float send = hi ? v[j] : v[j + w];
            const float keep = hi ? v[j + w] : v[j];
            v[j] = keep + __shfl_xor_sync(0xFFFFFFFFU, send, w);
        }
    }
    return v[0];
}

// 32 floats -> 16 packed half2 words (round to nearest even) and the "value is positive" bit of each element. The bit
// is taken from the fp32 value, as the reference takes its ReLU masks (mlp_backward.cu:944-1025 compare the fp32 copies):
// a positive value too small for fp16 rounds to +0 in the operand but still lets its gradient through.
__device__ __forceinline__ uint32_t pack_halfs(const float (&v)[32], uint32_t (&h)[16], bool bf16) {
    uint32_t bits = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        h[i] = ptx::pack_operand_pair(v[2 * i], v[2 * i + 1], bf16);
        bits |= (v[2 * i] > 0.0f ? 1U : 0U) << (2 * i);
        bits |= (v[2 * i + 1] > 0.0f ? 1U : 0U) << (2 * i + 1);
    }
    return bits;
}

}  // namespace detail

template <bool BWD>
__global__ void __launch_bounds__(ChainCfg::THREADS, 1)
tower_chain_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_tape_s,
                   const __grid_constant__ CUtensorMap tma_tape_t, const ChainArgs args) {
    using namespace ptx;
    constexpr int SW = ChainCfg::SW;
    constexpr uint32_t kStateCol = 256;  // first TMEM column of S

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + (((raw_addr + 1023U) & ~1023U) - raw_addr);
    uint8_t* act_s = smem;                           // fp16 copy of S, the A operand of the first MMA of a block
    uint8_t* act_t = smem + ChainCfg::ACT_BYTES;     // fp16 T, the A operand of the second
    uint8_t* w_ring = smem + 2 * ChainCfg::ACT_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(w_ring + SW * ChainCfg::W_STAGE_BYTES);
    uint64_t* w_full = bars;
    uint64_t* w_empty = w_full + SW;
    uint64_t* ready_s = w_empty + SW;   // [4] K chunk c of act_s is written
    uint64_t* ready_t = ready_s + 4;    // [4]
    uint64_t* mma_done = ready_t + 4;   // [2] D complete / S complete
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(mma_done + 2);
    volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_holder + 1);
    float* bias_slots = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);  // [warps per quadrant][chunks per warp][32]

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31U;
    const uint32_t H = args.H, R = args.R;
    const uint32_t KC = (H + 63U) / 64U;  // K chunks of an MMA
    const uint32_t NC = H / 32U;          // 32-column chunks of an epilogue

    if (threadIdx.x == 0) {
        for (int s = 0; s < SW; ++s) {
            mbar_init(&w_full[s], 1);
            mbar_init(&w_empty[s], 1);
        }
        for (uint32_t c = 0; c < 4U; ++c) {
            // one arrival per epilogue warp that owns a 32-column chunk inside K chunk c
            const uint32_t chunks = c < KC ? (NC - 2U * c >= 2U ? 2U : 1U) : 1U;
            mbar_init(&ready_s[c], 4U * chunks);
            mbar_init(&ready_t[c], 4U * chunks);
        }
        mbar_init(&mma_done[0], 1);
        mbar_init(&mma_done[1], 1);
        *cta_abort = 0;
        fence_barrier_init();
        prefetch_tensormap(&tma_w);
        prefetch_tensormap(&tma_tape_s);
        prefetch_tensormap(&tma_tape_t);
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        // ------------------------------- weight stream ------------------------------------
        if (lane == 0) {
            const uint32_t stage_bytes = BWD ? H * 128U : KC * 8192U;
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < args.tiles && ok; tile += gridDim.x) {
                for (uint32_t l = 0; l < 2U * R && ok; ++l) {
                    // forward visits W1_0, W2_0, W1_1, ...; backward W2_{R-1}, W1_{R-1}, W2_{R-2}, ...
                    const int32_t z = static_cast<int32_t>(BWD ? (2U * (R - 1U - (l >> 1)) + ((l & 1U) ^ 1U)) : l);
                    for (uint32_t c = 0; c < KC; ++c, ++it) {
                        const uint32_t s = it % SW, ph = (it / SW) & 1U;
                        if (!mbar_wait_spin(&w_empty[s], ph ^ 1U, cta_abort, kAbortChainWait)) { ok = false; break; }
                        uint8_t* dst = w_ring + s * ChainCfg::W_STAGE_BYTES;
                        mbar_arrive_expect_tx(&w_full[s], stage_bytes);
                        if (BWD) {
                            // B[N = in][K = out], K contiguous: one box 64(K) x H(N)
                            tma_load_3d(dst, &tma_w, static_cast<int32_t>(c * 64U), 0, z, &w_full[s]);
                        } else {
                            // B[K = in][N = out], N contiguous: boxes 64(N) x 64(K)
                            for (uint32_t g = 0; g < KC; ++g)
                                tma_load_3d(dst + g * 8192U, &tma_w, static_cast<int32_t>(g * 64U), static_cast<int32_t>(c * 64U), z, &w_full[s]);
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------- UMMA issuer --------------------------------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc_f16(128, H, false, !BWD, args.bf16 != 0U);
            uint32_t it = 0, uses = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < args.tiles && ok; tile += gridDim.x) {
                for (uint32_t kb = 0; kb < R && ok; ++kb, ++uses) {
                    for (uint32_t half = 0; half < 2U && ok; ++half) {
                        uint64_t* ready = half ? ready_t : ready_s;
                        const uint32_t a_base = smem_u32(half ? act_t : act_s);
                        const uint32_t d_addr = tmem_base + (half ? kStateCol : 0U);
                        for (uint32_t c = 0; c < KC; ++c, ++it) {
                            const uint32_t s = it % SW, ph = (it / SW) & 1U;
                            // (the issuing thread polls its barriers: waking from a suspended wait costs more than the hand-over itself)
                            if (!mbar_wait_spin(&ready[c], uses & 1U, cta_abort, kAbortChainWait)) { ok = false; break; }
                            if (!mbar_wait_spin(&w_full[s], ph, cta_abort, kAbortChainWait)) { ok = false; break; }
                            tc_fence_after();
                            const uint32_t a_addr = a_base + c * 16384U;
                            const uint32_t b_addr = smem_u32(w_ring + s * ChainCfg::W_STAGE_BYTES);
                            const uint32_t k_left = H - c * 64U;
                            const uint32_t ksteps = k_left >= 64U ? 4U : (k_left + 15U) / 16U;
                            // descriptors of the chunk's first K step; a later step only moves the start address (units of 16
                            // bytes, no carry out of the field). One thread issues everything: the full chunk is unrolled.
                            const uint64_t a_desc0 = make_smem_desc(a_addr, 16U, 1024U);
                            const uint64_t b_desc0 = BWD ? make_smem_desc(b_addr, 16U, 1024U) : make_smem_desc(b_addr, 8192U, 1024U);
                            constexpr uint64_t kStepA = 32U / 16U, kStepB = BWD ? 32U / 16U : 2048U / 16U;
                            // the second product of a block adds onto the state that already sits in TMEM
                            const uint32_t first = (half != 0U || c > 0U) ? 1U : 0U;
                            if (ksteps == 4U) {
#pragma unroll
                                for (uint32_t kk = 0; kk < 4U; ++kk) umma_f16(d_addr, a_desc0 + kk * kStepA, b_desc0 + kk * kStepB, idesc, kk == 0U ? first : 1U);
                            } else {
                                for (uint32_t kk = 0; kk < ksteps; ++kk) umma_f16(d_addr, a_desc0 + kk * kStepA, b_desc0 + kk * kStepB, idesc, kk == 0U ? first : 1U);
                            }
                            umma_commit(&w_empty[s]);
                        }
                        // the epilogue this commit releases overwrites the operand the PREVIOUS phase read and stored
                        bulk_wait_read_all();
                        if (ok) umma_commit(&mma_done[half]);
                        // Each operand panel is also a 64-column slice of a tape entry: T of this block, or the S the previous
                        // block produced (the S a tile starts with is on its tape already). Issued here, after the commit,
                        // the stores cost the MMA stream nothing.
                        if (ok && (half != 0U || kb > 0U)) {
                            const uint32_t k = BWD ? R - 1U - kb : kb;
                            const uint32_t entry = half ? k : (BWD ? k + 1U : k);
                            for (uint32_t c = 0; c < KC; ++c)
                                tma_store_3d(half ? &tma_tape_t : &tma_tape_s, (half ? act_t : act_s) + c * 16384U, static_cast<int32_t>(c * 64U),
                                             static_cast<int32_t>(tile * 128U), static_cast<int32_t>(entry));
                            bulk_commit_group();
                        }
                    }
                }
            }
            bulk_wait_all();  // the tape stores read this CTA's shared memory until they complete
        }
        __syncwarp();
    } else {
        // ------------------------------- epilogue -----------------------------------------
        const uint32_t ew = warp - 2U;
        const uint32_t quad = warp & 3U;       // TMEM lanes [32*quad, 32*quad+32)
        constexpr uint32_t SUBS = ChainCfg::EPI_WARPS / 4;  // warps per quadrant
        constexpr uint32_t WPW = 8U / SUBS;                  // 32-column chunks (and sign-bit words) per warp at most
        const uint32_t par = ew >> 2;          // this warp takes 32-column chunks par, par+SUBS, ...
        const uint32_t r = quad * 32U + lane;  // row inside the tile
        const uint32_t lane_addr = (quad * 32U) << 16;
        // byte offset of 16-byte unit u (0..7) of this row inside a 64-column panel, 128B swizzle
        auto unit_off = [&](uint32_t u) { return r * 128U + ((u ^ (r & 7U)) << 4); };
        auto store_operand = [&](uint8_t* act, uint32_t cc, const uint32_t (&h)[16]) {
            uint8_t* panel = act + (cc >> 1) * 16384U;
#pragma unroll
            for (uint32_t q = 0; q < 4U; ++q)
                *reinterpret_cast<uint4*>(panel + unit_off((cc & 1U) * 4U + q)) = make_uint4(h[4 * q], h[4 * q + 1], h[4 * q + 2], h[4 * q + 3]);
        };
        auto store_tape = [&](__half* row_ptr, uint32_t cc, const uint32_t (&h)[16]) {
            uint4* dst = reinterpret_cast<uint4*>(row_ptr + cc * 32U);
#pragma unroll
            for (uint32_t q = 0; q < 4U; ++q) dst[q] = make_uint4(h[4 * q], h[4 * q + 1], h[4 * q + 2], h[4 * q + 3]);
        };
        // lane 0 polls, the warp follows: the result is warp-uniform
        auto warp_wait = [&](uint64_t* bar, uint32_t parity) -> bool {
            uint32_t done = 0;
            if (lane == 0) done = mbar_wait_spin(bar, parity, cta_abort, kAbortChainWait) ? 1U : 0U;
            return __shfl_sync(0xFFFFFFFFU, done, 0) != 0U;
        };
        auto publish = [&](uint64_t* bar) {
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar);
        };
        // Bias of a layer: each lane fetches one value per chunk of its warp before the warp waits for the MMAs (the
        // load flies during the wait); after the wait the values go through a shared-memory slot so that every
        // thread can read all 32 of a chunk as broadcast vectors. The warps of one quadrant set share slots and write
        // identical values; a slot is rewritten only after the MMAs that needed every warp's previous epilogue.
        float bias_reg[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        auto fetch_bias = [&](uint32_t layer) {
            if (!BWD) {
#pragma unroll
                for (uint32_t ci = 0; ci < WPW; ++ci) {
                    const uint32_t cc = par + SUBS * ci;
                    if (cc < NC) bias_reg[ci] = __ldg(args.bias + layer * args.bias_stride + cc * 32U + lane);
                }
            }
        };
        auto stage_bias = [&]() {
            if (!BWD) {
#pragma unroll
                for (uint32_t ci = 0; ci < WPW; ++ci) bias_slots[(par * WPW + ci) * 32U + lane] = bias_reg[ci];
                __syncwarp();
            }
        };
        auto add_bias_relu = [&](float (&v)[32], uint32_t ci) {
            const float4* b = reinterpret_cast<const float4*>(bias_slots + (par * WPW + ci) * 32U);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float4 f = b[q];
                v[4 * q] = fmaxf(v[4 * q] + f.x, 0.0f);
                v[4 * q + 1] = fmaxf(v[4 * q + 1] + f.y, 0.0f);
                v[4 * q + 2] = fmaxf(v[4 * q + 2] + f.z, 0.0f);
                v[4 * q + 3] = fmaxf(v[4 * q + 3] + f.w, 0.0f);
            }
        };
        auto store_words = [&](uint32_t* dst, const uint32_t (&wd)[4]) {
            if (WPW == 4U) *reinterpret_cast<uint4*>(dst) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
            else *reinterpret_cast<uint2*>(dst) = make_uint2(wd[0], wd[1]);
        };
        auto load_words = [&](const uint32_t* src, uint32_t (&wd)[4]) {
            if (WPW == 4U) {
                const uint4 m = *reinterpret_cast<const uint4*>(src);
                wd[0] = m.x; wd[1] = m.y; wd[2] = m.z; wd[3] = m.w;
            } else {
                const uint2 m = *reinterpret_cast<const uint2*>(src);
                wd[0] = m.x; wd[1] = m.y;
            }
        };
        auto apply_mask = [&](float (&v)[32], uint32_t bits) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = ((bits >> j) & 1U) ? v[j] : 0.0f;
        };

        uint32_t uses = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < args.tiles && ok; tile += gridDim.x) {
            const uint64_t row = static_cast<uint64_t>(tile) * 128U + r;
            const bool row_ok = row < args.samples;
            const uint64_t bits_row = row * 8U + par * WPW;  // this warp's words of the row

            // ---- load the state: TMEM S, fp16 operand, (forward) sign bits of x_0
            {
                uint32_t words[4] = {0, 0, 0, 0};  // the first WPW are used
#pragma unroll
                for (uint32_t ci = 0; ci < WPW; ++ci) {
                    const uint32_t cc = par + SUBS * ci;
                    if (cc >= NC) break;
                    float v[32];
                    if (row_ok) {
                        const float4* src = reinterpret_cast<const float4*>(args.state_f32 + row * args.ld_f32 + cc * 32U);
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const float4 f = src[q];
                            v[4 * q] = f.x; v[4 * q + 1] = f.y; v[4 * q + 2] = f.z; v[4 * q + 3] = f.w;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = 0.0f;
                    }
                    uint32_t raw[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) raw[j] = __float_as_uint(v[j]);
                    tmem_st_32x32(tmem_base + lane_addr + kStateCol + cc * 32U, raw);
                    uint32_t h[16];
                    words[ci] = detail::pack_halfs(v, h, args.bf16 != 0U);
                    store_operand(act_s, cc, h);
                    tmem_st_wait();
                    publish(&ready_s[cc >> 1]);
                }
                if (!BWD) store_words(args.bits_s + bits_row, words);
            }

            for (uint32_t kb = 0; kb < R && ok; ++kb, ++uses) {
                const uint32_t k = BWD ? R - 1U - kb : kb;
                const bool last = kb + 1U == R;
                // ================= first epilogue: T from D =================
                {
                    uint32_t mwords[4] = {0, 0, 0, 0};
                    if (BWD) load_words(args.bits_t + k * args.bits_stride + bits_row, mwords);
                    uint32_t words[4] = {0, 0, 0, 0};  // the first WPW are used
                    fetch_bias(2U * k);
                    if (!warp_wait(&mma_done[0], uses & 1U)) { ok = false; break; }
                    tc_fence_after();
                    stage_bias();
#pragma unroll
                    for (uint32_t ci = 0; ci < WPW; ++ci) {
                        const uint32_t cc = par + SUBS * ci;
                        if (cc >= NC) break;
                        uint32_t raw[32];
                        tmem_ld_32x32(tmem_base + lane_addr + cc * 32U, raw);
                        tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
                        if (BWD) apply_mask(v, mwords[ci]);
                        else add_bias_relu(v, ci);
                        uint32_t h[16];
                        words[ci] = detail::pack_halfs(v, h, args.bf16 != 0U);
                        store_operand(act_t, cc, h);
                        publish(&ready_t[cc >> 1]);
                        if (BWD) {
                            const float total = detail::warp_column_sums(v, lane);
                            args.colsum[k * args.colsum_stride + (static_cast<uint64_t>(tile) * 4U + quad) * H + cc * 32U + lane] = total;
                        }
                    }
                    if (!BWD) store_words(args.bits_t + k * args.bits_stride + bits_row, words);
                }
                // ================= second epilogue: new S =================
                {
                    uint32_t mwords[4] = {0, 0, 0, 0};
                    if (BWD) load_words(args.bits_s + k * args.bits_stride + bits_row, mwords);
                    uint32_t words[4] = {0, 0, 0, 0};  // the first WPW are used
                    fetch_bias(2U * k + 1U);
                    if (!warp_wait(&mma_done[1], uses & 1U)) { ok = false; break; }
                    tc_fence_after();
                    stage_bias();
                    const uint32_t entry = BWD ? k : k + 1U;
                    __half* tape_row = args.tape_s + entry * args.tape_s_stride + row * args.ld_s;
#pragma unroll
                    for (uint32_t ci = 0; ci < WPW; ++ci) {
                        const uint32_t cc = par + SUBS * ci;
                        if (cc >= NC) break;
                        uint32_t raw[32];
                        tmem_ld_32x32(tmem_base + lane_addr + kStateCol + cc * 32U, raw);
                        tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
                        if (BWD) apply_mask(v, mwords[ci]);
                        else add_bias_relu(v, ci);
                        uint32_t h[16];
                        words[ci] = detail::pack_halfs(v, h, args.bf16 != 0U);
                        if (!last) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) raw[j] = __float_as_uint(v[j]);
                            tmem_st_32x32(tmem_base + lane_addr + kStateCol + cc * 32U, raw);
                            store_operand(act_s, cc, h);
                            tmem_st_wait();
                            publish(&ready_s[cc >> 1]);
                        }
                        if (row_ok && last) {  // no MMA consumes the last S of a tile, so no panel store either
                            store_tape(tape_row, cc, h);
                            if (!BWD) {
                                float4* dst = reinterpret_cast<float4*>(args.state_f32 + row * args.ld_f32 + cc * 32U);
#pragma unroll
                                for (int q = 0; q < 8; ++q) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                            }
                        }
                        if (BWD) {
                            const float total = detail::warp_column_sums(v, lane);
                            args.colsum[(R + k) * args.colsum_stride + (static_cast<uint64_t>(tile) * 4U + quad) * H + cc * 32U + lane] = total;
                        }
                    }
                    if (!BWD) store_words(args.bits_s + (k + 1U) * args.bits_stride + bits_row, words);
                    if (last) tc_fence_before();  // the next tile's state load overwrites the TMEM columns read here
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
