// Batch normalisation of the hidden layer's pre-activation and of every residual block's fc2 output (opt-in; the
// reference has no normalisation: its weights manifest says "normalization": "none",
// native/tools/mgt_native_train_smoke.cu:343). Training mode: statistics of the batch in flight - over ALL ranks when the
// caller installs a statistics exchange - biased variance, eps; running statistics kept for the export that folds the
// normalisation into the layer's weights.
//
//   forward   z[B][H] (fp32, bias added)  ->  mean, meansq per column  ->  [exchange: average over ranks]
//             y = gamma * (z - mean) * rstd + beta ;  hidden layer: x = relu(y) ;  block: x = relu(x + y)
//   backward  dpre (gradient w.r.t. the sum entering the ReLU, fp32) -> mean(dpre), mean(dpre * xhat) per column
//             -> [exchange] -> dz = gamma * rstd * (dpre - m1 - xhat * m2)   (16-bit operand of the GEMMs that follow)
//             dgamma = sum dpre * xhat, dbeta = sum dpre, bias gradient = sum dz (zero up to rounding)
//
// All kernels are plain HBM-bound passes over [B][H] tensors. A thread owns four neighbouring columns (one 16-byte load
// per row) and every fourth, fifth ... row of its CTA's slice of the batch, so that a warp reads whole rows and each
// thread keeps several independent loads in flight; the row lanes of a CTA are added in shared memory and the per-CTA
// partial sums in a second kernel, both in a fixed order (run-to-run deterministic). Row pitches are multiples of four
// floats (fp32 tensors) and of four 16-bit elements; columns of the last quad that lie beyond H are read but never used.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx_sm100.cuh"

namespace mgt {
namespace bn {

constexpr uint32_t kThreads = 256;
constexpr uint32_t kMaxBlocks = 592;  // partial rows per reduction
constexpr uint32_t kReduceParts = 128; // reduction kernels: threads that share one column (a power of two)
constexpr uint32_t kReduceCols = 8;   // columns per CTA of the reduction kernels

__host__ __device__ inline uint32_t BlocksFor(uint32_t rows, int sm_count) {
    const uint32_t want = (rows + 63U) / 64U;  // at least 64 rows per CTA
    const uint32_t cap = static_cast<uint32_t>(sm_count) * 4U < kMaxBlocks ? static_cast<uint32_t>(sm_count) * 4U : kMaxBlocks;
    return want < 1U ? 1U : (want < cap ? want : cap);
}

// Which columns and rows a thread owns: quads q0, q0 + QT, ... and rows first + lane, first + lane + RL, ...
struct Owner {
    uint32_t Q, QT, RL, lane, q0, r0, r1;
    bool active;
};
__device__ __forceinline__ Owner MakeOwner(uint32_t rows, uint32_t H) {
    Owner o;
    o.Q = (H + 3U) / 4U;
    o.QT = o.Q < kThreads ? o.Q : kThreads;
    o.RL = kThreads / o.QT;
    o.lane = threadIdx.x / o.QT;
    o.q0 = threadIdx.x % o.QT;
    o.active = o.lane < o.RL;
    const uint32_t rows_per = (rows + gridDim.x - 1U) / gridDim.x;
    o.r0 = min(rows, blockIdx.x * rows_per);
    o.r1 = min(rows, o.r0 + rows_per);
    return o;
}
__device__ __forceinline__ float4 Load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void LoadColumns(const float* v, uint32_t col, uint32_t H, float out[4], float fill) {
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) out[i] = col + i < H ? v[col + i] : fill;
}
__device__ __forceinline__ void Store4(float* p, const float v[4], uint32_t valid) {
    if (valid >= 4U) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        for (uint32_t i = 0; i < valid; ++i) p[i] = v[i];
    }
}
__device__ __forceinline__ void StoreOperand4(uint16_t* p, const float v[4], uint32_t valid, bool bf16) {
    if (valid >= 4U) {
        *reinterpret_cast<uint2*>(p) = make_uint2(ptx::pack_operand_pair(v[0], v[1], bf16), ptx::pack_operand_pair(v[2], v[3], bf16));
    } else {
        for (uint32_t i = 0; i < valid; ++i) p[i] = ptx::to_operand(v[i], bf16);
    }
}

// Adds the row lanes of a CTA (in lane order) and hands the sums of quad q to `emit(column, value index, sum)`.
template <uint32_t kValues, typename Emit>
__device__ __forceinline__ void AddRowLanes(const Owner& o, const float (&acc)[kValues][4], uint32_t q, uint32_t H, float* smem, Emit emit) {
    if (o.RL > 1U) {  // (then QT == Q and every thread runs the quad loop exactly once)
        if (o.active) {
#pragma unroll
            for (uint32_t v = 0; v < kValues; ++v)
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) smem[((o.lane * o.QT + o.q0) * kValues + v) * 4U + i] = acc[v][i];
        }
        __syncthreads();
        if (o.lane == 0U) {
#pragma unroll
            for (uint32_t v = 0; v < kValues; ++v)
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    float s = 0.0f;
                    for (uint32_t l = 0; l < o.RL; ++l) s += smem[((l * o.QT + o.q0) * kValues + v) * 4U + i];
                    if (q * 4U + i < H) emit(q * 4U + i, v, s);
                }
        }
        __syncthreads();
    } else {
#pragma unroll
        for (uint32_t v = 0; v < kValues; ++v)
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i)
                if (q * 4U + i < H) emit(q * 4U + i, v, acc[v][i]);
    }
}

// partial[blockIdx.x][0][h] = sum over this CTA's rows of a[r][h]; partial[blockIdx.x][1][h] = sum of a[r][h] * b[r][h]
// where b = a (forward: sums of z and z*z) or b = xhat recomputed from z (backward: sums of dpre and dpre * xhat).
template <bool kBackward>
__global__ void __launch_bounds__(kThreads)
ColumnMomentsKernel(const float* __restrict__ a, uint32_t ld_a, const float* __restrict__ z, uint32_t ld_z, const float* __restrict__ mean,
                    const float* __restrict__ rstd, uint32_t rows, uint32_t H, float* __restrict__ partial) {
    __shared__ float smem[kThreads * 2U * 4U];
    const Owner o = MakeOwner(rows, H);
    for (uint32_t q = o.q0; q < o.Q; q += o.QT) {
        float acc[2][4] = {};
        float mu[4] = {}, rs[4] = {};
        if (kBackward) {
            LoadColumns(mean, q * 4U, H, mu, 0.0f);
            LoadColumns(rstd, q * 4U, H, rs, 0.0f);
        }
        if (o.active) {
#pragma unroll 4
            for (uint32_t r = o.r0 + o.lane; r < o.r1; r += o.RL) {
                const float4 v4 = Load4(a + static_cast<uint64_t>(r) * ld_a + q * 4U);
                const float v[4] = {v4.x, v4.y, v4.z, v4.w};
                float w[4] = {v4.x, v4.y, v4.z, v4.w};
                if (kBackward) {
                    const float4 z4 = Load4(z + static_cast<uint64_t>(r) * ld_z + q * 4U);
                    w[0] = (z4.x - mu[0]) * rs[0]; w[1] = (z4.y - mu[1]) * rs[1]; w[2] = (z4.z - mu[2]) * rs[2]; w[3] = (z4.w - mu[3]) * rs[3];
                }
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    acc[0][i] += v[i];
                    acc[1][i] += v[i] * w[i];
                }
            }
        }
        AddRowLanes<2>(o, acc, q, H, smem, [&](uint32_t col, uint32_t which, float s) {
            partial[(static_cast<uint64_t>(blockIdx.x) * 2U + which) * H + col] = s;
        });
    }
}

// Sum of `blocks` partial rows, in a fixed order: kReduceParts threads share a column (each adds every kReduceParts-th
// row: at most five dependent loads for 592 rows), then a binary tree over their results in shared memory. Returns the
// total in the threads with part == 0.
__device__ __forceinline__ float AddPartialRows(const float* __restrict__ partial, uint32_t blocks, uint64_t row_stride, uint32_t col, bool in_range,
                                                uint32_t part, uint32_t c, float* smem) {
    float s = 0.0f;
    if (in_range) {
#pragma unroll 4
        for (uint32_t b = part; b < blocks; b += kReduceParts) s += partial[static_cast<uint64_t>(b) * row_stride + col];
    }
    smem[part * kReduceCols + c] = s;
    __syncthreads();
#pragma unroll
    for (uint32_t half = kReduceParts / 2U; half > 0U; half >>= 1) {
        if (part < half) smem[part * kReduceCols + c] += smem[(part + half) * kReduceCols + c];
        __syncthreads();
    }
    const float total = smem[c];
    __syncthreads();
    return total;
}

// out_mean[0][h], out_mean[1][h] = (sum over the partial rows) / rows ; optionally the plain sums to two gradient vectors
// (backward: dbeta, dgamma of THIS rank's samples - the gradient exchange averages them later).
// Grid: ceil(H / kReduceCols) CTAs of kReduceCols * kReduceParts threads.
__global__ void __launch_bounds__(kReduceCols * kReduceParts)
ReduceMomentsKernel(const float* __restrict__ partial, uint32_t blocks, uint32_t H, float inv_rows, float* __restrict__ out_mean,
                    float* __restrict__ grad_sum1, float* __restrict__ grad_sum2) {
    __shared__ float smem[kReduceCols * kReduceParts];
    const uint32_t c = threadIdx.x % kReduceCols, part = threadIdx.x / kReduceCols;
    const uint32_t h = blockIdx.x * kReduceCols + c;
    const bool ok = h < H;
    const float s1 = AddPartialRows(partial, blocks, 2ULL * H, h, ok, part, c, smem);
    const float s2 = AddPartialRows(partial + H, blocks, 2ULL * H, h, ok, part, c, smem);
    if (ok && part == 0U) {
        out_mean[h] = s1 * inv_rows;
        out_mean[H + h] = s2 * inv_rows;
        if (grad_sum1 != nullptr) grad_sum1[h] = s1;
        if (grad_sum2 != nullptr) grad_sum2[h] = s2;
    }
}

__global__ void __launch_bounds__(kReduceCols * kReduceParts)
ReduceSumsKernel(const float* __restrict__ partial, uint32_t blocks, uint32_t H, float* __restrict__ out) {
    __shared__ float smem[kReduceCols * kReduceParts];
    const uint32_t c = threadIdx.x % kReduceCols, part = threadIdx.x / kReduceCols;
    const uint32_t h = blockIdx.x * kReduceCols + c;
    const bool ok = h < H;
    const float s = AddPartialRows(partial, blocks, H, h, ok, part, c, smem);
    if (ok && part == 0U) out[h] = s;
}

// stats = {mean[H], meansq[H]} of the (global) batch -> saved mean/rstd of the layer, running statistics, and
// x = relu(y) (hidden layer) or x = relu(x + y) (block) in fp32 plus its 16-bit copy.
template <bool kResidual>
__global__ void __launch_bounds__(kThreads)
ApplyForwardKernel(const float* __restrict__ z, uint32_t ld_z, const float* __restrict__ stats, const float* __restrict__ gamma, const float* __restrict__ beta,
                   float eps, uint32_t rows, uint32_t H, float* __restrict__ x_f32, uint32_t ld_x, uint16_t* __restrict__ x_h, uint32_t ld_h, bool bf16,
                   float* __restrict__ save_mean, float* __restrict__ save_rstd, float* __restrict__ running, float momentum, float unbias) {
    const Owner o = MakeOwner(rows, H);
    for (uint32_t q = o.q0; q < o.Q; q += o.QT) {
        const uint32_t col = q * 4U, valid = min(4U, H - col);
        float mu[4], msq[4], g[4], bsh[4], rs[4];
        LoadColumns(stats, col, H, mu, 0.0f);
        LoadColumns(stats + H, col, H, msq, 1.0f);
        LoadColumns(gamma, col, H, g, 0.0f);
        LoadColumns(beta, col, H, bsh, 0.0f);
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const float var = fmaxf(msq[i] - mu[i] * mu[i], 0.0f);
            rs[i] = 1.0f / sqrtf(var + eps);
            if (blockIdx.x == 0 && o.lane == 0U && i < valid) {
                save_mean[col + i] = mu[i];
                save_rstd[col + i] = rs[i];
                if (running != nullptr) {
                    running[col + i] = (1.0f - momentum) * running[col + i] + momentum * mu[i];
                    running[H + col + i] = (1.0f - momentum) * running[H + col + i] + momentum * var * unbias;
                }
            }
        }
        if (!o.active) continue;
#pragma unroll 4
        for (uint32_t r = o.r0 + o.lane; r < o.r1; r += o.RL) {
            const float4 z4 = Load4(z + static_cast<uint64_t>(r) * ld_z + col);
            const float zv[4] = {z4.x, z4.y, z4.z, z4.w};
            float* xp = x_f32 + static_cast<uint64_t>(r) * ld_x + col;
            float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (kResidual) {
                const float4 x4 = Load4(xp);
                x[0] = x4.x; x[1] = x4.y; x[2] = x4.z; x[3] = x4.w;
            }
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) x[i] = fmaxf(x[i] + (g[i] * ((zv[i] - mu[i]) * rs[i]) + bsh[i]), 0.0f);
            Store4(xp, x, valid);
            StoreOperand4(x_h + static_cast<uint64_t>(r) * ld_h + col, x, valid, bf16);
        }
    }
}

// dz = gamma * rstd * (dpre - m1 - xhat * m2) as the 16-bit operand of the GEMMs that follow; partial column sums of dz
// (the gradient of the bias that precedes the normalisation) go to partial[blockIdx.x][h].
__global__ void __launch_bounds__(kThreads)
ApplyBackwardKernel(const float* __restrict__ dpre, uint32_t ld_d, const float* __restrict__ z, uint32_t ld_z, const float* __restrict__ mean,
                    const float* __restrict__ rstd, const float* __restrict__ gamma, const float* __restrict__ moments, uint32_t rows, uint32_t H,
                    uint16_t* __restrict__ dz_h, uint32_t ld_h, bool bf16, float* __restrict__ partial) {
    __shared__ float smem[kThreads * 4U];
    const Owner o = MakeOwner(rows, H);
    for (uint32_t q = o.q0; q < o.Q; q += o.QT) {
        const uint32_t col = q * 4U, valid = min(4U, H - col);
        float mu[4], rs[4], g[4], m1[4], m2[4];
        LoadColumns(mean, col, H, mu, 0.0f);
        LoadColumns(rstd, col, H, rs, 0.0f);
        LoadColumns(gamma, col, H, g, 0.0f);
        LoadColumns(moments, col, H, m1, 0.0f);
        LoadColumns(moments + H, col, H, m2, 0.0f);
        float acc[1][4] = {};
        if (o.active) {
#pragma unroll 4
            for (uint32_t r = o.r0 + o.lane; r < o.r1; r += o.RL) {
                const float4 z4 = Load4(z + static_cast<uint64_t>(r) * ld_z + col);
                const float4 d4 = Load4(dpre + static_cast<uint64_t>(r) * ld_d + col);
                const float zv[4] = {z4.x, z4.y, z4.z, z4.w}, dv[4] = {d4.x, d4.y, d4.z, d4.w};
                float dz[4];
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    const float xhat = (zv[i] - mu[i]) * rs[i];
                    dz[i] = (g[i] * rs[i]) * (dv[i] - m1[i] - xhat * m2[i]);
                    acc[0][i] += dz[i];
                }
                StoreOperand4(dz_h + static_cast<uint64_t>(r) * ld_h + col, dz, valid, bf16);
            }
        }
        AddRowLanes<1>(o, acc, q, H, smem, [&](uint32_t c, uint32_t, float s) { partial[static_cast<uint64_t>(blockIdx.x) * H + c] = s; });
    }
}

}  // namespace bn
}  // namespace mgt
