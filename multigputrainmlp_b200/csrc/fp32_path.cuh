// The reference's non-fp16 data flows (--linear-fp16 0 and/or --input-grad-fp16 0), on CUDA cores.
//
// These flags select fp32 activations and weights for the linear layers, and an fp32 (instead of fp16)
// gradient operand for the embedding table (native/cuda/mlp_backward.cu:1273-1510 with use_half_linear /
// use_half_input_grad false; the reference runs them as TF32 cuBLAS GEMMs). They are compatibility paths, not
// the benchmarked one: plain fp32 kernels with fixed summation orders, so results are deterministic and at
// least as accurate as the reference's TF32. Used by engine.cu only.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mgt {
namespace fp32path {

__device__ __forceinline__ float ToFloat(float x) { return x; }
__device__ __forceinline__ float ToFloat(__half x) { return __half2float(x); }

// C[M x N] = op(A)[M x K] * op(B)[K x N], fp32 accumulate in k order.
//   TA = false: A is [M][lda] (K contiguous)     TA = true: A is [K][lda] (M contiguous)
//   TB = false: B is [K][ldb] (N contiguous)     TB = true: B is [N][ldb] (K contiguous)
template <bool TA, bool TB, class TAe, class TBe>
__global__ void __launch_bounds__(256)
SgemmKernel(uint32_t M, uint32_t N, uint32_t K, const TAe* __restrict__ A, uint32_t lda, const TBe* __restrict__ B, uint32_t ldb,
            float* __restrict__ C, uint32_t ldc) {
    constexpr int T = 64, KT = 16;
    __shared__ float As[KT][T + 1];
    __shared__ float Bs[KT][T + 1];
    const uint32_t m0 = blockIdx.y * T, n0 = blockIdx.x * T;
    const uint32_t tx = threadIdx.x & 15U, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4] = {};
    for (uint32_t k0 = 0; k0 < K; k0 += KT) {
        for (uint32_t i = threadIdx.x; i < T * KT; i += 256U) {
            // A tile: element (m, k)
            const uint32_t am = TA ? (i % T) : (i / KT), ak = TA ? (i / T) : (i % KT);
            const uint32_t gm = m0 + am, gk = k0 + ak;
            As[ak][am] = (gm < M && gk < K) ? ToFloat(TA ? A[(uint64_t)gk * lda + gm] : A[(uint64_t)gm * lda + gk]) : 0.0f;
            const uint32_t bn = TB ? (i / KT) : (i % T), bk = TB ? (i % KT) : (i / T);
            const uint32_t gn = n0 + bn, gkb = k0 + bk;
            Bs[bk][bn] = (gn < N && gkb < K) ? ToFloat(TB ? B[(uint64_t)gn * ldb + gkb] : B[(uint64_t)gkb * ldb + gn]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < KT; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) C[(uint64_t)m * ldc + n] = acc[i][j];
        }
}

template <bool TA, bool TB, class TAe, class TBe>
inline cudaError_t Sgemm(cudaStream_t st, uint32_t M, uint32_t N, uint32_t K, const TAe* A, uint32_t lda, const TBe* B, uint32_t ldb, float* C, uint32_t ldc) {
    const dim3 grid((N + 63) / 64, (M + 63) / 64);
    SgemmKernel<TA, TB, TAe, TBe><<<grid, 256, 0, st>>>(M, N, K, A, lda, B, ldb, C, ldc);
    return cudaGetLastError();
}

// a1[s][h] = relu(b_in[h] + sum over positions, in position order, of W_in[pos*V + state[s][pos]][h])  (mlp_backward.cu:696-753)
__global__ void InputForwardKernel(const uint8_t* __restrict__ states, const float* __restrict__ w_in, const float* __restrict__ b_in, uint32_t B,
                                   uint32_t L, uint32_t V, uint32_t H1, float* __restrict__ a1) {
    const uint64_t total = (uint64_t)B * H1, stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint32_t s = (uint32_t)(i / H1), h = (uint32_t)(i - (uint64_t)s * H1);
        const uint8_t* st = states + (uint64_t)s * 80U;
        float sum = b_in[h];
        for (uint32_t p = 0; p < L; ++p) sum += w_in[((uint64_t)p * V + st[p]) * H1 + h];
        a1[i] = fmaxf(sum, 0.0f);
    }
}

// out = relu(z + bias[col] (+ res))
__global__ void BiasReluKernel(const float* __restrict__ z, const float* __restrict__ bias, const float* __restrict__ res, uint32_t cols, uint64_t total,
                               float* __restrict__ out) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        float v = z[i] + bias[i % cols];
        if (res != nullptr) v += res[i];
        out[i] = fmaxf(v, 0.0f);
    }
}

// out = (d (+ add)) * [act > 0]; optionally also rounded through fp16 (the operand form of the fp16 embedding gradient)
template <class Act>
__global__ void MaskKernel(const float* __restrict__ d, const float* __restrict__ add, const Act* __restrict__ act, uint32_t cols, uint32_t act_pitch,
                           uint64_t total, bool round_half, float* __restrict__ out, bool act_by_columns = false) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint64_t r = i / cols, c = i - r * cols;
        float v = d[i];
        if (add != nullptr) v += add[i];
        // act_by_columns: the activation is stored with one row per column of d (act[c][r])
        v = ToFloat(act[act_by_columns ? c * act_pitch + r : r * act_pitch + c]) > 0.0f ? v : 0.0f;
        out[i] = round_half ? __half2float(__float2half_rn(v)) : v;
    }
}

// dst[c] = sum over rows of src[r][c], rows in a fixed order (32 interleaved partial sums, then 0..31)
__global__ void __launch_bounds__(256)
ColumnSumKernel(const float* __restrict__ src, uint32_t rows, uint32_t cols, float* __restrict__ dst) {
    __shared__ float part[32][9];
    const uint32_t cl = threadIdx.x & 7U, g = threadIdx.x >> 3;
    const uint32_t c = blockIdx.x * 8U + cl;
    float sum = 0.0f;
    if (c < cols)
        for (uint32_t r = g; r < rows; r += 32U) sum += src[(uint64_t)r * cols + c];
    part[g][cl] = sum;
    __syncthreads();
    if (g == 0 && c < cols) {
        float total = part[0][cl];
        for (int q = 1; q < 32; ++q) total += part[q][cl];
        dst[c] = total;
    }
}

// dy = 2 (y - label) / n and per-block partial sums of (y - label)^2 / n   (mlp_backward.cu:1331-1340)
__global__ void __launch_bounds__(256)
LossKernel(const float* __restrict__ y, const float* __restrict__ labels, uint64_t total, float inv_n, float* __restrict__ dy, float* __restrict__ partial) {
    __shared__ float red[256];
    float sum = 0.0f;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const float diff = y[i] - labels[i];
        sum += diff * diff * inv_n;
        dy[i] = 2.0f * diff * inv_n;
    }
    red[threadIdx.x] = sum;
    __syncthreads();
    for (uint32_t s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = red[0];
}
__global__ void FinishLossKernel(const float* __restrict__ partial, uint32_t count, float* __restrict__ loss) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        float sum = 0.0f;
        for (uint32_t i = 0; i < count; ++i) sum += partial[i];
        *loss = sum;
    }
}
__global__ void AddIntoKernel(float* __restrict__ acc, const float* __restrict__ x, uint64_t total) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) acc[i] += x[i];
}
__global__ void AddBiasKernel(float* __restrict__ y, const float* __restrict__ bias, uint32_t cols, uint64_t total) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) y[i] += bias[i % cols];
}

// Embedding-table gradient without atomics: CTA (position p, 64-column slice) walks all samples in order and adds
// dz1[s][cols] into the shared-memory row of the class the sample has at p; two interleaved sample streams are
// combined in a fixed order. Writes all V rows of the position (zeros for classes no sample has).
template <class Dz>
__global__ void __launch_bounds__(128)
EmbeddingGradKernel(const uint8_t* __restrict__ states, const Dz* __restrict__ dz1, uint32_t dz_pitch, uint32_t B, uint32_t V, uint32_t H1,
                    float* __restrict__ grad_table) {
    extern __shared__ float acc[];  // [2][V][64]
    const uint32_t p = blockIdx.x, c0 = blockIdx.y * 64U;
    const uint32_t col = threadIdx.x & 63U, g = threadIdx.x >> 6;
    for (uint32_t i = threadIdx.x; i < 2U * V * 64U; i += 128U) acc[i] = 0.0f;
    __syncthreads();
    const uint32_t h = c0 + col;
    if (h < H1) {
        float* mine = acc + (uint64_t)g * V * 64U + col;
        for (uint32_t s = g; s < B; s += 2U) {
            const uint32_t v = states[(uint64_t)s * 80U + p];
            if (v < V) mine[v * 64U] += ToFloat(dz1[(uint64_t)s * dz_pitch + h]);
        }
    }
    __syncthreads();
    if (h < H1 && g == 0)
        for (uint32_t v = 0; v < V; ++v) grad_table[((uint64_t)p * V + v) * H1 + h] = acc[v * 64U + col] + acc[(uint64_t)V * 64U + v * 64U + col];
}

}  // namespace fp32path
}  // namespace mgt
