// On-GPU random-walk generator, bit-exact with the reference generator for the same
// (seed, epoch, step, rank, sample): native/cuda/random_walk_kernel.cu:7-64 and
// native/src/random_walk_cpu.cpp:32-66. Integer-only; HBM traffic is 100 bytes per sample.
//
// One thread walks one sample. The 18 move permutations live in shared memory; each thread keeps
// its two 72-byte state buffers in shared memory as well, laid out position-major so that the
// threads of a warp touch neighbouring bytes.
#include "../../include/mgt_b200.h"

#include <cuda_runtime.h>

namespace {

constexpr int kWalkThreads = 128;

__host__ __device__ inline uint64_t Mix64(uint64_t x) {
    x += 0x9e3779b97f4a7c15ULL;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ULL;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebULL;
    return x ^ (x >> 31);
}

// rng = Mix64(rng); value = rng % bound on the full 64-bit state
__device__ inline uint32_t NextBounded(uint64_t* state, uint32_t bound) {
    *state = Mix64(*state);
    return static_cast<uint32_t>(*state % bound);
}

__global__ void __launch_bounds__(kWalkThreads)
RandomWalkKernel(mgt_random_walk_config_t config, uint64_t base_seed, uint64_t epoch, uint64_t step, uint32_t global_rank,
                 const mgt_train_state_t* __restrict__ moves, const mgt_train_state_t* __restrict__ target,
                 mgt_train_state_t* __restrict__ states, float* __restrict__ labels, mgt_walk_meta_t* __restrict__ meta) {
    __shared__ uint8_t s_moves[MGT_MOVE_COUNT * MGT_STATE_LEN];
    __shared__ uint8_t s_state[2][MGT_STATE_LEN][kWalkThreads];
    __shared__ __align__(16) uint8_t s_out[kWalkThreads][MGT_STATE_STORAGE_LEN];

    const uint32_t tid = threadIdx.x;
    for (uint32_t i = tid; i < config.move_count * config.state_len; i += kWalkThreads) {
        const uint32_t mv = i / config.state_len, pos = i - mv * config.state_len;
        s_moves[mv * MGT_STATE_LEN + pos] = moves[mv].v[pos];
    }
    for (uint32_t pos = 0; pos < config.state_len; ++pos) s_state[0][pos][tid] = target->v[pos];
    __syncthreads();

    const uint32_t sample = blockIdx.x * kWalkThreads + tid;
    const bool active = sample < config.sample_count;

    uint64_t rng = base_seed;
    rng ^= Mix64(epoch + 0x100000001b3ULL);
    rng ^= Mix64(step + 0x9e3779b97f4a7c15ULL);
    rng ^= Mix64(static_cast<uint64_t>(global_rank) << 32);
    rng ^= Mix64(sample);

    const uint32_t depth_span = config.k_max - config.k_min + 1U;
    const uint32_t depth = active ? config.k_min + NextBounded(&rng, depth_span) : 0U;
    uint32_t last_move = config.move_count;
    uint32_t cur = 0;
    for (uint32_t d = 0; d < depth; ++d) {
        uint32_t move = NextBounded(&rng, config.move_count);
        if (last_move != config.move_count && move == last_move) {
            move = (move + 1U + NextBounded(&rng, config.move_count - 1U)) % config.move_count;
        }
        const uint8_t* def = s_moves + move * MGT_STATE_LEN;
        for (uint32_t i = 0; i < config.state_len; ++i) s_state[cur ^ 1U][i][tid] = s_state[cur][def[i]][tid];
        cur ^= 1U;
        last_move = move;
    }
    // stage the 80-byte record (pad bytes zero) and write it with 16-byte stores
    for (uint32_t i = 0; i < MGT_STATE_STORAGE_LEN; ++i) s_out[tid][i] = i < config.state_len ? s_state[cur][i][tid] : 0;
    if (active) {
        const uint4* src = reinterpret_cast<const uint4*>(s_out[tid]);
        uint4* dst = reinterpret_cast<uint4*>(states + sample);
#pragma unroll
        for (int q = 0; q < MGT_STATE_STORAGE_LEN / 16; ++q) dst[q] = src[q];
        labels[sample] = static_cast<float>(depth);
        mgt_walk_meta_t m;
        m.depth = depth;
        m.last_move = last_move;
        m.rng_counter = rng;
        meta[sample] = m;
    }
}

__global__ void ExpandScalarLabelsKernel(const float* __restrict__ scalar_labels, uint32_t samples, uint32_t output_dim, float* __restrict__ labels) {
    const uint64_t item = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t total = static_cast<uint64_t>(samples) * output_dim;
    if (item >= total) return;
    labels[item] = scalar_labels[item / output_dim];
}

}  // namespace

extern "C" {

mgt_status_t mgt_validate_random_walk_config(const mgt_random_walk_config_t* c) {
    if (c == nullptr) return MGT_INVALID_CONFIG;
    if (c->sample_count == 0 || c->k_min == 0 || c->k_min > c->k_max || c->move_count == 0 || c->move_count > MGT_MOVE_COUNT ||
        c->state_len == 0 || c->state_len > MGT_STATE_LEN || c->state_storage_len < c->state_len ||
        c->state_storage_len > MGT_STATE_STORAGE_LEN) {
        return MGT_INVALID_CONFIG;
    }
    return MGT_OK;
}

mgt_status_t mgt_launch_random_walk(const mgt_random_walk_config_t* config, uint64_t base_seed, uint64_t epoch, uint64_t step,
                                    uint32_t global_rank, const mgt_train_state_t* device_moves,
                                    const mgt_train_state_t* device_target, mgt_train_state_t* device_states,
                                    float* device_labels, mgt_walk_meta_t* device_meta, void* stream) {
    if (mgt_validate_random_walk_config(config) != MGT_OK || device_moves == nullptr || device_target == nullptr ||
        device_states == nullptr || device_labels == nullptr || device_meta == nullptr) {
        return MGT_INVALID_CONFIG;
    }
    const uint32_t blocks = (config->sample_count + kWalkThreads - 1U) / kWalkThreads;
    RandomWalkKernel<<<blocks, kWalkThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        *config, base_seed, epoch, step, global_rank, device_moves, device_target, device_states, device_labels, device_meta);
    return cudaGetLastError() == cudaSuccess ? MGT_OK : MGT_CUDA_FAILURE;
}

mgt_status_t mgt_launch_expand_scalar_labels(const float* device_scalar_labels, uint32_t samples, uint32_t output_dim,
                                             float* device_labels, void* stream) {
    if (device_scalar_labels == nullptr || device_labels == nullptr || samples == 0 || output_dim == 0) return MGT_INVALID_CONFIG;
    const uint64_t total = static_cast<uint64_t>(samples) * output_dim;
    const uint32_t blocks = static_cast<uint32_t>((total + 255ULL) / 256ULL);
    ExpandScalarLabelsKernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(device_scalar_labels, samples, output_dim, device_labels);
    return cudaGetLastError() == cudaSuccess ? MGT_OK : MGT_CUDA_FAILURE;
}

}  // extern "C"
