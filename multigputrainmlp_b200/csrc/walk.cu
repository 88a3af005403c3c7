// On-GPU random-walk generator, bit-exact with the reference generator for the same
// (seed, epoch, step, rank, sample): native/cuda/random_walk_kernel.cu:7-64 and
// native/src/random_walk_cpu.cpp:32-66. Integer-only; HBM traffic is 100 bytes per sample.
//
// One thread walks one sample. The 18 move permutations live in shared memory; each thread keeps its two 72-byte
// state buffers in shared memory as words of four positions, words of neighbouring threads next to each other:
// byte gathers of a warp then fall into 32 different banks and a move writes 18 words per thread instead of 72 bytes.
// The kernel is one warp's chain of instructions, as deep as the longest walk (about 775 instructions per move, three
// quarters of them the 72 byte gathers), so moves are applied two at a time: every CTA first composes the 18 x 18 pairs
// of permutations in shared memory (26 KB), the walk draws its moves one by one as the generator prescribes and gathers
// once per pair.
// The generator's `rng % bound` on the full 64-bit state is computed exactly with 32-bit multiplies
// (x mod b = ((hi mod b) * (2^32 mod b) + lo mod b) mod b, each step by a multiply-high with ceil(2^32 / b) and one
// correction), which is several times cheaper than a 64-bit remainder.
#include "../../include/mgt_b200.h"

#include <cuda_runtime.h>

namespace {

constexpr int kWalkThreads = 128;
constexpr int kStateWords = MGT_STATE_STORAGE_LEN / 4;  // 20 words hold the 72 positions (and the 8 pad bytes)

__host__ __device__ inline uint64_t Mix64(uint64_t x) {
    x += 0x9e3779b97f4a7c15ULL;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ULL;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebULL;
    return x ^ (x >> 31);
}

struct Bound {
    uint32_t b, magic, r32;  // magic = ceil(2^32 / b), r32 = 2^32 mod b; valid for 2 <= b <= 65535
};
__device__ inline Bound MakeBound(uint32_t b) {
    Bound q{b, 0U, 0U};
    if (b >= 2U && b <= 65535U) {
        q.magic = 0xFFFFFFFFU / b + 1U;
        q.r32 = (0xFFFFFFFFU % b + 1U) % b;
    }
    return q;
}
__device__ inline uint32_t Mod32(uint32_t n, const Bound& q) {
    if (q.magic == 0U) return q.b <= 1U ? 0U : n % q.b;
    uint32_t r = n - __umulhi(n, q.magic) * q.b;  // the quotient estimate is exact or one too large
    return r >= q.b ? r + q.b : r;
}
// rng = Mix64(rng); value = rng % bound on the full 64-bit state
__device__ inline uint32_t NextBounded(uint64_t* state, const Bound& q) {
    *state = Mix64(*state);
    const uint64_t x = *state;
    if (q.b <= 1U) return 0U;  // (a bound of 0 is a division by zero in the reference; never reached with valid configurations)
    if (q.magic == 0U) return static_cast<uint32_t>(x % q.b);
    const uint32_t h = Mod32(static_cast<uint32_t>(x >> 32), q), l = Mod32(static_cast<uint32_t>(x), q);
    return Mod32(h * q.r32 + l, q);
}

__global__ void __launch_bounds__(kWalkThreads)
RandomWalkKernel(mgt_random_walk_config_t config, uint64_t base_seed, uint64_t epoch, uint64_t step, uint32_t global_rank,
                 const mgt_train_state_t* __restrict__ moves, const mgt_train_state_t* __restrict__ target,
                 mgt_train_state_t* __restrict__ states, float* __restrict__ labels, mgt_walk_meta_t* __restrict__ meta) {
    __shared__ __align__(4) uint8_t s_moves[MGT_MOVE_COUNT * MGT_STATE_STORAGE_LEN];  // pad positions map to themselves
    // s_pairs[a][b][i] = moves[a][moves[b][i]]: "move a, then move b" as one gather (new[i] = old[move[i]] twice)
    __shared__ __align__(4) uint8_t s_pairs[MGT_MOVE_COUNT * MGT_MOVE_COUNT * MGT_STATE_STORAGE_LEN];
    __shared__ uint32_t s_state[2][kStateWords][kWalkThreads];

    const uint32_t tid = threadIdx.x;
    // Word wd of a record: the given bytes for positions below state_len. For a move (`as_move`) a pad position maps to
    // itself, and so does a source position outside the record - a malformed table must not make the gathers below index
    // outside the shared arrays; for a state the pad bytes are zero.
    auto keep_valid = [&](uint32_t given, uint32_t wd, bool as_move) -> uint32_t {
        uint32_t out = 0;
#pragma unroll
        for (uint32_t k = 0; k < 4U; ++k) {
            const uint32_t pos = wd * 4U + k;
            uint32_t byte = (given >> (8U * k)) & 0xFFU;
            if (as_move && byte >= static_cast<uint32_t>(MGT_STATE_STORAGE_LEN)) byte = pos;
            if (pos >= config.state_len) byte = as_move ? pos : 0U;
            out |= byte << (8U * k);
        }
        return out;
    };
    // the records are 80 bytes long and the arrays come from the device allocator: whole words can be read
    constexpr uint32_t kMoveWords = MGT_MOVE_COUNT * kStateWords;
    for (uint32_t i = tid; i < kMoveWords; i += kWalkThreads) {
        const uint32_t mv = i / kStateWords, wd = i - mv * kStateWords;
        const uint32_t given = mv < config.move_count ? reinterpret_cast<const uint32_t*>(moves[mv].v)[wd] : 0U;
        const uint32_t identity = 0x03020100U + wd * 0x04040404U;  // moves the puzzle does not have: never drawn, kept well-formed
        reinterpret_cast<uint32_t*>(s_moves)[i] = mv < config.move_count ? keep_valid(given, wd, true) : identity;
    }
    {
        const uint32_t* tw = reinterpret_cast<const uint32_t*>(target->v);
#pragma unroll
        for (uint32_t wd = 0; wd < kStateWords; ++wd) s_state[0][wd][tid] = keep_valid(__ldg(tw + wd), wd, false);
    }
    __syncthreads();
    // compose the pairs: one word (four positions) per item; pairs with a move the puzzle does not have are never read
    for (uint32_t i = tid; i < MGT_MOVE_COUNT * kMoveWords; i += kWalkThreads) {
        const uint32_t wd = i % kStateWords, ab = i / kStateWords;
        const uint32_t a = ab / MGT_MOVE_COUNT, b = ab - a * MGT_MOVE_COUNT;
        if (a >= config.move_count || b >= config.move_count) continue;
        const uint32_t inner = reinterpret_cast<const uint32_t*>(s_moves + b * MGT_STATE_STORAGE_LEN)[wd];
        const uint8_t* outer = s_moves + a * MGT_STATE_STORAGE_LEN;
        uint32_t packed = 0;
#pragma unroll
        for (uint32_t k = 0; k < 4U; ++k) packed |= static_cast<uint32_t>(outer[(inner >> (8U * k)) & 0xFFU]) << (8U * k);
        reinterpret_cast<uint32_t*>(s_pairs)[i] = packed;
    }
    __syncthreads();

    const uint32_t sample = blockIdx.x * kWalkThreads + tid;
    const bool active = sample < config.sample_count;

    uint64_t rng = base_seed;
    rng ^= Mix64(epoch + 0x100000001b3ULL);
    rng ^= Mix64(step + 0x9e3779b97f4a7c15ULL);
    rng ^= Mix64(static_cast<uint64_t>(global_rank) << 32);
    rng ^= Mix64(sample);

    const Bound span = MakeBound(config.k_max - config.k_min + 1U), all_moves = MakeBound(config.move_count), other_moves = MakeBound(config.move_count - 1U);
    const uint32_t depth = active ? config.k_min + NextBounded(&rng, span) : 0U;
    const uint32_t words = (config.state_len + 3U) / 4U;
    uint32_t last_move = config.move_count;
    uint32_t cur = 0;
    // the generator's next move (native/cuda/random_walk_kernel.cu:40-47: never the previous move again)
    auto draw = [&]() -> uint32_t {
        uint32_t move = NextBounded(&rng, all_moves);
        if (last_move != config.move_count && move == last_move) {
            move = Mod32(move + 1U + NextBounded(&rng, other_moves), all_moves);
        }
        last_move = move;
        return move;
    };
    // new[i] = old[def[i]] for the whole state
    auto apply = [&](const uint8_t* def_bytes) {
        const uint32_t* def = reinterpret_cast<const uint32_t*>(def_bytes);
        const uint8_t* src = reinterpret_cast<const uint8_t*>(&s_state[cur][0][0]);
        for (uint32_t wd = 0; wd < words; ++wd) {
            const uint32_t from = def[wd];  // four source positions
            uint32_t packed = 0;
#pragma unroll
            for (uint32_t k = 0; k < 4U; ++k) {
                const uint32_t pos = (from >> (8U * k)) & 0xFFU;
                packed |= static_cast<uint32_t>(src[((pos >> 2) * kWalkThreads + tid) * 4U + (pos & 3U)]) << (8U * k);
            }
            s_state[cur ^ 1U][wd][tid] = packed;
        }
        cur ^= 1U;
    };
    uint32_t d = 0;
    for (; d + 2U <= depth; d += 2U) {
        const uint32_t first = draw(), second = draw();
        apply(s_pairs + (first * MGT_MOVE_COUNT + second) * MGT_STATE_STORAGE_LEN);
    }
    if (d < depth) apply(s_moves + draw() * MGT_STATE_STORAGE_LEN);
    if (active) {
        // the 80-byte record (pad bytes zero) as five 16-byte stores
        uint4* dst = reinterpret_cast<uint4*>(states + sample);
#pragma unroll
        for (int q = 0; q < kStateWords / 4; ++q) {
            uint32_t wv[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t wd = q * 4 + k;
                uint32_t x = wd < words ? s_state[cur][wd][tid] : 0U;
                const uint32_t first = wd * 4U;  // positions at or beyond state_len are padding
                if (first + 4U > config.state_len) x &= first >= config.state_len ? 0U : (0xFFFFFFFFU >> (8U * (first + 4U - config.state_len)));
                wv[k] = x;
            }
            dst[q] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
        }
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
    // the kernel reads moves and target as words and writes a state record as five 16-byte vectors
    if ((reinterpret_cast<uintptr_t>(device_moves) & 3U) != 0 || (reinterpret_cast<uintptr_t>(device_target) & 3U) != 0 ||
        (reinterpret_cast<uintptr_t>(device_states) & 15U) != 0 || (reinterpret_cast<uintptr_t>(device_labels) & 3U) != 0 ||
        (reinterpret_cast<uintptr_t>(device_meta) & 7U) != 0) {
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
