// Gradient exchange between data-parallel ranks (one process per GPU, one node) over NVLink/NVSwitch
// peer memory, fused with the 1/W scaling and the AdamW update. Takes the place of the reference's
// NCCL wrapper + ScaleKernel + AdamW kernel (native/cuda/allreduce_nccl.cu:19-150,
// native/cuda/adamw.cu:8-46): result = (sum over ranks in rank order) * (1/W) -> AdamW, in fp32.
//
// Every rank owns one device allocation [gradient buffer | flag block] that all peers map through
// CUDA IPC. Handles are exchanged through files next to the caller's id file, the same rendezvous
// the reference uses for its NCCL id. A collective is one kernel per rank:
//   ready handshake  -> every rank tells every peer "my gradients for this call are in place"
//   small ranges     -> one-shot: each rank adds all W copies itself (identical order everywhere)
//   large ranges     -> two-shot: rank r adds slice r of all copies and writes the average into
//                       every rank's buffer
//   done handshake   -> nobody leaves (and overwrites its gradients) before all peers are finished
//   AdamW (+ fp16 mirror) on the averaged values, for the rank's own slice straight from registers.
// All waits on peers are bounded; when one runs out the kernel records a status and returns.
// Plain loads/stores on peer pointers only: no multicast of any kind.
#include "../../include/mgt_b200.h"
#include "adamw_math.cuh"

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <random>
#include <string>
#include <thread>

namespace {

constexpr uint32_t kMaxWorld = 8;
constexpr uint32_t kFlagReady = 0;     // [kMaxWorld] written by peers
constexpr uint32_t kFlagDone = 8;      // [kMaxWorld] written by peers
constexpr uint32_t kFlagCounter = 16;  // local: CTAs that finished their writes
constexpr uint32_t kFlagStatus = 17;   // local: 0 ok, else the wait that gave up
constexpr uint32_t kFlagPush = 32;     // [2][kMaxWorld] written by peers: "my vector of sequence s lies in your inbox" (slot s & 1)
constexpr uint32_t kFlagWords = 64;
constexpr uint64_t kPushMaxFloats = 1024;  // vectors up to 4 KB go by the push protocol (PushAllreduceKernel)
constexpr uint64_t kDefaultWaitLimitNs = 1000ULL * 1000ULL * 1000ULL;
constexpr uint32_t kCommThreads = 256;
constexpr uint32_t kPollSleepNs = 200;  // pause between two polls of a peer's flag (after the first few)
constexpr uint64_t kOneShotMaxFloats = 65536;  // 256 KB: below this a single pass over all copies is cheaper than two handshaken phases

struct CommDev {
    float* grad[kMaxWorld];
    uint32_t* flags[kMaxWorld];
    float* inbox[kMaxWorld];  // [2][kMaxWorld][kPushMaxFloats] on every rank
    uint32_t world;
    uint32_t rank;
    uint64_t wait_limit_ns;  // how long a kernel waits for a peer before it gives up
    uint32_t poll_sleep_ns;  // pause between two polls of a flag
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ld_peer_f1(const float* p) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Waits (bounded) until every peer has written at least `seq` into this rank's slot array.
__device__ bool WaitPeers(const CommDev& c, uint32_t base, uint32_t seq, int code) {
    __shared__ int s_fail;
    if (threadIdx.x == 0) s_fail = 0;
    __syncthreads();
    if (threadIdx.x < c.world && threadIdx.x != c.rank) {
        const uint32_t* slot = c.flags[c.rank] + base + threadIdx.x;
        const uint64_t start = timer_ns();
        uint32_t spins = 0;
        // sequence numbers only grow, so a later value also releases the wait
        while (static_cast<int32_t>(ld_acquire_sys(slot) - seq) < 0) {
            // back off between polls: hundreds of CTAs wait here at once, and their system-scope loads would otherwise
            // compete with the GEMM kernels this exchange runs beside
            if (spins >= 8U && c.poll_sleep_ns != 0U) __nanosleep(c.poll_sleep_ns);
            if ((++spins & 255U) == 0U && timer_ns() - start > c.wait_limit_ns) {
                s_fail = 1;
                atomicCAS(reinterpret_cast<int*>(c.flags[c.rank] + kFlagStatus), 0, code);
                break;
            }
        }
    }
    __syncthreads();
    return s_fail == 0;
}

struct AdamPtrs {
    float* w;
    __half* w_half;
    float* m;
    float* v;
};

template <bool kAdam>
__device__ __forceinline__ void Finish4(float4 avg, uint64_t i, float* own_grad, const AdamPtrs& a, const mgt::AdamWScalars& sc) {
    *reinterpret_cast<float4*>(own_grad + i) = avg;
    if (kAdam) {
        float4 wv = *reinterpret_cast<float4*>(a.w + i);
        float4 mv = *reinterpret_cast<float4*>(a.m + i);
        float4 vv = *reinterpret_cast<float4*>(a.v + i);
        wv.x = mgt::AdamWUpdateOne(sc, wv.x, avg.x, &mv.x, &vv.x);
        wv.y = mgt::AdamWUpdateOne(sc, wv.y, avg.y, &mv.y, &vv.y);
        wv.z = mgt::AdamWUpdateOne(sc, wv.z, avg.z, &mv.z, &vv.z);
        wv.w = mgt::AdamWUpdateOne(sc, wv.w, avg.w, &mv.w, &vv.w);
        *reinterpret_cast<float4*>(a.w + i) = wv;
        *reinterpret_cast<float4*>(a.m + i) = mv;
        *reinterpret_cast<float4*>(a.v + i) = vv;
        if (a.w_half != nullptr) {
            const __half2 h01 = __floats2half2_rn(wv.x, wv.y);
            const __half2 h23 = __floats2half2_rn(wv.z, wv.w);
            uint2 u;
            u.x = *reinterpret_cast<const uint32_t*>(&h01);
            u.y = *reinterpret_cast<const uint32_t*>(&h23);
            *reinterpret_cast<uint2*>(a.w_half + i) = u;
        }
    }
}

template <bool kAdam>
__device__ __forceinline__ void Finish1(float avg, uint64_t i, float* own_grad, const AdamPtrs& a, const mgt::AdamWScalars& sc) {
    own_grad[i] = avg;
    if (kAdam) {
        float mm = a.m[i], vv = a.v[i];
        const float nw = mgt::AdamWUpdateOne(sc, a.w[i], avg, &mm, &vv);
        a.w[i] = nw;
        a.m[i] = mm;
        a.v[i] = vv;
        if (a.w_half != nullptr) a.w_half[i] = __float2half_rn(nw);
    }
}

// Sum over ranks in rank order, times 1/W: what ncclAllReduce(sum) + ScaleKernel produce.
__device__ __forceinline__ float4 Average4(const CommDev& c, uint64_t i, float inv_w) {
    float4 s = ld_peer_f4(c.grad[0] + i);
    for (uint32_t p = 1; p < c.world; ++p) {
        const float4 x = ld_peer_f4(c.grad[p] + i);
        s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
    }
    s.x *= inv_w; s.y *= inv_w; s.z *= inv_w; s.w *= inv_w;
    return s;
}
__device__ __forceinline__ float Average1(const CommDev& c, uint64_t i, float inv_w) {
    float s = ld_peer_f1(c.grad[0] + i);
    for (uint32_t p = 1; p < c.world; ++p) s += ld_peer_f1(c.grad[p] + i);
    return s * inv_w;
}

// Elements [begin, end) of the flat buffer; begin/end need no alignment.
template <bool kAdam, bool kWritePeers>
__device__ void ReduceRange(const CommDev& c, uint64_t begin, uint64_t end, float inv_w, const AdamPtrs& a, const mgt::AdamWScalars& sc) {
    float* own = c.grad[c.rank];
    const uint64_t tid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t nthreads = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const uint64_t head_up = (begin + 3ULL) & ~3ULL;
    const uint64_t head_end = end < head_up ? end : head_up;
    const uint64_t body_end = head_end + ((end - head_end) & ~3ULL);
    for (uint64_t i = begin + tid; i < head_end; i += nthreads) {
        const float avg = Average1(c, i, inv_w);
        if (kWritePeers)
            for (uint32_t p = 0; p < c.world; ++p)
                if (p != c.rank) c.grad[p][i] = avg;
        Finish1<kAdam>(avg, i, own, a, sc);
    }
    // four vectors per thread and pass: 4 x world peer loads are in flight before the first sum, which is what it takes
    // to cover the NVLink round trip with 148 x 256 threads
    constexpr uint32_t kUnroll = 4;
    uint64_t i = head_end + tid * 4ULL;
    for (; i + (kUnroll - 1ULL) * nthreads * 4ULL < body_end; i += nthreads * 4ULL * kUnroll) {
        float4 acc[kUnroll];
#pragma unroll
        for (uint32_t u = 0; u < kUnroll; ++u) acc[u] = ld_peer_f4(c.grad[0] + i + u * nthreads * 4ULL);
        for (uint32_t p = 1; p < c.world; ++p) {
            float4 x[kUnroll];
#pragma unroll
            for (uint32_t u = 0; u < kUnroll; ++u) x[u] = ld_peer_f4(c.grad[p] + i + u * nthreads * 4ULL);
#pragma unroll
            for (uint32_t u = 0; u < kUnroll; ++u) { acc[u].x += x[u].x; acc[u].y += x[u].y; acc[u].z += x[u].z; acc[u].w += x[u].w; }
        }
#pragma unroll
        for (uint32_t u = 0; u < kUnroll; ++u) {
            const uint64_t j = i + u * nthreads * 4ULL;
            const float4 avg = make_float4(acc[u].x * inv_w, acc[u].y * inv_w, acc[u].z * inv_w, acc[u].w * inv_w);
            if (kWritePeers)
                for (uint32_t p = 0; p < c.world; ++p)
                    if (p != c.rank) *reinterpret_cast<float4*>(c.grad[p] + j) = avg;
            Finish4<kAdam>(avg, j, own, a, sc);
        }
    }
    for (; i < body_end; i += nthreads * 4ULL) {
        const float4 avg = Average4(c, i, inv_w);
        if (kWritePeers)
            for (uint32_t p = 0; p < c.world; ++p)
                if (p != c.rank) *reinterpret_cast<float4*>(c.grad[p] + i) = avg;
        Finish4<kAdam>(avg, i, own, a, sc);
    }
    for (uint64_t i = body_end + tid; i < end; i += nthreads) {
        const float avg = Average1(c, i, inv_w);
        if (kWritePeers)
            for (uint32_t p = 0; p < c.world; ++p)
                if (p != c.rank) c.grad[p][i] = avg;
        Finish1<kAdam>(avg, i, own, a, sc);
    }
}

// AdamW on averages that peers wrote into this rank's buffer.
__device__ void AdamRange(const CommDev& c, uint64_t begin, uint64_t end, const AdamPtrs& a, const mgt::AdamWScalars& sc) {
    float* own = c.grad[c.rank];
    const uint64_t tid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t nthreads = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const uint64_t head_up = (begin + 3ULL) & ~3ULL;
    const uint64_t head_end = end < head_up ? end : head_up;
    const uint64_t body_end = head_end + ((end - head_end) & ~3ULL);
    for (uint64_t i = begin + tid; i < head_end; i += nthreads) Finish1<true>(__ldcg(own + i), i, own, a, sc);
    for (uint64_t i = head_end + tid * 4ULL; i < body_end; i += nthreads * 4ULL) Finish4<true>(__ldcg(reinterpret_cast<const float4*>(own + i)), i, own, a, sc);
    for (uint64_t i = body_end + tid; i < end; i += nthreads) Finish1<true>(__ldcg(own + i), i, own, a, sc);
}

// Tiny vectors (batch-norm statistics, the output layer's gradient): one CTA, ONE one-way trip. Every rank writes its vector
// into slot [seq & 1][own rank] of every peer's inbox, then a flag; it waits for the W-1 flags in its own flag block and adds
// the W vectors in rank order (its own from its buffer). No ready and no done handshake: a peer can write sequence s + 2
// into the slot of sequence s only after it has finished s + 1, for which it needed this rank's vector of s + 1, which this
// rank sends only after it has read its inbox of s. 19 -> about 8 us per vector at 2 GPUs, and no growth with the rank count
// beyond the W - 1 stores (the handshaken one-shot kernel below takes 44 us at 4 GPUs).
template <bool kAdam>
__global__ void __launch_bounds__(kCommThreads)
PushAllreduceKernel(CommDev c, uint64_t offset, uint32_t count, uint32_t seq, mgt_adamw_config_t cfg, AdamPtrs a) {
    const float inv_w = 1.0f / static_cast<float>(c.world);
    mgt::AdamWScalars sc{};
    if (kAdam) sc = mgt::MakeAdamWScalars(cfg.step, cfg.learning_rate, cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay);
    const uint32_t slot = seq & 1U;
    float* own = c.grad[c.rank] + offset;
    for (uint32_t p = 0; p < c.world; ++p) {
        if (p == c.rank) continue;
        float* dst = c.inbox[p] + (static_cast<uint64_t>(slot) * kMaxWorld + c.rank) * kPushMaxFloats;
        for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) dst[i] = own[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < c.world && threadIdx.x != c.rank) st_release_sys(c.flags[threadIdx.x] + kFlagPush + slot * kMaxWorld + c.rank, seq);
    if (!WaitPeers(c, kFlagPush + slot * kMaxWorld, seq, 3)) return;
    const float* in = c.inbox[c.rank] + static_cast<uint64_t>(slot) * kMaxWorld * kPushMaxFloats;
    for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) {
        float sum = 0.0f;
        for (uint32_t p = 0; p < c.world; ++p) sum += p == c.rank ? own[i] : ld_peer_f1(in + static_cast<uint64_t>(p) * kPushMaxFloats + i);
        Finish1<kAdam>(sum * inv_w, offset + i, c.grad[c.rank], a, sc);
    }
}

// One-shot ranges run as ONE launch (kPhaseAll, at most 64 CTAs). Two-shot ranges run as two launches on the same stream:
// kPhaseReduce (ready handshake, reduce own slice, write it to every rank, last CTA signals "done") and kPhaseFinish
// (done handshake, AdamW on the slices the peers wrote). Split like this, no CTA of a large grid ever waits for something
// that another CTA of the SAME launch still has to do, so the grid need not be resident at once - it may queue behind the
// persistent GEMM kernels it overlaps with.
enum CommPhase : int { kPhaseAll = 0, kPhaseReduce = 1, kPhaseFinish = 2 };

template <bool kAdam>
__global__ void __launch_bounds__(kCommThreads)
AllreduceAverageKernel(CommDev c, uint64_t offset, uint64_t count, uint32_t seq, mgt_adamw_config_t cfg, AdamPtrs a, int phase) {
    const float inv_w = 1.0f / static_cast<float>(c.world);
    mgt::AdamWScalars sc{};
    if (kAdam) sc = mgt::MakeAdamWScalars(cfg.step, cfg.learning_rate, cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay);
    uint32_t* my_flags = c.flags[c.rank];
    const bool one_shot = phase == kPhaseAll;

    // two-shot slices: boundaries on multiples of 4 floats so that the bulk of every slice is 16-byte aligned
    uint64_t my_begin = offset, my_end = offset + count;
    if (!one_shot) {
        const uint64_t first4 = (offset + 3ULL) / 4ULL, last4 = (offset + count) / 4ULL;
        const uint64_t quads = last4 > first4 ? last4 - first4 : 0ULL;
        my_begin = c.rank == 0 ? offset : (first4 + quads * c.rank / c.world) * 4ULL;
        my_end = c.rank + 1 == c.world ? offset + count : (first4 + quads * (c.rank + 1) / c.world) * 4ULL;
    }
    // one-shot: every rank reads all copies, so nobody may overwrite its own copy before the done
    // handshake; each thread keeps its (at most one) float4 and two edge scalars in registers
    const uint64_t tid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t end = offset + count;
    const uint64_t head_up = (offset + 3ULL) & ~3ULL;
    const uint64_t head_end = end < head_up ? end : head_up;
    const uint64_t body_end = head_end + ((end - head_end) & ~3ULL);
    float4 keep4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float keep_head = 0.f, keep_tail = 0.f;

    if (phase != kPhaseFinish) {
        // ready handshake: the producer kernels of this rank finished before this kernel started
        if (blockIdx.x == 0 && threadIdx.x < c.world && threadIdx.x != c.rank) {
            __threadfence_system();
            st_release_sys(c.flags[threadIdx.x] + kFlagReady + c.rank, seq);
        }
        if (!WaitPeers(c, kFlagReady, seq, 1)) return;
        if (one_shot) {
            if (offset + tid < head_end) keep_head = Average1(c, offset + tid, inv_w);
            if (head_end + tid * 4ULL < body_end) keep4 = Average4(c, head_end + tid * 4ULL, inv_w);
            if (body_end + tid < end) keep_tail = Average1(c, body_end + tid, inv_w);
        } else {
            ReduceRange<kAdam, true>(c, my_begin, my_end, inv_w, a, sc);
        }
        // the last CTA of this rank to finish tells every peer
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            const uint32_t arrived = atomicAdd(my_flags + kFlagCounter, 1U);
            if (arrived == gridDim.x - 1U) {
                my_flags[kFlagCounter] = 0U;
                __threadfence_system();
                for (uint32_t p = 0; p < c.world; ++p)
                    if (p != c.rank) st_release_sys(c.flags[p] + kFlagDone + c.rank, seq);
            }
        }
        if (phase == kPhaseReduce) return;
    }

    // done handshake: nobody goes on (and overwrites its gradients) before all peers are finished
    if (!WaitPeers(c, kFlagDone, seq, 2)) return;

    if (one_shot) {
        float* own = c.grad[c.rank];
        if (offset + tid < head_end) Finish1<kAdam>(keep_head, offset + tid, own, a, sc);
        if (head_end + tid * 4ULL < body_end) Finish4<kAdam>(keep4, head_end + tid * 4ULL, own, a, sc);
        if (body_end + tid < end) Finish1<kAdam>(keep_tail, body_end + tid, own, a, sc);
    } else if (kAdam) {
        AdamRange(c, offset, my_begin, a, sc);
        AdamRange(c, my_end, offset + count, a, sc);
    }
}

struct Handshake {
    char magic[8];
    uint64_t nonce;
    uint64_t bytes;
    cudaIpcMemHandle_t handle;
};

bool WriteFileAtomic(const std::string& path, const void* data, size_t bytes) {
    const std::string tmp = path + ".tmp";
    {
        std::ofstream out(tmp, std::ios::binary | std::ios::trunc);
        if (!out) return false;
        out.write(static_cast<const char*>(data), static_cast<std::streamsize>(bytes));
        if (!out) return false;
    }
    return std::rename(tmp.c_str(), path.c_str()) == 0;
}

// Polls like the reference's id-file reader: 300 attempts, 100 ms apart (allreduce_nccl.cu:38-49).
bool ReadFilePolling(const std::string& path, void* data, size_t bytes) {
    for (int attempt = 0; attempt < 300; ++attempt) {
        std::ifstream in(path, std::ios::binary);
        if (in) {
            in.read(static_cast<char*>(data), static_cast<std::streamsize>(bytes));
            if (in.gcount() == static_cast<std::streamsize>(bytes)) return true;
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(100));
    }
    return false;
}

}  // namespace

struct mgt_comm {
    int device = 0;
    uint32_t world = 1, rank = 0;
    uint64_t gradient_floats = 0;
    uint8_t* local = nullptr;             // [gradient buffer | flag block]
    void* peer_base[kMaxWorld] = {};
    CommDev dev{};
    uint32_t seq = 0;
    int sm_count = 148;
    uint64_t launches = 0;
    std::string id_file;
    uint64_t nonce = 0;
    uint64_t barrier_seq = 0;  // host barriers passed so far
    bool dead = false;         // a wait ran out: the flag state of the ranks no longer agrees, nothing more is launched
};

extern "C" {

mgt_status_t mgt_comm_create(int32_t device_id, uint32_t world_size, uint32_t global_rank, const char* id_file,
                             uint64_t gradient_floats, mgt_comm_t** out) {
    if (out == nullptr || world_size == 0 || world_size > kMaxWorld || global_rank >= world_size || gradient_floats == 0 || device_id < 0) return MGT_INVALID_CONFIG;
    if (world_size > 1 && (id_file == nullptr || id_file[0] == '\0')) return MGT_INVALID_CONFIG;  // allreduce_nccl.cu:66-68
    *out = nullptr;
    if (cudaSetDevice(device_id) != cudaSuccess) return MGT_CUDA_FAILURE;
    auto* c = new mgt_comm();
    c->device = device_id;
    c->world = world_size;
    c->rank = global_rank;
    c->gradient_floats = gradient_floats;
    cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, device_id);
    const uint64_t grad_bytes = (gradient_floats * 4ULL + 255ULL) & ~255ULL;
    const uint64_t inbox_bytes = 2ULL * kMaxWorld * kPushMaxFloats * 4ULL;
    const uint64_t bytes = grad_bytes + kFlagWords * 4ULL + inbox_bytes;
    if (cudaMalloc(&c->local, bytes) != cudaSuccess || cudaMemset(c->local, 0, bytes) != cudaSuccess) {
        delete c;
        return MGT_CUDA_FAILURE;
    }
    c->dev.world = world_size;
    c->dev.rank = global_rank;
    c->dev.wait_limit_ns = kDefaultWaitLimitNs;
    c->dev.poll_sleep_ns = kPollSleepNs;
    c->peer_base[global_rank] = c->local;
    if (world_size > 1) {
        c->id_file = id_file;
        // rank 0 publishes a nonce (the role of the NCCL unique id); every rank then publishes the IPC
        // handle of its allocation under that nonce, so files of an earlier run are never picked up
        Handshake mine{};
        std::memcpy(mine.magic, "MGTIPC1", 8);
        if (global_rank == 0) {
            std::random_device rd;
            c->nonce = (static_cast<uint64_t>(rd()) << 32) ^ rd() ^ static_cast<uint64_t>(std::chrono::steady_clock::now().time_since_epoch().count());
            uint8_t id[128] = {};
            std::memcpy(id, "MGTID01", 8);
            std::memcpy(id + 8, &c->nonce, 8);
            if (!WriteFileAtomic(c->id_file, id, sizeof(id))) { cudaFree(c->local); delete c; return MGT_IO_FAILURE; }
        } else {
            uint8_t id[128] = {};
            if (!ReadFilePolling(c->id_file, id, sizeof(id)) || std::memcmp(id, "MGTID01", 8) != 0) { cudaFree(c->local); delete c; return MGT_IO_FAILURE; }
            std::memcpy(&c->nonce, id + 8, 8);
        }
        mine.nonce = c->nonce;
        mine.bytes = bytes;
        if (cudaIpcGetMemHandle(&mine.handle, c->local) != cudaSuccess) { cudaFree(c->local); delete c; return MGT_CUDA_FAILURE; }
        char suffix[64];
        std::snprintf(suffix, sizeof(suffix), ".%016llx.%u", static_cast<unsigned long long>(c->nonce), global_rank);
        if (!WriteFileAtomic(c->id_file + suffix, &mine, sizeof(mine))) { cudaFree(c->local); delete c; return MGT_IO_FAILURE; }
        for (uint32_t p = 0; p < world_size; ++p) {
            if (p == global_rank) continue;
            Handshake theirs{};
            std::snprintf(suffix, sizeof(suffix), ".%016llx.%u", static_cast<unsigned long long>(c->nonce), p);
            if (!ReadFilePolling(c->id_file + suffix, &theirs, sizeof(theirs)) || theirs.nonce != c->nonce || theirs.bytes != bytes) {
                cudaFree(c->local); delete c; return MGT_IO_FAILURE;
            }
            if (cudaIpcOpenMemHandle(&c->peer_base[p], theirs.handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                cudaFree(c->local); delete c; return MGT_NCCL_FAILURE;
            }
        }
    }
    for (uint32_t p = 0; p < world_size; ++p) {
        c->dev.grad[p] = reinterpret_cast<float*>(c->peer_base[p]);
        c->dev.flags[p] = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(c->peer_base[p]) + grad_bytes);
        c->dev.inbox[p] = reinterpret_cast<float*>(static_cast<uint8_t*>(c->peer_base[p]) + grad_bytes + kFlagWords * 4ULL);
    }
    *out = c;
    return MGT_OK;
}

float* mgt_comm_gradient_buffer(mgt_comm_t* c) { return c == nullptr ? nullptr : reinterpret_cast<float*>(c->local); }

uint64_t mgt_comm_launch_count(const mgt_comm_t* c) { return c == nullptr ? 0 : c->launches; }

static mgt_status_t LaunchAllreduce(mgt_comm_t* c, uint64_t offset, uint64_t count, const mgt_adamw_config_t* adam, float* w,
                                    uint16_t* w_half, float* m, float* v, void* stream) {
    if (c == nullptr || count == 0 || offset + count > c->gradient_floats) return MGT_INVALID_CONFIG;
    if (c->dead) return MGT_DEVICE_TIMEOUT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    AdamPtrs a{w, reinterpret_cast<__half*>(w_half), m, v};
    mgt_adamw_config_t cfg{};
    if (adam != nullptr) {
        if (mgt_validate_adamw_config(adam) != MGT_OK || w == nullptr || m == nullptr || v == nullptr) return MGT_INVALID_CONFIG;
        if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15U) return MGT_INVALID_CONFIG;
        cfg = *adam;
        // the optimizer state is addressed with the same flat offsets as the gradient buffer
    }
    const uint64_t quads = (count + 3ULL) / 4ULL;
    const uint64_t want = (quads + kCommThreads - 1ULL) / kCommThreads;  // one-shot ranges: one float4 per thread (at most 64 CTAs)
    const bool one_shot = count <= kOneShotMaxFloats;
    const uint32_t seq = ++c->seq;
    auto launch = [&](uint32_t grid, int phase) {
        if (adam != nullptr) {
            AllreduceAverageKernel<true><<<grid, kCommThreads, 0, st>>>(c->dev, offset, count, seq, cfg, a, phase);
        } else {
            AllreduceAverageKernel<false><<<grid, kCommThreads, 0, st>>>(c->dev, offset, count, seq, cfg, a, phase);
        }
        ++c->launches;
    };
    if (count <= kPushMaxFloats && c->world > 1) {
        if (adam != nullptr) {
            PushAllreduceKernel<true><<<1, kCommThreads, 0, st>>>(c->dev, offset, static_cast<uint32_t>(count), seq, cfg, a);
        } else {
            PushAllreduceKernel<false><<<1, kCommThreads, 0, st>>>(c->dev, offset, static_cast<uint32_t>(count), seq, cfg, a);
        }
        ++c->launches;
    } else if (one_shot) {
        // every CTA waits for the peers' "done" after its own reads, so these (at most 64) CTAs must be able to be resident
        // together: they are, one per SM, also beside a persistent GEMM CTA (256 threads, no shared memory)
        launch(static_cast<uint32_t>(want < 1 ? 1 : want), kPhaseAll);
    } else {
        // up to four CTAs per SM cover the NVLink round trip; the grid may queue (see CommPhase)
        const uint64_t cap = static_cast<uint64_t>(c->sm_count) * 4ULL;
        launch(static_cast<uint32_t>(want < cap ? want : cap), kPhaseReduce);
        const uint64_t rest = adam != nullptr ? want : 1ULL;  // without the update the second launch only waits for the peers
        launch(static_cast<uint32_t>(rest < cap ? rest : cap), kPhaseFinish);
    }
    return cudaGetLastError() == cudaSuccess ? MGT_OK : MGT_CUDA_FAILURE;
}

mgt_status_t mgt_comm_allreduce_average(mgt_comm_t* c, const mgt_allreduce_config_t* config, float* device_gradients, void* stream) {
    if (c == nullptr || config == nullptr || device_gradients == nullptr || config->world_size == 0 || config->element_count == 0 ||
        config->global_rank >= config->world_size) return MGT_INVALID_CONFIG;
    if (config->world_size != c->world || config->global_rank != c->rank) return MGT_INVALID_CONFIG;  // allreduce_nccl.cu:127-129
    float* base = reinterpret_cast<float*>(c->local);
    if (device_gradients < base || device_gradients + config->element_count > base + c->gradient_floats) return MGT_INVALID_CONFIG;
    return LaunchAllreduce(c, static_cast<uint64_t>(device_gradients - base), config->element_count, nullptr, nullptr, nullptr, nullptr, nullptr, stream);
}

mgt_status_t mgt_comm_allreduce_average_adamw(mgt_comm_t* c, uint64_t param_offset, uint64_t param_count, const mgt_adamw_config_t* adamw,
                                              float* device_weights, uint16_t* device_weights_half, float* device_m, float* device_v, void* stream) {
    if (adamw == nullptr) return MGT_INVALID_CONFIG;
    return LaunchAllreduce(c, param_offset, param_count, adamw, device_weights, device_weights_half, device_m, device_v, stream);
}

mgt_status_t mgt_comm_check(mgt_comm_t* c, void* stream, int32_t* out_code) {
    if (c == nullptr) return MGT_INVALID_CONFIG;
    if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) return MGT_CUDA_FAILURE;
    const uint64_t grad_bytes = (c->gradient_floats * 4ULL + 255ULL) & ~255ULL;
    uint32_t* status = reinterpret_cast<uint32_t*>(c->local + grad_bytes) + kFlagStatus;
    uint32_t code = 0;
    if (cudaMemcpy(&code, status, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return MGT_CUDA_FAILURE;
    if (out_code) *out_code = static_cast<int32_t>(code);
    if (code != 0 || c->dead) {
        // CTAs that gave up never reached the arrival counter and the peers' sequence numbers no longer match this
        // rank's: the communicator stays unusable. Weights that a fused update touched before the wait ran out are
        // undefined (some slices updated, some not).
        cudaMemset(status, 0, 4);
        cudaMemset(reinterpret_cast<uint32_t*>(c->local + grad_bytes) + kFlagCounter, 0, 4);
        c->dead = true;
        return MGT_DEVICE_TIMEOUT;
    }
    return MGT_OK;
}

mgt_status_t mgt_comm_set_wait_limit_ms(mgt_comm_t* c, uint32_t milliseconds) {
    if (c == nullptr || milliseconds == 0 || milliseconds > 60000U) return MGT_INVALID_CONFIG;
    c->dev.wait_limit_ns = static_cast<uint64_t>(milliseconds) * 1000000ULL;
    return MGT_OK;
}

mgt_status_t mgt_comm_host_barrier(mgt_comm_t* c, uint32_t timeout_ms) {
    if (c == nullptr) return MGT_INVALID_CONFIG;
    if (c->world <= 1) return MGT_OK;
    // every rank publishes "<id file>.<nonce>.b<seq>.<rank>" and waits for the files of all the others; a rank removes
    // its file of the barrier before the last one, which every peer has passed by then
    const uint64_t seq = ++c->barrier_seq;
    auto name = [&](uint64_t q, uint32_t r) {
        char suffix[96];
        std::snprintf(suffix, sizeof(suffix), ".%016llx.b%llu.%u", static_cast<unsigned long long>(c->nonce), static_cast<unsigned long long>(q), r);
        return c->id_file + suffix;
    };
    const uint8_t mark = 1;
    if (!WriteFileAtomic(name(seq, c->rank), &mark, 1)) return MGT_IO_FAILURE;
    const auto start = std::chrono::steady_clock::now();
    for (uint32_t p = 0; p < c->world; ++p) {
        if (p == c->rank) continue;
        for (;;) {
            std::ifstream in(name(seq, p), std::ios::binary);
            if (in) break;
            if (std::chrono::steady_clock::now() - start > std::chrono::milliseconds(timeout_ms)) return MGT_IO_FAILURE;
            std::this_thread::sleep_for(std::chrono::milliseconds(2));
        }
    }
    if (seq >= 2) std::remove(name(seq - 2, c->rank).c_str());
    return MGT_OK;
}

mgt_status_t mgt_comm_destroy(mgt_comm_t* c) {
    if (c == nullptr) return MGT_OK;
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    for (uint32_t p = 0; p < c->world; ++p)
        if (p != c->rank && c->peer_base[p] != nullptr) cudaIpcCloseMemHandle(c->peer_base[p]);
    if (c->local) cudaFree(c->local);
    if (c->world > 1 && !c->id_file.empty()) {
        char suffix[96];
        std::snprintf(suffix, sizeof(suffix), ".%016llx.%u", static_cast<unsigned long long>(c->nonce), c->rank);
        std::remove((c->id_file + suffix).c_str());
        // the file of the last barrier stays: a peer may still be reading it
        if (c->barrier_seq >= 2) {
            std::snprintf(suffix, sizeof(suffix), ".%016llx.b%llu.%u", static_cast<unsigned long long>(c->nonce), static_cast<unsigned long long>(c->barrier_seq - 1), c->rank);
            std::remove((c->id_file + suffix).c_str());
        }
    }
    delete c;
    return MGT_OK;
}

}  // extern "C"
