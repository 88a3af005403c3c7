// Thin inline-PTX wrappers for sm_100a: mbarrier (bounded waits), TMA tiled loads,
// tcgen05 (TMEM allocation, UMMA issue, commit, TMEM loads) and the descriptor encodings.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mgt {
namespace ptx {

// Device-side error codes written to the engine's status word when a bounded wait gives up.
enum DeviceAbort : int {
    kAbortNone = 0,
    kAbortProducerWait = 1,
    kAbortMmaWait = 2,
    kAbortEpilogueWait = 3,
    kAbortSynthWait = 4,
    kAbortPeerWait = 5,
    kAbortChainWait = 6,
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Every wait in the kernels is bounded: after kWaitLimitNs without progress the waiter raises the
// CTA-wide abort word (shared memory) and returns false; all roles then leave their loops, let the
// copies already in flight land, free TMEM and return. The host reads the status word afterwards.
constexpr uint64_t kWaitLimitNs = 1000ULL * 1000ULL * 1000ULL;

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* cta_abort, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63U) == 0U) {
            if (*cta_abort != 0) return false;
            if (global_timer_ns() - start > kWaitLimitNs) {
                *cta_abort = code;
                return false;
            }
        }
    }
    return true;
}

// The same bound, but polling with the non-suspending test_wait: for hand-overs on a latency-critical chain,
// where the time try_wait may take to resume a waiter matters.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, volatile int* cta_abort, int code) {
    if (mbar_test_wait(bar, parity)) return true;
    const uint64_t start = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_test_wait(bar, parity)) {
        if ((++spins & 1023U) == 0U) {
            if (*cta_abort != 0) return false;
            if (global_timer_ns() - start > kWaitLimitNs) {
                *cta_abort = code;
                return false;
            }
        }
    }
    return true;
}

// Named barrier over `threads` threads (a multiple of 32); id 0 is __syncthreads' own barrier.
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// Barrier plus AND-reduction of a predicate: every participant receives the same answer.
__device__ __forceinline__ bool named_bar_and(uint32_t id, uint32_t threads, bool pred) {
    uint32_t out;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 p, %3, 0;\n\t"
        "bar.red.and.pred q, %1, %2, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(out)
        : "r"(id), "r"(threads), "r"(static_cast<uint32_t>(pred))
        : "memory");
    return out != 0;
}

__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void prefetch_tensormap(const void* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tiled TMA load into this CTA's shared memory (never multicast), completion on an mbarrier.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* map, int32_t x, int32_t y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// The same for a 3-D tensor (x innermost): used when one descriptor spans a stack of equally shaped matrices.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* map, int32_t x, int32_t y, int32_t z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// 3-D tiled TMA store from this CTA's shared memory (bulk-group completion); rows/columns outside the tensor are clipped.
__device__ __forceinline__ void tma_store_3d(const void* map, const void* smem_src, int32_t x, int32_t y, int32_t z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all bulk stores of this thread have finished READING shared memory / have completed
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---- tcgen05 / TMEM -------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_holder, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_holder)), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], fp16 inputs, fp32 accumulate, issued by ONE thread.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the mbarrier once every UMMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives lane (base_lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// The reverse: thread t of the warp writes its 32 values to lane (base_lane + t), 32 consecutive columns.
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
          "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
          "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- descriptors ----------------------------------------------------------------------------
// Shared-memory matrix descriptor (64-bit): start address >> 4 in bits [0,14), leading byte
// offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), descriptor version 1 in [46,48),
// layout type in [61,64) with 2 = 128-byte swizzle.
//  K-major 128B swizzle : rows of 128 bytes (64 halfs of K), 8-row groups SBO bytes apart; LBO unused.
//  MN-major 128B swizzle: K-rows of 128 bytes (64 halfs of M/N), 8-K-row groups SBO bytes apart,
//                         64-element M/N groups LBO bytes apart.
__host__ __device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFU);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFU) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFU) << 32;
    d |= 1ULL << 46;
    d |= 2ULL << 61;
    return d;
}

// Instruction descriptor for kind::f16 with fp16 A/B and fp32 accumulator:
// c_format(F32=1) bits [4,6), a_format/b_format (F16=0) bits [7,10)/[10,13), a_major bit 15,
// b_major bit 16 (0 = K-major, 1 = MN-major), N>>3 in bits [17,23), M>>4 in bits [24,29).
// bf16: both operands bfloat16 (format code 1) instead of fp16 (format code 0); the accumulator stays fp32.
__host__ __device__ constexpr uint32_t make_idesc_f16(uint32_t m, uint32_t n, bool a_mn_major, bool b_mn_major, bool bf16 = false) {
    return (1U << 4) | ((bf16 ? 1U : 0U) << 7) | ((bf16 ? 1U : 0U) << 10) | ((a_mn_major ? 1U : 0U) << 15) | ((b_mn_major ? 1U : 0U) << 16) |
           ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---- 16-bit operand formats -------------------------------------------------------------------
// The reference computes with fp16 operands; bfloat16 is this library's option. Both round to nearest even.
__device__ __forceinline__ uint32_t pack_operand_pair(float lo, float hi, bool bf16) {
    if (bf16) {
        const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&p);
    }
    const __half2 p = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&p);
}
__device__ __forceinline__ uint16_t to_operand(float x, bool bf16) {
    if (bf16) return __bfloat16_as_ushort(__float2bfloat16_rn(x));
    return __half_as_ushort(__float2half_rn(x));
}
__device__ __forceinline__ float from_operand(uint16_t bits, bool bf16) {
    if (bf16) return __uint_as_float(static_cast<uint32_t>(bits) << 16);
    return __half2float(__ushort_as_half(bits));
}
__device__ __forceinline__ uint16_t operand_one(bool bf16) { return bf16 ? 0x3F80 : 0x3C00; }

}  // namespace ptx
}  // namespace mgt
