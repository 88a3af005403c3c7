// Loss + gradient engine: forward, MSE loss and backward of the residual MLP on tcgen05 tensor
// cores, behind the C ABI of include/mgt_b200.h. Follows the data flow of the reference's fp16
// path (native/cuda/mlp_backward.cu:1228-1510): fp16 operands rounded at the same tensors, fp32
// accumulation, fp32 master biases for the hidden/residual layers, fp16 mirror for the embedding
// table and its bias. What differs is how it is computed:
//   * the embedding layer and its gradient are one-hot GEMMs whose one-hot operand is synthesised
//     in shared memory from the 80-byte states (never materialised in HBM);
//   * bias, ReLU, residual add, ReLU-mask and the fp16 down-cast are epilogues of the GEMMs;
//   * bias gradients are fp32 column sums taken in the epilogue that produces each dz tensor
//     (the reference sums the fp32 dz, not its fp16 copy: tiny gradients that underflow in fp16
//     still reach the bias), reduced over CTAs in a fixed order;
//   * activations are kept once (fp16 tape + one in-place fp32 residual stream).
#include "../../include/mgt_b200.h"
#include "batch_norm.cuh"
#include "fp32_path.cuh"
#include "tower_chain.cuh"
#include "umma_gemm.cuh"

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace mgt {
namespace {

// ---- flat parameter layout (native/cuda/mlp_backward.cu:25-36) -----------------------------
inline uint64_t BlockParams(const mgt_mlp_shape_t& s) { return 2ULL * ((uint64_t)s.hd2 * s.hd2 + s.hd2); }
inline uint64_t InputBias(const mgt_mlp_shape_t& s) { return (uint64_t)s.state_len * s.state_value_pad * s.hd1; }
inline uint64_t HiddenWeight(const mgt_mlp_shape_t& s) { return InputBias(s) + s.hd1; }
inline uint64_t HiddenBias(const mgt_mlp_shape_t& s) { return HiddenWeight(s) + (uint64_t)s.hd1 * s.hd2; }
inline uint64_t ResidualBase(const mgt_mlp_shape_t& s) { return HiddenBias(s) + s.hd2; }
inline uint64_t OutputWeight(const mgt_mlp_shape_t& s) { return ResidualBase(s) + (uint64_t)s.residual_blocks * BlockParams(s); }
inline uint64_t OutputBias(const mgt_mlp_shape_t& s) { return OutputWeight(s) + (uint64_t)s.hd2 * s.output_dim; }
inline uint64_t ParamCount(const mgt_mlp_shape_t& s) { return OutputBias(s) + s.output_dim; }
inline uint64_t Fc1W(const mgt_mlp_shape_t& s, uint32_t b) { return ResidualBase(s) + (uint64_t)b * BlockParams(s); }
inline uint64_t Fc1B(const mgt_mlp_shape_t& s, uint32_t b) { return Fc1W(s, b) + (uint64_t)s.hd2 * s.hd2; }
inline uint64_t Fc2W(const mgt_mlp_shape_t& s, uint32_t b) { return Fc1B(s, b) + s.hd2; }
inline uint64_t Fc2B(const mgt_mlp_shape_t& s, uint32_t b) { return Fc2W(s, b) + (uint64_t)s.hd2 * s.hd2; }

inline uint64_t RoundUp(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

bool ValidShape(const mgt_mlp_shape_t* s) {
    return s != nullptr && s->state_len > 0 && s->state_len <= MGT_STATE_LEN && s->state_value_pad > 0 &&
           s->state_value_pad <= MGT_STATE_VALUE_PAD && s->hd1 > 0 && s->hd1 <= MGT_MAX_HD1 && s->hd2 > 0 &&
           s->hd2 <= MGT_MAX_HD2 && s->residual_blocks <= MGT_MAX_RESIDUAL_BLOCKS && s->output_dim > 0;
}

// ---- workspace ------------------------------------------------------------------------------
// All offsets are in bytes from a 1024-byte aligned base inside the caller's float arena.
struct Workspace {
    uint32_t B, H1, H2, R, OUT, IN;
    uint32_t p_bt;    // pitch (halfs) of the tensors kept with one row per hd1 column (a1, dz1): samples rounded to 8
    uint64_t off_rowsum, rowsum_rows;  // partial row sums of the hidden layer's dX GEMM (input-bias gradient)
    uint64_t off_bits_h1;              // sign words of the embedding layer's pre-activation: [hd1][ld_bits_h1]
    uint32_t ld_bits_h1;
    uint32_t p_act;   // pitch (halfs) of x_h / r1_h, rounded to 8
    uint32_t p_dz;    // pitch (halfs) of dz tensors over H2
    uint32_t p_f32;   // pitch (floats) of the fp32 residual / gradient streams
    uint32_t p_w1, p_w2, p_wout;  // pitches of the internal fp16 weight copy
    uint64_t off_a1, off_x, off_r1, off_xf, off_dzf, off_dz2, off_dz1t, off_dz1, off_partial, off_head, off_wint, off_dy, off_dyh, off_colsum;
    uint64_t colsum_floats, colsum_slot_floats, dz_stride;
    uint64_t off_bits, bits_stride;  // ReLU sign bits of the residual tower: 2R+1 entries of bits_stride words
    uint64_t x_stride, r1_stride;  // bytes between consecutive blocks' tensors
    uint64_t partial_floats, head_blocks;
    // batch normalisation (only planned when it is on): fp32 pre-activations of the R+1 normalised layers, their saved
    // mean / rstd, partial sums of the reductions, the statistics vector when the caller gives no exchange buffer
    uint64_t off_bn_z, bn_z_stride, off_bn_save, off_bn_partial, off_bn_stats;
    uint64_t total_bytes;
};

constexpr uint32_t kHeadBlocks = 296;   // two CTAs per SM on a 148-SM part
constexpr uint32_t kHeadThreads = 256;

// The scratch for per-CTA partial sums is sized by the SM count: never below the B200's 148, so that the size the
// query reports (it has no engine, it asks the current device) covers the launch on any sm_100 part.
inline uint32_t PlanSmCount(int device_sms) { return device_sms > 148 ? static_cast<uint32_t>(device_sms) : 148U; }
inline uint32_t CurrentDeviceSmCount() {
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
        cudaGetLastError();
        return 148U;
    }
    return PlanSmCount(sms);
}

Workspace PlanWorkspace(const mgt_mlp_shape_t& s, uint32_t B, uint32_t sm_count, bool batch_norm = false) {
    Workspace w{};
    w.B = B; w.H1 = s.hd1; w.H2 = s.hd2; w.R = s.residual_blocks; w.OUT = s.output_dim;
    w.IN = s.state_len * s.state_value_pad;
    w.p_act = (uint32_t)RoundUp(s.hd2, 8);
    w.p_dz = (uint32_t)RoundUp(s.hd2, 8);
    w.p_bt = (uint32_t)RoundUp(B, 8);
    w.p_f32 = (uint32_t)RoundUp(s.hd2, 4);
    w.p_w1 = (uint32_t)RoundUp(s.hd1, 8);
    w.p_w2 = (uint32_t)RoundUp(s.hd2, 8);
    w.p_wout = (uint32_t)RoundUp(s.output_dim, 8);
    uint64_t off = 0;
    auto take = [&](uint64_t bytes) { const uint64_t o = off; off = RoundUp(off + bytes, 1024); return o; };
    // a1 and dz1 lie as [hd1][samples]: the way the two embedding GEMMs produce and consume them
    const uint64_t hidden_act_bytes = (uint64_t)s.hd1 * w.p_bt * 2;
    w.off_a1 = take(hidden_act_bytes);
    w.x_stride = RoundUp((uint64_t)B * w.p_act * 2, 1024);
    w.off_x = take(w.x_stride * (w.R + 1));
    w.r1_stride = w.x_stride;
    w.off_r1 = take(w.r1_stride * (w.R > 0 ? w.R : 1));
    w.off_xf = take((uint64_t)B * w.p_f32 * 4);
    w.off_dzf = take((uint64_t)B * w.p_f32 * 4);
    // gradients w.r.t. pre-activations, kept for the whole backward pass so that the weight gradients of all
    // residual blocks can be computed by two grouped GEMMs at the end: tape[0] belongs to the hidden layer,
    // tape[k+1] to fc2 of block k; dz1t[k] to fc1 of block k
    w.dz_stride = RoundUp((uint64_t)B * w.p_dz * 2, 1024);
    w.off_dz2 = take(w.dz_stride * (w.R + 1));
    w.off_dz1t = take(w.dz_stride * (w.R > 0 ? w.R : 1));
    w.off_dz1 = take(hidden_act_bytes);
    // split-K partials: at most one CTA wave of [128 x 256] fp32 tiles plus slack for tile padding
    const uint64_t hidden_units = (uint64_t)((s.hd1 + 127) / 128) * ((s.hd2 + 255) / 256);
    const uint64_t resid_units = (uint64_t)((s.hd2 + 127) / 128) * ((s.hd2 + 255) / 256);
    const uint64_t hidden_splits = hidden_units >= sm_count ? 1 : sm_count / hidden_units;
    const uint64_t resid_splits = resid_units >= sm_count ? 1 : sm_count / resid_units;
    const uint64_t p1 = hidden_splits * (uint64_t)s.hd1 * s.hd2;
    const uint64_t group_units = resid_units * (w.R > 0 ? w.R : 1);
    const uint64_t group_splits = group_units >= sm_count ? 1 : sm_count / group_units;
    const uint64_t p2 = group_splits * (w.R > 0 ? w.R : 1) * (uint64_t)s.hd2 * s.hd2;
    (void)resid_splits;
    w.partial_floats = p1 > p2 ? p1 : p2;
    w.off_partial = take(w.partial_floats * 4);
    w.head_blocks = kHeadBlocks;
    w.off_head = take((uint64_t)kHeadBlocks * (2ULL * s.hd2 + 2) * 4);
    // per-warp column sums: one slot per residual dX GEMM (2R of them)
    const uint64_t chain_tiles = (B + 127) / 128;
    const uint64_t slot_rows = (uint64_t)sm_count * 16 > chain_tiles * 4 ? (uint64_t)sm_count * 16 : chain_tiles * 4;  // up to 16 epilogue warps per CTA
    w.colsum_slot_floats = slot_rows * s.hd2;
    w.colsum_floats = w.colsum_slot_floats * 2 * (w.R > 0 ? w.R : 1);
    w.off_colsum = take(w.colsum_floats * 4);
    w.rowsum_rows = 2ULL * ((B + 255) / 256);  // two epilogue warps per lane quadrant, one N tile per 256 samples
    w.off_rowsum = take(w.rowsum_rows * s.hd1 * 4);
    w.ld_bits_h1 = (uint32_t)RoundUp((B + 31) / 32, 8);  // (32-byte rows)
    w.off_bits_h1 = take((uint64_t)s.hd1 * w.ld_bits_h1 * 4);
    w.bits_stride = chain_tiles * 128 * 8;
    w.off_bits = take(w.bits_stride * 4 * (2 * w.R + 1));
    // internal fp16 weight copy (used when the caller's mirror cannot be addressed by TMA as it lies)
    const uint64_t wint_halfs = (uint64_t)(w.IN + 1) * w.p_w1 + (uint64_t)s.hd1 * w.p_w2 + 2ULL * w.R * s.hd2 * w.p_w2 + (uint64_t)s.hd2 * w.p_wout;
    w.off_wint = take(wint_halfs * 2 + 1024ULL * (2 * w.R + 4));
    w.off_dy = take((uint64_t)B * s.output_dim * 4);
    w.off_dyh = take((uint64_t)B * w.p_wout * 2);
    if (batch_norm) {
        w.bn_z_stride = RoundUp((uint64_t)B * w.p_f32 * 4, 1024);
        w.off_bn_z = take(w.bn_z_stride * (w.R + 1));
        w.off_bn_save = take((uint64_t)(w.R + 1) * 2 * s.hd2 * 4);
        w.off_bn_partial = take((uint64_t)bn::kMaxBlocks * 2 * s.hd2 * 4);
        w.off_bn_stats = take(2ULL * s.hd2 * 4);
    }
    w.total_bytes = off + 1024;  // slack to align the caller's base
    return w;
}

// ---- engine -----------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct MapKey {
    const void* base;
    uint64_t inner, outer, pitch;
    uint32_t box_inner, box_outer;
    uint64_t layers = 0, layer_stride = 0;  // 3-D maps only
    bool operator==(const MapKey& o) const {
        return base == o.base && inner == o.inner && outer == o.outer && pitch == o.pitch && box_inner == o.box_inner && box_outer == o.box_outer &&
               layers == o.layers && layer_stride == o.layer_stride;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        uint64_t h = reinterpret_cast<uint64_t>(k.base);
        auto mix = [&](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ULL + (h << 6) + (h >> 2); };
        mix(k.inner); mix(k.outer); mix(k.pitch); mix(k.box_inner); mix(k.box_outer); mix(k.layers); mix(k.layer_stride);
        return (size_t)h;
    }
};

}  // namespace
}  // namespace mgt

struct mgt_engine {
    int device = 0;
    int sm_count = 148;
    int* status_word = nullptr;  // device
    mgt::EncodeTiledFn encode = nullptr;
    std::unordered_map<mgt::MapKey, CUtensorMap, mgt::MapKeyHash> maps;
    std::mutex mu;
    cudaEvent_t ev_last = nullptr, ev_now = nullptr;
    uint64_t launches = 0;  // kernels launched through this engine (host-side count)
    bool layered_tower = false;  // MGT_RESIDUAL_PATH=layered: per-layer GEMMs instead of the fused residual-tower kernels (both are tested)
    mgt_gradient_ready_fn early_fn = nullptr;  // mgt_engine_set_early_range_hook
    void* early_user = nullptr;
    mgt_train_options_t options{MGT_OPERAND_FP16, MGT_LOSS_MSE, 0, 1.0e-5f};  // mgt_engine_set_train_options
    // mgt_engine_set_batch_norm_state
    float* bn_running = nullptr;
    float bn_momentum = 0.1f;
    uint32_t bn_world = 1;
    float* bn_exchange_buffer = nullptr;
    mgt_stats_exchange_fn bn_exchange = nullptr;
    void* bn_exchange_user = nullptr;
    bool bf16_now = false;  // operand format of the launch being enqueued (set by mgt_launch_mlp_loss_grad, off otherwise)

    // fp16 3-D tensor map (a stack of `layers` equal matrices `layer_stride_bytes` apart), 128-byte swizzle, box depth 1
    bool Map3D(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t layers, uint64_t pitch_elems, uint64_t layer_stride_bytes,
               uint32_t box_inner, uint32_t box_outer) {
        mgt::MapKey key{base, inner, outer, pitch_elems, box_inner, box_outer};
        key.layers = layers;
        key.layer_stride = layer_stride_bytes;
        std::lock_guard<std::mutex> lock(mu);
        auto it = maps.find(key);
        if (it != maps.end()) { *out = it->second; return true; }
        if ((reinterpret_cast<uintptr_t>(base) & 15U) != 0 || ((pitch_elems * 2) & 15U) != 0 || (layer_stride_bytes & 15U) != 0 || box_inner * 2 > 128 || box_outer > 256) return false;
        const cuuint64_t dims[3] = {inner, outer, layers};
        const cuuint64_t strides[2] = {pitch_elems * 2, layer_stride_bytes};
        const cuuint32_t box[3] = {box_inner, box_outer, 1};
        const cuuint32_t elem[3] = {1, 1, 1};
        CUtensorMap m;
        const CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return false;
        if (maps.size() > 4096) maps.clear();
        maps.emplace(key, m);
        *out = m;
        return true;
    }

    // fp16 2-D tensor map with 128-byte swizzle: `inner` contiguous elements per row, `outer` rows.
    bool Map(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch_elems, uint32_t box_inner, uint32_t box_outer) {
        const mgt::MapKey key{base, inner, outer, pitch_elems, box_inner, box_outer};
        std::lock_guard<std::mutex> lock(mu);
        auto it = maps.find(key);
        if (it != maps.end()) { *out = it->second; return true; }
        if ((reinterpret_cast<uintptr_t>(base) & 15U) != 0 || ((pitch_elems * 2) & 15U) != 0 || box_inner * 2 > 128 || box_outer > 256) return false;
        const cuuint64_t dims[2] = {inner, outer};
        const cuuint64_t strides[1] = {pitch_elems * 2};
        const cuuint32_t box[2] = {box_inner, box_outer};
        const cuuint32_t elem[2] = {1, 1};
        CUtensorMap m;
        const CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return false;
        if (maps.size() > 4096) maps.clear();
        maps.emplace(key, m);
        *out = m;
        return true;
    }
};

namespace mgt {
namespace {

template <class Cfg>
mgt_status_t LaunchGemm(mgt_engine* e, const CUtensorMap& ta, const CUtensorMap& tb, GemmArgs args, cudaStream_t stream) {
    // the opt-in shared-memory size is a per-device attribute of each kernel instantiation
    static std::mutex attr_mu;
    static bool attr_done[64] = {};
    if (e->device < 0 || e->device >= 64) return MGT_INVALID_CONFIG;
    {
        std::lock_guard<std::mutex> lock(attr_mu);
        if (!attr_done[e->device]) {
            if (cudaFuncSetAttribute(umma_gemm_kernel<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) return MGT_CUDA_FAILURE;
            attr_done[e->device] = true;
        }
    }
    const uint64_t units = (uint64_t)args.m_tiles * args.n_tiles * args.splits * (Cfg::GROUPED ? args.groups : 1U);
    if (units == 0) return MGT_INVALID_CONFIG;
    uint32_t grid = (uint32_t)(units < (uint64_t)e->sm_count ? units : (uint64_t)e->sm_count);
    if (Cfg::BSTAT) {
        // every unit of a CTA must share the N tile: unit = mt * n_tiles + nt advances by the grid size
        if (args.splits != 1 || args.k_chunks > (uint32_t)Cfg::SB || args.n_tiles > (uint32_t)e->sm_count) return MGT_INVALID_CONFIG;
        if (grid >= args.n_tiles) grid = grid / args.n_tiles * args.n_tiles;
    }
    args.status = e->status_word;
    args.bf16 = e->bf16_now ? 1U : 0U;
    umma_gemm_kernel<Cfg><<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, args);
    ++e->launches;
    return cudaGetLastError() == cudaSuccess ? MGT_OK : MGT_CUDA_FAILURE;
}

// Tile configurations. BN = 224 serves the p888 residual width without padded MMA columns.
template <int BN, Epi EPI> using CfgFwd = GemmCfg<BN, 1, false, BSource::kTmaMN, EPI, 3, 3>;   // act[K-major] x W[K][N]
template <int BN, Epi EPI> using CfgDx = GemmCfg<BN, 1, false, BSource::kTmaK, EPI, 3, 3>;     // dz[K-major] x W[N][K]
// B-stationary forms for reductions of at most 256 (the residual width): weights stay in shared memory
template <int BN, Epi EPI> using CfgFwdS = GemmCfg<BN, 1, false, BSource::kTmaMN, EPI, 3, 4, true>;
template <int BN, Epi EPI> using CfgDxS = GemmCfg<BN, 1, false, BSource::kTmaK, EPI, 3, 4, true>;
template <int BN> using CfgDw = GemmCfg<BN, 1, true, BSource::kTmaMN, Epi::kPartialF32, 3, 3>; // act^T x dz
// The hidden layer with its wide side (hd1) as rows: a1 and dz1 are kept as [hd1][samples], the way the two embedding GEMMs
// produce and consume them, so that their epilogues and the hidden dX epilogue move 64 contiguous bytes per lane
template <int BN, Epi EPI> using CfgFwdRows = GemmCfg<BN, 1, true, BSource::kTmaMN, EPI, 3, 3>;        // a1T[K][M] x W[K][N]
template <int BN> using CfgDwRows = GemmCfg<BN, 1, false, BSource::kTmaMN, Epi::kPartialF32, 3, 3>;    // a1T[M][K] x dz[K][N]
using CfgDxRows = GemmCfg<256, 1, false, BSource::kTmaK, Epi::kMaskRowsumF16, 4, 4>;                   // W[M][K] x dz[N][K] -> dz1T[M][N]
template <int BN> using CfgDwG = GemmCfg<BN, 1, true, BSource::kTmaMN, Epi::kPartialF32, 3, 3, false, true>; // R stacked act^T x dz
// Two 256-column accumulators per unit (all of TMEM) and a two-stage one-hot ring. Measured alternatives at p888: 2 x 192
// columns with a three-stage ring 1.44 ms, one double-buffered 256-column accumulator (epilogue under the next unit's
// MMAs, but the table tile re-read twice as often) 1.37 ms, this form 1.14 ms: the K loop already issues MMAs back to back.
using CfgEmbFwd = GemmCfg<256, 2, true, BSource::kOneHotFwd, Epi::kEmbFwdRows, 4, 2>;   // table[K][M] x onehot -> a1T[M][N]
using CfgEmbGrad = GemmCfg<256, 2, false, BSource::kOneHotGrad, Epi::kEmbGrad, 4, 2>;    // dz1T[M][K] x onehot -> grad[N][M]
// (One accumulator per unit with two units in flight - the epilogue of one draining under the MMAs of the next, operand
// ring four deep - was measured at p888: forward 1.40 ms against 1.22 ms, gradient 1.56 ms against 1.13 ms. A K chunk
// costs about a thousand cycles in hand-overs whatever it feeds, so it should feed eight MMAs, not four.)
using CfgDbgKK = GemmCfg<256, 1, false, BSource::kTmaK, Epi::kPartialF32, 3, 3>;
using CfgDbgKM = GemmCfg<256, 1, false, BSource::kTmaMN, Epi::kPartialF32, 3, 3>;
using CfgDbgMK = GemmCfg<256, 1, true, BSource::kTmaK, Epi::kPartialF32, 3, 3>;

inline uint32_t PickBN(uint32_t n) { return n <= 224 ? 224U : 256U; }

GemmArgs BaseArgs(uint32_t M, uint32_t N, uint32_t K, uint32_t bn_total, uint32_t splits) {
    GemmArgs a{};
    a.M = M; a.N = N; a.K = K;
    a.m_tiles = (M + 127) / 128;
    a.n_tiles = (N + bn_total - 1) / bn_total;
    a.k_chunks = (K + 63) / 64;
    a.groups = 1;
    a.splits = splits < 1 ? 1 : (splits > a.k_chunks ? a.k_chunks : splits);
    return a;
}

// ---- small kernels ------------------------------------------------------------------------------

// fp32 [rows][cols] (pitch src_pitch) -> fp16 or bfloat16 [rows][dst_pitch], round-to-nearest-even.
__global__ void RepackHalfKernel(const float* __restrict__ src, uint32_t rows, uint32_t cols, uint32_t src_pitch, __half* __restrict__ dst, uint32_t dst_pitch,
                                 bool bf16) {
    const uint64_t total = (uint64_t)rows * cols;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    uint16_t* out = reinterpret_cast<uint16_t*>(dst);
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint32_t r = (uint32_t)(i / cols), c = (uint32_t)(i - (uint64_t)r * cols);
        out[(uint64_t)r * dst_pitch + c] = ptx::to_operand(src[(uint64_t)r * src_pitch + c], bf16);
    }
}

// grad[i] = sum over splits (fixed order) of partial[split][i]; loads of eight splits are in flight at once
__global__ void __launch_bounds__(256)
ReducePartialsKernel(const float* __restrict__ partial, uint32_t splits, uint64_t count, float* __restrict__ out) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        float sum = partial[i];
        uint32_t s = 1;
        for (; s + 8U <= splits; s += 8U) {
            float x[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) x[q] = partial[(uint64_t)(s + q) * count + i];
#pragma unroll
            for (int q = 0; q < 8; ++q) sum += x[q];
        }
        for (; s < splits; ++s) sum += partial[(uint64_t)s * count + i];
        out[i] = sum;
    }
}

// dst[c] = sum over rows r of src[r * row_stride + col_offset + c], in a fixed order: each of 32 row
// groups adds its rows (r = g, g+32, ...) and the groups are then added 0..31. One CTA per 8 columns,
// so that a few-hundred-column reduction still spreads over dozens of SMs.
constexpr uint32_t kReduceCols = 8;
__global__ void __launch_bounds__(256)
ReduceRowsKernel(const float* __restrict__ src, uint32_t rows, uint64_t row_stride, uint32_t col_offset, uint32_t cols, float* __restrict__ dst) {
    __shared__ float s_part[32][kReduceCols + 1];
    const uint32_t cl = threadIdx.x & (kReduceCols - 1U), g = threadIdx.x / kReduceCols;
    const uint32_t c = blockIdx.x * kReduceCols + cl;
    float sum = 0.0f;
    if (c < cols) {
        const float* p = src + col_offset + c;
        uint32_t r = g;
        for (; r + 96U < rows; r += 128U) {
            const float a0 = p[(uint64_t)r * row_stride];
            const float a1 = p[(uint64_t)(r + 32U) * row_stride];
            const float a2 = p[(uint64_t)(r + 64U) * row_stride];
            const float a3 = p[(uint64_t)(r + 96U) * row_stride];
            sum += a0; sum += a1; sum += a2; sum += a3;
        }
        for (; r < rows; r += 32U) sum += p[(uint64_t)r * row_stride];
    }
    s_part[g][cl] = sum;
    __syncthreads();
    if (g == 0 && c < cols) {
        float total = s_part[0][cl];
#pragma unroll
        for (int q = 1; q < 32; ++q) total += s_part[q][cl];
        dst[c] = total;
    }
}

// The three reductions behind HeadOut1Kernel in one launch: items [0, H2] -> grad W_out and grad b_out (contiguous in the
// parameter layout), item H2 + 1 -> the loss, items [H2 + 2, 2 H2 + 2) -> the bias gradient of the layer below the head.
// Same thread-to-row assignment and order of additions as ReduceRowsKernel.
__global__ void __launch_bounds__(256)
ReduceHeadKernel(const float* __restrict__ src, uint32_t rows, uint32_t H2, float* __restrict__ grad_out_layer, float* __restrict__ loss,
                 float* __restrict__ bias_below) {
    __shared__ float s_part[32][kReduceCols + 1];
    const uint32_t items = 2U * H2 + 2U;
    const uint32_t cl = threadIdx.x & (kReduceCols - 1U), g = threadIdx.x / kReduceCols;
    const uint32_t c = blockIdx.x * kReduceCols + cl;
    float sum = 0.0f;
    if (c < items) {
        const float* p = src + c;
        uint32_t r = g;
        for (; r + 96U < rows; r += 128U) {
            const float a0 = p[(uint64_t)r * items];
            const float a1 = p[(uint64_t)(r + 32U) * items];
            const float a2 = p[(uint64_t)(r + 64U) * items];
            const float a3 = p[(uint64_t)(r + 96U) * items];
            sum += a0; sum += a1; sum += a2; sum += a3;
        }
        for (; r < rows; r += 32U) sum += p[(uint64_t)r * items];
    }
    s_part[g][cl] = sum;
    __syncthreads();
    if (g == 0 && c < items) {
        float total = s_part[0][cl];
#pragma unroll
        for (int q = 1; q < 32; ++q) total += s_part[q][cl];
        if (c <= H2) grad_out_layer[c] = total;
        else if (c == H2 + 1U) *loss = total;
        else bias_below[c - H2 - 2U] = total;
    }
}

// The two reducers above for a stack of problems: blockIdx.y selects the problem.
__global__ void __launch_bounds__(256)
ReducePartialsGroupedKernel(const float* __restrict__ partial, uint32_t splits, uint64_t count, float* __restrict__ out, uint64_t out_group_stride) {
    const float* src = partial + (uint64_t)blockIdx.y * splits * count;
    float* dst = out + (uint64_t)blockIdx.y * out_group_stride;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        float sum = src[i];
        for (uint32_t s = 1; s < splits; ++s) sum += src[(uint64_t)s * count + i];
        dst[i] = sum;
    }
}

struct ReduceDestinations { uint64_t offset[2 * MGT_MAX_RESIDUAL_BLOCKS]; };  // element offsets into the gradient array

__global__ void __launch_bounds__(256)
ReduceRowsGroupedKernel(const float* __restrict__ src, uint32_t rows, uint32_t cols, uint64_t slot_stride, float* __restrict__ grad, ReduceDestinations dst) {
    __shared__ float s_part[32][kReduceCols + 1];
    const uint32_t cl = threadIdx.x & (kReduceCols - 1U), g = threadIdx.x / kReduceCols;
    const uint32_t c = blockIdx.x * kReduceCols + cl;
    float sum = 0.0f;
    if (c < cols) {
        const float* p = src + (uint64_t)blockIdx.y * slot_stride + c;
        uint32_t r = g;
        for (; r + 96U < rows; r += 128U) {
            const float a0 = p[(uint64_t)r * cols];
            const float a1 = p[(uint64_t)(r + 32U) * cols];
            const float a2 = p[(uint64_t)(r + 64U) * cols];
            const float a3 = p[(uint64_t)(r + 96U) * cols];
            sum += a0; sum += a1; sum += a2; sum += a3;
        }
        for (; r < rows; r += 32U) sum += p[(uint64_t)r * cols];
    }
    s_part[g][cl] = sum;
    __syncthreads();
    if (g == 0 && c < cols) {
        float total = s_part[0][cl];
#pragma unroll
        for (int q = 1; q < 32; ++q) total += s_part[q][cl];
        grad[dst.offset[blockIdx.y] + c] = total;
    }
}

// Output head for output_dim == 1 (native/cuda/mlp_backward.cu:891-931): y = b + <x, w> with fp32
// master weights, diff, dy = 2 diff / B, loss term diff^2 / B, dcur = w * dy, then the ReLU mask of
// the last block. One warp per sample (grid-stride); per-CTA partial sums go to
// partials[CTA][2*H2+2] = { grad W_out[H2], grad b_out, loss, column sums of dz[H2] } and are added
// in a fixed order by ReduceRowsKernel.
constexpr int kHeadMaxPerLane = MGT_MAX_HD2 / 32;
constexpr size_t kHeadStagedSmemLimit = 160U * 1024U;  // dynamic shared memory of HeadOutNKernel with staged weights (two CTAs per SM at up to 96 KB)
__global__ void __launch_bounds__(kHeadThreads)
HeadOut1Kernel(const float* __restrict__ w_out, const float* __restrict__ b_out, const float* __restrict__ labels, const float* __restrict__ x,
               uint32_t p_f32, uint32_t B, uint32_t H2, float* __restrict__ dzf, __half* __restrict__ dz_h, uint32_t p_dz, float* __restrict__ partials,
               bool bf16) {
    __shared__ float s_acc[kHeadThreads / 32][2 * MGT_MAX_HD2 + 2];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31U;
    const uint32_t warps_total = gridDim.x * (kHeadThreads / 32);
    const float inv_n = 1.0f / static_cast<float>(B);
    const float bias = *b_out;
    float wreg[kHeadMaxPerLane], gacc[kHeadMaxPerLane], dacc[kHeadMaxPerLane];
#pragma unroll
    for (int q = 0; q < kHeadMaxPerLane; ++q) {
        const uint32_t j = q * 32 + lane;
        wreg[q] = j < H2 ? w_out[j] : 0.0f;
        gacc[q] = 0.0f;
        dacc[q] = 0.0f;
    }
    float gb = 0.0f, loss = 0.0f;
    // The row and the label of the warp's next sample are fetched before the current one is worked on: one sample is a
    // chain of load -> five shuffles -> stores, and a warp that waits for each load in turn leaves HBM idle.
    float xn[kHeadMaxPerLane], label_next = 0.0f;
    auto fetch = [&](uint32_t b) {
        const float* row = x + (uint64_t)b * p_f32;
#pragma unroll
        for (int q = 0; q < kHeadMaxPerLane; ++q) {
            const uint32_t j = q * 32 + lane;
            xn[q] = (b < B && j < H2) ? row[j] : 0.0f;
        }
        label_next = b < B ? labels[b] : 0.0f;
    };
    fetch(blockIdx.x * (kHeadThreads / 32) + warp);
    for (uint32_t b = blockIdx.x * (kHeadThreads / 32) + warp; b < B; b += warps_total) {
        float xv[kHeadMaxPerLane];
        const float label = label_next;
        float dot = 0.0f;
#pragma unroll
        for (int q = 0; q < kHeadMaxPerLane; ++q) {
            xv[q] = xn[q];
            dot += xv[q] * wreg[q];
        }
        fetch(b + warps_total);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFU, dot, o);
        const float diff = (bias + dot) - label;
        const float dy = 2.0f * diff * inv_n;
        if (lane == 0) { gb += dy; loss += diff * diff * inv_n; }
#pragma unroll
        for (int q = 0; q < kHeadMaxPerLane; ++q) {
            const uint32_t j = q * 32 + lane;
            if (j < H2) {
                gacc[q] += xv[q] * dy;
                const float d = xv[q] > 0.0f ? wreg[q] * dy : 0.0f;
                dacc[q] += d;
                dzf[(uint64_t)b * p_f32 + j] = d;
                reinterpret_cast<uint16_t*>(dz_h)[(uint64_t)b * p_dz + j] = ptx::to_operand(d, bf16);
            }
        }
    }
#pragma unroll
    for (int q = 0; q < kHeadMaxPerLane; ++q) {
        const uint32_t j = q * 32 + lane;
        if (j < H2) { s_acc[warp][j] = gacc[q]; s_acc[warp][H2 + 2 + j] = dacc[q]; }
    }
    if (lane == 0) { s_acc[warp][H2] = gb; s_acc[warp][H2 + 1] = loss; }
    __syncthreads();
    for (uint32_t j = threadIdx.x; j < 2 * H2 + 2; j += kHeadThreads) {
        float sum = 0.0f;
        for (int wi = 0; wi < kHeadThreads / 32; ++wi) sum += s_acc[wi][j];
        partials[(uint64_t)blockIdx.x * (2 * H2 + 2) + j] = sum;
    }
}

// Output head for output_dim > 1 (native/cuda/mlp_backward.cu:1341-1363): 16-bit operands, fp32 accumulate, dy rounded to
// the operand format for the two products that follow. kCrossEntropy = false: the reference's MSE against the labels.
// kCrossEntropy = true (no counterpart in the reference): the outputs are per-depth logits, class = depth - 1 (the labels
// carry the walk depth in every output slot), loss = mean over the batch of -log softmax(y)[class],
// dy = (softmax(y) - onehot(class)) / B. One warp per sample, plain SIMT (B x OUT x H2 multiply-adds twice). kStageW: the
// output weights are converted once per CTA into shared memory ([H2][OUT | 1] floats: rows for the forward product, a
// lane per row without bank conflicts for the backward one); read from global memory instead, the lane-per-row access of
// the backward product touches 32 sectors per instruction and the kernel is bound by L2 (5.4 ms instead of 0.5 ms at
// batch 131072, hd2 512, 29 outputs).
template <bool kCrossEntropy, bool kStageW>
__global__ void __launch_bounds__(kHeadThreads)
HeadOutNKernel(const __half* __restrict__ w_out_h, uint32_t p_wout, const float* __restrict__ b_out, const float* __restrict__ labels,
               const __half* __restrict__ x_h, uint32_t p_act, const float* __restrict__ x_f32, uint32_t p_f32, uint32_t B, uint32_t H2, uint32_t OUT,
               float* __restrict__ dy, __half* __restrict__ dy_h, uint32_t p_dy, float* __restrict__ dzf, __half* __restrict__ dz_h, uint32_t p_dz,
               float* __restrict__ partials, bool bf16) {
    extern __shared__ float s_dyn[];  // per warp: OUT floats (logits, then rounded dy); then the staged weights
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31U;
    const uint32_t warps_total = gridDim.x * (kHeadThreads / 32);
    float* s_dy = s_dyn + warp * OUT;
    const uint16_t* wq = reinterpret_cast<const uint16_t*>(w_out_h);
    const uint32_t outp = OUT | 1U;
    float* w_s = s_dyn + (kHeadThreads / 32) * OUT;
    if (kStageW) {
        for (uint32_t i = threadIdx.x; i < H2 * OUT; i += kHeadThreads) {
            const uint32_t j = i / OUT, o = i % OUT;
            w_s[j * outp + o] = ptx::from_operand(wq[(uint64_t)j * p_wout + o], bf16);
        }
        __syncthreads();
    }
    auto weight = [&](uint32_t j, uint32_t o) -> float { return kStageW ? w_s[j * outp + o] : ptx::from_operand(wq[(uint64_t)j * p_wout + o], bf16); };
    const float inv_n = 1.0f / static_cast<float>(kCrossEntropy ? (uint64_t)B : (uint64_t)B * OUT);
    float loss = 0.0f;
    float dacc[kHeadMaxPerLane];
#pragma unroll
    for (int q = 0; q < kHeadMaxPerLane; ++q) dacc[q] = 0.0f;
    for (uint32_t b = blockIdx.x * (kHeadThreads / 32) + warp; b < B; b += warps_total) {
        const uint16_t* row = reinterpret_cast<const uint16_t*>(x_h) + (uint64_t)b * p_act;
        float mx = -3.0e38f;
        for (uint32_t o = lane; o < OUT; o += 32) {
            float acc = 0.0f;
            for (uint32_t j = 0; j < H2; ++j) acc += ptx::from_operand(row[j], bf16) * weight(j, o);
            const float y = acc + b_out[o];
            s_dy[o] = y;
            mx = fmaxf(mx, y);
        }
        float log_sum = 0.0f;
        uint32_t cls = 0;
        if (kCrossEntropy) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFU, mx, o));
            __syncwarp();
            float sum = 0.0f;
            for (uint32_t o = lane; o < OUT; o += 32) sum += expf(s_dy[o] - mx);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFU, sum, o);
            log_sum = logf(sum) + mx;
            // a depth outside 1..OUT cannot come from the walk generator with k_max <= OUT; clamp instead of reading out of bounds
            const int c = __float2int_rn(labels[(uint64_t)b * OUT]) - 1;
            cls = static_cast<uint32_t>(c < 0 ? 0 : (c >= static_cast<int>(OUT) ? static_cast<int>(OUT) - 1 : c));
        }
        for (uint32_t o = lane; o < OUT; o += 32) {
            const float y = s_dy[o];
            float d;
            if (kCrossEntropy) {
                d = (expf(y - log_sum) - (o == cls ? 1.0f : 0.0f)) * inv_n;
                if (o == cls) loss += (log_sum - y) * inv_n;
            } else {
                const float diff = y - labels[(uint64_t)b * OUT + o];
                d = 2.0f * diff * inv_n;
                loss += diff * diff * inv_n;
            }
            dy[(uint64_t)b * OUT + o] = d;
            const uint16_t dh = ptx::to_operand(d, bf16);
            reinterpret_cast<uint16_t*>(dy_h)[(uint64_t)b * p_dy + o] = dh;
            s_dy[o] = ptx::from_operand(dh, bf16);
        }
        __syncwarp();
#pragma unroll
        for (int q = 0; q < kHeadMaxPerLane; ++q) {
            const uint32_t j = q * 32 + lane;
            if (j < H2) {
                float acc = 0.0f;
                for (uint32_t o = 0; o < OUT; ++o) acc += s_dy[o] * weight(j, o);
                const float d = x_f32[(uint64_t)b * p_f32 + j] > 0.0f ? acc : 0.0f;
                dacc[q] += d;
                dzf[(uint64_t)b * p_f32 + j] = d;
                reinterpret_cast<uint16_t*>(dz_h)[(uint64_t)b * p_dz + j] = ptx::to_operand(d, bf16);
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) loss += __shfl_xor_sync(0xFFFFFFFFU, loss, o);
    __shared__ float s_part[kHeadThreads / 32][MGT_MAX_HD2 + 1];
    if (lane == 0) s_part[warp][0] = loss;
#pragma unroll
    for (int q = 0; q < kHeadMaxPerLane; ++q) {
        const uint32_t j = q * 32 + lane;
        if (j < H2) s_part[warp][1 + j] = dacc[q];
    }
    __syncthreads();
    for (uint32_t j = threadIdx.x; j < H2 + 1; j += kHeadThreads) {
        float sum = 0.0f;
        for (int wi = 0; wi < kHeadThreads / 32; ++wi) sum += s_part[wi][j];
        partials[(uint64_t)blockIdx.x * (H2 + 1) + j] = sum;
    }
}

// grad b_out[o] = sum_b dy[b][o]: one CTA per output, rows dealt to the threads and added in a fixed tree.
__global__ void __launch_bounds__(256)
HeadOutNBiasGradKernel(const float* __restrict__ dy, uint32_t B, uint32_t OUT, float* __restrict__ grad_b) {
    __shared__ float s_sum[256];
    const uint32_t o = blockIdx.x;
    float sum = 0.0f;
    for (uint32_t b = threadIdx.x; b < B; b += 256U) sum += dy[(uint64_t)b * OUT + o];
    s_sum[threadIdx.x] = sum;
    __syncthreads();
    for (uint32_t w = 128U; w > 0U; w >>= 1) {
        if (threadIdx.x < w) s_sum[threadIdx.x] += s_sum[threadIdx.x + w];
        __syncthreads();
    }
    if (threadIdx.x == 0) grad_b[o] = s_sum[0];
}

inline uint32_t GridFor(uint64_t items, uint32_t threads, int sm_count) {
    const uint64_t want = (items + threads - 1) / threads;
    const uint64_t cap = (uint64_t)sm_count * 8;
    return (uint32_t)(want < 1 ? 1 : (want < cap ? want : cap));
}

struct StageTimer {
    mgt_engine* e;
    cudaStream_t stream;
    mgt_backward_profile_t* profile;
    bool Start() {
        if (!profile) return true;
        std::memset(profile, 0, sizeof(*profile));
        if (!e->ev_last && cudaEventCreate(&e->ev_last) != cudaSuccess) return false;
        if (!e->ev_now && cudaEventCreate(&e->ev_now) != cudaSuccess) return false;
        return cudaEventRecord(e->ev_last, stream) == cudaSuccess;
    }
    // As in the reference, every mark synchronises the host (native/cuda/mlp_backward.cu:211-221).
    bool Mark(float* dst) {
        if (!profile) return true;
        float ms = 0.0f;
        if (cudaEventRecord(e->ev_now, stream) != cudaSuccess) return false;
        if (cudaEventSynchronize(e->ev_now) != cudaSuccess) return false;
        if (cudaEventElapsedTime(&ms, e->ev_last, e->ev_now) != cudaSuccess) return false;
        *dst += ms;  // a stage may be visited twice (its dX part and, later, its dW part): Start() zeroed the profile
        std::swap(e->ev_last, e->ev_now);
        return true;
    }
};

#define MGT_TRY(...)                          \
    do {                                      \
        const mgt_status_t _st = (__VA_ARGS__); \
        if (_st != MGT_OK) return _st;        \
    } while (0)
#define MGT_MAP(...)                               \
    do {                                           \
        if (!(__VA_ARGS__)) return MGT_CUDA_FAILURE; \
    } while (0)

// D = act[M x K, K-major] * W[K x N, row-major] with a forward epilogue.
template <Epi EPI>
mgt_status_t GemmForward(mgt_engine* e, cudaStream_t st, const __half* act, uint32_t act_pitch, const __half* w, uint32_t w_pitch,
                         uint32_t M, uint32_t N, uint32_t K, GemmArgs epi) {
    const uint32_t bn = PickBN(N);
    GemmArgs a = BaseArgs(M, N, K, bn, 1);
    a.bias = epi.bias; a.out_f32 = epi.out_f32; a.ld_f32 = epi.ld_f32; a.out_f16 = epi.out_f16; a.ld_f16 = epi.ld_f16;
    a.add_f32 = epi.add_f32; a.ld_add = epi.ld_add; a.mask = epi.mask; a.ld_mask = epi.ld_mask;
    CUtensorMap ta, tb;
    MGT_MAP(e->Map(&ta, act, K, M, act_pitch, 64, 128));
    MGT_MAP(e->Map(&tb, w, N, K, w_pitch, 64, 64));
    if (a.k_chunks <= 4) return bn == 224 ? LaunchGemm<CfgFwdS<224, EPI>>(e, ta, tb, a, st) : LaunchGemm<CfgFwdS<256, EPI>>(e, ta, tb, a, st);
    return bn == 224 ? LaunchGemm<CfgFwd<224, EPI>>(e, ta, tb, a, st) : LaunchGemm<CfgFwd<256, EPI>>(e, ta, tb, a, st);
}

// The same product with the activation stored as actT[K][M] (one row per input column): an MN-major A operand.
template <Epi EPI>
mgt_status_t GemmForwardRows(mgt_engine* e, cudaStream_t st, const __half* act_t, uint32_t act_t_pitch, const __half* w, uint32_t w_pitch,
                             uint32_t M, uint32_t N, uint32_t K, GemmArgs epi) {
    const uint32_t bn = PickBN(N);
    GemmArgs a = BaseArgs(M, N, K, bn, 1);
    a.bias = epi.bias; a.out_f32 = epi.out_f32; a.ld_f32 = epi.ld_f32; a.out_f16 = epi.out_f16; a.ld_f16 = epi.ld_f16;
    a.add_f32 = epi.add_f32; a.ld_add = epi.ld_add; a.mask = epi.mask; a.ld_mask = epi.ld_mask;
    CUtensorMap ta, tb;
    MGT_MAP(e->Map(&ta, act_t, M, K, act_t_pitch, 64, 64));
    MGT_MAP(e->Map(&tb, w, N, K, w_pitch, 64, 64));
    return bn == 224 ? LaunchGemm<CfgFwdRows<224, EPI>>(e, ta, tb, a, st) : LaunchGemm<CfgFwdRows<256, EPI>>(e, ta, tb, a, st);
}

// How a dX GEMM is run: tile width, form, grid, and the rows of its column-sum scratch (one per epilogue warp of every CTA).
struct BackpropPlan {
    uint32_t bn;
    bool stationary;
    uint32_t grid, rows;
};
BackpropPlan PlanBackprop(const mgt_engine* e, uint32_t M, uint32_t N, uint32_t K) {
    BackpropPlan p{};
    const uint32_t sm = (uint32_t)e->sm_count;
    p.bn = PickBN(N);
    const GemmArgs a = BaseArgs(M, N, K, p.bn, 1);
    p.stationary = a.k_chunks <= 4 && a.n_tiles <= sm;
    const uint64_t units = (uint64_t)a.m_tiles * a.n_tiles;
    p.grid = (uint32_t)(units < (uint64_t)sm ? units : (uint64_t)sm);
    if (p.stationary && p.grid >= a.n_tiles) p.grid = p.grid / a.n_tiles * a.n_tiles;  // as LaunchGemm picks it
    p.rows = p.grid * 8U;
    return p;
}

// dX[M x N] = dz[M x K, K-major] * W[N x K, row-major]^T with a backward epilogue that produces the
// next dz tensor; its fp32 column sums (a bias gradient) go to `colsum` (zeroed by the caller,
// PlanBackprop().rows rows of N) and, if bias_grad is given, are reduced into bias_grad[N] right away.
template <Epi EPI>
mgt_status_t GemmBackpropInput(mgt_engine* e, cudaStream_t st, const __half* dz, uint32_t dz_pitch, const __half* w, uint32_t w_pitch,
                               uint32_t M, uint32_t N, uint32_t K, GemmArgs epi, float* colsum, float* bias_grad) {
    const BackpropPlan p = PlanBackprop(e, M, N, K);
    GemmArgs a = BaseArgs(M, N, K, p.bn, 1);
    a.out_f32 = epi.out_f32; a.ld_f32 = epi.ld_f32; a.out_f16 = epi.out_f16; a.ld_f16 = epi.ld_f16;
    a.add_f32 = epi.add_f32; a.ld_add = epi.ld_add; a.mask = epi.mask; a.ld_mask = epi.ld_mask;
    a.colsum = colsum;
    CUtensorMap ta, tb;
    MGT_MAP(e->Map(&ta, dz, K, M, dz_pitch, 64, 128));
    MGT_MAP(e->Map(&tb, w, K, N, w_pitch, 64, p.bn));
    if (p.stationary) {
        MGT_TRY(p.bn == 224 ? LaunchGemm<CfgDxS<224, EPI>>(e, ta, tb, a, st) : LaunchGemm<CfgDxS<256, EPI>>(e, ta, tb, a, st));
    } else {
        MGT_TRY(p.bn == 224 ? LaunchGemm<CfgDx<224, EPI>>(e, ta, tb, a, st) : LaunchGemm<CfgDx<256, EPI>>(e, ta, tb, a, st));
    }
    if (bias_grad != nullptr) {
        ReduceRowsKernel<<<(N + kReduceCols - 1) / kReduceCols, 256, 0, st>>>(colsum, p.rows, N, 0, N, bias_grad);
        ++e->launches;
    }
    return cudaGetLastError() == cudaSuccess ? MGT_OK : MGT_CUDA_FAILURE;
}

// The weight gradients of all residual blocks for one of the two linear layers in ONE launch:
// grad_g[in x out] = act_g^T * dz_g for g = 0..groups-1, where act_g / dz_g are slices of two tapes and
// grad_g lie `grad_group_stride` floats apart. Split-K with a fixed-order reduction.
mgt_status_t GemmGradWeightsGrouped(mgt_engine* e, cudaStream_t st, const __half* act_tape, uint32_t act_pitch, uint64_t act_stride_bytes,
                                    const __half* dz_tape, uint32_t dz_pitch, uint64_t dz_stride_bytes, uint32_t groups, uint32_t samples,
                                    uint32_t in_dim, uint32_t out_dim, float* partial, uint64_t partial_floats, float* grad_first, uint64_t grad_group_stride) {
    const uint32_t M = in_dim, N = out_dim, K = samples;
    const uint32_t bn = PickBN(N);
    GemmArgs a = BaseArgs(M, N, K, bn, 1);
    const uint64_t tiles = (uint64_t)a.m_tiles * a.n_tiles * groups;
    uint32_t splits = tiles >= (uint64_t)e->sm_count ? 1U : (uint32_t)(e->sm_count / tiles);
    const uint64_t per_split = (uint64_t)M * N;
    if ((uint64_t)splits * groups * per_split > partial_floats) splits = (uint32_t)(partial_floats / (per_split * groups));
    if (splits < 1) return MGT_CAPACITY_EXCEEDED;
    a = BaseArgs(M, N, K, bn, splits);
    a.groups = groups;
    a.partial = partial;
    CUtensorMap ta, tb;
    MGT_MAP(e->Map3D(&ta, act_tape, M, K, groups, act_pitch, act_stride_bytes, 64, 64));
    MGT_MAP(e->Map3D(&tb, dz_tape, N, K, groups, dz_pitch, dz_stride_bytes, 64, 64));
    MGT_TRY(bn == 224 ? LaunchGemm<CfgDwG<224>>(e, ta, tb, a, st) : LaunchGemm<CfgDwG<256>>(e, ta, tb, a, st));
    const dim3 grid(GridFor(per_split, 256, e->sm_count) / (groups > 4 ? 4 : 1) + 1, groups);
    ReducePartialsGroupedKernel<<<grid, 256, 0, st>>>(partial, a.splits, per_split, grad_first, grad_group_stride);
    ++e->launches;
    return cudaGetLastError() == cudaSuccess ? MGT_OK : MGT_CUDA_FAILURE;
}

// grad[in x out] = act^T * dz, reduced over the batch with split-K and a fixed-order reduction.
mgt_status_t GemmGradWeights(mgt_engine* e, cudaStream_t st, const __half* act, uint32_t act_pitch, const __half* dz, uint32_t dz_pitch,
                             uint32_t samples, uint32_t in_dim, uint32_t out_dim, float* partial, uint64_t partial_floats, float* grad_out) {
    const uint32_t M = in_dim, N = out_dim, K = samples;
    const uint32_t bn = PickBN(N);
    GemmArgs a = BaseArgs(M, N, K, bn, 1);
    const uint64_t tiles = (uint64_t)a.m_tiles * a.n_tiles;
    uint32_t splits = tiles >= (uint64_t)e->sm_count ? 1U : (uint32_t)(e->sm_count / tiles);
    const uint64_t per_split = (uint64_t)M * N;
    if ((uint64_t)splits * per_split > partial_floats) splits = (uint32_t)(partial_floats / per_split);
    if (splits < 1) return MGT_CAPACITY_EXCEEDED;
    a = BaseArgs(M, N, K, bn, splits);
    a.partial = partial;
    CUtensorMap ta, tb;
    MGT_MAP(e->Map(&ta, act, M, K, act_pitch, 64, 64));
    MGT_MAP(e->Map(&tb, dz, N, K, dz_pitch, 64, 64));
    MGT_TRY(bn == 224 ? LaunchGemm<CfgDw<224>>(e, ta, tb, a, st) : LaunchGemm<CfgDw<256>>(e, ta, tb, a, st));
    ReducePartialsKernel<<<GridFor(per_split, 256, e->sm_count), 256, 0, st>>>(partial, a.splits, per_split, grad_out);
    ++e->launches;
    return cudaGetLastError() == cudaSuccess ? MGT_OK : MGT_CUDA_FAILURE;
}

// grad[in x out] = act^T * dz with the activation stored as actT[in][samples]: a K-major A operand.
mgt_status_t GemmGradWeightsRows(mgt_engine* e, cudaStream_t st, const __half* act_t, uint32_t act_t_pitch, const __half* dz, uint32_t dz_pitch,
                                 uint32_t samples, uint32_t in_dim, uint32_t out_dim, float* partial, uint64_t partial_floats, float* grad_out) {
    const uint32_t M = in_dim, N = out_dim, K = samples;
    const uint32_t bn = PickBN(N);
    GemmArgs a = BaseArgs(M, N, K, bn, 1);
    const uint64_t tiles = (uint64_t)a.m_tiles * a.n_tiles;
    uint32_t splits = tiles >= (uint64_t)e->sm_count ? 1U : (uint32_t)(e->sm_count / tiles);
    const uint64_t per_split = (uint64_t)M * N;
    if ((uint64_t)splits * per_split > partial_floats) splits = (uint32_t)(partial_floats / per_split);
    if (splits < 1) return MGT_CAPACITY_EXCEEDED;
    a = BaseArgs(M, N, K, bn, splits);
    a.partial = partial;
    CUtensorMap ta, tb;
    MGT_MAP(e->Map(&ta, act_t, K, M, act_t_pitch, 64, 128));
    MGT_MAP(e->Map(&tb, dz, N, K, dz_pitch, 64, 64));
    MGT_TRY(bn == 224 ? LaunchGemm<CfgDwRows<224>>(e, ta, tb, a, st) : LaunchGemm<CfgDwRows<256>>(e, ta, tb, a, st));
    ReducePartialsKernel<<<GridFor(per_split, 256, e->sm_count), 256, 0, st>>>(partial, a.splits, per_split, grad_out);
    ++e->launches;
    return cudaGetLastError() == cudaSuccess ? MGT_OK : MGT_CUDA_FAILURE;
}

// dxT[N_in x samples] = (W[N_in x K] * dz[samples x K]^T) * [mask bit]: the hidden layer's dX with its wide side as rows; the
// mask words are the ones the embedding forward wrote beside its activation.
// Row sums of the result (the bias gradient of the layer below) are reduced into bias_grad[N_in] in a fixed order.
mgt_status_t GemmBackpropInputRows(mgt_engine* e, cudaStream_t st, const __half* w, uint32_t w_pitch, const __half* dz, uint32_t dz_pitch, uint32_t samples,
                                   uint32_t in_dim, uint32_t out_dim, uint32_t* mask_bits, uint32_t ld_bits, __half* dx_t, uint32_t t_pitch, float* rowsum,
                                   uint64_t rowsum_rows, float* bias_grad) {
    GemmArgs a = BaseArgs(in_dim, samples, out_dim, CfgDxRows::BN, 1);
    const uint64_t rows = (uint64_t)a.n_tiles * CfgDxRows::EPI_STRIDE;
    if (rows > rowsum_rows) return MGT_CAPACITY_EXCEEDED;
    a.bits = mask_bits; a.ld_bits = ld_bits; a.out_f16 = dx_t; a.ld_f16 = t_pitch; a.rowsum = rowsum;
    CUtensorMap ta, tb;
    MGT_MAP(e->Map(&ta, w, out_dim, in_dim, w_pitch, 64, 128));
    MGT_MAP(e->Map(&tb, dz, out_dim, samples, dz_pitch, 64, CfgDxRows::BN));
    MGT_TRY(LaunchGemm<CfgDxRows>(e, ta, tb, a, st));
    ReduceRowsKernel<<<(in_dim + kReduceCols - 1) / kReduceCols, 256, 0, st>>>(rowsum, (uint32_t)rows, in_dim, 0, in_dim, bias_grad);
    ++e->launches;
    return cudaGetLastError() == cudaSuccess ? MGT_OK : MGT_CUDA_FAILURE;
}

// The residual tower in one launch per direction; see tower_chain.cuh. Shapes it takes: hd2 a multiple of 32 up to 256.
bool ChainEligible(const mgt_engine* e, const mgt_mlp_shape_t& s) {
    return s.residual_blocks > 0 && s.hd2 % 32U == 0 && s.hd2 >= 32U && s.hd2 <= 256U && !e->layered_tower;
}

template <bool BWD>
mgt_status_t LaunchChain(mgt_engine* e, cudaStream_t st, const __half* w_first, uint32_t w_pitch, uint64_t w_layer_stride_bytes, uint32_t tape_s_entries,
                         uint32_t tape_t_entries, ChainArgs a) {
    static std::mutex attr_mu;
    static bool attr_done[64] = {};
    {
        std::lock_guard<std::mutex> lock(attr_mu);
        if (e->device >= 0 && e->device < 64 && !attr_done[e->device]) {
            if (cudaFuncSetAttribute(tower_chain_kernel<BWD>, cudaFuncAttributeMaxDynamicSharedMemorySize, ChainCfg::SMEM_BYTES) != cudaSuccess) return MGT_CUDA_FAILURE;
            attr_done[e->device] = true;
        }
    }
    CUtensorMap tw, ts, tt;
    MGT_MAP(e->Map3D(&tw, w_first, a.H, a.H, 2ULL * a.R, w_pitch, w_layer_stride_bytes, 64, BWD ? a.H : 64));
    // the tapes as stacks of [samples][H] matrices; a store box is one operand panel: 64 columns x 128 rows
    MGT_MAP(e->Map3D(&ts, a.tape_s, a.H, a.samples, tape_s_entries, a.ld_s, a.tape_s_stride * 2, 64, 128));
    MGT_MAP(e->Map3D(&tt, a.tape_t, a.H, a.samples, tape_t_entries, a.ld_t, a.tape_t_stride * 2, 64, 128));
    a.status = e->status_word;
    a.bf16 = e->bf16_now ? 1U : 0U;
    const uint32_t grid = a.tiles < (uint32_t)e->sm_count ? a.tiles : (uint32_t)e->sm_count;
    tower_chain_kernel<BWD><<<grid, ChainCfg::THREADS, ChainCfg::SMEM_BYTES, st>>>(tw, ts, tt, a);
    ++e->launches;
    return cudaGetLastError() == cudaSuccess ? MGT_OK : MGT_CUDA_FAILURE;
}

// ---- the fp32 data flow (use_half_linear == 0), mlp_backward.cu:1273-1510 without the fp16 copies -----------------
struct Fp32Workspace {
    uint64_t a1, x, r1, z, y, dy, d0, d1, dz1, lossp, total;  // float offsets
};
Fp32Workspace PlanFp32(const mgt_mlp_shape_t& s, uint32_t B) {
    Fp32Workspace w{};
    uint64_t off = 0;
    auto take = [&](uint64_t n) { const uint64_t at = off; off += (n + 63) & ~63ULL; return at; };
    const uint64_t bh2 = (uint64_t)B * s.hd2, bh1 = (uint64_t)B * s.hd1;
    w.a1 = take(bh1);
    w.x = take(bh2 * (s.residual_blocks + 1ULL));
    w.r1 = take(bh2 * (s.residual_blocks > 0 ? s.residual_blocks : 1ULL));
    w.z = take(bh2);
    w.y = take((uint64_t)B * s.output_dim);
    w.dy = take((uint64_t)B * s.output_dim);
    w.d0 = take(bh2);
    w.d1 = take(bh2);
    w.dz1 = take(bh1);
    w.lossp = take(1024);
    w.total = off + 64;
    return w;
}
uint64_t Fp32WorkspaceFloats(const mgt_mlp_shape_t& s, uint32_t B) { return PlanFp32(s, B).total; }

template <class F>
mgt_status_t LaunchFp32Path(mgt_engine* e, const mgt_mlp_shape_t& s, const float* w, const uint8_t* states, const float* labels, uint32_t B, float* loss,
                            float* grad, float* workspace, bool half_ig, mgt_backward_profile_t* profile, F&& notify, cudaStream_t st) {
    using namespace mgt::fp32path;
    const Fp32Workspace ws = PlanFp32(s, B);
    float* base = reinterpret_cast<float*>(RoundUp(reinterpret_cast<uintptr_t>(workspace), 256));
    const uint32_t H1 = s.hd1, H2 = s.hd2, R = s.residual_blocks, OUT = s.output_dim, L = s.state_len, V = s.state_value_pad;
    const uint64_t bh2 = (uint64_t)B * H2, bh1 = (uint64_t)B * H1;
    float* a1 = base + ws.a1;
    auto x = [&](uint32_t k) { return base + ws.x + bh2 * k; };
    auto r1 = [&](uint32_t k) { return base + ws.r1 + bh2 * k; };
    float *z = base + ws.z, *y = base + ws.y, *dy = base + ws.dy, *d0 = base + ws.d0, *d1 = base + ws.d1, *dz1 = base + ws.dz1, *lossp = base + ws.lossp;
    const int sm = e->sm_count;
    auto blocks = [&](uint64_t n) { return GridFor(n, 256, sm); };
    auto ok = [&]() { return cudaGetLastError() == cudaSuccess; };
    auto colsum = [&](const float* src, uint32_t cols, float* dst) {
        ColumnSumKernel<<<(cols + 7) / 8, 256, 0, st>>>(src, B, cols, dst);
        ++e->launches;
    };
    StageTimer timer{e, st, profile};
    if (!timer.Start()) return MGT_CUDA_FAILURE;

    InputForwardKernel<<<blocks(bh1), 256, 0, st>>>(states, w, w + InputBias(s), B, L, V, H1, a1);
    ++e->launches;
    if (!ok() || !timer.Mark(profile ? &profile->input_forward_ms : nullptr)) return MGT_CUDA_FAILURE;
    // hidden layer and residual blocks (y = x W, weights row-major [in][out])
    if (Sgemm<false, false>(st, B, H2, H1, a1, H1, w + HiddenWeight(s), H2, z, H2) != cudaSuccess) return MGT_CUDA_FAILURE;
    BiasReluKernel<<<blocks(bh2), 256, 0, st>>>(z, w + HiddenBias(s), nullptr, H2, bh2, x(0));
    e->launches += 2;
    if (!ok() || !timer.Mark(profile ? &profile->hidden_forward_ms : nullptr)) return MGT_CUDA_FAILURE;
    for (uint32_t k = 0; k < R; ++k) {
        if (Sgemm<false, false>(st, B, H2, H2, x(k), H2, w + Fc1W(s, k), H2, z, H2) != cudaSuccess) return MGT_CUDA_FAILURE;
        BiasReluKernel<<<blocks(bh2), 256, 0, st>>>(z, w + Fc1B(s, k), nullptr, H2, bh2, r1(k));
        if (Sgemm<false, false>(st, B, H2, H2, r1(k), H2, w + Fc2W(s, k), H2, z, H2) != cudaSuccess) return MGT_CUDA_FAILURE;
        BiasReluKernel<<<blocks(bh2), 256, 0, st>>>(z, w + Fc2B(s, k), x(k), H2, bh2, x(k + 1));
        e->launches += 4;
    }
    if (!ok() || !timer.Mark(profile ? &profile->residual_forward_ms : nullptr)) return MGT_CUDA_FAILURE;
    // output layer, loss, dL/dy, gradients of the output layer, gradient entering the tower
    const uint64_t by = (uint64_t)B * OUT;
    if (Sgemm<false, false>(st, B, OUT, H2, x(R), H2, w + OutputWeight(s), OUT, y, OUT) != cudaSuccess) return MGT_CUDA_FAILURE;
    AddBiasKernel<<<blocks(by), 256, 0, st>>>(y, w + OutputBias(s), OUT, by);
    const uint32_t loss_blocks = (uint32_t)(blocks(by) < 1024 ? blocks(by) : 1024);
    LossKernel<<<loss_blocks, 256, 0, st>>>(y, labels, by, 1.0f / (float)by, dy, lossp);
    FinishLossKernel<<<1, 32, 0, st>>>(lossp, loss_blocks, loss);
    if (Sgemm<true, false>(st, H2, OUT, B, x(R), H2, dy, OUT, grad + OutputWeight(s), OUT) != cudaSuccess) return MGT_CUDA_FAILURE;
    colsum(dy, OUT, grad + OutputBias(s));
    if (Sgemm<false, true>(st, B, H2, OUT, dy, OUT, w + OutputWeight(s), OUT, d0, H2) != cudaSuccess) return MGT_CUDA_FAILURE;
    e->launches += 6;
    MGT_TRY(notify(OutputWeight(s), (uint64_t)H2 * OUT + OUT));
    if (!ok() || !timer.Mark(profile ? &profile->output_ms : nullptr)) return MGT_CUDA_FAILURE;
    // residual blocks backward: d0 holds dL/dx_{k+1}
    for (uint32_t rb = R; rb > 0; --rb) {
        const uint32_t k = rb - 1U;
        MaskKernel<float><<<blocks(bh2), 256, 0, st>>>(d0, nullptr, x(k + 1), H2, H2, bh2, false, d0);  // dz2, in place
        colsum(d0, H2, grad + Fc2B(s, k));
        if (Sgemm<true, false>(st, H2, H2, B, r1(k), H2, d0, H2, grad + Fc2W(s, k), H2) != cudaSuccess) return MGT_CUDA_FAILURE;
        if (Sgemm<false, true>(st, B, H2, H2, d0, H2, w + Fc2W(s, k), H2, z, H2) != cudaSuccess) return MGT_CUDA_FAILURE;
        MGT_TRY(notify(Fc2W(s, k), (uint64_t)H2 * H2 + H2));  // after the last reader of W2_k
        MaskKernel<float><<<blocks(bh2), 256, 0, st>>>(z, nullptr, r1(k), H2, H2, bh2, false, d1);       // dz1 of the block
        colsum(d1, H2, grad + Fc1B(s, k));
        if (Sgemm<true, false>(st, H2, H2, B, x(k), H2, d1, H2, grad + Fc1W(s, k), H2) != cudaSuccess) return MGT_CUDA_FAILURE;
        if (Sgemm<false, true>(st, B, H2, H2, d1, H2, w + Fc1W(s, k), H2, z, H2) != cudaSuccess) return MGT_CUDA_FAILURE;
        MGT_TRY(notify(Fc1W(s, k), (uint64_t)H2 * H2 + H2));
        AddIntoKernel<<<blocks(bh2), 256, 0, st>>>(d0, z, bh2);  // dL/dx_k = dz2 + dz1 W1^T
        e->launches += 7;
    }
    if (!ok() || !timer.Mark(profile ? &profile->residual_backward_ms : nullptr)) return MGT_CUDA_FAILURE;
    // hidden layer backward
    MaskKernel<float><<<blocks(bh2), 256, 0, st>>>(d0, nullptr, x(0), H2, H2, bh2, false, d0);  // dzh
    colsum(d0, H2, grad + HiddenBias(s));
    if (Sgemm<true, false>(st, H1, H2, B, a1, H1, d0, H2, grad + HiddenWeight(s), H2) != cudaSuccess) return MGT_CUDA_FAILURE;
    if (Sgemm<false, true>(st, B, H1, H2, d0, H2, w + HiddenWeight(s), H2, dz1, H1) != cudaSuccess) return MGT_CUDA_FAILURE;
    MGT_TRY(notify(HiddenWeight(s), (uint64_t)H1 * H2 + H2));
    MaskKernel<float><<<blocks(bh1), 256, 0, st>>>(dz1, nullptr, a1, H1, H1, bh1, false, dz1);
    colsum(dz1, H1, grad + InputBias(s));  // the reference sums the fp32 dz1 (mlp_backward.cu:1505)
    if (half_ig) MaskKernel<float><<<blocks(bh1), 256, 0, st>>>(dz1, nullptr, a1, H1, H1, bh1, true, dz1);  // fp16 operand of the embedding gradient
    e->launches += 5;
    if (!ok() || !timer.Mark(profile ? &profile->hidden_backward_ms : nullptr)) return MGT_CUDA_FAILURE;
    EmbeddingGradKernel<float><<<dim3(L, (H1 + 63) / 64), 128, 2ULL * V * 64 * sizeof(float), st>>>(states, dz1, H1, B, V, H1, grad);
    ++e->launches;
    MGT_TRY(notify(0, (uint64_t)L * V * H1 + H1));
    if (!ok() || !timer.Mark(profile ? &profile->input_grad_ms : nullptr)) return MGT_CUDA_FAILURE;
    return MGT_OK;
}

struct HalfWeights {
    const __half* in_table; uint32_t p1;     // [(IN+1)][p1], row IN is the input bias
    const __half* wh; uint32_t p2;            // [H1][p2]
    const __half* w1[MGT_MAX_RESIDUAL_BLOCKS];
    const __half* w2[MGT_MAX_RESIDUAL_BLOCKS];
    const __half* wout; uint32_t pout;        // [H2][pout]
};

}  // namespace
}  // namespace mgt

using namespace mgt;

extern "C" {

const char* mgt_status_name(mgt_status_t status) {
    switch (status) {
        case MGT_OK: return "ok";
        case MGT_INVALID_CONFIG: return "invalid_config";
        case MGT_INVALID_PUZZLE: return "invalid_puzzle";
        case MGT_CAPACITY_EXCEEDED: return "capacity_exceeded";
        case MGT_CUDA_FAILURE: return "cuda_failure";
        case MGT_NCCL_FAILURE: return "nccl_failure";
        case MGT_IO_FAILURE: return "io_failure";
        case MGT_DEVICE_TIMEOUT: return "device_timeout";
    }
    return "unknown";
}

const char* mgt_version(void) { return "mgt_b200 0.1 (sm_100a)"; }

mgt_status_t mgt_validate_mlp_shape(const mgt_mlp_shape_t* shape) { return ValidShape(shape) ? MGT_OK : MGT_INVALID_CONFIG; }

uint64_t mgt_mlp_param_count(const mgt_mlp_shape_t* shape) { return ValidShape(shape) ? ParamCount(*shape) : 0; }

mgt_status_t mgt_engine_create(int32_t device_id, mgt_engine_t** out_engine) {
    if (out_engine == nullptr || device_id < 0) return MGT_INVALID_CONFIG;
    *out_engine = nullptr;
    if (cudaSetDevice(device_id) != cudaSuccess) return MGT_CUDA_FAILURE;
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device_id) != cudaSuccess) return MGT_CUDA_FAILURE;
    if (prop.major != 10) {
        std::fprintf(stderr, "mgt_b200: device %d is sm_%d%d; this library only runs on sm_100a (B200)\n", device_id, prop.major, prop.minor);
        return MGT_CUDA_FAILURE;
    }
    auto* e = new mgt_engine();
    e->device = device_id;
    e->sm_count = prop.multiProcessorCount;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || fn == nullptr) {
        delete e;
        return MGT_CUDA_FAILURE;
    }
    e->encode = reinterpret_cast<EncodeTiledFn>(fn);
    if (const char* path = std::getenv("MGT_RESIDUAL_PATH")) e->layered_tower = std::strcmp(path, "layered") == 0;
    if (cudaMalloc(&e->status_word, sizeof(int)) != cudaSuccess || cudaMemset(e->status_word, 0, sizeof(int)) != cudaSuccess) {
        delete e;
        return MGT_CUDA_FAILURE;
    }
    *out_engine = e;
    return MGT_OK;
}

mgt_status_t mgt_engine_destroy(mgt_engine_t* e) {
    if (e == nullptr) return MGT_OK;
    if (e->ev_last) cudaEventDestroy(e->ev_last);
    if (e->ev_now) cudaEventDestroy(e->ev_now);
    if (e->status_word) cudaFree(e->status_word);
    delete e;
    return MGT_OK;
}

uint64_t mgt_engine_launch_count(const mgt_engine_t* e) { return e == nullptr ? 0 : e->launches; }

mgt_status_t mgt_engine_check(mgt_engine_t* e, void* stream, int32_t* out_device_code) {
    if (e == nullptr) return MGT_INVALID_CONFIG;
    int code = 0;
    if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) return MGT_CUDA_FAILURE;
    if (cudaMemcpy(&code, e->status_word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return MGT_CUDA_FAILURE;
    if (out_device_code) *out_device_code = code;
    if (code != 0) {
        cudaMemset(e->status_word, 0, sizeof(int));
        return MGT_DEVICE_TIMEOUT;
    }
    return MGT_OK;
}

static uint64_t WorkspaceFloats(const mgt_mlp_shape_t* shape, uint32_t sample_count, uint32_t chunks, int32_t use_half_input_grad, int32_t use_half_linear,
                                bool batch_norm) {
    if (!ValidShape(shape) || sample_count == 0 || chunks == 0) return 0;
    if (!use_half_linear) return batch_norm ? 0 : Fp32WorkspaceFloats(*shape, sample_count);
    const Workspace w = PlanWorkspace(*shape, sample_count, CurrentDeviceSmCount(), batch_norm);
    // fp32 embedding-gradient operand: da1 and dz1 [samples][hd1] in fp32 behind the tensor-core workspace
    const uint64_t extra = use_half_input_grad ? 0 : 2ULL * sample_count * shape->hd1;
    return (w.total_bytes + 3) / 4 + extra + (extra ? 256 : 0);
}

uint64_t mgt_mlp_loss_grad_workspace_floats(const mgt_mlp_shape_t* shape, uint32_t sample_count, uint32_t chunks,
                                            int32_t use_half_input_grad, int32_t use_half_linear) {
    return WorkspaceFloats(shape, sample_count, chunks, use_half_input_grad, use_half_linear, false);
}

uint64_t mgt_mlp_loss_grad_workspace_floats_with_options(const mgt_mlp_shape_t* shape, uint32_t sample_count, uint32_t chunks, int32_t use_half_input_grad,
                                                         int32_t use_half_linear, const mgt_train_options_t* options) {
    return WorkspaceFloats(shape, sample_count, chunks, use_half_input_grad, use_half_linear, options != nullptr && options->batch_norm != 0);
}

uint64_t mgt_bn_param_count(const mgt_mlp_shape_t* shape) { return ValidShape(shape) ? 2ULL * (shape->residual_blocks + 1ULL) * shape->hd2 : 0; }

mgt_status_t mgt_engine_set_batch_norm_state(mgt_engine_t* e, float* device_running_stats, float momentum, uint32_t world_size, float* device_exchange_buffer,
                                             mgt_stats_exchange_fn exchange, void* user) {
    if (e == nullptr || !(momentum >= 0.0f && momentum <= 1.0f) || world_size == 0) return MGT_INVALID_CONFIG;
    if ((exchange != nullptr) != (device_exchange_buffer != nullptr)) return MGT_INVALID_CONFIG;
    e->bn_running = device_running_stats;
    e->bn_momentum = momentum;
    e->bn_world = world_size;
    e->bn_exchange_buffer = device_exchange_buffer;
    e->bn_exchange = exchange;
    e->bn_exchange_user = user;
    return MGT_OK;
}

mgt_status_t mgt_launch_mlp_loss_grad(mgt_engine_t* e, const mgt_mlp_shape_t* shape, const float* w, const uint16_t* w_half_u16,
                                      const mgt_train_state_t* states, const float* labels, uint32_t B, float* loss, float* grad,
                                      float* workspace, uint64_t workspace_floats, uint32_t chunks, uint32_t ppb, int32_t half_ig,
                                      int32_t half_lin, mgt_backward_profile_t* profile, mgt_gradient_ready_fn ready, void* ready_user,
                                      void* stream_v, uint32_t position_tile) {
    (void)position_tile;
    if (e == nullptr || !ValidShape(shape) || w == nullptr || states == nullptr || labels == nullptr || loss == nullptr || grad == nullptr ||
        B == 0 || workspace == nullptr || chunks == 0 || ppb == 0) {
        return MGT_INVALID_CONFIG;
    }
    const mgt_mlp_shape_t s = *shape;
    const bool bnorm = e->options.batch_norm != 0;
    const bool options_set = e->options.operand_format != MGT_OPERAND_FP16 || e->options.loss_kind != MGT_LOSS_MSE || bnorm;
    if (options_set && !half_lin) return MGT_INVALID_CONFIG;  // the options belong to the tensor-core data flow
    if (e->options.loss_kind == MGT_LOSS_CROSS_ENTROPY && s.output_dim < 2U) return MGT_INVALID_CONFIG;
    struct FormatScope {  // the operand format applies to the kernels enqueued by this call only
        mgt_engine* e;
        ~FormatScope() { e->bf16_now = false; }
    } format_scope{e};
    e->bf16_now = half_lin && e->options.operand_format == MGT_OPERAND_BF16;
    if (!half_lin) {
        // fp32 linear layers: the CUDA-core path (fp32_path.cuh); half_ig only selects the rounding of its embedding-gradient operand
        if (workspace_floats < Fp32WorkspaceFloats(s, B)) return MGT_CAPACITY_EXCEEDED;
        uint32_t id = 0;
        auto tell = [&](uint64_t off, uint64_t count) -> mgt_status_t {
            if (ready == nullptr) return MGT_OK;
            return ready(ready_user, id++, off, count, stream_v) == MGT_OK ? MGT_OK : MGT_CUDA_FAILURE;
        };
        return LaunchFp32Path(e, s, w, reinterpret_cast<const uint8_t*>(states), labels, B, loss, grad, workspace, half_ig != 0, profile, tell,
                              static_cast<cudaStream_t>(stream_v));
    }
    const Workspace ws = PlanWorkspace(s, B, PlanSmCount(e->sm_count), bnorm);
    const uint64_t f32_extra = half_ig ? 0 : 2ULL * B * s.hd1;  // da1, dz1 in fp32 for the fp32 embedding gradient
    if (workspace_floats < (ws.total_bytes + 3) / 4 + f32_extra + (f32_extra ? 256 : 0)) return MGT_CAPACITY_EXCEEDED;
    cudaStream_t st = static_cast<cudaStream_t>(stream_v);
    uint8_t* base = reinterpret_cast<uint8_t*>(RoundUp(reinterpret_cast<uintptr_t>(workspace), 1024));
    float* da1_f32 = reinterpret_cast<float*>(RoundUp(reinterpret_cast<uintptr_t>(workspace + (ws.total_bytes + 3) / 4), 256));  // behind the tensor-core workspace
    float* dz1_f32 = da1_f32 + (uint64_t)B * s.hd1;
    __half* a1_h = reinterpret_cast<__half*>(base + ws.off_a1);
    auto x_h = [&](uint32_t k) { return reinterpret_cast<__half*>(base + ws.off_x + ws.x_stride * k); };
    auto r1_h = [&](uint32_t k) { return reinterpret_cast<__half*>(base + ws.off_r1 + ws.r1_stride * k); };
    float* x_f32 = reinterpret_cast<float*>(base + ws.off_xf);
    float* dzf = reinterpret_cast<float*>(base + ws.off_dzf);
    auto dz_tape = [&](uint32_t k) { return reinterpret_cast<__half*>(base + ws.off_dz2 + ws.dz_stride * k); };   // [0] hidden, [k+1] fc2 of block k
    auto dz1_tape = [&](uint32_t k) { return reinterpret_cast<__half*>(base + ws.off_dz1t + ws.dz_stride * k); };  // fc1 of block k
    __half* dz1_h = reinterpret_cast<__half*>(base + ws.off_dz1);
    float* partial = reinterpret_cast<float*>(base + ws.off_partial);
    float* head_partial = reinterpret_cast<float*>(base + ws.off_head);
    float* colsum = reinterpret_cast<float*>(base + ws.off_colsum);
    const uint32_t H1 = s.hd1, H2 = s.hd2, R = s.residual_blocks, OUT = s.output_dim, IN = ws.IN;

    StageTimer timer{e, st, profile};
    if (!timer.Start()) return MGT_CUDA_FAILURE;
    uint32_t ready_id = 0;
    auto notify = [&](uint64_t off, uint64_t count) -> mgt_status_t {
        if (ready == nullptr) return MGT_OK;
        const mgt_status_t r = ready(ready_user, ready_id++, off, count, stream_v);
        return r == MGT_OK ? MGT_OK : MGT_CUDA_FAILURE;  // the reference maps a failing callback to kCudaFailure
    };

    // ---- batch normalisation (opt-in): fp32 pre-activations z of every normalised layer are kept, layer 0 = hidden
    // layer, layer k + 1 = fc2 of block k; gamma/beta and their gradients follow the reference's parameters
    const uint64_t bn_base = ParamCount(s);
    auto z_tape = [&](uint32_t layer) { return reinterpret_cast<float*>(base + ws.off_bn_z + ws.bn_z_stride * layer); };
    auto bn_mean = [&](uint32_t layer) { return reinterpret_cast<float*>(base + ws.off_bn_save) + 2ULL * layer * H2; };
    auto bn_rstd = [&](uint32_t layer) { return bn_mean(layer) + H2; };
    float* bn_partial = reinterpret_cast<float*>(base + ws.off_bn_partial);
    float* bn_stats = bnorm && e->bn_exchange_buffer != nullptr ? e->bn_exchange_buffer : reinterpret_cast<float*>(base + ws.off_bn_stats);
    const uint32_t bn_blocks = bn::BlocksFor(B, e->sm_count);
    const uint32_t bn_reduce_grid = (H2 + bn::kReduceCols - 1U) / bn::kReduceCols, bn_reduce_threads = bn::kReduceCols * bn::kReduceParts;
    auto bn_exchange = [&]() -> mgt_status_t {
        if (e->bn_exchange == nullptr) return MGT_OK;
        return e->bn_exchange(e->bn_exchange_user, bn_stats, 2ULL * H2, stream_v) == MGT_OK ? MGT_OK : MGT_CUDA_FAILURE;
    };
    // z_tape(layer) -> x_f32 / x_h(layer): x = relu(bn(z)) for the hidden layer, relu(x + bn(z)) for a block
    auto bn_forward = [&](uint32_t layer) -> mgt_status_t {
        bn::ColumnMomentsKernel<false><<<bn_blocks, bn::kThreads, 0, st>>>(z_tape(layer), ws.p_f32, nullptr, 0, nullptr, nullptr, B, H2, bn_partial);
        bn::ReduceMomentsKernel<<<bn_reduce_grid, bn_reduce_threads, 0, st>>>(bn_partial, bn_blocks, H2, 1.0f / (float)B, bn_stats, nullptr, nullptr);
        MGT_TRY(bn_exchange());
        const float* gamma = w + bn_base + 2ULL * layer * H2;
        float* running = e->bn_running != nullptr ? e->bn_running + 2ULL * layer * H2 : nullptr;
        const double n = (double)B * e->bn_world;
        const float unbias = n > 1.0 ? (float)(n / (n - 1.0)) : 1.0f;
        uint16_t* xh = reinterpret_cast<uint16_t*>(x_h(layer));
        if (layer == 0U) {
            bn::ApplyForwardKernel<false><<<bn_blocks, bn::kThreads, 0, st>>>(z_tape(layer), ws.p_f32, bn_stats, gamma, gamma + H2, e->options.bn_eps, B, H2, x_f32,
                                                                             ws.p_f32, xh, ws.p_act, e->bf16_now, bn_mean(layer), bn_rstd(layer), running,
                                                                             e->bn_momentum, unbias);
        } else {
            bn::ApplyForwardKernel<true><<<bn_blocks, bn::kThreads, 0, st>>>(z_tape(layer), ws.p_f32, bn_stats, gamma, gamma + H2, e->options.bn_eps, B, H2, x_f32,
                                                                            ws.p_f32, xh, ws.p_act, e->bf16_now, bn_mean(layer), bn_rstd(layer), running,
                                                                            e->bn_momentum, unbias);
        }
        e->launches += 3;
        return cudaGetLastError() == cudaSuccess ? MGT_OK : MGT_CUDA_FAILURE;
    };
    // dzf (gradient w.r.t. the sum entering the ReLU above the layer) -> dz_tape(layer) = gradient w.r.t. z, plus the
    // gradients of gamma, beta and of the bias inside z
    auto bn_backward = [&](uint32_t layer, float* bias_grad) -> mgt_status_t {
        bn::ColumnMomentsKernel<true><<<bn_blocks, bn::kThreads, 0, st>>>(dzf, ws.p_f32, z_tape(layer), ws.p_f32, bn_mean(layer), bn_rstd(layer), B, H2, bn_partial);
        float* dgamma = grad + bn_base + 2ULL * layer * H2;
        bn::ReduceMomentsKernel<<<bn_reduce_grid, bn_reduce_threads, 0, st>>>(bn_partial, bn_blocks, H2, 1.0f / (float)B, bn_stats, dgamma + H2, dgamma);
        MGT_TRY(bn_exchange());
        bn::ApplyBackwardKernel<<<bn_blocks, bn::kThreads, 0, st>>>(dzf, ws.p_f32, z_tape(layer), ws.p_f32, bn_mean(layer), bn_rstd(layer), w + bn_base + 2ULL * layer * H2,
                                                                    bn_stats, B, H2, reinterpret_cast<uint16_t*>(dz_tape(layer)), ws.p_dz, e->bf16_now, bn_partial);
        bn::ReduceSumsKernel<<<bn_reduce_grid, bn_reduce_threads, 0, st>>>(bn_partial, bn_blocks, H2, bias_grad);
        e->launches += 4;
        return cudaGetLastError() == cudaSuccess ? MGT_OK : MGT_CUDA_FAILURE;
    };

    // ---- fp16 weights: the caller's mirror as it lies when TMA can address it, else a padded copy
    HalfWeights hw{};
    const __half* w_half = reinterpret_cast<const __half*>(w_half_u16);
    // (the caller's mirror is fp16 by contract: with bfloat16 operands the copy is rebuilt from the fp32 weights each call)
    const bool direct = w_half != nullptr && !e->bf16_now && (H1 % 8U) == 0 && (H2 % 8U) == 0 && (reinterpret_cast<uintptr_t>(w_half) & 15U) == 0;
    if (direct) {
        hw.in_table = w_half; hw.p1 = H1;
        hw.wh = w_half + HiddenWeight(s); hw.p2 = H2;
        for (uint32_t k = 0; k < R; ++k) { hw.w1[k] = w_half + Fc1W(s, k); hw.w2[k] = w_half + Fc2W(s, k); }
        hw.wout = w_half + OutputWeight(s); hw.pout = OUT;
    } else {
        uint8_t* cur = base + ws.off_wint;
        auto repack = [&](const float* src, uint32_t rows, uint32_t cols, uint32_t pitch) -> const __half* {
            __half* dst = reinterpret_cast<__half*>(cur);
            cur += RoundUp((uint64_t)rows * pitch * 2, 1024);
            cudaMemsetAsync(dst, 0, (uint64_t)rows * pitch * 2, st);
            RepackHalfKernel<<<GridFor((uint64_t)rows * cols, 256, e->sm_count), 256, 0, st>>>(src, rows, cols, cols, dst, pitch, e->bf16_now);
            ++e->launches;
            return dst;
        };
        hw.p1 = ws.p_w1; hw.p2 = ws.p_w2; hw.pout = ws.p_wout;
        hw.in_table = repack(w, IN + 1, H1, ws.p_w1);
        hw.wh = repack(w + HiddenWeight(s), H1, H2, ws.p_w2);
        for (uint32_t k = 0; k < R; ++k) {
            hw.w1[k] = repack(w + Fc1W(s, k), H2, H2, ws.p_w2);
            hw.w2[k] = repack(w + Fc2W(s, k), H2, H2, ws.p_w2);
        }
        hw.wout = repack(w + OutputWeight(s), H2, OUT, ws.p_wout);
        if (cudaGetLastError() != cudaSuccess) return MGT_CUDA_FAILURE;
    }

    // ---- embedding forward: a1 = relu([onehot | 1] * [W_in ; b_in])  (mlp_backward.cu:755-832)
    {
        GemmArgs a = BaseArgs(H1, B, IN + 1, CfgEmbFwd::NACC * CfgEmbFwd::BN, 1);
        a.out_f16 = a1_h; a.ld_f16 = ws.p_bt;
        a.bits = reinterpret_cast<uint32_t*>(base + ws.off_bits_h1); a.ld_bits = ws.ld_bits_h1;
        a.states = reinterpret_cast<const uint8_t*>(states); a.state_len = s.state_len; a.value_pad = s.state_value_pad; a.samples = B; a.in_rows = IN;
        CUtensorMap ta;
        MGT_MAP(e->Map(&ta, hw.in_table, H1, IN + 1, hw.p1, 64, 64));
        MGT_TRY(LaunchGemm<CfgEmbFwd>(e, ta, ta, a, st));
    }
    if (!timer.Mark(profile ? &profile->input_forward_ms : nullptr)) return MGT_CUDA_FAILURE;

    // ---- hidden layer: x0 = relu(a1 * Wh + bh)  (mlp_backward.cu:1281-1291)
    {
        GemmArgs epi{};
        epi.bias = w + HiddenBias(s); epi.out_f32 = x_f32; epi.ld_f32 = ws.p_f32; epi.out_f16 = x_h(0); epi.ld_f16 = ws.p_act;
        if (bnorm) {
            epi.out_f32 = z_tape(0);
            MGT_TRY(GemmForwardRows<Epi::kBiasF32>(e, st, a1_h, ws.p_bt, hw.wh, hw.p2, B, H2, H1, epi));
            MGT_TRY(bn_forward(0));
        } else {
            MGT_TRY(GemmForwardRows<Epi::kBiasReluF32F16>(e, st, a1_h, ws.p_bt, hw.wh, hw.p2, B, H2, H1, epi));
        }
    }
    if (!timer.Mark(profile ? &profile->hidden_forward_ms : nullptr)) return MGT_CUDA_FAILURE;

    // ---- residual blocks forward (mlp_backward.cu:1294-1323)
    const bool chain = ChainEligible(e, s) && !bnorm;  // batch statistics need the whole batch between two layers: one kernel per layer
    const uint64_t w_layer_stride = R > 0 ? (uint64_t)(reinterpret_cast<const uint8_t*>(hw.w2[0]) - reinterpret_cast<const uint8_t*>(hw.w1[0])) : 16;
    ChainArgs ca{};
    ca.samples = B; ca.H = H2; ca.R = R; ca.tiles = (B + 127U) / 128U;
    ca.ld_f32 = ws.p_f32;
    ca.bits_s = reinterpret_cast<uint32_t*>(base + ws.off_bits);
    ca.bits_t = ca.bits_s + ws.bits_stride * (R + 1);
    ca.bits_stride = ws.bits_stride;
    if (chain) {
        ChainArgs f = ca;
        f.state_f32 = x_f32;
        f.bias = w + Fc1B(s, 0); f.bias_stride = (uint64_t)H2 * H2 + H2;
        f.tape_s = x_h(0); f.tape_s_stride = ws.x_stride / 2; f.ld_s = ws.p_act;
        f.tape_t = r1_h(0); f.tape_t_stride = ws.r1_stride / 2; f.ld_t = ws.p_act;
        MGT_TRY(LaunchChain<false>(e, st, hw.w1[0], hw.p2, w_layer_stride, R + 1, R, f));
    }
    for (uint32_t k = 0; k < R && !chain; ++k) {
        GemmArgs e1{};
        e1.bias = w + Fc1B(s, k); e1.out_f16 = r1_h(k); e1.ld_f16 = ws.p_act;
        MGT_TRY(GemmForward<Epi::kBiasReluF16>(e, st, x_h(k), ws.p_act, hw.w1[k], hw.p2, B, H2, H2, e1));
        GemmArgs e2{};
        e2.bias = w + Fc2B(s, k); e2.add_f32 = x_f32; e2.ld_add = ws.p_f32; e2.out_f32 = x_f32; e2.ld_f32 = ws.p_f32;
        e2.out_f16 = x_h(k + 1); e2.ld_f16 = ws.p_act;
        if (bnorm) {
            e2.out_f32 = z_tape(k + 1U);
            MGT_TRY(GemmForward<Epi::kBiasF32>(e, st, r1_h(k), ws.p_act, hw.w2[k], hw.p2, B, H2, H2, e2));
            MGT_TRY(bn_forward(k + 1U));
            continue;
        }
        MGT_TRY(GemmForward<Epi::kBiasResReluF32F16>(e, st, r1_h(k), ws.p_act, hw.w2[k], hw.p2, B, H2, H2, e2));
    }
    if (!timer.Mark(profile ? &profile->residual_forward_ms : nullptr)) return MGT_CUDA_FAILURE;

    // ---- output head, loss and the gradient entering the last block (mlp_backward.cu:1327-1364)
    __half* dz_cur = dz_tape(R);   // fp16 copy of the gradient w.r.t. the pre-activation the head feeds
    // the head also yields the fp32 column sums of dz: the bias gradient of the layer below it
    float* head_bias_dst = grad + (R > 0 ? Fc2B(s, R - 1) : HiddenBias(s));
    if (OUT == 1U) {
        HeadOut1Kernel<<<kHeadBlocks, kHeadThreads, 0, st>>>(w + OutputWeight(s), w + OutputBias(s), labels, x_f32, ws.p_f32, B, H2, dzf, dz_cur, ws.p_dz, head_partial, e->bf16_now);
        ReduceHeadKernel<<<(2 * H2 + 2 + kReduceCols - 1) / kReduceCols, 256, 0, st>>>(head_partial, kHeadBlocks, H2, grad + OutputWeight(s), loss, head_bias_dst);
        e->launches += 2;
    } else {
        float* dy = reinterpret_cast<float*>(base + ws.off_dy);
        __half* dy_h = reinterpret_cast<__half*>(base + ws.off_dyh);
        const size_t warp_smem = (kHeadThreads / 32) * OUT * sizeof(float);
        const size_t staged_smem = warp_smem + (size_t)H2 * (OUT | 1U) * sizeof(float);
        const bool stage_w = staged_smem <= kHeadStagedSmemLimit;
        const bool ce = e->options.loss_kind == MGT_LOSS_CROSS_ENTROPY;
        auto launch_head = [&](auto kernel, size_t smem) -> bool {
            if (smem > 48U * 1024U && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kHeadStagedSmemLimit) != cudaSuccess) return false;
            kernel<<<kHeadBlocks, kHeadThreads, smem, st>>>(hw.wout, hw.pout, w + OutputBias(s), labels, x_h(R), ws.p_act, x_f32, ws.p_f32, B, H2, OUT, dy, dy_h, ws.p_wout,
                                                           dzf, dz_cur, ws.p_dz, head_partial, e->bf16_now);
            return true;
        };
        const bool launched = stage_w ? (ce ? launch_head(HeadOutNKernel<true, true>, staged_smem) : launch_head(HeadOutNKernel<false, true>, staged_smem))
                                      : (ce ? launch_head(HeadOutNKernel<true, false>, warp_smem) : launch_head(HeadOutNKernel<false, false>, warp_smem));
        if (!launched) return MGT_CUDA_FAILURE;
        ReduceRowsKernel<<<1, 256, 0, st>>>(head_partial, kHeadBlocks, H2 + 1, 0, 1, loss);
        ReduceRowsKernel<<<(H2 + kReduceCols - 1) / kReduceCols, 256, 0, st>>>(head_partial, kHeadBlocks, H2 + 1, 1, H2, head_bias_dst);
        HeadOutNBiasGradKernel<<<OUT, 256, 0, st>>>(dy, B, OUT, grad + OutputBias(s));
        e->launches += 4;
        if (cudaGetLastError() != cudaSuccess) return MGT_CUDA_FAILURE;
        // grad W_out = x_R^T * dy (16-bit operands, fp32 accumulate, mlp_backward.cu:1349-1354): the split-K weight-gradient GEMM
        MGT_TRY(GemmGradWeights(e, st, x_h(R), ws.p_act, dy_h, ws.p_wout, B, H2, OUT, partial, ws.partial_floats, grad + OutputWeight(s)));
    }
    if (cudaGetLastError() != cudaSuccess) return MGT_CUDA_FAILURE;
    MGT_TRY(notify(OutputWeight(s), (uint64_t)H2 * OUT + OUT));
    if (!timer.Mark(profile ? &profile->output_ms : nullptr)) return MGT_CUDA_FAILURE;

    // ---- residual blocks backward (mlp_backward.cu:1367-1413). First the chain of input-gradient GEMMs,
    // block R-1 down to 0; every dz tensor is kept. dzf holds the running fp32 gradient (skip connection).
    const uint32_t dx_rows = PlanBackprop(e, B, H2, H2).rows;
    if (R > 0 && !chain && cudaMemsetAsync(colsum, 0, ws.colsum_floats * sizeof(float), st) != cudaSuccess) return MGT_CUDA_FAILURE;
    uint32_t colsum_rows = dx_rows;
    if (chain) {
        ChainArgs b = ca;
        b.state_f32 = dzf;
        b.tape_s = dz_tape(0); b.tape_s_stride = ws.dz_stride / 2; b.ld_s = ws.p_dz;
        b.tape_t = dz1_tape(0); b.tape_t_stride = ws.dz_stride / 2; b.ld_t = ws.p_dz;
        b.colsum = colsum; b.colsum_stride = ws.colsum_slot_floats;
        MGT_TRY(LaunchChain<true>(e, st, hw.w1[0], hw.p2, w_layer_stride, R + 1, R, b));
        colsum_rows = ca.tiles * 4U;
    }
    for (uint32_t rb = R; rb > 0 && !chain; --rb) {
        const uint32_t k = rb - 1U;
        if (bnorm) MGT_TRY(bn_backward(k + 1U, grad + Fc2B(s, k)));  // dz_tape(k + 1) = gradient w.r.t. the fc2 output; dzf goes down the skip path as it is
        GemmArgs d2{};  // dz1 = (dz2 * W2^T) * [r1 > 0]
        d2.mask = r1_h(k); d2.ld_mask = ws.p_act; d2.out_f16 = dz1_tape(k); d2.ld_f16 = ws.p_dz;
        MGT_TRY(GemmBackpropInput<Epi::kMaskF16>(e, st, dz_tape(k + 1), ws.p_dz, hw.w2[k], hw.p2, B, H2, H2, d2, colsum + ws.colsum_slot_floats * k, nullptr));
        GemmArgs d1{};  // next dz = (dz1 * W1^T + dz2) * [x_k > 0]: ReLU of the previous block (or of the hidden layer)
        d1.add_f32 = dzf; d1.ld_add = ws.p_f32; d1.out_f32 = dzf; d1.ld_f32 = ws.p_f32; d1.mask = x_h(k); d1.ld_mask = ws.p_act;
        d1.out_f16 = dz_tape(k); d1.ld_f16 = ws.p_dz;
        MGT_TRY(GemmBackpropInput<Epi::kAddMaskF32F16>(e, st, dz1_tape(k), ws.p_dz, hw.w1[k], hw.p2, B, H2, H2, d1,
                                                        colsum + ws.colsum_slot_floats * (R + k), nullptr));
    }
    if (!timer.Mark(profile ? &profile->residual_backward_ms : nullptr)) return MGT_CUDA_FAILURE;

    // Order of what follows: the dX GEMMs run first, down to the embedding gradient; the weight-gradient GEMMs of the tower
    // and of the hidden layer (which only read tapes) come last. The embedding table is 86 % of the parameters: this way
    // its gradient is complete - and the early-range hook can hand it to the exchange - while a third of a millisecond
    // of weight-gradient work is still to run. The gradient-ready notifications keep the reference's order.

    // ---- hidden layer backward, dX part (mlp_backward.cu:1417-1438): dz_tape(0) = dcur * [x0 > 0]
    dz_cur = dz_tape(0);
    if (bnorm) MGT_TRY(bn_backward(0, grad + HiddenBias(s)));
    if (half_ig) {
        // dz1T = (Wh * dzh^T) * [pre-activation of a1 > 0], the input-bias gradient from its row sums
        MGT_TRY(GemmBackpropInputRows(e, st, hw.wh, hw.p2, dz_cur, ws.p_dz, B, H1, H2, reinterpret_cast<uint32_t*>(base + ws.off_bits_h1), ws.ld_bits_h1, dz1_h,
                                      ws.p_bt, reinterpret_cast<float*>(base + ws.off_rowsum), ws.rowsum_rows, grad + InputBias(s)));
    } else {
        // --input-grad-fp16 0: the embedding gradient wants dz1 in fp32 (mlp_backward.cu:1433-1504, float one-hot GEMM).
        // da1 from the same fp16 operands with fp32 accumulation, masked in fp32, then the table gradient on CUDA cores.
        using namespace mgt::fp32path;
        const uint64_t bh1 = (uint64_t)B * H1;
        if (Sgemm<false, true>(st, B, H1, H2, dz_cur, ws.p_dz, hw.wh, hw.p2, da1_f32, H1) != cudaSuccess) return MGT_CUDA_FAILURE;
        MaskKernel<__half><<<GridFor(bh1, 256, e->sm_count), 256, 0, st>>>(da1_f32, nullptr, a1_h, H1, ws.p_bt, bh1, false, dz1_f32, true);
        ColumnSumKernel<<<(H1 + 7) / 8, 256, 0, st>>>(dz1_f32, B, H1, grad + InputBias(s));
        e->launches += 3;
        if (cudaGetLastError() != cudaSuccess) return MGT_CUDA_FAILURE;
    }
    if (!timer.Mark(profile ? &profile->hidden_backward_ms : nullptr)) return MGT_CUDA_FAILURE;

    // ---- embedding gradient: grad W_in = onehot^T * dz1  (mlp_backward.cu:1440-1504); the input-bias
    // gradient (mlp_backward.cu:1505) is the column sum written by the GEMM above
    if (!half_ig) {
        using namespace mgt::fp32path;
        EmbeddingGradKernel<float><<<dim3(s.state_len, (H1 + 63) / 64), 128, 2ULL * s.state_value_pad * 64 * sizeof(float), st>>>(
            reinterpret_cast<const uint8_t*>(states), dz1_f32, H1, B, s.state_value_pad, H1, grad);
        ++e->launches;
        if (cudaGetLastError() != cudaSuccess) return MGT_CUDA_FAILURE;
    } else {
        const uint32_t unit_rows = CfgEmbGrad::NACC * CfgEmbGrad::BN;
        GemmArgs a = BaseArgs(H1, IN, B, unit_rows, 1);
        const uint64_t tiles = (uint64_t)a.m_tiles * a.n_tiles;
        // Two splits keep fp32 atomics order-independent (0 + a + b == 0 + b + a); use them when one
        // split would leave a large part of the last wave idle.
        const uint64_t waves1 = (tiles + e->sm_count - 1) / e->sm_count;
        const uint64_t waves2 = (2 * tiles + e->sm_count - 1) / e->sm_count;
        const uint32_t splits = (a.k_chunks >= 2 && waves2 < 2 * waves1) ? 2U : 1U;
        a = BaseArgs(H1, IN, B, unit_rows, splits);
        a.out_f32 = grad; a.ld_f32 = H1;
        a.states = reinterpret_cast<const uint8_t*>(states); a.state_len = s.state_len; a.value_pad = s.state_value_pad; a.samples = B;
        a.in_rows = 0xFFFFFFFFU;  // no all-ones row in this direction
        if (a.splits > 1 && cudaMemsetAsync(grad, 0, (uint64_t)IN * H1 * sizeof(float), st) != cudaSuccess) return MGT_CUDA_FAILURE;
        CUtensorMap ta;
        MGT_MAP(e->Map(&ta, dz1_h, B, H1, ws.p_bt, 64, 128));
        MGT_TRY(LaunchGemm<CfgEmbGrad>(e, ta, ta, a, st));
    }
    // table and input bias are complete: tell a caller who asked to hear of it before the weight-gradient GEMMs are enqueued
    if (e->early_fn != nullptr && e->early_fn(e->early_user, 2U * R + 2U, 0, InputBias(s) + H1, stream_v) != MGT_OK) return MGT_CUDA_FAILURE;
    if (!timer.Mark(profile ? &profile->input_grad_ms : nullptr)) return MGT_CUDA_FAILURE;

    if (R > 0) {
        // weight gradients of all blocks: two grouped split-K GEMMs (fc2: r1_k^T dz2_k, fc1: x_k^T dz1_k)
        MGT_TRY(GemmGradWeightsGrouped(e, st, r1_h(0), ws.p_act, ws.r1_stride, dz_tape(1), ws.p_dz, ws.dz_stride, R, B, H2, H2, partial,
                                       ws.partial_floats, grad + Fc2W(s, 0), BlockParams(s)));
        MGT_TRY(GemmGradWeightsGrouped(e, st, x_h(0), ws.p_act, ws.x_stride, dz1_tape(0), ws.p_dz, ws.dz_stride, R, B, H2, H2, partial,
                                       ws.partial_floats, grad + Fc1W(s, 0), BlockParams(s)));
        // bias gradients: column sums of dz1_k -> b1_k, of the dz each fc1 GEMM produced -> b2_{k-1} (hidden bias for k = 0)
        ReduceDestinations dst{};
        for (uint32_t k = 0; k < R; ++k) {
            dst.offset[k] = Fc1B(s, k);
            dst.offset[R + k] = k > 0 ? Fc2B(s, k - 1) : HiddenBias(s);
        }
        // (with batch normalisation b2_k and the hidden bias got their gradients from the normalisation's backward pass)
        ReduceRowsGroupedKernel<<<dim3((H2 + kReduceCols - 1) / kReduceCols, bnorm ? R : 2 * R), 256, 0, st>>>(colsum, colsum_rows, H2, ws.colsum_slot_floats, grad, dst);
        ++e->launches;
        if (cudaGetLastError() != cudaSuccess) return MGT_CUDA_FAILURE;
        for (uint32_t rb = R; rb > 0; --rb) {
            MGT_TRY(notify(Fc2W(s, rb - 1U), (uint64_t)H2 * H2 + H2));
            MGT_TRY(notify(Fc1W(s, rb - 1U), (uint64_t)H2 * H2 + H2));
        }
    }
    if (!timer.Mark(profile ? &profile->residual_backward_ms : nullptr)) return MGT_CUDA_FAILURE;

    // ---- hidden layer backward, dW part; every kernel that reads the hidden weights was enqueued long before, so a caller
    // may update the range in place as soon as it is announced
    MGT_TRY(GemmGradWeightsRows(e, st, a1_h, ws.p_bt, dz_cur, ws.p_dz, B, H1, H2, partial, ws.partial_floats, grad + HiddenWeight(s)));
    MGT_TRY(notify(HiddenWeight(s), (uint64_t)H1 * H2 + H2));
    if (!timer.Mark(profile ? &profile->hidden_backward_ms : nullptr)) return MGT_CUDA_FAILURE;
    MGT_TRY(notify(0, InputBias(s) + H1));
    if (bnorm) MGT_TRY(notify(bn_base, 2ULL * (R + 1ULL) * H2));
    return MGT_OK;
}

mgt_status_t mgt_engine_set_train_options(mgt_engine_t* e, const mgt_train_options_t* options) {
    if (e == nullptr || options == nullptr) return MGT_INVALID_CONFIG;
    if (options->operand_format != MGT_OPERAND_FP16 && options->operand_format != MGT_OPERAND_BF16) return MGT_INVALID_CONFIG;
    if (options->loss_kind != MGT_LOSS_MSE && options->loss_kind != MGT_LOSS_CROSS_ENTROPY) return MGT_INVALID_CONFIG;
    if (options->batch_norm != 0 && !(options->bn_eps > 0.0f)) return MGT_INVALID_CONFIG;
    e->options = *options;
    return MGT_OK;
}

mgt_status_t mgt_engine_set_early_range_hook(mgt_engine_t* e, mgt_gradient_ready_fn fn, void* user) {
    if (e == nullptr) return MGT_INVALID_CONFIG;
    e->early_fn = fn;
    e->early_user = user;
    return MGT_OK;
}

mgt_status_t mgt_debug_gemm(mgt_engine_t* e, const uint16_t* a, uint32_t lda, int32_t a_mn, const uint16_t* b, uint32_t ldb, int32_t b_mn,
                            float* d, uint32_t m, uint32_t n, uint32_t k, uint32_t splits, float* partial_scratch, void* stream) {
    if (e == nullptr || a == nullptr || b == nullptr || d == nullptr || m == 0 || n == 0 || k == 0 || splits == 0) return MGT_INVALID_CONFIG;
    if (splits > 1 && partial_scratch == nullptr) return MGT_INVALID_CONFIG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    GemmArgs args = BaseArgs(m, n, k, 256, splits);
    // with a single split the accumulator tiles go straight into d, as 16-byte vectors when n is a multiple of 4
    if (args.splits == 1 && (n & 3U) == 0U && (reinterpret_cast<uintptr_t>(d) & 15U) != 0U) return MGT_INVALID_CONFIG;
    if ((reinterpret_cast<uintptr_t>(d) & 3U) != 0U) return MGT_INVALID_CONFIG;
    if (args.splits > 1 && (n & 3U) == 0U && (reinterpret_cast<uintptr_t>(partial_scratch) & 15U) != 0U) return MGT_INVALID_CONFIG;
    args.partial = args.splits > 1 ? partial_scratch : d;
    CUtensorMap ta, tb;
    const __half* ah = reinterpret_cast<const __half*>(a);
    const __half* bh = reinterpret_cast<const __half*>(b);
    if (a_mn) { MGT_MAP(e->Map(&ta, ah, m, k, lda, 64, 64)); } else { MGT_MAP(e->Map(&ta, ah, k, m, lda, 64, 128)); }
    if (b_mn) { MGT_MAP(e->Map(&tb, bh, n, k, ldb, 64, 64)); } else { MGT_MAP(e->Map(&tb, bh, k, n, ldb, 64, 256)); }
    mgt_status_t r;
    if (a_mn && b_mn) r = LaunchGemm<CfgDw<256>>(e, ta, tb, args, st);
    else if (a_mn) r = LaunchGemm<CfgDbgMK>(e, ta, tb, args, st);
    else if (b_mn) r = LaunchGemm<CfgDbgKM>(e, ta, tb, args, st);
    else r = LaunchGemm<CfgDbgKK>(e, ta, tb, args, st);
    if (r != MGT_OK) return r;
    if (args.splits > 1) {
        ReducePartialsKernel<<<GridFor((uint64_t)m * n, 256, e->sm_count), 256, 0, st>>>(partial_scratch, args.splits, (uint64_t)m * n, d);
        if (cudaGetLastError() != cudaSuccess) return MGT_CUDA_FAILURE;
    }
    return MGT_OK;
}

}  // extern "C"

// ---- split-K GEMM whose scratch is part of the library image ------------------------------------
// Device memory that this library reserves at load time on every GPU that uses it: the split-K
// partial sums of mgt_gemm_split_k_static_scratch and that entry point's status word.
static __device__ __align__(256) float g_static_partials[MGT_STATIC_SCRATCH_FLOATS];
static __device__ int g_static_status;

namespace {
struct StaticSlot {
    mgt_engine* engine = nullptr;   // host-side object only: descriptor cache, SM count, status-word address
    float* partials = nullptr;      // device address of g_static_partials on that device
};
StaticSlot g_static_slots[64];
std::mutex g_static_mu;

// One-time set-up per device, with that device current: resolve the DEVICE addresses of the two
// symbols above (in host code their names are only host-side handles) and look up the tensor-map
// encoder. Allocates no device memory.
mgt_status_t StaticSlotFor(int device, StaticSlot** out) {
    if (device < 0 || device >= 64) return MGT_INVALID_CONFIG;
    std::lock_guard<std::mutex> lock(g_static_mu);
    StaticSlot& slot = g_static_slots[device];
    if (slot.engine == nullptr) {
        void* partials = nullptr;
        void* status = nullptr;
        if (cudaGetSymbolAddress(&partials, g_static_partials) != cudaSuccess || partials == nullptr) return MGT_CUDA_FAILURE;
        if (cudaGetSymbolAddress(&status, g_static_status) != cudaSuccess || status == nullptr) return MGT_CUDA_FAILURE;
        cudaDeviceProp prop{};
        if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return MGT_CUDA_FAILURE;
        if (prop.major != 10) {
            std::fprintf(stderr, "mgt_b200: device %d is sm_%d%d; this library only runs on sm_100a (B200)\n", device, prop.major, prop.minor);
            return MGT_CUDA_FAILURE;
        }
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || fn == nullptr) return MGT_CUDA_FAILURE;
        auto* e = new mgt_engine();
        e->device = device;
        e->sm_count = prop.multiProcessorCount;
        e->encode = reinterpret_cast<EncodeTiledFn>(fn);
        e->status_word = static_cast<int*>(status);
        slot.engine = e;
        slot.partials = static_cast<float*>(partials);
    }
    *out = &slot;
    return MGT_OK;
}
}  // namespace

extern "C" mgt_status_t mgt_gemm_split_k_static_scratch(const uint16_t* a, uint32_t lda, int32_t a_mn, const uint16_t* b, uint32_t ldb, int32_t b_mn,
                                                        float* d, uint32_t m, uint32_t n, uint32_t k, uint32_t splits, void* stream) {
    if (a == nullptr || b == nullptr || d == nullptr || m == 0 || n == 0 || k == 0 || splits == 0) return MGT_INVALID_CONFIG;
    const uint32_t k_chunks = (k + 63U) / 64U;
    const uint64_t used_splits = splits > k_chunks ? k_chunks : splits;
    if (used_splits > 1 && used_splits * m * n > static_cast<uint64_t>(MGT_STATIC_SCRATCH_FLOATS)) {
        std::fprintf(stderr, "mgt_gemm_split_k_static_scratch: %llu splits of a %u x %u result need %llu floats of scratch, the built-in buffer holds %u\n",
                     static_cast<unsigned long long>(used_splits), m, n, static_cast<unsigned long long>(used_splits * m * n),
                     static_cast<unsigned>(MGT_STATIC_SCRATCH_FLOATS));
        return MGT_CAPACITY_EXCEEDED;
    }
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return MGT_CUDA_FAILURE;
    StaticSlot* slot = nullptr;
    MGT_TRY(StaticSlotFor(device, &slot));
    // every valid element of the partial planes is written before the reduction reads it, so nothing
    // needs clearing between calls; what an earlier call left beyond that is never read
    return mgt_debug_gemm(slot->engine, a, lda, a_mn, b, ldb, b_mn, d, m, n, k, splits, slot->partials, stream);
}

extern "C" mgt_status_t mgt_static_scratch_check(void* stream, int32_t* out_device_code) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return MGT_CUDA_FAILURE;
    StaticSlot* slot = nullptr;
    MGT_TRY(StaticSlotFor(device, &slot));
    // the hidden per-device engine's status word is the built-in g_static_status: same read-and-clear as mgt_engine_check
    return mgt_engine_check(slot->engine, stream, out_device_code);
}
