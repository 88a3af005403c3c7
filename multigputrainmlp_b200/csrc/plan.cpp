// Plan of a training run (see host_plan.hpp). Pure host code, no CUDA.
#include "host_plan.hpp"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <functional>
#include <map>

namespace mgt {
namespace host {
namespace {

uint64_t RoundUp64(uint64_t v, uint64_t a) { return a == 0 ? v : (v + a - 1) / a * a; }
uint32_t RoundUp32(uint32_t v, uint32_t a) { return a == 0 ? v : (v + a - 1) / a * a; }
bool PowerOfTwo(uint32_t v) { return v != 0 && (v & (v - 1)) == 0; }

bool ToU32(const char* text, uint32_t* out) {
    // std::stoul semantics of the reference: leading digits are enough, the value must fit 32 bits
    char* end = nullptr;
    if (text == nullptr || *text == '\0') return false;
    const char* p = text;
    while (*p == ' ' || *p == '\t' || *p == '\n') ++p;
    if (*p == '-') {  // stoul accepts a sign and wraps; such values never fit 32 bits in a meaningful way
        const unsigned long v = std::strtoul(text, &end, 10);
        if (end == text) return false;
        *out = static_cast<uint32_t>(v);
        return v <= 0xffffffffUL;
    }
    const unsigned long v = std::strtoul(text, &end, 10);
    if (end == text) return false;
    *out = static_cast<uint32_t>(v);
    return v <= 0xffffffffUL;
}
bool ToU64(const char* text, uint64_t* out) {
    char* end = nullptr;
    if (text == nullptr || *text == '\0') return false;
    const unsigned long long v = std::strtoull(text, &end, 10);
    if (end == text) return false;
    *out = v;
    return true;
}
bool ToF32(const char* text, float* out) {
    char* end = nullptr;
    if (text == nullptr || *text == '\0') return false;
    const float v = std::strtof(text, &end);
    if (end == text) return false;
    *out = v;
    return true;
}
bool ToBool(const char* text, bool* out) {  // tool:434-445
    static const char* yes[] = {"1", "true", "yes", "on"};
    static const char* no[] = {"0", "false", "no", "off"};
    for (const char* y : yes) if (std::strcmp(text, y) == 0) { *out = true; return true; }
    for (const char* n : no) if (std::strcmp(text, n) == 0) { *out = false; return true; }
    return false;
}

}  // namespace

bool ParseTrainOptions(int argc, const char* const* argv, TrainOptions* o) {
    using Setter = std::function<bool(const char*)>;
    auto u32 = [](uint32_t* dst) { return Setter([dst](const char* v) { return ToU32(v, dst); }); };
    auto u64 = [](uint64_t* dst) { return Setter([dst](const char* v) { return ToU64(v, dst); }); };
    auto f32 = [](float* dst) { return Setter([dst](const char* v) { return ToF32(v, dst); }); };
    auto flag = [](bool* dst) { return Setter([dst](const char* v) { return ToBool(v, dst); }); };
    auto text = [](std::string* dst) { return Setter([dst](const char* v) { *dst = v; return true; }); };
    const std::map<std::string, Setter> table = {
        {"--output-dir", text(&o->output_dir)}, {"--steps", u32(&o->steps)}, {"--device-id", u32(&o->device_id)},
        {"--world-size", u32(&o->world_size)}, {"--global-rank", u32(&o->global_rank)}, {"--local-rank", u32(&o->local_rank)},
        {"--group-id", u32(&o->group_id)}, {"--target-id", u32(&o->target_id)}, {"--state-len", u32(&o->state_len)},
        {"--state-value-count", u32(&o->state_value_count)}, {"--move-count", u32(&o->move_count)},
        {"--state-alignment", u32(&o->state_alignment)}, {"--batch-size", u32(&o->batch_size)}, {"--k-min", u32(&o->k_min)},
        {"--k-max", u32(&o->k_max)}, {"--walkers", u32(&o->walkers)}, {"--hd1", u32(&o->hd1)}, {"--hd2", u32(&o->hd2)},
        {"--nrd", u32(&o->nrd)}, {"--output-dim", u32(&o->output_dim)}, {"--hidden-alignment", u32(&o->hidden_alignment)},
        {"--gradient-carousel-slots", u32(&o->gradient_carousel_slots)},
        {"--input-grad-partial-chunks", u32(&o->input_grad_partial_chunks)},
        {"--input-grad-positions-per-block", u32(&o->input_grad_positions_per_block)},
        {"--input-grad-position-tile", u32(&o->input_grad_position_tile)}, {"--input-grad-fp16", flag(&o->input_grad_fp16)},
        {"--linear-fp16", flag(&o->linear_fp16)}, {"--persistent-half-weights", flag(&o->persistent_half_weights)},
        {"--allreduce-bucket-bytes", u64(&o->allreduce_bucket_bytes)}, {"--lt-workspace-bytes", u64(&o->lt_workspace_bytes)},
        {"--seed", u64(&o->seed)}, {"--lr", f32(&o->lr)}, {"--weight-decay", f32(&o->weight_decay)},
        {"--write-artifacts", flag(&o->write_artifacts)}, {"--backward-profile", flag(&o->backward_profile)},
        {"--overlap-allreduce", flag(&o->overlap_allreduce)}, {"--nccl-id-file", text(&o->nccl_id_file)},
        {"--resume-checkpoint", text(&o->resume_checkpoint)},
        {"--checkpoint-period-steps", u32(&o->checkpoint_period_steps)}, {"--resume-step", flag(&o->resume_step)},
        {"--puzzle-json", text(&o->puzzle_json)}, {"--target-bin", text(&o->target_bin)},
        {"--operand-format", text(&o->operand_format)}, {"--loss", text(&o->loss)},
        {"--batch-norm", flag(&o->batch_norm)}, {"--bn-eps", f32(&o->bn_eps)}, {"--bn-momentum", f32(&o->bn_momentum)},
    };
    for (int i = 1; i < argc; i += 2) {
        if (i + 1 >= argc) return false;
        const auto it = table.find(argv[i]);
        if (it == table.end() || !it->second(argv[i + 1])) return false;
    }
    return ValidateTrainOptions(*o);
}

bool ValidateTrainOptions(const TrainOptions& o) {
    if (o.steps == 0 || o.world_size == 0 || o.global_rank >= o.world_size || o.batch_size == 0) return false;
    if (o.state_len == 0 || o.state_value_count == 0 || o.move_count == 0) return false;
    if (!PowerOfTwo(o.state_alignment) || !PowerOfTwo(o.hidden_alignment)) return false;
    if (o.hd1 == 0 || o.hd2 == 0 || o.output_dim == 0) return false;
    if (o.k_min == 0 || o.k_min > o.k_max) return false;
    if (!(o.lr > 0.0f) || o.weight_decay < 0.0f) return false;
    if (o.world_size > 128) return false;  // kMaxRuntimeDevices, config.hpp:22
    if (o.gradient_carousel_slots == 0 || o.input_grad_partial_chunks == 0 || o.input_grad_positions_per_block == 0) return false;
    if (o.allreduce_bucket_bytes == 0 || o.allreduce_bucket_bytes % sizeof(float) != 0) return false;
    if (o.operand_format != "fp16" && o.operand_format != "bf16") return false;
    if (o.loss != "mse" && o.loss != "ce") return false;
    if (o.loss == "ce" && (o.output_dim < 2 || o.k_max > o.output_dim)) return false;  // one logit per walk depth
    if ((o.loss == "ce" || o.operand_format == "bf16" || o.batch_norm) && !o.linear_fp16) return false;
    if (o.batch_norm && (!(o.bn_eps > 0.0f) || !(o.bn_momentum >= 0.0f && o.bn_momentum <= 1.0f))) return false;
    return true;
}

const char* ParamRoleName(ParamRole role) {
    static const char* names[] = {"unknown", "input_embedding", "input_bias", "hidden_weight", "hidden_bias", "residual_fc1_weight",
                                  "residual_fc1_bias", "residual_fc2_weight", "residual_fc2_bias", "output_weight", "output_bias"};
    const uint32_t i = static_cast<uint32_t>(role);
    return i <= 10 ? names[i] : names[0];
}
const char* LinearPhaseName(uint32_t phase) { return phase == 1 ? "forward" : phase == 2 ? "backward_weights" : phase == 3 ? "backward_input" : "unknown"; }
const char* LinearBackendName(uint32_t b) { return b == 1 ? "custom_kernel" : b == 2 ? "library_tensorop" : b == 3 ? "cutlass_large_k_reduction_candidate" : "unknown"; }

const char* InputGradBackendName(const TrainOptions& o) {
    if (o.input_grad_position_tile > 0) return o.input_grad_fp16 ? "position_tiled_one_hot_half_gemm" : "position_tiled_one_hot_float_gemm";
    if (o.input_grad_partial_chunks > 1) return "position_chunked_owner_write";
    if (o.input_grad_positions_per_block > 1) return "position_group_owner_write";
    return o.input_grad_fp16 ? "dense_one_hot_half_gemm" : "dense_one_hot_float_gemm";
}

namespace {

// The backend class the reference would pick (native/src/train_plan.cpp:35-48); kept in the manifest
// because consumers of linear_ops.json read it, although every op here runs on this library's kernels.
uint32_t BackendClass(ParamRole role, uint32_t phase, uint32_t m, uint32_t n, uint32_t k, uint32_t output_dim) {
    if (role == ParamRole::kInputEmbedding && phase == 1) return 1;
    if (role == ParamRole::kOutputWeight && output_dim == 1) return 1;
    if (role == ParamRole::kInputEmbedding && phase == 2 && m >= 4096 && n >= 4096 && k >= 8192) return 3;
    return 2;
}

void PushOp(std::vector<LinearOp>* ops, uint32_t phase, ParamRole role, uint32_t block, bool ta, bool tb, uint32_t m, uint32_t n,
            uint32_t k, uint32_t output_dim, bool tail) {
    LinearOp op{};
    op.op_id = static_cast<uint32_t>(ops->size());
    op.phase = phase; op.role = role; op.block_index = block; op.transpose_a = ta; op.transpose_b = tb;
    op.m = m; op.n = n; op.k = k;
    op.lhs_rows = ta ? k : m; op.lhs_cols = ta ? m : k;
    op.rhs_rows = tb ? n : k; op.rhs_cols = tb ? k : n;
    op.output_rows = m; op.output_cols = n;
    op.backend = BackendClass(role, phase, m, n, k, output_dim);
    op.tensor_core_eligible = m && n && k && m % 8 == 0 && n % 8 == 0 && k % 8 == 0;
    op.logical_tail_masked = tail;
    ops->push_back(op);
}

}  // namespace

bool BuildTrainPlan(const TrainOptions& o, TrainPlan* out) {
    if (out == nullptr || !ValidateTrainOptions(o)) return false;
    TrainPlan p{};
    p.options = o;
    if (p.options.walkers == 0) p.options.walkers = o.k_max == 0 ? 0 : o.batch_size / o.k_max;  // tool:463
    p.padded_state_dim = RoundUp32(o.state_len, o.state_alignment);
    p.state_capacity_bytes = p.padded_state_dim;
    p.fits_state_record = p.state_capacity_bytes <= 80;
    p.physical_hd1 = RoundUp32(o.hd1, o.hidden_alignment);
    p.physical_hd2 = RoundUp32(o.hd2, o.hidden_alignment);
    const uint32_t in_rows = o.state_len * o.state_value_count;
    const uint32_t H1 = p.physical_hd1, H2 = p.physical_hd2;

    // parameter blocks in flat order (native/src/model_layout.cpp:40-126)
    auto add = [&](ParamRole role, uint32_t lr, uint32_t lc, uint32_t pr, uint32_t pc, uint32_t block) {
        ParamBlock b{};
        b.role = role; b.block_index = block; b.rows = pr; b.cols = pc; b.logical_rows = lr; b.logical_cols = lc;
        b.offset_bytes = p.total_bytes;
        b.size_bytes = static_cast<uint64_t>(pr) * pc * sizeof(float);
        b.param_offset = p.total_params;
        p.blocks.push_back(b);
        p.total_bytes = RoundUp64(p.total_bytes + b.size_bytes, 64);
        p.total_params += static_cast<uint64_t>(pr) * pc;
        p.logical_params += static_cast<uint64_t>(lr) * lc;
    };
    add(ParamRole::kInputEmbedding, in_rows, o.hd1, in_rows, H1, 0);
    add(ParamRole::kInputBias, 1, o.hd1, 1, H1, 0);
    add(ParamRole::kHiddenWeight, o.hd1, o.hd2, H1, H2, 0);
    add(ParamRole::kHiddenBias, 1, o.hd2, 1, H2, 0);
    for (uint32_t b = 0; b < o.nrd; ++b) {
        add(ParamRole::kResidualFc1Weight, o.hd2, o.hd2, H2, H2, b);
        add(ParamRole::kResidualFc1Bias, 1, o.hd2, 1, H2, b);
        add(ParamRole::kResidualFc2Weight, o.hd2, o.hd2, H2, H2, b);
        add(ParamRole::kResidualFc2Bias, 1, o.hd2, 1, H2, b);
    }
    add(ParamRole::kOutputWeight, o.hd2, o.output_dim, H2, o.output_dim, 0);
    add(ParamRole::kOutputBias, 1, o.output_dim, 1, o.output_dim, 0);
    if (p.total_params == 0 || p.total_bytes == 0) return false;

    // gradient buckets: the padded byte total cut into bucket-sized pieces (train_plan.cpp:10-29)
    p.gradient_bucket_count = static_cast<uint32_t>((p.total_bytes + o.allreduce_bucket_bytes - 1) / o.allreduce_bucket_bytes);

    // linear-operation manifest (train_plan.cpp:82-155): forward ops, then backward in execution order
    const uint32_t B = o.batch_size, OUT = o.output_dim;
    const bool t1 = o.hd1 != H1, t2 = o.hd2 != H2;
    std::vector<LinearOp>& ops = p.linear_ops;
    PushOp(&ops, 1, ParamRole::kInputEmbedding, 0, false, false, B, H1, o.state_len, OUT, t1);
    PushOp(&ops, 1, ParamRole::kHiddenWeight, 0, false, false, B, H2, H1, OUT, t1 || t2);
    for (uint32_t b = 0; b < o.nrd; ++b) {
        PushOp(&ops, 1, ParamRole::kResidualFc1Weight, b, false, false, B, H2, H2, OUT, t2);
        PushOp(&ops, 1, ParamRole::kResidualFc2Weight, b, false, false, B, H2, H2, OUT, t2);
    }
    PushOp(&ops, 1, ParamRole::kOutputWeight, 0, false, false, B, OUT, H2, OUT, t2);
    PushOp(&ops, 2, ParamRole::kOutputWeight, 0, true, false, H2, OUT, B, OUT, t2);
    PushOp(&ops, 3, ParamRole::kOutputWeight, 0, false, true, B, H2, OUT, OUT, t2);
    for (uint32_t rb = o.nrd; rb > 0; --rb) {
        const uint32_t b = rb - 1;
        PushOp(&ops, 2, ParamRole::kResidualFc2Weight, b, true, false, H2, H2, B, OUT, t2);
        PushOp(&ops, 3, ParamRole::kResidualFc2Weight, b, false, true, B, H2, H2, OUT, t2);
        PushOp(&ops, 2, ParamRole::kResidualFc1Weight, b, true, false, H2, H2, B, OUT, t2);
        PushOp(&ops, 3, ParamRole::kResidualFc1Weight, b, false, true, B, H2, H2, OUT, t2);
    }
    PushOp(&ops, 2, ParamRole::kHiddenWeight, 0, true, false, H1, H2, B, OUT, t1 || t2);
    PushOp(&ops, 3, ParamRole::kHiddenWeight, 0, false, true, B, H1, H2, OUT, t1 || t2);
    PushOp(&ops, 2, ParamRole::kInputEmbedding, 0, true, false, in_rows, H1, B, OUT, t1);

    // per-rank byte budget (native/src/memory_plan.cpp:30-69)
    MemoryPlan& mp = p.memory;
    auto a256 = [](uint64_t v) { return RoundUp64(v, 256); };
    mp.weights_bytes = mp.optimizer_m_bytes = mp.optimizer_v_bytes = mp.gradient_bytes = p.total_bytes;
    mp.gradient_carousel_bytes = mp.gradient_bytes * o.gradient_carousel_slots;
    mp.states_bytes = static_cast<uint64_t>(B) * p.padded_state_dim;
    mp.labels_bytes = static_cast<uint64_t>(B) * OUT * sizeof(float);
    mp.walk_meta_bytes = static_cast<uint64_t>(B) * 16;
    const uint64_t a1 = a256(static_cast<uint64_t>(B) * H1 * 4), a2 = a256(static_cast<uint64_t>(B) * H2 * 4);
    const uint64_t tape = a256(static_cast<uint64_t>(B) * H2 * o.nrd * 3ULL * 4), outb = a256(static_cast<uint64_t>(B) * OUT * 4);
    mp.layout_generate_bytes = a256(mp.states_bytes + mp.labels_bytes + mp.walk_meta_bytes);
    mp.layout_forward_bytes = a256(a1 + a2 + tape + outb);
    mp.layout_backward_bytes = a256(outb + a2 + tape + a1);
    mp.layout_allreduce_bytes = mp.gradient_bytes * o.gradient_carousel_slots;
    mp.layout_checkpoint_bytes = a256(mp.weights_bytes + 4096);
    mp.training_scratch_bytes = std::max({mp.layout_generate_bytes, mp.layout_forward_bytes, mp.layout_backward_bytes,
                                          mp.layout_allreduce_bytes, mp.layout_checkpoint_bytes});
    mp.total_rank_bytes = a256(mp.weights_bytes + mp.optimizer_m_bytes + mp.optimizer_v_bytes + mp.gradient_carousel_bytes + mp.training_scratch_bytes);
    if (mp.total_rank_bytes == 0 || p.gradient_bucket_count == 0) return false;
    *out = std::move(p);
    return true;
}

void BuildCyclicPuzzle(const TrainPlan& plan, uint8_t* moves, uint8_t* target) {
    const uint32_t L = plan.options.state_len, mc = plan.options.move_count;
    std::memset(moves, 0, 18 * 80);
    std::memset(target, 0, 80);
    for (uint32_t mv = 0; mv < 18; ++mv)
        for (uint32_t i = 0; i < L && i < 80; ++i) moves[mv * 80 + i] = static_cast<uint8_t>(mv < mc ? (i + mv + 1) % L : i);
    for (uint32_t i = 0; i < L && i < 80; ++i) target[i] = static_cast<uint8_t>(i);
}

int LoadPuzzleFiles(const std::string& group_json, const std::string& target_bin, uint32_t group_id, uint32_t state_len, uint32_t move_count,
                    uint8_t* moves, uint8_t* target) {
    if (moves == nullptr || target == nullptr || state_len == 0 || state_len > 72 || move_count == 0 || move_count > 18) return 2;
    std::ifstream json(group_json, std::ios::binary);
    if (!json) return 6;
    // every run of digits (with an optional leading minus) is a value; names and punctuation are skipped
    std::vector<long long> values;
    {
        long long value = 0;
        bool in_number = false, negative = false;
        char ch = 0, prev = 0;
        auto flush = [&]() {
            if (in_number) values.push_back(negative ? -value : value);
            in_number = false;
            negative = false;
            value = 0;
        };
        while (json.get(ch)) {
            if (ch >= '0' && ch <= '9') {
                if (!in_number) negative = prev == '-';
                in_number = true;
                if (value < (1LL << 40)) value = value * 10 + (ch - '0');
            } else {
                flush();
            }
            prev = ch;
        }
        flush();
    }
    const size_t required = 3 + static_cast<size_t>(move_count) * state_len;
    if (values.size() < required) return 2;
    if (values[0] != static_cast<long long>(group_id) || values[1] != static_cast<long long>(state_len) || values[2] != static_cast<long long>(move_count)) return 2;
    std::memset(moves, 0, 18 * 80);
    size_t pos = 3;
    for (uint32_t mv = 0; mv < 18; ++mv) {
        uint8_t* rec = moves + mv * 80;
        if (mv < move_count) {
            bool seen[80] = {};
            for (uint32_t i = 0; i < state_len; ++i) {
                const long long v = values[pos++];
                if (v < 0 || v >= static_cast<long long>(state_len) || seen[v]) return 2;  // not a permutation
                seen[v] = true;
                rec[i] = static_cast<uint8_t>(v);
            }
            for (uint32_t i = state_len; i < 80; ++i) rec[i] = static_cast<uint8_t>(i);  // pad positions stay where they are
        } else {
            for (uint32_t i = 0; i < 80; ++i) rec[i] = static_cast<uint8_t>(i);
        }
    }
    std::ifstream bin(target_bin, std::ios::binary);
    if (!bin) return 6;
    std::memset(target, 0, 80);
    bin.read(reinterpret_cast<char*>(target), state_len);
    if (bin.gcount() != static_cast<std::streamsize>(state_len)) return 2;
    char extra = 0;
    if (bin.read(&extra, 1)) return 2;  // longer than one state
    return 0;
}

void InitialWeights(std::vector<float>* w) {
    for (uint64_t i = 0; i < w->size(); ++i) (*w)[i] = static_cast<float>((static_cast<int>(i % 29) - 14) * 0.0001);
}

}  // namespace host
}  // namespace mgt
