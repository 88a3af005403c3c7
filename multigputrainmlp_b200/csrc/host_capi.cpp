// C entry points over the host-side plan and artefact writers (see include/mgt_b200.h).
#include "../../include/mgt_b200.h"
#include "host_plan.hpp"

#include <cmath>
#include <algorithm>
#include <filesystem>
#include <string>
#include <vector>

using namespace mgt::host;

namespace {
bool PlanFromArgs(int32_t argc, const char* const* argv, TrainPlan* plan) {
    TrainOptions o;
    std::vector<const char*> full;
    full.push_back("mgt_native_train");
    for (int32_t i = 0; i < argc; ++i) full.push_back(argv[i]);
    if (!ParseTrainOptions(static_cast<int>(full.size()), full.data(), &o)) return false;
    return BuildTrainPlan(o, plan);
}
}  // namespace

extern "C" {

mgt_status_t mgt_plan_summary(int32_t argc, const char* const* argv, uint64_t* out, uint32_t out_count) {
    TrainPlan p;
    if (out == nullptr || out_count < MGT_PLAN_SUMMARY_FIELDS || !PlanFromArgs(argc, argv, &p)) return MGT_INVALID_CONFIG;
    const uint64_t v[MGT_PLAN_SUMMARY_FIELDS] = {
        p.padded_state_dim, p.physical_hd1, p.physical_hd2, p.blocks.size(), p.linear_ops.size(), p.gradient_bucket_count,
        p.total_params, p.total_bytes, p.memory.total_rank_bytes, p.memory.training_scratch_bytes, p.logical_params,
        p.fits_state_record ? 1ULL : 0ULL, p.memory.states_bytes, p.memory.layout_allreduce_bytes, p.options.walkers, p.state_capacity_bytes};
    for (uint32_t i = 0; i < MGT_PLAN_SUMMARY_FIELDS; ++i) out[i] = v[i];
    return MGT_OK;
}

mgt_status_t mgt_plan_linear_op(int32_t argc, const char* const* argv, uint32_t index, uint32_t* out, uint32_t out_count) {
    TrainPlan p;
    if (out == nullptr || out_count < MGT_PLAN_LINEAR_OP_FIELDS || !PlanFromArgs(argc, argv, &p) || index >= p.linear_ops.size()) return MGT_INVALID_CONFIG;
    const LinearOp& op = p.linear_ops[index];
    const uint32_t v[MGT_PLAN_LINEAR_OP_FIELDS] = {op.op_id, op.phase, static_cast<uint32_t>(op.role), op.block_index, op.transpose_a ? 1U : 0U,
                                                   op.transpose_b ? 1U : 0U, op.m, op.n, op.k, op.backend, op.tensor_core_eligible ? 1U : 0U,
                                                   op.logical_tail_masked ? 1U : 0U, op.lhs_rows, op.rhs_cols};
    for (uint32_t i = 0; i < MGT_PLAN_LINEAR_OP_FIELDS; ++i) out[i] = v[i];
    return MGT_OK;
}

mgt_status_t mgt_plan_write_files(int32_t argc, const char* const* argv, const char* dir, int32_t overlap_allreduce, int32_t comm_enabled, int32_t resumed) {
    TrainPlan p;
    if (dir == nullptr || !PlanFromArgs(argc, argv, &p)) return MGT_INVALID_CONFIG;
    std::error_code ec;
    std::filesystem::create_directories(dir, ec);
    const bool ok = WriteMetadataEnv(dir, p, overlap_allreduce != 0, comm_enabled != 0, resumed != 0) && WriteLayersJson(dir, p) && WriteLinearOpsManifest(dir, p);
    return ok ? MGT_OK : MGT_IO_FAILURE;
}

mgt_status_t mgt_format_step_record(int32_t argc, const char* const* argv, const mgt_step_record_t* record, int32_t overlap_allreduce, int32_t comm_enabled,
                                    int32_t resumed, char* start_line, char* log_line, char* profile_row, uint32_t capacity) {
    TrainPlan p;
    if (record == nullptr || capacity == 0 || !PlanFromArgs(argc, argv, &p)) return MGT_INVALID_CONFIG;
    StepRecord r{};
    r.step = record->step; r.loss = record->loss; r.step_ms = record->step_ms; r.walk_ms = record->walk_ms; r.backward_ms = record->backward_ms;
    r.allreduce_ms = record->allreduce_ms; r.adam_ms = record->adam_ms; r.memory_bytes = record->memory_bytes;
    r.overlap_ranges = record->overlap_ranges; r.overlap_chunks = record->overlap_chunks;
    for (int i = 0; i < 7; ++i) r.bw[i] = record->backward_stage_ms[i];
    auto put = [&](char* dst, const std::string& text) {
        if (dst == nullptr) return true;
        if (text.size() + 1 > capacity) return false;
        std::copy(text.begin(), text.end(), dst);
        dst[text.size()] = '\0';
        return true;
    };
    const bool ok = put(start_line, StartLogLine(p, overlap_allreduce != 0, comm_enabled != 0, resumed != 0)) && put(log_line, StepLogLine(p, r)) &&
                    put(profile_row, StepProfileRow(p, r, overlap_allreduce != 0));
    return ok ? MGT_OK : MGT_CAPACITY_EXCEEDED;
}

uint16_t mgt_export_float_to_fp16(float value) { return ExportFloatToFp16(value); }

mgt_status_t mgt_fold_batch_norm(const mgt_mlp_shape_t* shape, float* weights, const float* scale_shift, const float* running_stats, float eps) {
    if (shape == nullptr || weights == nullptr || scale_shift == nullptr || running_stats == nullptr || !(eps > 0.0f)) return MGT_INVALID_CONFIG;
    if (mgt_validate_mlp_shape(shape) != MGT_OK) return MGT_INVALID_CONFIG;
    const uint64_t H1 = shape->hd1, H2 = shape->hd2, R = shape->residual_blocks;
    const uint64_t hidden_w = (uint64_t)shape->state_len * shape->state_value_pad * H1 + H1, hidden_b = hidden_w + H1 * H2, tower = hidden_b + H2;
    // y = gamma * (z - mean) / sqrt(var + eps) + beta with z = x W + b  ==  x (W diag(s)) + ((b - mean) s + beta),  s = gamma / sqrt(var + eps)
    auto fold = [&](uint64_t layer, float* w, uint64_t rows, float* b) {
        const float* gamma = scale_shift + 2ULL * layer * H2;
        const float* beta = gamma + H2;
        const float* mean = running_stats + 2ULL * layer * H2;
        const float* var = mean + H2;
        for (uint64_t j = 0; j < H2; ++j) {
            const float s = gamma[j] / std::sqrt(var[j] + eps);
            for (uint64_t i = 0; i < rows; ++i) w[i * H2 + j] *= s;
            b[j] = (b[j] - mean[j]) * s + beta[j];
        }
    };
    fold(0, weights + hidden_w, H1, weights + hidden_b);
    for (uint64_t k = 0; k < R; ++k) {
        float* fc2_w = weights + tower + k * 2ULL * (H2 * H2 + H2) + H2 * H2 + H2;
        fold(k + 1ULL, fc2_w, H2, fc2_w + H2 * H2);
    }
    return MGT_OK;
}

mgt_status_t mgt_load_puzzle_definition(const char* group_json, const char* target_bin, uint32_t group_id, uint32_t state_len, uint32_t move_count,
                                        mgt_train_state_t* moves, mgt_train_state_t* target) {
    if (group_json == nullptr || target_bin == nullptr || moves == nullptr || target == nullptr) return MGT_INVALID_PUZZLE;
    return static_cast<mgt_status_t>(LoadPuzzleFiles(group_json, target_bin, group_id, state_len, move_count, reinterpret_cast<uint8_t*>(moves),
                                                     reinterpret_cast<uint8_t*>(target)));
}

mgt_status_t mgt_write_run_artifacts(int32_t argc, const char* const* argv, const char* dir, const float* weights, const float* adam_m, const float* adam_v) {
    TrainPlan p;
    if (dir == nullptr || weights == nullptr || adam_m == nullptr || adam_v == nullptr || !PlanFromArgs(argc, argv, &p)) return MGT_INVALID_CONFIG;
    const std::vector<float> w(weights, weights + p.total_params), m(adam_m, adam_m + p.total_params), v(adam_v, adam_v + p.total_params);
    std::error_code ec;
    std::filesystem::create_directories(dir, ec);
    return WriteWeights(dir, p, w) && WriteCheckpoint(dir, p, w, m, v) ? MGT_OK : MGT_IO_FAILURE;
}

mgt_status_t mgt_read_checkpoint(const char* checkpoint_dir, uint64_t param_count, float* weights, float* adam_m, float* adam_v) {
    if (checkpoint_dir == nullptr || param_count == 0 || weights == nullptr || adam_m == nullptr || adam_v == nullptr) return MGT_INVALID_CONFIG;
    std::vector<float> w(param_count), m(param_count), v(param_count);
    if (!ReadCheckpoint(checkpoint_dir, &w, &m, &v)) return MGT_IO_FAILURE;
    std::copy(w.begin(), w.end(), weights);
    std::copy(m.begin(), m.end(), adam_m);
    std::copy(v.begin(), v.end(), adam_v);
    return MGT_OK;
}

}  // extern "C"
