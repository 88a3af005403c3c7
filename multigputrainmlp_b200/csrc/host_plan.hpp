// Host-side plan of a training run: configuration, flat parameter layout, linear-operation
// manifest, gradient buckets and the per-rank byte budget. These numbers feed metadata.env,
// layers.json, linear_ops.json and profile.jsonl, whose contents are part of the drop-in contract.
// Counterparts in the reference: native/include/mgt/config.hpp, model_layout.hpp, train_plan.hpp,
// memory_plan.hpp and their .cpp files.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace mgt {
namespace host {

// Command-line options of mgt_native_train with the binary's defaults
// (native/tools/mgt_native_train_smoke.cu:26-65).
struct TrainOptions {
    std::string output_dir = "runs/native-smoke";
    uint32_t steps = 4, device_id = 0, world_size = 1, global_rank = 0, local_rank = 0;
    uint32_t group_id = 888, target_id = 0, state_len = 72, state_value_count = 72, move_count = 18, state_alignment = 16;
    uint32_t batch_size = 64, k_min = 1, k_max = 9, walkers = 0;
    uint32_t hd1 = 5, hd2 = 3, nrd = 1, output_dim = 1, hidden_alignment = 8;
    uint32_t gradient_carousel_slots = 3, input_grad_partial_chunks = 1, input_grad_positions_per_block = 1, input_grad_position_tile = 0;
    bool input_grad_fp16 = true, linear_fp16 = true, persistent_half_weights = true;
    uint64_t allreduce_bucket_bytes = 4ULL << 20, lt_workspace_bytes = 0, seed = 1234;
    float lr = 0.0001f, weight_decay = 0.0f;
    bool write_artifacts = true, backward_profile = false, overlap_allreduce = true;
    std::string nccl_id_file, resume_checkpoint;
    // beyond the reference's flag set (both default to its behaviour): write the checkpoint every N steps, and let a
    // resumed run continue the step count the checkpoint was written at instead of restarting it at 0
    std::string puzzle_json, target_bin;  // a puzzle definition from files instead of the built-in cyclic shifts
    uint32_t checkpoint_period_steps = 0;
    bool resume_step = false;
    // options of the loss+gradient launch that the reference does not have (mgt_train_options_t): "fp16" | "bf16", "mse" | "ce"
    std::string operand_format = "fp16", loss = "mse";
    // batch normalisation of the hidden layer and of every block's fc2 output (statistics over all ranks); the scale/shift
    // vectors and the running statistics live beside the reference's files, and the exported weights have them folded in
    bool batch_norm = false;
    float bn_eps = 1.0e-5f, bn_momentum = 0.1f;
};

// Every flag takes exactly one value; unknown flags, missing values and unparsable values fail
// (tool:525-613). Returns false where the reference prints its usage text and exits 1.
bool ParseTrainOptions(int argc, const char* const* argv, TrainOptions* out);
// The checks of ValidateTrainConfig (native/src/train_plan.cpp:168-185) plus the binary's own
// (steps > 0, rank < world, batch > 0; tool:611-612).
bool ValidateTrainOptions(const TrainOptions& o);

enum class ParamRole : uint32_t {  // native/include/mgt/model_layout.hpp:17-28
    kInputEmbedding = 1, kInputBias, kHiddenWeight, kHiddenBias, kResidualFc1Weight, kResidualFc1Bias,
    kResidualFc2Weight, kResidualFc2Bias, kOutputWeight, kOutputBias
};
const char* ParamRoleName(ParamRole role);

struct ParamBlock {
    ParamRole role;
    uint32_t block_index;
    uint32_t rows, cols;                  // physical
    uint32_t logical_rows, logical_cols;
    uint64_t offset_bytes, size_bytes;    // blocks are laid 64-byte aligned in this accounting
    uint64_t param_offset;                // offset in the unpadded flat array the kernels use
};

struct LinearOp {  // native/include/mgt/train_plan.hpp:44-63
    uint32_t op_id, phase, block_index;   // phase: 1 forward, 2 backward_weights, 3 backward_input
    ParamRole role;
    bool transpose_a, transpose_b;
    uint32_t m, n, k, lhs_rows, lhs_cols, rhs_rows, rhs_cols, output_rows, output_cols;
    uint32_t backend;                     // 1 custom_kernel, 2 library_tensorop, 3 cutlass_large_k_reduction_candidate
    bool tensor_core_eligible, logical_tail_masked;
};

struct MemoryPlan {  // native/include/mgt/memory_plan.hpp:23-39
    uint64_t weights_bytes, optimizer_m_bytes, optimizer_v_bytes, gradient_bytes, gradient_carousel_bytes;
    uint64_t states_bytes, labels_bytes, walk_meta_bytes;
    uint64_t layout_generate_bytes, layout_forward_bytes, layout_backward_bytes, layout_allreduce_bytes, layout_checkpoint_bytes;
    uint64_t training_scratch_bytes, total_rank_bytes;
};

struct TrainPlan {
    TrainOptions options;
    uint32_t padded_state_dim = 0, physical_hd1 = 0, physical_hd2 = 0;
    uint64_t state_capacity_bytes = 0;
    bool fits_state_record = false;       // state fits the 80-byte record the kernels use
    std::vector<ParamBlock> blocks;
    uint64_t total_params = 0, logical_params = 0, total_bytes = 0;
    uint32_t gradient_bucket_count = 0;
    std::vector<LinearOp> linear_ops;
    MemoryPlan memory{};
};

// BuildTrainPlan (native/src/train_plan.cpp:204-230). False = invalid configuration.
bool BuildTrainPlan(const TrainOptions& options, TrainPlan* out);

// Name the reference reports for the input-gradient back-end its flags would select (tool:93-102).
const char* InputGradBackendName(const TrainOptions& o);
const char* LinearPhaseName(uint32_t phase);
const char* LinearBackendName(uint32_t backend);

// ---- artefacts (native/tools/mgt_native_train_smoke.cu:184-404, 888-895) -----------------------
uint16_t ExportFloatToFp16(float value);  // the trainer's software converter (tool:215-229), not IEEE RN-even
bool WriteLinearOpsManifest(const std::string& dir, const TrainPlan& plan);
bool WriteMetadataEnv(const std::string& dir, const TrainPlan& plan, bool overlap_allreduce, bool comm_enabled, bool resumed);
bool WriteLayersJson(const std::string& dir, const TrainPlan& plan);
bool WriteWeights(const std::string& dir, const TrainPlan& plan, const std::vector<float>& weights);
bool WriteCheckpoint(const std::string& dir, const TrainPlan& plan, const std::vector<float>& w, const std::vector<float>& m, const std::vector<float>& v);
bool ReadCheckpoint(const std::string& checkpoint_dir, std::vector<float>* w, std::vector<float>* m, std::vector<float>* v);
std::string StartLogLine(const TrainPlan& plan, bool overlap_allreduce, bool comm_enabled, bool resumed);

struct StepRecord {
    uint32_t step;
    float loss, step_ms, walk_ms, backward_ms, allreduce_ms, adam_ms;
    uint64_t memory_bytes;
    uint32_t overlap_ranges, overlap_chunks;
    float bw[7];  // input_forward, hidden_forward, residual_forward, output, residual_backward, hidden_backward, input_grad
};
std::string StepLogLine(const TrainPlan& plan, const StepRecord& r);
std::string StepProfileRow(const TrainPlan& plan, const StepRecord& r, bool overlap_allreduce);

// Built-in puzzle of the trainer: cyclic shifts, identity target (tool:117-140). 18 move records + 1 target record of 80 bytes.
void BuildCyclicPuzzle(const TrainPlan& plan, uint8_t* moves_18x80, uint8_t* target_80);
// A puzzle definition from files (the format of the reference's LoadPuzzleDefinition, native/src/puzzle_io.cpp:48-97):
// the integers of the JSON text in order are group id, state length, move count, then move_count permutations of
// 0..state_len-1; the target is exactly state_len raw bytes. Returns 0 ok, 2 invalid_puzzle, 6 io_failure.
int LoadPuzzleFiles(const std::string& group_json, const std::string& target_bin, uint32_t group_id, uint32_t state_len, uint32_t move_count,
                    uint8_t* moves_18x80, uint8_t* target_80);
// Deterministic initial weights (tool:648-650).
void InitialWeights(std::vector<float>* weights);

}  // namespace host
}  // namespace mgt
