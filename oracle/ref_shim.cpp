// C-ABI shim over the reference's own CPU library (test infrastructure only).
// Compiled together with the reference's sources by oracle/Makefile into
// oracle/_ref/libmgt_ref.so; used to validate the restatement in oracle.cpp, to generate the
// golden vectors under tests/golden/ and as the timed CPU baseline. The reference sources are
// compiled where they lie; nothing of them is copied into this repository.
#include "mgt/puzzle_io.hpp"
#include "mgt/allreduce.hpp"
#include "mgt/mlp_cpu_ref.hpp"
#include "mgt/random_walk.hpp"
#include "mgt/train_plan.hpp"

#include <cstring>
#include <span>

extern "C" {

int ref_random_walks(const unsigned char* moves, const unsigned char* target, unsigned long long seed,
                     unsigned long long epoch, unsigned long long step, unsigned rank, unsigned k_min,
                     unsigned k_max, unsigned samples, unsigned char* states, float* labels, void* meta) {
    mgt::PuzzleDefinition puzzle{};
    std::memcpy(puzzle.moves.data(), moves, sizeof(mgt::TrainStateStorage) * mgt::kMoveCount);
    std::memcpy(&puzzle.target, target, sizeof(mgt::TrainStateStorage));
    const mgt::WalkRequest request{seed, epoch, step, rank, k_min, k_max, samples};
    return static_cast<int>(mgt::GenerateRandomWalksCpu(puzzle, request, reinterpret_cast<mgt::TrainStateStorage*>(states),
                                                        labels, static_cast<mgt::WalkMeta*>(meta)));
}

unsigned long long ref_param_count(const unsigned* shape6) {
    const mgt::CpuMlpShape shape{shape6[0], shape6[1], shape6[2], shape6[3], shape6[4], shape6[5]};
    return mgt::CpuMlpParamCount(shape);
}

int ref_mlp_forward(const unsigned* shape6, const float* weights, const unsigned char* states, unsigned samples, float* outputs) {
    const mgt::CpuMlpShape shape{shape6[0], shape6[1], shape6[2], shape6[3], shape6[4], shape6[5]};
    return static_cast<int>(mgt::CpuMlpForward(shape, std::span<const float>(weights, mgt::CpuMlpParamCount(shape)),
                                               reinterpret_cast<const mgt::TrainStateStorage*>(states), samples, outputs));
}

int ref_mlp_loss_grad(const unsigned* shape6, const float* weights, const unsigned char* states, const float* labels,
                      unsigned samples, float* loss, float* grad) {
    const mgt::CpuMlpShape shape{shape6[0], shape6[1], shape6[2], shape6[3], shape6[4], shape6[5]};
    return static_cast<int>(mgt::CpuMlpLossAndGrad(shape, std::span<const float>(weights, mgt::CpuMlpParamCount(shape)),
                                                   reinterpret_cast<const mgt::TrainStateStorage*>(states), labels, samples, loss, grad));
}

int ref_adamw(float* weights, const float* grad, float* m, float* v, unsigned long long n, unsigned long long step,
              float lr, float beta1, float beta2, float eps, float wd) {
    return static_cast<int>(mgt::CpuAdamWStep(weights, grad, m, v, n, step, lr, beta1, beta2, eps, wd));
}

// Plan numbers used by the planner tests. out[0..]: padded_state_dim, physical_hd1, physical_hd2,
// blocks, linear_ops, gradient_buckets, total_params, total_bytes, total_rank_bytes, training_scratch_bytes.
int ref_plan_numbers(unsigned state_len, unsigned value_count, unsigned move_count, unsigned state_alignment,
                     unsigned hd1, unsigned hd2, unsigned nrd, unsigned output_dim, unsigned hidden_alignment,
                     unsigned batch, unsigned long long bucket_bytes, unsigned world, unsigned long long* out) {
    mgt::TrainConfig config = mgt::MakeArchiveP888TrainConfig();
    config.puzzle.raw_state_dim = state_len;
    config.puzzle.state_value_count = value_count;
    config.puzzle.move_count = move_count;
    config.puzzle.state_alignment = state_alignment;
    config.model.hd1 = hd1;
    config.model.hd2 = hd2;
    config.model.residual_blocks = nrd;
    config.model.output_dim = output_dim;
    config.model.hidden_alignment = hidden_alignment;
    config.train.batch_size = batch;
    config.runtime.allreduce_bucket_bytes = bucket_bytes;
    config.runtime.device_count = world;
    config.runtime.mode = world == 1 ? mgt::RuntimeMode::kSingleGpu : mgt::RuntimeMode::kMultiGpu;
    mgt::TrainPlan plan{};
    const mgt::Status status = mgt::BuildTrainPlan(config, &plan);
    if (status != mgt::Status::kOk) return static_cast<int>(status);
    out[0] = plan.padded_state_dim;
    out[1] = plan.layout.physical_hd1;
    out[2] = plan.layout.physical_hd2;
    out[3] = plan.layout.blocks.size();
    out[4] = plan.linear_ops.size();
    out[5] = plan.gradient_buckets.size();
    out[6] = plan.layout.total_params;
    out[7] = plan.layout.total_bytes;
    out[8] = plan.memory.total_rank_bytes;
    out[9] = plan.memory.training_scratch_bytes;
    return 0;
}

// One linear-op row: out[0..13] = op_id, phase, role, block_index, ta, tb, m, n, k, backend, tc_eligible, tail_masked, lhs_rows, rhs_cols
int ref_plan_linear_op(unsigned state_len, unsigned value_count, unsigned hd1, unsigned hd2, unsigned nrd,
                       unsigned output_dim, unsigned batch, unsigned index, unsigned* out) {
    mgt::TrainConfig config = mgt::MakeArchiveP888TrainConfig();
    config.puzzle.raw_state_dim = state_len;
    config.puzzle.state_value_count = value_count;
    config.model.hd1 = hd1;
    config.model.hd2 = hd2;
    config.model.residual_blocks = nrd;
    config.model.output_dim = output_dim;
    config.train.batch_size = batch;
    mgt::TrainPlan plan{};
    if (mgt::BuildTrainPlan(config, &plan) != mgt::Status::kOk || index >= plan.linear_ops.size()) return 1;
    const mgt::LinearOpPlan& op = plan.linear_ops[index];
    out[0] = op.op_id;
    out[1] = static_cast<unsigned>(op.phase);
    out[2] = static_cast<unsigned>(op.role);
    out[3] = op.block_index;
    out[4] = static_cast<unsigned>(op.transpose_a);
    out[5] = static_cast<unsigned>(op.transpose_b);
    out[6] = op.m;
    out[7] = op.n;
    out[8] = op.k;
    out[9] = static_cast<unsigned>(op.backend);
    out[10] = op.tensor_core_eligible ? 1U : 0U;
    out[11] = op.logical_tail_masked ? 1U : 0U;
    out[12] = op.lhs_rows;
    out[13] = op.rhs_cols;
    return 0;
}

// LoadPuzzleDefinition (native/src/puzzle_io.cpp:48-97): 18 move records and the target, 80 bytes each.
int ref_load_puzzle(const char* group_json, const char* target_bin, unsigned char* moves, unsigned char* target) {
    mgt::PuzzleDefinition puzzle{};
    const mgt::Status st = mgt::LoadPuzzleDefinition(group_json, target_bin, &puzzle);
    if (st != mgt::Status::kOk) return static_cast<int>(st);
    for (unsigned mv = 0; mv < mgt::kMoveCount; ++mv)
        for (unsigned i = 0; i < mgt::kStateStorageLen; ++i) moves[mv * mgt::kStateStorageLen + i] = puzzle.moves[mv].v[i];
    for (unsigned i = 0; i < mgt::kStateStorageLen; ++i) target[i] = puzzle.target.v[i];
    return 0;
}

}  // extern "C"
