// mgt_native_train: one process per GPU rank. Same command line, same output files and the same
// step loop as the reference trainer (native/tools/mgt_native_train_smoke.cu:619-930); the device
// work goes through the C ABI of libmgt_b200 (include/mgt_b200.h).
//
//   per step:  record step_start -> random walks -> forward/loss/backward (gradient-ready
//              notifications schedule the peer gradient exchange, fused with AdamW, on a second
//              stream, also with a single rank) -> wait for the exchange -> AdamW (non-overlapped mode only)
//              -> record step_stop, synchronise, read the loss, write train.log / profile.jsonl
#include "../../include/mgt_b200.h"
#include "host_plan.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <filesystem>
#include <fstream>
#include <iostream>
#include <vector>

using namespace mgt::host;

namespace {

#define CUDA_OK(expr) ((expr) == cudaSuccess)

// Gradient-ready ranges -> exchange launches (the role of ScheduleGradientAllreduce, tool:494-523).
// The exchange is fused with the AdamW update; the engine announces a range only after the last kernel that
// reads its weights is enqueued, so ranges go out as they are announced.
struct ExchangeContext {
    bool enabled = false;
    mgt_comm_t* comm = nullptr;
    cudaStream_t comm_stream = nullptr;
    std::vector<cudaEvent_t>* events = nullptr;
    uint64_t bucket_params = 0;
    mgt_adamw_config_t adamw{};
    float* w = nullptr;
    uint16_t* w_half = nullptr;
    float* m = nullptr;
    float* v = nullptr;
    float* grad = nullptr;
    uint32_t world_size = 1, global_rank = 0;
    bool early_update_after_backward = true;  // the early range: exchange under the weight-gradient GEMMs, AdamW once backward has ended
    bool have_deferred = false;
    cudaEvent_t early_done = nullptr;  // recorded behind the exchange of the deferred range
    uint64_t deferred_offset = 0, deferred_count = 0;
    uint32_t scheduled_ranges = 0, scheduled_chunks = 0, next_event = 0, expected_ranges = 0;
    bool have_pending = false;
    uint64_t pending_offset = 0, pending_count = 0;
    bool failed = false;
    bool have_early = false;  // the early-range hook already sent [early_begin, early_end)
    uint64_t early_begin = 0, early_end = 0;

    // `whole`: no chunking - for the range(s) left when backward has ended and nothing remains to overlap with.
    // `exchange_only`: average the gradients now, leave the AdamW update of the range to the caller (UpdateDeferred).
    bool LaunchRange(uint64_t offset, uint64_t count, cudaStream_t producer, bool whole, bool exchange_only = false) {
        cudaEvent_t ev = (*events)[next_event++ % events->size()];
        if (!CUDA_OK(cudaEventRecord(ev, producer)) || !CUDA_OK(cudaStreamWaitEvent(comm_stream, ev, 0))) return false;
        while (count > 0) {
            const uint64_t chunk = whole ? count : std::min<uint64_t>(count, bucket_params);
            if (exchange_only) {
                const mgt_allreduce_config_t ar{world_size, global_rank, 0, chunk};
                if (mgt_comm_allreduce_average(comm, &ar, grad + offset, comm_stream) != MGT_OK) return false;
            } else if (mgt_comm_allreduce_average_adamw(comm, offset, chunk, &adamw, w, w_half, m, v, comm_stream) != MGT_OK) {
                return false;
            }
            offset += chunk;
            count -= chunk;
            ++scheduled_chunks;
        }
        return true;
    }
    bool Flush(cudaStream_t producer, bool whole = false) {
        if (!have_pending) return true;
        have_pending = false;
        return LaunchRange(pending_offset, pending_count, producer, whole);
    }
    // AdamW of the range whose exchange ran without it; `stream` has already waited for the exchange.
    bool UpdateDeferred(cudaStream_t stream) {
        if (!have_deferred) return true;
        have_deferred = false;
        mgt_adamw_config_t cfg = adamw;
        cfg.param_count = deferred_count;
        const uint64_t o = deferred_offset;
        const mgt_status_t st = w_half != nullptr ? mgt_launch_adamw_with_half_mirror(&cfg, w + o, w_half + o, grad + o, m + o, v + o, stream)
                                                  : mgt_launch_adamw(&cfg, w + o, grad + o, m + o, v + o, stream);
        return st == MGT_OK;
    }
};

mgt_status_t OnGradientReady(void* user, uint32_t ready_id, uint64_t offset, uint64_t count, void* producer_stream) {
    auto* ctx = static_cast<ExchangeContext*>(user);
    if (ctx == nullptr || !ctx->enabled) return MGT_OK;
    if (ctx->comm == nullptr || ctx->comm_stream == nullptr || ctx->events == nullptr || ctx->bucket_params == 0 || count == 0) return MGT_INVALID_CONFIG;
    (void)ready_id;
    ++ctx->scheduled_ranges;
    // The engine announces a range after the last kernel that reads its weights, so the fused exchange + update can go
    // out without holding it back for safety. It is held back for another reason: every launch costs a handshake with all
    // peers, and backward announces the ranges of the residual blocks end to end (last block first, the hidden layer
    // below them), so ranges that touch in memory are joined while the sum stays within one bucket. The range that closes
    // backward (the embedding table) is kept for Flush(whole): nothing is left to overlap with, so it is not cut up.
    if (ctx->have_early && ctx->early_begin == offset && ctx->early_end <= offset + count) {
        // leading blocks of this range went out through the hook: only the rest is left
        count = offset + count - ctx->early_end;
        offset = ctx->early_end;
        if (count == 0) return MGT_OK;
    }
    if (ctx->have_pending) {
        const bool touches = offset + count == ctx->pending_offset || ctx->pending_offset + ctx->pending_count == offset;
        if (touches && ctx->pending_count + count <= ctx->bucket_params) {
            ctx->pending_offset = std::min(ctx->pending_offset, offset);
            ctx->pending_count += count;
            return MGT_OK;
        }
        if (!ctx->Flush(static_cast<cudaStream_t>(producer_stream))) { ctx->failed = true; return MGT_NCCL_FAILURE; }
    }
    ctx->have_pending = true;
    ctx->pending_offset = offset;
    ctx->pending_count = count;
    return MGT_OK;
}

// The engine's early-range hook: a leading block of the embedding table's gradient is complete while the kernel that
// computes the next block still runs, so it goes out now, whole, and is exchanged and updated under that kernel.
mgt_status_t OnEarlyRange(void* user, uint32_t ready_id, uint64_t offset, uint64_t count, void* producer_stream) {
    auto* ctx = static_cast<ExchangeContext*>(user);
    if (ctx == nullptr || !ctx->enabled) return MGT_OK;
    (void)ready_id;
    if (ctx->comm == nullptr || ctx->comm_stream == nullptr || ctx->events == nullptr || count == 0) return MGT_INVALID_CONFIG;
    if (ctx->have_early && offset != ctx->early_end) return MGT_INVALID_CONFIG;  // blocks come in order, end to end
    // The AdamW update moves 30 bytes per parameter through HBM and would fight the HBM-bound weight-gradient GEMMs that
    // run now; the NVLink exchange alone hardly touches local memory. So the update of this range is left for later,
    // unless an earlier early range is still waiting for its own (then this one takes the fused path).
    const bool defer = ctx->early_update_after_backward && !ctx->have_deferred;
    if (!ctx->Flush(static_cast<cudaStream_t>(producer_stream)) || !ctx->LaunchRange(offset, count, static_cast<cudaStream_t>(producer_stream), true, defer)) {
        ctx->failed = true;
        return MGT_NCCL_FAILURE;
    }
    if (defer) {
        if (ctx->early_done != nullptr && !CUDA_OK(cudaEventRecord(ctx->early_done, ctx->comm_stream))) return MGT_CUDA_FAILURE;
        ctx->have_deferred = true;
        ctx->deferred_offset = offset;
        ctx->deferred_count = count;
    }
    if (!ctx->have_early) ctx->early_begin = offset;
    ctx->have_early = true;
    ctx->early_end = offset + count;
    return MGT_OK;
}

// Batch-norm statistics over all ranks: a second, small communicator driven from the compute stream (one communicator
// belongs to one stream; the gradient exchange keeps its own).
struct StatsContext {
    mgt_comm_t* comm = nullptr;
    uint32_t world_size = 1, global_rank = 0;
};
mgt_status_t OnStatsExchange(void* user, float* device_buffer, uint64_t float_count, void* stream) {
    auto* ctx = static_cast<StatsContext*>(user);
    if (ctx == nullptr || ctx->comm == nullptr) return MGT_INVALID_CONFIG;
    const mgt_allreduce_config_t ar{ctx->world_size, ctx->global_rank, 0, float_count};
    return mgt_comm_allreduce_average(ctx->comm, &ar, device_buffer, stream);
}

// checkpoint/batch_norm.f32.bin: scale/shift, their AdamW moments, running statistics - four sections of `count` floats,
// beside the reference's checkpoint files, which keep their format.
bool WriteBatchNormState(const std::string& dir, const std::vector<float>& scale_shift, const std::vector<float>& m, const std::vector<float>& v,
                         const std::vector<float>& running, uint32_t layers, uint32_t width, float eps, float momentum) {
    std::ofstream data(dir + "/checkpoint/batch_norm.f32.bin", std::ios::binary | std::ios::trunc);
    for (const std::vector<float>* section : {&scale_shift, &m, &v, &running})
        data.write(reinterpret_cast<const char*>(section->data()), static_cast<std::streamsize>(section->size() * sizeof(float)));
    std::ofstream man(dir + "/checkpoint/batch_norm.json", std::ios::trunc);
    man << "{\n  \"format\": \"mgt_batch_norm_state_v1\",\n  \"layers\": " << layers << ",\n  \"width\": " << width << ",\n  \"eps\": " << eps
        << ",\n  \"momentum\": " << momentum << ",\n  \"dtype\": \"f32\",\n  \"sections\": [\"scale_shift\", \"adam_m\", \"adam_v\", \"running_stats\"],\n"
        << "  \"section_floats\": " << scale_shift.size() << ",\n  \"layer_layout\": \"layer 0 = hidden layer, layer k+1 = residual block k; scale_shift: gamma[width], "
        << "beta[width]; running_stats: mean[width], var[width]\"\n}\n";
    return static_cast<bool>(data) && static_cast<bool>(man);
}
bool ReadBatchNormState(const std::string& checkpoint_dir, std::vector<float>* scale_shift, std::vector<float>* m, std::vector<float>* v, std::vector<float>* running) {
    std::ifstream data(checkpoint_dir + "/batch_norm.f32.bin", std::ios::binary);
    if (!data) return false;
    for (std::vector<float>* section : {scale_shift, m, v, running})
        data.read(reinterpret_cast<char*>(section->data()), static_cast<std::streamsize>(section->size() * sizeof(float)));
    return static_cast<bool>(data);
}

const char kUsage[] =
    "usage: mgt_native_train --output-dir DIR --steps N --device-id ID --world-size N --global-rank R --local-rank R "
    "[--batch-size N --k-min N --k-max N --hd1 N --hd2 N --nrd N --write-artifacts 0|1 --backward-profile 0|1 --overlap-allreduce 0|1 "
    "--input-grad-partial-chunks N --input-grad-positions-per-block N --input-grad-position-tile N --input-grad-fp16 0|1 --linear-fp16 0|1 "
    "--persistent-half-weights 0|1 --lt-workspace-bytes N --nccl-id-file PATH --resume-checkpoint DIR "
    "--checkpoint-period-steps N --resume-step 0|1 --puzzle-json PATH --target-bin PATH --operand-format fp16|bf16 --loss mse|ce --batch-norm 0|1 --bn-eps X --bn-momentum X]\n";

}  // namespace

int main(int argc, char** argv) {
    TrainOptions opt;
    if (!ParseTrainOptions(argc, argv, &opt)) {
        std::cerr << kUsage;
        return EXIT_FAILURE;
    }
    int device_count = 0;
    if (!CUDA_OK(cudaGetDeviceCount(&device_count)) || device_count <= static_cast<int>(opt.device_id)) return EXIT_FAILURE;
    if (!CUDA_OK(cudaSetDevice(static_cast<int>(opt.device_id)))) return EXIT_FAILURE;

    TrainPlan plan;
    if (!BuildTrainPlan(opt, &plan)) return EXIT_FAILURE;
    if (!plan.fits_state_record || opt.state_len > MGT_STATE_LEN || opt.state_value_count > MGT_STATE_VALUE_PAD || opt.move_count > MGT_MOVE_COUNT) {
        std::cerr << "current CUDA smoke path supports puzzles fitting TrainStateStorage only\n";
        return EXIT_FAILURE;
    }
    // the device model uses the PHYSICAL (padded) hidden sizes; padded tails are trained (tool:641)
    const mgt_mlp_shape_t shape{opt.state_len, opt.state_value_count, plan.physical_hd1, plan.physical_hd2, opt.nrd, opt.output_dim};
    const uint32_t B = opt.batch_size;
    const uint64_t P = plan.total_params;
    if (mgt_mlp_param_count(&shape) != P) return EXIT_FAILURE;

    // trained floats on the device: the reference's parameters, then (with --batch-norm 1) the scale/shift vectors
    const uint64_t NBN = opt.batch_norm ? mgt_bn_param_count(&shape) : 0;
    const uint64_t T = P + NBN;
    std::vector<float> weights(P), adam_m(P, 0.0f), adam_v(P, 0.0f);
    std::vector<float> bn_scale_shift(NBN, 0.0f), bn_m(NBN, 0.0f), bn_v(NBN, 0.0f), bn_running(NBN, 0.0f);
    for (uint64_t i = 0; i < NBN; ++i) {
        const bool first_half = (i / shape.hd2) % 2ULL == 0;
        bn_scale_shift[i] = first_half ? 1.0f : 0.0f;  // gamma = 1, beta = 0
        bn_running[i] = first_half ? 0.0f : 1.0f;      // mean = 0, var = 1
    }
    InitialWeights(&weights);
    const bool resumed = !opt.resume_checkpoint.empty();
    if (resumed && !ReadCheckpoint(opt.resume_checkpoint, &weights, &adam_m, &adam_v)) return EXIT_FAILURE;
    if (resumed && NBN != 0 && !ReadBatchNormState(opt.resume_checkpoint, &bn_scale_shift, &bn_m, &bn_v, &bn_running)) {
        std::cerr << "--batch-norm 1: " << opt.resume_checkpoint << "/batch_norm.f32.bin not found or too short\n";
        return EXIT_FAILURE;
    }
    // Step numbering of a resumed run: the reference restarts at 0 (tool:765,830), which replays the first walk batches
    // and AdamW bias corrections. With --resume-step 1 the count written beside the checkpoint (checkpoint/step.txt; the
    // manifest itself stays byte-compatible) is continued, so that N + M steps in two runs equal N + M steps in one.
    uint32_t first_step = 0;
    if (resumed && opt.resume_step) {
        std::ifstream in(opt.resume_checkpoint + "/step.txt");
        if (!(in >> first_step)) {
            std::cerr << "--resume-step 1: " << opt.resume_checkpoint << "/step.txt not found or unreadable\n";
            return EXIT_FAILURE;
        }
    }
    uint8_t moves[18 * 80], target[80];
    if (opt.puzzle_json.empty() != opt.target_bin.empty()) {
        std::cerr << "--puzzle-json and --target-bin go together\n";
        return EXIT_FAILURE;
    }
    if (opt.puzzle_json.empty()) {
        BuildCyclicPuzzle(plan, moves, target);  // the reference trainer's only puzzle (tool:117-140)
    } else {
        const int st = LoadPuzzleFiles(opt.puzzle_json, opt.target_bin, opt.group_id, opt.state_len, opt.move_count, moves, target);
        if (st != 0) {
            std::cerr << "puzzle definition: " << mgt_status_name(static_cast<mgt_status_t>(st)) << "\n";
            return EXIT_FAILURE;
        }
    }

    mgt_engine_t* engine = nullptr;
    if (mgt_engine_create(static_cast<int32_t>(opt.device_id), &engine) != MGT_OK) return EXIT_FAILURE;
    const mgt_train_options_t train_options{opt.operand_format == "bf16" ? MGT_OPERAND_BF16 : MGT_OPERAND_FP16, opt.loss == "ce" ? MGT_LOSS_CROSS_ENTROPY : MGT_LOSS_MSE,
                                            opt.batch_norm ? 1 : 0, opt.bn_eps};
    if (mgt_engine_set_train_options(engine, &train_options) != MGT_OK) return EXIT_FAILURE;
    // the communicator stands where the reference creates its NCCL context, also for one rank (tool:708-713)
    mgt_comm_t* comm = nullptr;
    if (mgt_comm_create(static_cast<int32_t>(opt.device_id), opt.world_size, opt.global_rank, opt.nccl_id_file.empty() ? nullptr : opt.nccl_id_file.c_str(), T, &comm) != MGT_OK) {
        return EXIT_FAILURE;
    }
    mgt_comm_t* stats_comm = nullptr;
    StatsContext stats_ctx;
    if (NBN != 0 && opt.world_size > 1) {
        const std::string stats_id = opt.nccl_id_file + ".bn";
        if (mgt_comm_create(static_cast<int32_t>(opt.device_id), opt.world_size, opt.global_rank, stats_id.c_str(), 2ULL * shape.hd2, &stats_comm) != MGT_OK) return EXIT_FAILURE;
        stats_ctx.comm = stats_comm;
        stats_ctx.world_size = opt.world_size;
        stats_ctx.global_rank = opt.global_rank;
    }
    const bool comm_enabled = true;

    float* d_bn_running = nullptr;
    float *d_w = nullptr, *d_labels = nullptr, *d_walk_labels = nullptr, *d_loss = nullptr, *d_ws = nullptr, *d_m = nullptr, *d_v = nullptr;
    uint16_t* d_w_half = nullptr;
    mgt_train_state_t *d_states = nullptr, *d_moves = nullptr, *d_target = nullptr;
    mgt_walk_meta_t* d_meta = nullptr;
    float* d_grad = mgt_comm_gradient_buffer(comm);  // peers map this buffer; with one rank it is plain device memory
    const uint64_t ws_floats = mgt_mlp_loss_grad_workspace_floats_with_options(&shape, B, opt.input_grad_partial_chunks, opt.input_grad_fp16, opt.linear_fp16, &train_options);
    if (ws_floats == 0 || d_grad == nullptr) return EXIT_FAILURE;
    cudaStream_t compute = nullptr, comm_stream = nullptr;
    bool ok = CUDA_OK(cudaMalloc(&d_w, T * 4)) && (!(opt.linear_fp16 && opt.persistent_half_weights) || CUDA_OK(cudaMalloc(&d_w_half, T * 2))) &&
              (NBN == 0 || CUDA_OK(cudaMalloc(&d_bn_running, NBN * 4))) &&
              CUDA_OK(cudaMalloc(&d_labels, static_cast<uint64_t>(B) * opt.output_dim * 4)) &&
              (opt.output_dim == 1 || CUDA_OK(cudaMalloc(&d_walk_labels, static_cast<uint64_t>(B) * 4))) && CUDA_OK(cudaMalloc(&d_loss, 4)) &&
              CUDA_OK(cudaMalloc(&d_ws, ws_floats * 4)) && CUDA_OK(cudaMalloc(&d_m, T * 4)) && CUDA_OK(cudaMalloc(&d_v, T * 4)) &&
              CUDA_OK(cudaMalloc(&d_states, static_cast<uint64_t>(B) * 80)) && CUDA_OK(cudaMalloc(&d_meta, static_cast<uint64_t>(B) * 16)) &&
              CUDA_OK(cudaMalloc(&d_moves, 18 * 80)) && CUDA_OK(cudaMalloc(&d_target, 80)) &&
              CUDA_OK(cudaStreamCreateWithFlags(&compute, cudaStreamNonBlocking)) && CUDA_OK(cudaStreamCreateWithFlags(&comm_stream, cudaStreamNonBlocking));
    if (!ok) return EXIT_FAILURE;
    ok = CUDA_OK(cudaMemcpy(d_w, weights.data(), P * 4, cudaMemcpyHostToDevice)) && CUDA_OK(cudaMemcpy(d_m, adam_m.data(), P * 4, cudaMemcpyHostToDevice)) &&
         CUDA_OK(cudaMemcpy(d_v, adam_v.data(), P * 4, cudaMemcpyHostToDevice)) && CUDA_OK(cudaMemcpy(d_moves, moves, sizeof(moves), cudaMemcpyHostToDevice)) &&
         CUDA_OK(cudaMemcpy(d_target, target, sizeof(target), cudaMemcpyHostToDevice));
    if (!ok) return EXIT_FAILURE;
    if (NBN != 0) {
        ok = CUDA_OK(cudaMemcpy(d_w + P, bn_scale_shift.data(), NBN * 4, cudaMemcpyHostToDevice)) && CUDA_OK(cudaMemcpy(d_m + P, bn_m.data(), NBN * 4, cudaMemcpyHostToDevice)) &&
             CUDA_OK(cudaMemcpy(d_v + P, bn_v.data(), NBN * 4, cudaMemcpyHostToDevice)) && CUDA_OK(cudaMemcpy(d_bn_running, bn_running.data(), NBN * 4, cudaMemcpyHostToDevice));
        if (!ok) return EXIT_FAILURE;
        if (mgt_engine_set_batch_norm_state(engine, d_bn_running, opt.bn_momentum, opt.world_size, stats_comm != nullptr ? mgt_comm_gradient_buffer(stats_comm) : nullptr,
                                            stats_comm != nullptr ? OnStatsExchange : nullptr, &stats_ctx) != MGT_OK) return EXIT_FAILURE;
    }
    if (d_w_half != nullptr && mgt_launch_float_to_half(d_w, T, d_w_half, compute) != MGT_OK) return EXIT_FAILURE;

    std::filesystem::create_directories(opt.output_dir);
    std::ofstream log(std::filesystem::path(opt.output_dir) / "train.log");
    std::ofstream profile(std::filesystem::path(opt.output_dir) / "profile.jsonl");
    cudaEvent_t ev_start, ev_walk, ev_backward, ev_allreduce, ev_stop, ev_comm_done, ev_early_done;
    if (!CUDA_OK(cudaEventCreate(&ev_start)) || !CUDA_OK(cudaEventCreate(&ev_walk)) || !CUDA_OK(cudaEventCreate(&ev_backward)) ||
        !CUDA_OK(cudaEventCreate(&ev_allreduce)) || !CUDA_OK(cudaEventCreate(&ev_stop)) ||
        !CUDA_OK(cudaEventCreateWithFlags(&ev_comm_done, cudaEventDisableTiming)) ||
        !CUDA_OK(cudaEventCreateWithFlags(&ev_early_done, cudaEventDisableTiming))) return EXIT_FAILURE;
    const bool overlap = comm_enabled && opt.overlap_allreduce && opt.world_size > 1;
    const uint32_t expected_ranges = 2U * opt.nrd + 3U + (NBN != 0 ? 1U : 0U);  // batch norm: one more range, the scale/shift vectors
    std::vector<cudaEvent_t> ready_events;
    if (overlap) {
        ready_events.resize(expected_ranges + 1U, nullptr);
        for (cudaEvent_t& ev : ready_events)
            if (!CUDA_OK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming))) return EXIT_FAILURE;
    }
    log << StartLogLine(plan, overlap, comm_enabled, resumed);

    const mgt_random_walk_config_t walk_cfg{B, opt.k_min, opt.k_max, opt.move_count, opt.state_len, plan.padded_state_dim};
    float last_loss = 0.0f;
    auto write_checkpoint = [&](uint32_t steps_done, bool with_weights) -> bool {
        if (!CUDA_OK(cudaMemcpy(weights.data(), d_w, P * 4, cudaMemcpyDeviceToHost)) || !CUDA_OK(cudaMemcpy(adam_m.data(), d_m, P * 4, cudaMemcpyDeviceToHost)) ||
            !CUDA_OK(cudaMemcpy(adam_v.data(), d_v, P * 4, cudaMemcpyDeviceToHost))) return false;
        if (NBN != 0 && (!CUDA_OK(cudaMemcpy(bn_scale_shift.data(), d_w + P, NBN * 4, cudaMemcpyDeviceToHost)) || !CUDA_OK(cudaMemcpy(bn_m.data(), d_m + P, NBN * 4, cudaMemcpyDeviceToHost)) ||
                         !CUDA_OK(cudaMemcpy(bn_v.data(), d_v + P, NBN * 4, cudaMemcpyDeviceToHost)) ||
                         !CUDA_OK(cudaMemcpy(bn_running.data(), d_bn_running, NBN * 4, cudaMemcpyDeviceToHost)))) return false;
        if (with_weights) {
            // the weights/ files describe a network without normalisation: fold it in with the running statistics
            std::vector<float> exported = weights;
            if (NBN != 0 && mgt_fold_batch_norm(&shape, exported.data(), bn_scale_shift.data(), bn_running.data(), opt.bn_eps) != MGT_OK) return false;
            if (!WriteWeights(opt.output_dir, plan, exported)) return false;
        }
        if (!WriteCheckpoint(opt.output_dir, plan, weights, adam_m, adam_v)) return false;
        if (NBN != 0 && !WriteBatchNormState(opt.output_dir, bn_scale_shift, bn_m, bn_v, bn_running, opt.nrd + 1U, shape.hd2, opt.bn_eps, opt.bn_momentum)) return false;
        std::ofstream out(opt.output_dir + "/checkpoint/step.txt", std::ios::trunc);
        out << steps_done << "\n";
        return static_cast<bool>(out);
    };
    // The exchange kernels wait at most a second for a peer, so the ranks meet on the host wherever they may have
    // drifted apart: after start-up (allocations, uploads, module load) and after every checkpoint write.
    constexpr uint32_t kHostBarrierTimeoutMs = 600000;
    if (!CUDA_OK(cudaDeviceSynchronize()) || mgt_comm_host_barrier(comm, kHostBarrierTimeoutMs) != MGT_OK) return EXIT_FAILURE;
    for (uint32_t step = first_step; step < first_step + opt.steps; ++step) {
        if (!CUDA_OK(cudaEventRecord(ev_start, compute))) return EXIT_FAILURE;
        float* walk_labels = opt.output_dim == 1 ? d_labels : d_walk_labels;
        if (mgt_launch_random_walk(&walk_cfg, opt.seed, 0, step, opt.global_rank, d_moves, d_target, d_states, walk_labels, d_meta, compute) != MGT_OK) return EXIT_FAILURE;
        if (opt.output_dim > 1 && mgt_launch_expand_scalar_labels(d_walk_labels, B, opt.output_dim, d_labels, compute) != MGT_OK) return EXIT_FAILURE;
        if (!CUDA_OK(cudaEventRecord(ev_walk, compute))) return EXIT_FAILURE;

        // the resumed run restarts its step counter, as the reference does (tool:765,830)
        const mgt_adamw_config_t adamw{T, static_cast<uint64_t>(step) + 1ULL, opt.lr, 0.9f, 0.999f, 1.0e-8f, opt.weight_decay};
        ExchangeContext exchange;
        if (overlap) {
            exchange.enabled = true;
            exchange.comm = comm;
            exchange.comm_stream = comm_stream;
            exchange.events = &ready_events;
            exchange.bucket_params = std::max<uint64_t>(1ULL, opt.allreduce_bucket_bytes / sizeof(float));
            exchange.adamw = adamw;
            exchange.expected_ranges = expected_ranges;
            exchange.w = d_w; exchange.w_half = d_w_half; exchange.m = d_m; exchange.v = d_v; exchange.grad = d_grad;
            exchange.world_size = opt.world_size; exchange.global_rank = opt.global_rank;
            exchange.early_done = ev_early_done;
        }
        if (mgt_engine_set_early_range_hook(engine, overlap ? OnEarlyRange : nullptr, overlap ? &exchange : nullptr) != MGT_OK) return EXIT_FAILURE;
        mgt_backward_profile_t bw{};
        const mgt_status_t st = mgt_launch_mlp_loss_grad(engine, &shape, d_w, d_w_half, d_states, d_labels, B, d_loss, d_grad, d_ws, ws_floats,
                                                         opt.input_grad_partial_chunks, opt.input_grad_positions_per_block, opt.input_grad_fp16,
                                                         opt.linear_fp16, opt.backward_profile ? &bw : nullptr, overlap ? OnGradientReady : nullptr,
                                                         overlap ? &exchange : nullptr, compute, opt.input_grad_position_tile);
        if (st != MGT_OK) {
            log << "rank=" << opt.global_rank << " step=" << step << " phase=backward status=" << mgt_status_name(st) << " status_code=" << st << "\n";
            std::cerr << "backward failed: " << mgt_status_name(st) << " (" << st << ")\n";
            return EXIT_FAILURE;
        }
        if (!CUDA_OK(cudaEventRecord(ev_backward, compute))) return EXIT_FAILURE;
        uint32_t overlap_ranges = 0, overlap_chunks = 0;
        bool weights_updated = false;
        if (overlap) {
            if (exchange.failed || exchange.scheduled_ranges != expected_ranges || !exchange.Flush(compute, true)) return EXIT_FAILURE;
            overlap_ranges = exchange.scheduled_ranges;
            overlap_chunks = exchange.scheduled_chunks;
            if (!CUDA_OK(cudaEventRecord(ev_comm_done, comm_stream))) return EXIT_FAILURE;
            // the deferred update needs only its own range's exchange: it runs beside the tail of the exchange
            if (exchange.have_deferred && !CUDA_OK(cudaStreamWaitEvent(compute, ev_early_done, 0))) return EXIT_FAILURE;
            if (!exchange.UpdateDeferred(compute) || !CUDA_OK(cudaStreamWaitEvent(compute, ev_comm_done, 0))) return EXIT_FAILURE;
            weights_updated = true;  // AdamW ran inside the exchange kernels
        } else if (opt.world_size > 1) {
            const mgt_allreduce_config_t ar{opt.world_size, opt.global_rank, step, T};
            if (mgt_comm_allreduce_average(comm, &ar, d_grad, compute) != MGT_OK) return EXIT_FAILURE;
            overlap_chunks = 1;
        }
        if (!CUDA_OK(cudaEventRecord(ev_allreduce, compute))) return EXIT_FAILURE;
        if (!weights_updated) {
            const mgt_status_t ad = d_w_half != nullptr ? mgt_launch_adamw_with_half_mirror(&adamw, d_w, d_w_half, d_grad, d_m, d_v, compute)
                                                        : mgt_launch_adamw(&adamw, d_w, d_grad, d_m, d_v, compute);
            if (ad != MGT_OK) return EXIT_FAILURE;
        }
        if (!CUDA_OK(cudaEventRecord(ev_stop, compute)) || !CUDA_OK(cudaEventSynchronize(ev_stop))) return EXIT_FAILURE;

        StepRecord rec{};
        rec.step = step;
        if (!CUDA_OK(cudaEventElapsedTime(&rec.step_ms, ev_start, ev_stop)) || !CUDA_OK(cudaEventElapsedTime(&rec.walk_ms, ev_start, ev_walk)) ||
            !CUDA_OK(cudaEventElapsedTime(&rec.backward_ms, ev_walk, ev_backward)) || !CUDA_OK(cudaEventElapsedTime(&rec.allreduce_ms, ev_backward, ev_allreduce)) ||
            !CUDA_OK(cudaEventElapsedTime(&rec.adam_ms, ev_allreduce, ev_stop))) return EXIT_FAILURE;
        if (!CUDA_OK(cudaMemcpy(&last_loss, d_loss, 4, cudaMemcpyDeviceToHost))) return EXIT_FAILURE;
        int32_t code = 0;
        if (mgt_engine_check(engine, compute, &code) != MGT_OK || mgt_comm_check(comm, comm_stream, &code) != MGT_OK ||
            (stats_comm != nullptr && mgt_comm_check(stats_comm, compute, &code) != MGT_OK)) {
            std::cerr << "device wait timed out (code " << code << ")\n";
            return EXIT_FAILURE;
        }
        size_t free_bytes = 0, total_bytes = 0;
        if (!CUDA_OK(cudaMemGetInfo(&free_bytes, &total_bytes))) return EXIT_FAILURE;
        rec.loss = last_loss;
        rec.memory_bytes = total_bytes - free_bytes;
        rec.overlap_ranges = overlap_ranges;
        rec.overlap_chunks = overlap_chunks;
        const float bwv[7] = {bw.input_forward_ms, bw.hidden_forward_ms, bw.residual_forward_ms, bw.output_ms, bw.residual_backward_ms, bw.hidden_backward_ms, bw.input_grad_ms};
        std::copy(bwv, bwv + 7, rec.bw);
        log << StepLogLine(plan, rec);
        profile << StepProfileRow(plan, rec, overlap);
        const uint32_t done = step + 1U;
        if (opt.checkpoint_period_steps != 0 && done % opt.checkpoint_period_steps == 0 && done != first_step + opt.steps) {
            // every rank passes here at the same steps, whether or not it writes files itself
            if (opt.write_artifacts && !write_checkpoint(done, false)) return EXIT_FAILURE;
            if (mgt_comm_host_barrier(comm, kHostBarrierTimeoutMs) != MGT_OK) return EXIT_FAILURE;
        }
    }

    if (opt.write_artifacts && !write_checkpoint(first_step + opt.steps, true)) return EXIT_FAILURE;
    if (!WriteMetadataEnv(opt.output_dir, plan, overlap, comm_enabled, resumed) || !WriteLayersJson(opt.output_dir, plan) ||
        !WriteLinearOpsManifest(opt.output_dir, plan)) return EXIT_FAILURE;

    if (mgt_comm_destroy(comm) != MGT_OK || mgt_comm_destroy(stats_comm) != MGT_OK) return EXIT_FAILURE;
    mgt_engine_destroy(engine);
    for (cudaEvent_t ev : ready_events) cudaEventDestroy(ev);
    for (cudaEvent_t ev : {ev_start, ev_walk, ev_backward, ev_allreduce, ev_stop, ev_comm_done, ev_early_done}) cudaEventDestroy(ev);
    for (void* p : {static_cast<void*>(d_target), static_cast<void*>(d_moves), static_cast<void*>(d_meta), static_cast<void*>(d_states), static_cast<void*>(d_v),
                    static_cast<void*>(d_m), static_cast<void*>(d_ws), static_cast<void*>(d_loss), static_cast<void*>(d_labels), static_cast<void*>(d_walk_labels),
                    static_cast<void*>(d_w_half), static_cast<void*>(d_w), static_cast<void*>(d_bn_running)})
        if (p != nullptr) cudaFree(p);
    cudaStreamDestroy(comm_stream);
    cudaStreamDestroy(compute);
    std::cout << "native_train_smoke_ok loss=" << last_loss << "\n";
    return EXIT_SUCCESS;
}
