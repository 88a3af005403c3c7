/*
 * mgt_b200 - C ABI of the B200-native (sm_100a) training-step library.
 *
 * Drop-in boundary for the per-step data-parallel training hot path of MultiGPUTrainMLP:
 * the functions below take the place of the reference's in-process launch API
 * (namespace mgt_cuda, native/cuda/mgt_cuda/ *.cuh). Conventions kept from the reference:
 *   - every function returns an int32 status with the reference's numeric values
 *     (native/include/mgt/status.hpp:5-13); nothing throws;
 *   - launches are asynchronous on the caller's stream (a cudaStream_t passed as void*);
 *   - all device buffers are owned by the caller; the library allocates nothing per step.
 * Differences: cuBLAS/cuBLASLt handles are replaced by one opaque engine handle, and the
 * workspace is much smaller than the reference's (query it, do not assume).
 *
 * Plain pointers and sizes only: no C++ or torch types cross this boundary.
 */
#ifndef MGT_B200_H_
#define MGT_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* native/include/mgt/status.hpp:5-13; values above 6 are additions of this library. */
typedef int32_t mgt_status_t;
enum {
    MGT_OK = 0,
    MGT_INVALID_CONFIG = 1,
    MGT_INVALID_PUZZLE = 2,
    MGT_CAPACITY_EXCEEDED = 3,
    MGT_CUDA_FAILURE = 4,
    MGT_NCCL_FAILURE = 5,
    MGT_IO_FAILURE = 6,
    MGT_DEVICE_TIMEOUT = 7 /* a bounded device-side wait ran out; the context stays usable */
};

/* Compile-time limits of the reference (native/include/mgt/config.hpp:8-11,32-35). */
#define MGT_STATE_LEN 72
#define MGT_STATE_STORAGE_LEN 80
#define MGT_STATE_VALUE_PAD 72
#define MGT_MOVE_COUNT 18
/* native/cuda/mlp_forward.cu:7-9 */
#define MGT_MAX_HD1 4096
#define MGT_MAX_HD2 512
#define MGT_MAX_RESIDUAL_BLOCKS 32

/* 80-byte state record, 16-byte walk record: native/include/mgt/static_contracts.hpp:11-19. */
typedef struct { uint8_t v[MGT_STATE_STORAGE_LEN]; } mgt_train_state_t;
typedef struct { uint32_t depth; uint32_t last_move; uint64_t rng_counter; } mgt_walk_meta_t;

/* ---- on-GPU random-walk generator ------------------------------------------------------
 * Replaces mgt_cuda::RandomWalkKernelConfig / ValidateRandomWalkKernelConfig /
 * LaunchRandomWalkKernel (native/cuda/mgt_cuda/random_walk_kernel.cuh:10-29,
 * native/cuda/random_walk_kernel.cu:66-99). Bit-exact with the reference for the same
 * (seed, epoch, step, rank, sample). Alignment of the device arrays (checked, MGT_INVALID_CONFIG otherwise): moves, target and
 * labels 4 bytes, meta 8 bytes, states 16 bytes - what any device allocation satisfies. */
typedef struct {
    uint32_t sample_count;
    uint32_t k_min;
    uint32_t k_max;
    uint32_t move_count;
    uint32_t state_len;
    uint32_t state_storage_len;
} mgt_random_walk_config_t;

mgt_status_t mgt_validate_random_walk_config(const mgt_random_walk_config_t* config);
mgt_status_t mgt_launch_random_walk(const mgt_random_walk_config_t* config, uint64_t base_seed, uint64_t epoch,
                                    uint64_t step, uint32_t global_rank, const mgt_train_state_t* device_moves,
                                    const mgt_train_state_t* device_target, mgt_train_state_t* device_states,
                                    float* device_labels, mgt_walk_meta_t* device_meta, void* stream);

/* Replaces ExpandScalarLabelsKernel (native/tools/mgt_native_train_smoke.cu:74-80). */
mgt_status_t mgt_launch_expand_scalar_labels(const float* device_scalar_labels, uint32_t samples, uint32_t output_dim,
                                             float* device_labels, void* stream);

/* ---- model shape -------------------------------------------------------------------------
 * Replaces mgt_cuda::CudaMlpShape / ValidateCudaMlpShape (native/cuda/mgt_cuda/mlp_forward.cuh:9-18,
 * native/cuda/mlp_forward.cu:89-97). Flat parameter layout: native/cuda/mlp_backward.cu:25-36. */
typedef struct {
    uint32_t state_len;
    uint32_t state_value_pad;
    uint32_t hd1;
    uint32_t hd2;
    uint32_t residual_blocks;
    uint32_t output_dim;
} mgt_mlp_shape_t;

mgt_status_t mgt_validate_mlp_shape(const mgt_mlp_shape_t* shape);
uint64_t mgt_mlp_param_count(const mgt_mlp_shape_t* shape);

/* ---- engine handle -----------------------------------------------------------------------
 * Takes the place of the cublasHandle_t / cublasLtHandle_t pair of the reference signatures
 * (native/cuda/mgt_cuda/mlp_backward.cuh:224-287): it caches TMA descriptors and owns a
 * 4-byte device status word. Create once per device, before the step loop. */
typedef struct mgt_engine mgt_engine_t;
mgt_status_t mgt_engine_create(int32_t device_id, mgt_engine_t** out_engine);
mgt_status_t mgt_engine_destroy(mgt_engine_t* engine);
/* Synchronises `stream`, then reads and clears the device status word: MGT_OK, or
 * MGT_DEVICE_TIMEOUT if a kernel gave up on a bounded wait since the last call. */
mgt_status_t mgt_engine_check(mgt_engine_t* engine, void* stream, int32_t* out_device_code);
/* Kernels launched through this engine so far (host-side count; no counterpart in the reference). */
uint64_t mgt_engine_launch_count(const mgt_engine_t* engine);

/* ---- loss + gradient (forward, MSE loss, backward) -----------------------------------------
 * Replaces MlpLossGradWorkspaceFloats (native/cuda/mgt_cuda/mlp_backward.cuh:27-43) and the
 * LaunchMlpLossGrad...ExternalHalf family (mlp_backward.cuh:224-314,
 * native/cuda/mlp_backward.cu:1228-1510). */
typedef struct {
    float input_forward_ms;
    float hidden_forward_ms;
    float residual_forward_ms;
    float output_ms;
    float residual_backward_ms;
    float hidden_backward_ms;
    float input_grad_ms;
} mgt_backward_profile_t; /* mlp_backward.cuh:11-19 */

/* mlp_backward.cuh:21-25. Called synchronously on the launching thread, 2*residual_blocks+3 times
 * per launch, in the reference's order: output, (fc2, fc1) of each block from last to first,
 * hidden, embedding+input bias. Stronger than the reference: when a range is announced, every kernel of
 * this launch that reads the WEIGHTS of that range has already been enqueued on producer_stream, so a
 * caller may exchange the gradient range and update those weights in place behind an event recorded at
 * that moment (the reference announces a layer before the GEMM that back-propagates through it). */
typedef mgt_status_t (*mgt_gradient_ready_fn)(void* user, uint32_t ready_id, uint64_t param_offset,
                                              uint64_t param_count, void* producer_stream);

/* Options of the loss+gradient launch that the reference does not have (it computes with fp16 operands and an MSE loss
 * only: native/include/mgt/config.hpp:37-40, native/cuda/mlp_backward.cu:932-943). The defaults are the reference's;
 * nothing in the reference pins the others - they are checked against this repository's CPU restatement, which is
 * pinned by finite differences.
 *   operand_format  MGT_OPERAND_BF16: bfloat16 operands (weights, activations, dz tensors) with fp32 accumulation, the
 *                   same rounding points as the fp16 flow. device_weights_half of the launch is then ignored (it is
 *                   fp16 by contract): the bfloat16 copy is rebuilt from the fp32 weights inside the workspace.
 *   loss_kind       MGT_LOSS_CROSS_ENTROPY (output_dim >= 2): the outputs are per-depth logits, class = depth - 1 where
 *                   the labels carry the walk depth in every output slot (what mgt_launch_expand_scalar_labels writes),
 *                   loss = mean over the batch of -log softmax(y)[class].
 *   batch_norm      1: training-mode batch normalisation (biased batch variance, bn_eps) of the hidden layer's
 *                   pre-activation (before its ReLU) and of every residual block's fc2 output (before the skip add). The
 *                   scale/shift vectors follow the reference's parameters in device_weights and device_grad: layer 0 =
 *                   hidden layer, layer k + 1 = block k, each gamma[hd2] then beta[hd2] - mgt_bn_param_count() more
 *                   floats in both arrays, announced to gradient_ready as ONE more range after the reference's last one
 *                   (2*residual_blocks + 4 calls). The workspace is larger: ask
 *                   mgt_mlp_loss_grad_workspace_floats_with_options. See mgt_engine_set_batch_norm_state for the
 *                   statistics over all ranks and the running statistics.
 * All need use_half_linear = 1; with use_half_linear = 0 a launch with options set returns MGT_INVALID_CONFIG. */
enum { MGT_OPERAND_FP16 = 0, MGT_OPERAND_BF16 = 1 };
enum { MGT_LOSS_MSE = 0, MGT_LOSS_CROSS_ENTROPY = 1 };
typedef struct {
    int32_t operand_format;
    int32_t loss_kind;
    int32_t batch_norm;
    float bn_eps; /* > 0 when batch_norm is set (1e-5 is the usual value) */
} mgt_train_options_t;
mgt_status_t mgt_engine_set_train_options(mgt_engine_t* engine, const mgt_train_options_t* options);
uint64_t mgt_mlp_loss_grad_workspace_floats_with_options(const mgt_mlp_shape_t* shape, uint32_t sample_count,
                                                         uint32_t input_grad_partial_chunks, int32_t use_half_input_grad,
                                                         int32_t use_half_linear, const mgt_train_options_t* options);
uint64_t mgt_bn_param_count(const mgt_mlp_shape_t* shape); /* 2 * (residual_blocks + 1) * hd2; 0 = invalid shape */

/* Batch statistics over all ranks ("sync" batch norm) and running statistics; both optional.
 *   exchange(user, device_buffer, float_count, stream) is called on the launching thread, 2 * (residual_blocks + 1)
 *   times per launch (once per layer in forward, once in backward), and must enqueue on `stream` an in-place AVERAGE of
 *   device_buffer[0..float_count) over all ranks (float_count = 2 * hd2: forward mean and mean of squares, backward
 *   mean(dy) and mean(dy * xhat) of this rank's samples; every rank holds the same number of samples).
 *   device_exchange_buffer is where the engine puts those numbers - e.g. the buffer of a second, small mgt_comm (one
 *   communicator is driven from one stream: the gradient exchange keeps its own). Both NULL: statistics of this rank only.
 *   device_running_stats, if not NULL: (residual_blocks + 1) x {mean[hd2], var[hd2]}, updated every launch as
 *   running = (1 - momentum) * running + momentum * batch (variance unbiased over world_size * sample_count samples). */
typedef mgt_status_t (*mgt_stats_exchange_fn)(void* user, float* device_buffer, uint64_t float_count, void* stream);
mgt_status_t mgt_engine_set_batch_norm_state(mgt_engine_t* engine, float* device_running_stats, float momentum,
                                             uint32_t world_size, float* device_exchange_buffer,
                                             mgt_stats_exchange_fn exchange, void* user);

/* Early-range hook (optional; no counterpart in the reference). The embedding table and the input bias are 86 % of the
 * p888 parameters and the reference announces them last. This library computes their gradient BEFORE the weight-gradient
 * GEMMs of the residual blocks and of the hidden layer, and calls `hook` (same signature and rules as gradient_ready;
 * ready_id = the id the closing announcement will carry) the moment the kernels producing that range are enqueued, so
 * that a caller can exchange it while that remaining work runs. The gradient_ready calls are unchanged - same count,
 * order and ranges as the reference, the embedding range last - so a caller that acted on the hook skips the range
 * (or handles only what the hook did not name) there. NULL removes the hook. */
mgt_status_t mgt_engine_set_early_range_hook(mgt_engine_t* engine, mgt_gradient_ready_fn hook, void* user);

/* Number of floats of caller-owned scratch the launch needs (0 = invalid arguments). */
uint64_t mgt_mlp_loss_grad_workspace_floats(const mgt_mlp_shape_t* shape, uint32_t sample_count,
                                            uint32_t input_grad_partial_chunks, int32_t use_half_input_grad,
                                            int32_t use_half_linear);

/* device_weights_half may be NULL (the fp16 mirror is then rebuilt from device_weights each call).
 * input_grad_partial_chunks / positions_per_block / position_tile select among the reference's
 * input-gradient back-ends; they are validated like the reference does and otherwise ignored:
 * this library has one back-end (one-hot operand synthesised in shared memory for tcgen05). */
mgt_status_t mgt_launch_mlp_loss_grad(mgt_engine_t* engine, const mgt_mlp_shape_t* shape, const float* device_weights,
                                      const uint16_t* device_weights_half, const mgt_train_state_t* device_states,
                                      const float* device_labels, uint32_t sample_count, float* device_loss,
                                      float* device_grad, float* workspace, uint64_t workspace_floats,
                                      uint32_t input_grad_partial_chunks, uint32_t input_grad_positions_per_block,
                                      int32_t use_half_input_grad, int32_t use_half_linear,
                                      mgt_backward_profile_t* profile, mgt_gradient_ready_fn gradient_ready,
                                      void* gradient_ready_user, void* stream, uint32_t input_grad_position_tile);

/* ---- AdamW ---------------------------------------------------------------------------------
 * Replaces AdamWKernelConfig / ValidateAdamWKernelConfig / LaunchAdamWKernel /
 * LaunchAdamWKernelWithHalfMirror (native/cuda/mgt_cuda/adamw.cuh:10-34, native/cuda/adamw.cu:8-88). */
typedef struct {
    uint64_t param_count;
    uint64_t step;
    float learning_rate;
    float beta1;
    float beta2;
    float eps;
    float weight_decay;
} mgt_adamw_config_t;

mgt_status_t mgt_validate_adamw_config(const mgt_adamw_config_t* config);
mgt_status_t mgt_launch_adamw(const mgt_adamw_config_t* config, float* device_weights, const float* device_grad,
                              float* device_m, float* device_v, void* stream);
mgt_status_t mgt_launch_adamw_with_half_mirror(const mgt_adamw_config_t* config, float* device_weights,
                                               uint16_t* device_weights_half, const float* device_grad,
                                               float* device_m, float* device_v, void* stream);
/* Replaces FloatToHalfMirrorKernel (native/tools/mgt_native_train_smoke.cu:68-72). */
mgt_status_t mgt_launch_float_to_half(const float* device_values, uint64_t count, uint16_t* device_half, void* stream);

/* ---- gradient exchange between data-parallel ranks --------------------------------------------
 * Replaces the reference's NCCL wrapper (native/cuda/mgt_cuda/allreduce_nccl.cuh:14-24,
 * native/cuda/allreduce_nccl.cu:58-150) with peer-to-peer loads/stores over NVLink/NVSwitch.
 * One process per GPU on one node, world_size <= 8. mgt_comm_create stands where
 * CreateNcclRankContext stands: ranks rendezvous through `id_file` (rank 0 writes it, the others
 * poll for up to 30 s) and exchange CUDA IPC handles through files next to it. The communicator
 * owns the gradient buffer (peers must be able to map it): pass mgt_comm_gradient_buffer() as the
 * device_grad of mgt_launch_mlp_loss_grad. world_size 1 needs no id file and exchanges nothing. */
typedef struct mgt_comm mgt_comm_t;
typedef struct {
    uint32_t world_size;
    uint32_t global_rank;
    uint64_t collective_seq;
    uint64_t element_count;
} mgt_allreduce_config_t; /* native/include/mgt/allreduce.hpp:9-14 */

mgt_status_t mgt_comm_create(int32_t device_id, uint32_t world_size, uint32_t global_rank, const char* id_file,
                             uint64_t gradient_floats, mgt_comm_t** out_comm);
mgt_status_t mgt_comm_destroy(mgt_comm_t* comm);
float* mgt_comm_gradient_buffer(mgt_comm_t* comm);
/* In place on a range of the gradient buffer: sum over ranks (rank order) then * 1/world_size.
 * Replaces NcclAllreduceAverageFloat (allreduce_nccl.cu:120-150). Every rank must make the same
 * calls in the same order. */
mgt_status_t mgt_comm_allreduce_average(mgt_comm_t* comm, const mgt_allreduce_config_t* config, float* device_gradients,
                                        void* stream);
/* The same exchange fused with the AdamW update (and fp16 mirror, may be NULL) of parameters
 * [param_offset, param_offset + param_count): replaces allreduce + ScaleKernel + AdamW kernel
 * (allreduce_nccl.cu:130-148, native/cuda/adamw.cu:35-46). weights/m/v are the flat full-model
 * arrays; the gradient buffer afterwards holds the averaged gradient as in the reference. */
mgt_status_t mgt_comm_allreduce_average_adamw(mgt_comm_t* comm, uint64_t param_offset, uint64_t param_count,
                                              const mgt_adamw_config_t* adamw, float* device_weights,
                                              uint16_t* device_weights_half, float* device_m, float* device_v, void* stream);
/* Synchronises `stream` and reads the communicator's status: MGT_OK or MGT_DEVICE_TIMEOUT (a peer did
 * not show up within the wait limit; out_code 1 = ready wait, 2 = done wait). A timeout is final for this
 * communicator: the ranks' flag state no longer agrees, so every later exchange call and check returns
 * MGT_DEVICE_TIMEOUT without launching anything, and parameters that a fused update had already touched are
 * undefined. Destroy it, restore weights/m/v from a checkpoint and create a new one.
 * (The reference's NCCL call has no timeout at all: a dead peer hangs it, allreduce_nccl.cu:130.) */
mgt_status_t mgt_comm_check(mgt_comm_t* comm, void* stream, int32_t* out_code);
/* How long an exchange kernel waits for a peer before it gives up (default 1000 ms, at most 60 000).
 * The limit also bounds how far apart the ranks may ENTER a collective, so ranks that do unequal host
 * work between steps (checkpoint files, start-up) meet at mgt_comm_host_barrier first. No counterpart
 * in the reference. */
mgt_status_t mgt_comm_set_wait_limit_ms(mgt_comm_t* comm, uint32_t milliseconds);
/* Host-side rendezvous of all ranks through small files beside the id file (no GPU work, no kernel):
 * returns when every rank has called it the same number of times, or MGT_IO_FAILURE after timeout_ms.
 * world_size 1: returns at once. No counterpart in the reference. */
mgt_status_t mgt_comm_host_barrier(mgt_comm_t* comm, uint32_t timeout_ms);
uint64_t mgt_comm_launch_count(const mgt_comm_t* comm);

/* ---- run plan and output files (host only, no GPU) --------------------------------------------
 * The configuration travels as the trainer's own command line: `argv` holds flag/value pairs in
 * the grammar of mgt_native_train (native/tools/mgt_native_train_smoke.cu:525-613), without the
 * program name. Replaces BuildTrainPlan (native/src/train_plan.cpp:204-230) and the trainer's
 * writers (tool:184-404, 888-895); file contents are byte-compatible with the reference's. */
#define MGT_PLAN_SUMMARY_FIELDS 16
#define MGT_PLAN_LINEAR_OP_FIELDS 14
/* out: padded_state_dim, physical_hd1, physical_hd2, param blocks, linear ops, gradient buckets,
 * total_params, total_bytes, total_rank_bytes, training_scratch_bytes, logical_params,
 * fits_state_record, states_bytes, layout_allreduce_bytes, walkers, state_capacity_bytes */
mgt_status_t mgt_plan_summary(int32_t argc, const char* const* argv, uint64_t* out, uint32_t out_count);
/* out: op_id, phase, role, block_index, transpose_a, transpose_b, m, n, k, backend class,
 * tensor_core_eligible, logical_tail_masked, lhs_rows, rhs_cols (native/include/mgt/train_plan.hpp:44-63) */
mgt_status_t mgt_plan_linear_op(int32_t argc, const char* const* argv, uint32_t index, uint32_t* out, uint32_t out_count);
/* metadata.env, layers.json, linear_ops.json (tool:184-214, 888-895) */
mgt_status_t mgt_plan_write_files(int32_t argc, const char* const* argv, const char* dir, int32_t overlap_allreduce,
                                  int32_t comm_enabled, int32_t resumed);
/* One step as the trainer logs it: the "phase=start" line of train.log (tool:750-762), the per-step line of train.log
 * (tool:856-858) and the row of profile.jsonl (tool:859-875), each zero-terminated into a caller buffer of `capacity`
 * bytes (NULL = not wanted). The trainer binary writes its files through the same formatters. */
typedef struct {
    uint32_t step;
    float loss, step_ms, walk_ms, backward_ms, allreduce_ms, adam_ms;
    uint64_t memory_bytes;
    uint32_t overlap_ranges, overlap_chunks;
    float backward_stage_ms[7]; /* the fields of mgt_backward_profile_t, in its order */
} mgt_step_record_t;
mgt_status_t mgt_format_step_record(int32_t argc, const char* const* argv, const mgt_step_record_t* record,
                                    int32_t overlap_allreduce, int32_t comm_enabled, int32_t resumed, char* start_line,
                                    char* log_line, char* profile_row, uint32_t capacity);
/* Folds trained batch normalisation (mgt_train_options_t.batch_norm) into the layers it follows, with the RUNNING
 * statistics: the hidden layer's and every fc2's weight columns are scaled by gamma / sqrt(var + eps) and the biases
 * become (b - mean) * that + beta. Host arrays; weights (the reference's layout, mgt_mlp_param_count floats) are changed
 * in place and then describe a network without normalisation - what the weights/ files hold ("normalization": "none",
 * native/tools/mgt_native_train_smoke.cu:343). scale_shift and running_stats: mgt_bn_param_count floats each, layer 0 =
 * hidden layer, layer k + 1 = block k; {gamma, beta} resp. {mean, var} of hd2 floats per layer. */
mgt_status_t mgt_fold_batch_norm(const mgt_mlp_shape_t* shape, float* weights, const float* scale_shift,
                                 const float* running_stats, float eps);
/* The trainer's software float->fp16 converter used for weights/ files (tool:215-229). */
uint16_t mgt_export_float_to_fp16(float value);
/* weights/ (fp16 per-layer files + manifest + weights.f32.bin) and checkpoint/ (tool:241-390) from host arrays. */
mgt_status_t mgt_write_run_artifacts(int32_t argc, const char* const* argv, const char* dir, const float* weights,
                                     const float* adam_m, const float* adam_v);
/* checkpoint/state.f32.bin = weights | adam_m | adam_v (tool:392-404) */
mgt_status_t mgt_read_checkpoint(const char* checkpoint_dir, uint64_t param_count, float* weights, float* adam_m, float* adam_v);

/* Replaces LoadPuzzleDefinition (native/include/mgt/puzzle_io.hpp, native/src/puzzle_io.cpp:48-97): the integers of the
 * JSON text are group id, state length, move count and move_count permutations; the target file holds exactly
 * state_len bytes. `moves` receives MGT_MOVE_COUNT records (unused ones are the identity), pad positions of a move map
 * to themselves, pad bytes of the target are 0. The reference fixes group 888 / 72 / 18; here they are arguments.
 * Returns MGT_OK, MGT_INVALID_PUZZLE or MGT_IO_FAILURE. Host only. */
mgt_status_t mgt_load_puzzle_definition(const char* group_json, const char* target_bin, uint32_t group_id, uint32_t state_len,
                                        uint32_t move_count, mgt_train_state_t* moves, mgt_train_state_t* target);

/* ---- diagnostics ---------------------------------------------------------------------------
 * One plain GEMM through the tcgen05 kernel, used by the parity tests to pin each operand form.
 * D[M x N] fp32 = A * B with fp16 operands; a_mn_major: A stored [K][M] (else [M][K]);
 * b_mn_major: B stored [K][N] (else [N][K]); lda/ldb are row pitches in elements.
 * d must be 4-byte aligned, and 16-byte aligned when a single split is used (splits == 1 or k <= 64) and
 * n is a multiple of 4 (the accumulator tiles are then stored to d as 16-byte vectors); partial_scratch must
 * be 16-byte aligned when n is a multiple of 4. Otherwise MGT_INVALID_CONFIG, nothing is launched.
 * No counterpart in the reference. */
mgt_status_t mgt_debug_gemm(mgt_engine_t* engine, const uint16_t* a, uint32_t lda, int32_t a_mn_major,
                            const uint16_t* b, uint32_t ldb, int32_t b_mn_major, float* d, uint32_t m, uint32_t n,
                            uint32_t k, uint32_t splits, float* partial_scratch, void* stream);

/* Split-K GEMM that allocates nothing. No counterpart in the reference.
 *
 * Same computation and arguments as mgt_debug_gemm, for callers that cannot obtain device memory
 * themselves: a host application that has handed all of HBM to its own memory pool, or a
 * latency-critical loop in which a cudaMalloc (which synchronises the whole device) is not
 * acceptable. Such a caller has nowhere to put the split-K partial sums, so they live in a buffer
 * that is part of the library image: MGT_STATIC_SCRATCH_FLOATS floats (16 MiB) of device memory
 * on every GPU that loads the library, held until the process exits. No engine handle is needed
 * and neither this call nor anything it calls uses cudaMalloc, cudaFree or another device allocator.
 *
 * Limit: min(splits, ceil(k/64)) * m * n <= MGT_STATIC_SCRATCH_FLOATS when more than one split is
 * used; beyond that the call returns MGT_CAPACITY_EXCEEDED and says why on stderr.
 * The first call on each device looks up the device addresses of the built-in buffers and the
 * tensor-map encoder (host work only); make that first call before starting any stream capture.
 * All calls on a device share the one buffer: calls that may overlap on the GPU (different
 * streams) race on it - keep them on one stream or order them with events.
 * d has the alignment rule of mgt_debug_gemm. The kernels' bounded waits report into a status word that is
 * built into the library as well; read it with mgt_static_scratch_check. */
#define MGT_STATIC_SCRATCH_FLOATS (4u << 20)
mgt_status_t mgt_gemm_split_k_static_scratch(const uint16_t* a, uint32_t lda, int32_t a_mn_major, const uint16_t* b,
                                             uint32_t ldb, int32_t b_mn_major, float* d, uint32_t m, uint32_t n,
                                             uint32_t k, uint32_t splits, void* stream);
/* What mgt_engine_check is for an engine, for mgt_gemm_split_k_static_scratch on the current device:
 * synchronises `stream`, reads and clears the built-in status word. MGT_OK, or MGT_DEVICE_TIMEOUT when a
 * kernel of an earlier call gave up on a bounded wait (d of that call is then undefined). Allocates nothing.
 * No counterpart in the reference. */
mgt_status_t mgt_static_scratch_check(void* stream, int32_t* out_device_code);

const char* mgt_status_name(mgt_status_t status);
const char* mgt_version(void);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif

#endif /* MGT_B200_H_ */
