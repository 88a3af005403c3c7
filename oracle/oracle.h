/*
 * CPU oracle for the per-step training hot path (TEST INFRASTRUCTURE ONLY).
 *
 * This library is a plain, single-threaded restatement of the reference's algorithms.
 * It exists so that the CUDA kernels can be checked; it is never linked into, imported by
 * or executed from the shipped library, the trainer binary or the product Python package.
 * Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may use it.
 *
 * Parity status: pinned. Every function here is compared against the reference's own CPU
 * code (built from the reference sources into oracle/_ref/libmgt_ref.so by oracle/Makefile)
 * and against golden vectors generated from that build (tests/golden/).
 * The fp16 rounding-point model (orc_mlp_loss_grad_mixed) has no CPU counterpart in the
 * reference: it restates the data flow of the reference's GPU fp16 path
 * (native/cuda/mlp_backward.cu:1273-1507) and is pinned to the fp32 reference through the
 * reference's own mixed-precision envelope (loss 2e-3 + 2e-2*scale, grad rel-L2 8e-2).
 */
#ifndef MGT_ORACLE_H_
#define MGT_ORACLE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same numeric values as the reference's mgt::Status (native/include/mgt/status.hpp:5-13). */
enum { ORC_OK = 0, ORC_INVALID_CONFIG = 1 };

#define ORC_STATE_STORAGE_LEN 80 /* native/include/mgt/config.hpp:32-35 */

typedef struct {
    uint32_t depth;
    uint32_t last_move;
    uint64_t rng_counter;
} orc_walk_meta_t; /* native/include/mgt/static_contracts.hpp:15-19 */

typedef struct {
    uint32_t state_len;
    uint32_t state_value_pad;
    uint32_t hd1;
    uint32_t hd2;
    uint32_t residual_blocks;
    uint32_t output_dim;
} orc_mlp_shape_t; /* native/include/mgt/mlp_cpu_ref.hpp:9-16 */

uint64_t orc_mix64(uint64_t x); /* native/src/random_walk_cpu.cpp:7-12 */

/* native/src/random_walk_cpu.cpp:32-66 with runtime move_count/state_len as in
 * native/cuda/random_walk_kernel.cu:19-64. moves: move_count records of 80 bytes. */
int orc_random_walks(const uint8_t* moves, const uint8_t* target, uint32_t move_count,
                     uint32_t state_len, uint32_t state_storage_len, uint64_t base_seed,
                     uint64_t epoch, uint64_t step, uint32_t global_rank, uint32_t k_min,
                     uint32_t k_max, uint32_t sample_count, uint8_t* states, float* labels,
                     orc_walk_meta_t* meta);

/* Built-in puzzle of the trainer: native/tools/mgt_native_train_smoke.cu:117-140. */
void orc_build_cyclic_puzzle(uint32_t state_len, uint32_t move_count, uint32_t max_moves,
                             uint8_t* moves, uint8_t* target);

uint64_t orc_mlp_param_count(const orc_mlp_shape_t* shape); /* mlp_cpu_ref.cpp:40-51 */

/* native/src/mlp_cpu_ref.cpp:129-147 */
int orc_mlp_forward(const orc_mlp_shape_t* shape, const float* weights, const uint8_t* states,
                    uint32_t sample_count, float* outputs);

/* native/src/mlp_cpu_ref.cpp:149-251 (true fp32, sample-major accumulation order). */
int orc_mlp_loss_grad(const orc_mlp_shape_t* shape, const float* weights, const uint8_t* states,
                      const float* labels, uint32_t sample_count, float* loss, float* grad);

/* The reference's GPU fp16 data flow (native/cuda/mlp_backward.cu:1273-1507) on the CPU:
 * fp16 round-to-nearest-even at the same tensors, fp32 accumulation, fp32 master biases
 * for hidden/residual layers, fp16 mirror for the embedding table and its bias.
 * half_linear / half_input_grad mirror --linear-fp16 / --input-grad-fp16. */
int orc_mlp_loss_grad_mixed(const orc_mlp_shape_t* shape, const float* weights,
                            const uint8_t* states, const float* labels, uint32_t sample_count,
                            int half_linear, int half_input_grad, float* loss, float* grad);

/* The same data flow with the options the reference does NOT have (so nothing in the reference pins them; they are
 * pinned by finite differences in tests/test_oracle.py and are the checker for the library's opt-in extensions):
 *   operand_format  ORC_OPERAND_BF16: operands rounded to bfloat16 (round to nearest even) instead of fp16
 *   loss_kind       ORC_LOSS_CROSS_ENTROPY: per-depth logits (output_dim classes), class = depth - 1, mean over the
 *                   batch of -log softmax; labels keep the trainer's layout (the depth in every output slot)
 *   batch_norm      training-mode batch normalisation (batch statistics, biased variance, eps) of the hidden layer's
 *                   pre-activation and of every block's fc2 output before it joins the skip path. Its scale and shift
 *                   follow the reference's parameters in `weights`/`grad`: layer 0 = hidden, layer k + 1 = block k,
 *                   each gamma[hd2] then beta[hd2] (orc_bn_param_count floats). bn_batch_stats (may be NULL) receives
 *                   mean[hd2], var[hd2] per layer.
 * With all options off this IS orc_mlp_loss_grad_mixed. */
enum { ORC_OPERAND_FP16 = 0, ORC_OPERAND_BF16 = 1 };
enum { ORC_LOSS_MSE = 0, ORC_LOSS_CROSS_ENTROPY = 1 };
typedef struct {
    int half_linear;
    int half_input_grad;
    int operand_format;
    int loss_kind;
    int batch_norm;
    float bn_eps;
} orc_train_options_t;
uint64_t orc_bn_param_count(const orc_mlp_shape_t* shape);
int orc_mlp_loss_grad_ex(const orc_mlp_shape_t* shape, const float* weights, const uint8_t* states,
                         const float* labels, uint32_t sample_count, const orc_train_options_t* options,
                         float* loss, float* grad, float* bn_batch_stats);
uint16_t orc_float_to_bf16_rn(float value);
float orc_bf16_to_float(uint16_t bits);

/* native/src/mlp_cpu_ref.cpp:253-276; half_mirror (may be NULL) as adamw.cu:35-46. */
int orc_adamw_step(float* weights, const float* grad, float* m, float* v, uint64_t param_count,
                   uint64_t step, float lr, float beta1, float beta2, float eps,
                   float weight_decay, uint16_t* half_mirror);

/* IEEE round-to-nearest-even float->half (what __float2half_rn does) and back. */
uint16_t orc_float_to_half_rn(float value);
float orc_half_to_float(uint16_t bits);

/* The trainer's software converter used for weights/.fp16 files:
 * native/tools/mgt_native_train_smoke.cu:215-229 (round-half-up, flushes exp < -10). */
uint16_t orc_export_float_to_fp16(float value);

/* Allreduce average: sum over ranks in rank order then *(1/W)
 * (native/cuda/allreduce_nccl.cu:120-150, native/src/allreduce.cpp:17-26). */
void orc_allreduce_average(const float* const* rank_grads, uint32_t world_size, uint64_t count,
                           float* out);

#ifdef __cplusplus
}
#endif

#endif /* MGT_ORACLE_H_ */
