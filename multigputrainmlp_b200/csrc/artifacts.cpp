// Output files of a training run, byte-compatible with the reference trainer's
// (native/tools/mgt_native_train_smoke.cu:184-404, 750-762, 856-895): train.log lines,
// profile.jsonl rows, metadata.env, layers.json, linear_ops.json, the fp16 weight export consumed
// by the beam-search project and the fp32 checkpoint. Pure host code.
#include "host_plan.hpp"

#include <cstring>
#include <filesystem>
#include <fstream>
#include <iomanip>
#include <sstream>

namespace mgt {
namespace host {
namespace {

namespace fs = std::filesystem;

// Offsets into the flat fp32 parameter array (native/cuda/mlp_backward.cu:25-36).
struct Flat {
    uint64_t in_table, in_bias, hid_w, hid_b, res_base, blk, out_w, out_b;
    explicit Flat(const TrainPlan& p) {
        const uint64_t H1 = p.physical_hd1, H2 = p.physical_hd2;
        in_table = 0;
        in_bias = static_cast<uint64_t>(p.options.state_len) * p.options.state_value_count * H1;
        hid_w = in_bias + H1;
        hid_b = hid_w + H1 * H2;
        res_base = hid_b + H2;
        blk = 2 * (H2 * H2 + H2);
        out_w = res_base + p.options.nrd * blk;
        out_b = out_w + H2 * p.options.output_dim;
    }
};

// Copies a [rows x cols] matrix into a zero-padded [rows x pitch] one and writes it as fp16.
bool WriteMatrixFp16(const fs::path& path, const float* src, uint64_t rows, uint64_t cols, uint64_t pitch) {
    std::ofstream out(path, std::ios::binary);
    if (!out) return false;
    std::vector<uint16_t> line(pitch);
    for (uint64_t r = 0; r < rows; ++r) {
        for (uint64_t c = 0; c < pitch; ++c) line[c] = ExportFloatToFp16(c < cols ? src[r * cols + c] : 0.0f);
        out.write(reinterpret_cast<const char*>(line.data()), static_cast<std::streamsize>(pitch * sizeof(uint16_t)));
    }
    return static_cast<bool>(out);
}

}  // namespace

uint16_t ExportFloatToFp16(float value) {
    // round-half-up on the mantissa, flush below 2^-25... kept exactly as the consumer of the files expects
    uint32_t bits;
    std::memcpy(&bits, &value, sizeof(bits));
    const uint32_t sign = (bits >> 16) & 0x8000U;
    const int32_t exp = static_cast<int32_t>((bits >> 23) & 0xffU) - 112;
    uint32_t mant = bits & 0x7fffffU;
    if (exp <= 0) {
        if (exp < -10) return static_cast<uint16_t>(sign);
        mant = (mant | 0x800000U) >> static_cast<uint32_t>(1 - exp);
        return static_cast<uint16_t>(sign | ((mant + 0x1000U) >> 13));
    }
    if (exp >= 31) return static_cast<uint16_t>(sign | 0x7c00U);
    return static_cast<uint16_t>(sign | (static_cast<uint32_t>(exp) << 10) | ((mant + 0x1000U) >> 13));
}

bool WriteLinearOpsManifest(const std::string& dir, const TrainPlan& plan) {
    std::ofstream out(fs::path(dir) / "linear_ops.json");
    if (!out) return false;
    out << "{\n  \"format\": \"mgt_linear_ops_v1\",\n  \"op_count\": " << plan.linear_ops.size() << ",\n  \"linear_ops\": [\n";
    for (size_t i = 0; i < plan.linear_ops.size(); ++i) {
        const LinearOp& op = plan.linear_ops[i];
        out << "    {\"op_id\": " << op.op_id << ", \"phase\": \"" << LinearPhaseName(op.phase) << "\", \"role\": \"" << ParamRoleName(op.role)
            << "\", \"block_index\": " << op.block_index << ", \"transpose_a\": \"" << (op.transpose_a ? "T" : "N") << "\", \"transpose_b\": \""
            << (op.transpose_b ? "T" : "N") << "\", \"m\": " << op.m << ", \"n\": " << op.n << ", \"k\": " << op.k << ", \"lhs_rows\": " << op.lhs_rows
            << ", \"lhs_cols\": " << op.lhs_cols << ", \"rhs_rows\": " << op.rhs_rows << ", \"rhs_cols\": " << op.rhs_cols
            << ", \"output_rows\": " << op.output_rows << ", \"output_cols\": " << op.output_cols << ", \"backend\": \"" << LinearBackendName(op.backend)
            << "\", \"tensor_core_eligible\": " << (op.tensor_core_eligible ? "true" : "false")
            << ", \"logical_tail_masked\": " << (op.logical_tail_masked ? "true" : "false") << "}" << (i + 1 == plan.linear_ops.size() ? "\n" : ",\n");
    }
    out << "  ]\n}\n";
    return static_cast<bool>(out);
}

bool WriteMetadataEnv(const std::string& dir, const TrainPlan& plan, bool overlap, bool comm_enabled, bool resumed) {
    const TrainOptions& o = plan.options;
    std::ofstream out(fs::path(dir) / "metadata.env");
    if (!out) return false;
    const std::pair<const char*, std::string> rows[] = {
        {"MODEL_MODE", "MLP2RB"}, {"OUTPUT_DIM", std::to_string(o.output_dim)}, {"WORLD_SIZE", std::to_string(o.world_size)},
        {"GLOBAL_RANK", std::to_string(o.global_rank)}, {"LOCAL_RANK", std::to_string(o.local_rank)}, {"DEVICE_ID", std::to_string(o.device_id)},
        {"HD1", std::to_string(o.hd1)}, {"PHYSICAL_HD1", std::to_string(plan.physical_hd1)}, {"HD2", std::to_string(o.hd2)},
        {"PHYSICAL_HD2", std::to_string(plan.physical_hd2)}, {"NUM_CLASSES", std::to_string(o.state_value_count)}, {"NRD", std::to_string(o.nrd)},
        {"K_MIN", std::to_string(o.k_min)}, {"K_MAX", std::to_string(o.k_max)}, {"BATCH_SIZE", std::to_string(o.batch_size)},
        {"GRADIENT_CAROUSEL_SLOTS", std::to_string(o.gradient_carousel_slots)}, {"LT_WORKSPACE_BYTES", std::to_string(o.lt_workspace_bytes)},
        {"INPUT_GRAD_PARTIAL_CHUNKS", std::to_string(o.input_grad_partial_chunks)},
        {"INPUT_GRAD_POSITIONS_PER_BLOCK", std::to_string(o.input_grad_positions_per_block)},
        {"INPUT_GRAD_POSITION_TILE", std::to_string(o.input_grad_position_tile)}, {"INPUT_GRAD_FP16", o.input_grad_fp16 ? "1" : "0"},
        {"INPUT_GRAD_BACKEND", InputGradBackendName(o)}, {"LINEAR_FP16", o.linear_fp16 ? "1" : "0"},
        {"PERSISTENT_HALF_WEIGHTS", o.persistent_half_weights ? "1" : "0"}, {"OVERLAP_ALLREDUCE", overlap ? "1" : "0"},
        {"GRADIENT_BUCKETS", std::to_string(plan.gradient_bucket_count)}, {"NCCL_ENABLED", comm_enabled ? "1" : "0"},
        {"RESUME_CHECKPOINT", resumed ? "1" : "0"}, {"ARTIFACTS_WRITTEN", o.write_artifacts ? "1" : "0"},
        {"NUM_PARAMETERS", std::to_string(plan.total_params)},
    };
    for (const auto& row : rows) out << row.first << "=" << row.second << "\n";
    return static_cast<bool>(out);
}

bool WriteLayersJson(const std::string& dir, const TrainPlan& plan) {
    const TrainOptions& o = plan.options;
    std::ofstream out(fs::path(dir) / "layers.json");
    if (!out) return false;
    out << "{\n  \"model_mode\": \"MLP2RB\",\n  \"output_dim\": " << o.output_dim << ",\n  \"state_len\": " << o.state_len
        << ",\n  \"state_storage_len\": " << plan.padded_state_dim << ",\n  \"num_classes\": " << o.state_value_count << ",\n  \"hd1\": " << o.hd1
        << ",\n  \"physical_hd1\": " << plan.physical_hd1 << ",\n  \"hd2\": " << o.hd2 << ",\n  \"physical_hd2\": " << plan.physical_hd2
        << ",\n  \"nrd\": " << o.nrd << ",\n  \"artifacts_written\": " << (o.write_artifacts ? "true" : "false")
        << ",\n  \"num_parameters\": " << plan.total_params << "\n}\n";
    return static_cast<bool>(out);
}

bool WriteWeights(const std::string& dir, const TrainPlan& plan, const std::vector<float>& w) {
    const TrainOptions& o = plan.options;
    if (w.size() != plan.total_params) return false;
    const fs::path wd = fs::path(dir) / "weights";
    std::error_code ec;
    fs::create_directories(wd, ec);
    {
        std::ofstream flat(wd / "weights.f32.bin", std::ios::binary);
        if (!flat) return false;
        flat.write(reinterpret_cast<const char*>(w.data()), static_cast<std::streamsize>(w.size() * sizeof(float)));
        if (!flat) return false;
    }
    const Flat f(plan);
    const uint64_t H1 = plan.physical_hd1, H2 = plan.physical_hd2, OUT = o.output_dim;
    const uint64_t E1 = (H1 + 7) / 8 * 8, E2 = (H2 + 7) / 8 * 8;  // exported hidden sizes are multiples of 8 (tool:259-260)
    const uint64_t in_rows = static_cast<uint64_t>(o.state_len) * o.state_value_count;
    bool ok = WriteMatrixFp16(wd / "input_weight_hxk.fp16", w.data() + f.in_table, in_rows, H1, E1) &&
              WriteMatrixFp16(wd / "input_bias.fp16", w.data() + f.in_bias, 1, H1, E1) &&
              WriteMatrixFp16(wd / "hidden_weight_hxk.fp16", w.data() + f.hid_w, H1, H2, E2) &&
              WriteMatrixFp16(wd / "hidden_bias.fp16", w.data() + f.hid_b, 1, H2, E2);
    // hidden_weight has E1 rows in the file: rows beyond H1 (if any) are zero
    if (ok && E1 > H1) {
        std::ofstream app(wd / "hidden_weight_hxk.fp16", std::ios::binary | std::ios::app);
        std::vector<uint16_t> zeros(E2 * (E1 - H1), 0);
        app.write(reinterpret_cast<const char*>(zeros.data()), static_cast<std::streamsize>(zeros.size() * 2));
        ok = static_cast<bool>(app);
    }
    for (uint32_t b = 0; ok && b < o.nrd; ++b) {
        const uint64_t base = f.res_base + b * f.blk;
        const std::string stem = "residual" + std::to_string(b);
        auto square = [&](const std::string& name, uint64_t off) {
            if (!WriteMatrixFp16(wd / name, w.data() + off, H2, H2, E2)) return false;
            if (E2 > H2) {
                std::ofstream app(wd / name, std::ios::binary | std::ios::app);
                std::vector<uint16_t> zeros(E2 * (E2 - H2), 0);
                app.write(reinterpret_cast<const char*>(zeros.data()), static_cast<std::streamsize>(zeros.size() * 2));
                return static_cast<bool>(app);
            }
            return true;
        };
        ok = square(stem + "_fc1_weight_hxk.fp16", base) && WriteMatrixFp16(wd / (stem + "_fc1_bias.fp16"), w.data() + base + H2 * H2, 1, H2, E2) &&
             square(stem + "_fc2_weight_hxk.fp16", base + H2 * H2 + H2) &&
             WriteMatrixFp16(wd / (stem + "_fc2_bias.fp16"), w.data() + base + 2 * H2 * H2 + H2, 1, H2, E2);
    }
    if (ok) {
        ok = WriteMatrixFp16(wd / "output_weight_hxk.fp16", w.data() + f.out_w, H2, OUT, OUT);
        if (ok && E2 > H2) {
            std::ofstream app(wd / "output_weight_hxk.fp16", std::ios::binary | std::ios::app);
            std::vector<uint16_t> zeros(OUT * (E2 - H2), 0);
            app.write(reinterpret_cast<const char*>(zeros.data()), static_cast<std::streamsize>(zeros.size() * 2));
            ok = static_cast<bool>(app);
        }
        ok = ok && WriteMatrixFp16(wd / "output_bias.fp16", w.data() + f.out_b, 1, OUT, OUT);
    }
    if (!ok) return false;
    std::ofstream man(wd / "manifest.json", std::ios::binary);
    if (!man) return false;
    man << "{\n  \"format\": \"stream1_weights\",\n  \"version\": 1,\n  \"state_len\": " << o.state_len << ",\n  \"num_classes\": " << o.state_value_count
        << ",\n  \"logical_num_classes\": " << o.state_value_count << ",\n  \"hd1\": " << E1 << ",\n  \"hd2\": " << E2 << ",\n  \"original_hd1\": " << o.hd1
        << ",\n  \"original_hd2\": " << o.hd2 << ",\n  \"hidden_alignment\": 8,\n  \"nrd\": " << o.nrd << ",\n  \"output_dim\": " << OUT
        << ",\n  \"dtype\": \"fp16\",\n  \"normalization\": \"none\",\n  \"layout\": \"row-major input activations times weight_hxk\",\n"
        << "  \"flat_debug_weights\": \"weights.f32.bin\"\n}\n";
    return static_cast<bool>(man);
}

bool WriteCheckpoint(const std::string& dir, const TrainPlan& plan, const std::vector<float>& w, const std::vector<float>& m, const std::vector<float>& v) {
    const TrainOptions& o = plan.options;
    if (w.size() != m.size() || w.size() != v.size()) return false;
    const fs::path cd = fs::path(dir) / "checkpoint";
    std::error_code ec;
    fs::create_directories(cd, ec);
    std::ofstream data(cd / "state.f32.bin", std::ios::binary);
    if (!data) return false;
    for (const std::vector<float>* section : {&w, &m, &v})
        data.write(reinterpret_cast<const char*>(section->data()), static_cast<std::streamsize>(section->size() * sizeof(float)));
    if (!data) return false;
    std::ofstream man(cd / "manifest.json", std::ios::binary);
    if (!man) return false;
    man << "{\n  \"format\": \"mgt_train_checkpoint\",\n  \"version\": 1,\n  \"step\": " << o.steps << ",\n  \"model_mode\": \"MLP2RB\",\n  \"output_dim\": "
        << o.output_dim << ",\n  \"state_len\": " << o.state_len << ",\n  \"state_storage_len\": " << plan.padded_state_dim << ",\n  \"num_classes\": "
        << o.state_value_count << ",\n  \"hd1\": " << o.hd1 << ",\n  \"physical_hd1\": " << plan.physical_hd1 << ",\n  \"hd2\": " << o.hd2
        << ",\n  \"physical_hd2\": " << plan.physical_hd2 << ",\n  \"nrd\": " << o.nrd << ",\n  \"optimizer\": \"AdamW\",\n  \"weight_decay\": "
        << o.weight_decay << ",\n  \"dtype\": \"float32\",\n  \"data\": \"state.f32.bin\",\n  \"sections\": [\"weights\", \"adam_m\", \"adam_v\"],\n"
        << "  \"params_per_section\": " << w.size() << "\n}\n";
    return static_cast<bool>(man);
}

bool ReadCheckpoint(const std::string& checkpoint_dir, std::vector<float>* w, std::vector<float>* m, std::vector<float>* v) {
    if (!w || !m || !v || w->size() != m->size() || w->size() != v->size()) return false;
    std::ifstream data(fs::path(checkpoint_dir) / "state.f32.bin", std::ios::binary);
    if (!data) return false;
    for (std::vector<float>* section : {w, m, v})
        data.read(reinterpret_cast<char*>(section->data()), static_cast<std::streamsize>(section->size() * sizeof(float)));
    return static_cast<bool>(data);
}

std::string StartLogLine(const TrainPlan& plan, bool overlap, bool comm_enabled, bool resumed) {
    const TrainOptions& o = plan.options;
    std::ostringstream s;
    s << "rank=" << o.global_rank << " local_rank=" << o.local_rank << " device=" << o.device_id << " world_size=" << o.world_size
      << " phase=start batch_states=" << o.batch_size << " hd1=" << o.hd1 << " physical_hd1=" << plan.physical_hd1 << " hd2=" << o.hd2
      << " physical_hd2=" << plan.physical_hd2 << " nrd=" << o.nrd << " k_min=" << o.k_min << " k_max=" << o.k_max
      << " input_grad_partial_chunks=" << o.input_grad_partial_chunks << " input_grad_positions_per_block=" << o.input_grad_positions_per_block
      << " input_grad_position_tile=" << o.input_grad_position_tile << " input_grad_fp16=" << (o.input_grad_fp16 ? 1 : 0)
      << " input_grad_backend=" << InputGradBackendName(o) << " linear_fp16=" << (o.linear_fp16 ? 1 : 0)
      << " persistent_half_weights=" << (o.persistent_half_weights ? 1 : 0) << " lt_workspace_bytes=" << o.lt_workspace_bytes
      << " overlap_allreduce=" << (overlap ? 1 : 0) << " nccl=" << (comm_enabled ? 1 : 0) << " resumed=" << (resumed ? 1 : 0) << "\n";
    return s.str();
}

std::string StepLogLine(const TrainPlan& plan, const StepRecord& r) {
    std::ostringstream s;
    s << "rank=" << plan.options.global_rank << " step=" << r.step << " phase=train loss=" << r.loss << " step_ms=" << r.step_ms
      << " walk_ms=" << r.walk_ms << " backward_ms=" << r.backward_ms << " allreduce_ms=" << r.allreduce_ms << " adam_ms=" << r.adam_ms
      << " memory_bytes=" << r.memory_bytes << "\n";
    return s.str();
}

std::string StepProfileRow(const TrainPlan& plan, const StepRecord& r, bool overlap) {
    // Fixed notation; three digits from "milliseconds" up to "loss", six from "loss" on (tool:859-875).
    const TrainOptions& o = plan.options;
    std::ostringstream s;
    s << std::fixed;
    s << "{\"rank\":" << o.global_rank << ",\"device\":" << o.device_id << ",\"step\":" << r.step << ",\"phase\":\"train\",\"milliseconds\":"
      << std::setprecision(3) << r.step_ms << ",\"walk_ms\":" << r.walk_ms << ",\"backward_ms\":" << r.backward_ms << ",\"allreduce_ms\":" << r.allreduce_ms
      << ",\"adam_ms\":" << r.adam_ms << ",\"batch_states\":" << o.batch_size << ",\"loss\":" << std::setprecision(6) << r.loss
      << ",\"memory_bytes\":" << r.memory_bytes << ",\"gradient_slots\":" << o.gradient_carousel_slots << ",\"gradient_buckets\":" << plan.gradient_bucket_count
      << ",\"input_grad_fp16\":" << (o.input_grad_fp16 ? 1 : 0) << ",\"input_grad_position_tile\":" << o.input_grad_position_tile
      << ",\"input_grad_backend\":\"" << InputGradBackendName(o) << "\",\"linear_fp16\":" << (o.linear_fp16 ? 1 : 0)
      << ",\"persistent_half_weights\":" << (o.persistent_half_weights ? 1 : 0) << ",\"lt_workspace_bytes\":" << o.lt_workspace_bytes
      << ",\"overlap_allreduce\":" << (overlap ? 1 : 0) << ",\"overlap_ranges\":" << r.overlap_ranges << ",\"overlap_chunks\":" << r.overlap_chunks
      << ",\"bw_input_forward_ms\":" << r.bw[0] << ",\"bw_hidden_forward_ms\":" << r.bw[1] << ",\"bw_residual_forward_ms\":" << r.bw[2]
      << ",\"bw_output_ms\":" << r.bw[3] << ",\"bw_residual_backward_ms\":" << r.bw[4] << ",\"bw_hidden_backward_ms\":" << r.bw[5]
      << ",\"bw_input_grad_ms\":" << r.bw[6] << ",\"status\":\"ok\"}\n";
    return s.str();
}

}  // namespace host
}  // namespace mgt
