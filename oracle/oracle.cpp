// CPU oracle (test infrastructure only, see oracle.h). Plain scalar loops on purpose.
#include "oracle.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

namespace {

struct Offsets {
    uint64_t input_table, input_bias, hidden_weight, hidden_bias, residual_base, output_weight,
        output_bias, total;
};

uint64_t BlockParams(const orc_mlp_shape_t& s) { return 2ULL * ((uint64_t)s.hd2 * s.hd2 + s.hd2); }

// Flat parameter layout: native/src/mlp_cpu_ref.cpp:40-51.
Offsets BuildOffsets(const orc_mlp_shape_t& s) {
    Offsets o{};
    o.input_table = 0;
    o.input_bias = (uint64_t)s.state_len * s.state_value_pad * s.hd1;
    o.hidden_weight = o.input_bias + s.hd1;
    o.hidden_bias = o.hidden_weight + (uint64_t)s.hd1 * s.hd2;
    o.residual_base = o.hidden_bias + s.hd2;
    o.output_weight = o.residual_base + (uint64_t)s.residual_blocks * BlockParams(s);
    o.output_bias = o.output_weight + (uint64_t)s.hd2 * s.output_dim;
    o.total = o.output_bias + s.output_dim;
    return o;
}
uint64_t Fc1W(const orc_mlp_shape_t& s, const Offsets& o, uint32_t b) { return o.residual_base + (uint64_t)b * BlockParams(s); }
uint64_t Fc1B(const orc_mlp_shape_t& s, const Offsets& o, uint32_t b) { return Fc1W(s, o, b) + (uint64_t)s.hd2 * s.hd2; }
uint64_t Fc2W(const orc_mlp_shape_t& s, const Offsets& o, uint32_t b) { return Fc1B(s, o, b) + s.hd2; }
uint64_t Fc2B(const orc_mlp_shape_t& s, const Offsets& o, uint32_t b) { return Fc2W(s, o, b) + (uint64_t)s.hd2 * s.hd2; }

// Limits of the reference's device shape check: native/cuda/mlp_forward.cu:7-9,89-97.
bool ValidShape(const orc_mlp_shape_t& s) {
    return s.state_len > 0 && s.state_len <= 72 && s.state_value_pad > 0 && s.state_value_pad <= 72 &&
           s.hd1 > 0 && s.hd2 > 0 && s.residual_blocks <= 64 && s.output_dim > 0;
}

inline float Relu(float x) { return x > 0.0f ? x : 0.0f; }

struct Tape {
    std::vector<float> z1, a1, z2, a2, rz1, ra1, rz2, rout;
    explicit Tape(const orc_mlp_shape_t& s)
        : z1(s.hd1), a1(s.hd1), z2(s.hd2), a2(s.hd2), rz1((uint64_t)s.residual_blocks * s.hd2),
          ra1((uint64_t)s.residual_blocks * s.hd2), rz2((uint64_t)s.residual_blocks * s.hd2), rout(s.hd2) {}
};

// native/src/mlp_cpu_ref.cpp:62-126
int ForwardOne(const orc_mlp_shape_t& s, const Offsets& o, const float* w, const uint8_t* state, Tape* t, float* output) {
    for (uint32_t h = 0; h < s.hd1; ++h) t->z1[h] = w[o.input_bias + h];
    for (uint32_t pos = 0; pos < s.state_len; ++pos) {
        const uint32_t value = state[pos];
        if (value >= s.state_value_pad) return ORC_INVALID_CONFIG;
        const uint64_t base = o.input_table + ((uint64_t)pos * s.state_value_pad + value) * s.hd1;
        for (uint32_t h = 0; h < s.hd1; ++h) t->z1[h] += w[base + h];
    }
    for (uint32_t h = 0; h < s.hd1; ++h) t->a1[h] = Relu(t->z1[h]);
    for (uint32_t j = 0; j < s.hd2; ++j) {
        float sum = w[o.hidden_bias + j];
        for (uint32_t h = 0; h < s.hd1; ++h) sum += t->a1[h] * w[o.hidden_weight + (uint64_t)h * s.hd2 + j];
        t->z2[j] = sum;
        t->a2[j] = Relu(sum);
        t->rout[j] = t->a2[j];
    }
    for (uint32_t b = 0; b < s.residual_blocks; ++b) {
        const uint64_t f1w = Fc1W(s, o, b), f1b = Fc1B(s, o, b), f2w = Fc2W(s, o, b), f2b = Fc2B(s, o, b);
        const uint64_t base = (uint64_t)b * s.hd2;
        for (uint32_t j = 0; j < s.hd2; ++j) {
            float sum = w[f1b + j];
            for (uint32_t i = 0; i < s.hd2; ++i) sum += t->rout[i] * w[f1w + (uint64_t)i * s.hd2 + j];
            t->rz1[base + j] = sum;
            t->ra1[base + j] = Relu(sum);
        }
        for (uint32_t j = 0; j < s.hd2; ++j) {
            float sum = w[f2b + j];
            for (uint32_t i = 0; i < s.hd2; ++i) sum += t->ra1[base + i] * w[f2w + (uint64_t)i * s.hd2 + j];
            t->rz2[base + j] = sum;
        }
        // The reference updates residual_out inside the j loop; each element only depends on
        // its own column, so a second loop gives the same values.
        for (uint32_t j = 0; j < s.hd2; ++j) t->rout[j] = Relu(t->rout[j] + t->rz2[base + j]);
    }
    for (uint32_t out = 0; out < s.output_dim; ++out) {
        float y = w[o.output_bias + out];
        for (uint32_t j = 0; j < s.hd2; ++j) y += t->rout[j] * w[o.output_weight + (uint64_t)j * s.output_dim + out];
        output[out] = y;
    }
    return ORC_OK;
}

}  // namespace

extern "C" {

uint64_t orc_mix64(uint64_t x) {
    x += 0x9e3779b97f4a7c15ULL;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ULL;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebULL;
    return x ^ (x >> 31);
}

static uint32_t NextBounded(uint64_t* state, uint32_t bound) {
    *state = orc_mix64(*state);
    return (uint32_t)(*state % bound);
}

int orc_random_walks(const uint8_t* moves, const uint8_t* target, uint32_t move_count, uint32_t state_len,
                     uint32_t state_storage_len, uint64_t base_seed, uint64_t epoch, uint64_t step,
                     uint32_t global_rank, uint32_t k_min, uint32_t k_max, uint32_t sample_count,
                     uint8_t* states, float* labels, orc_walk_meta_t* meta) {
    if (!moves || !target || !states || !labels || !meta) return ORC_INVALID_CONFIG;
    if (sample_count == 0 || k_min == 0 || k_min > k_max) return ORC_INVALID_CONFIG;
    if (move_count == 0 || move_count > 18 || state_len == 0 || state_len > 72 ||
        state_storage_len < state_len || state_storage_len > ORC_STATE_STORAGE_LEN) return ORC_INVALID_CONFIG;
    const uint32_t span = k_max - k_min + 1U;
    for (uint32_t sample = 0; sample < sample_count; ++sample) {
        uint64_t rng = base_seed;
        rng ^= orc_mix64(epoch + 0x100000001b3ULL);
        rng ^= orc_mix64(step + 0x9e3779b97f4a7c15ULL);
        rng ^= orc_mix64((uint64_t)global_rank << 32);
        rng ^= orc_mix64(sample);
        const uint32_t depth = k_min + NextBounded(&rng, span);
        uint8_t cur[ORC_STATE_STORAGE_LEN], next[ORC_STATE_STORAGE_LEN];
        std::memcpy(cur, target, ORC_STATE_STORAGE_LEN);
        uint32_t last = move_count;
        for (uint32_t d = 0; d < depth; ++d) {
            uint32_t mv = NextBounded(&rng, move_count);
            if (last != move_count && mv == last) mv = (mv + 1U + NextBounded(&rng, move_count - 1U)) % move_count;
            const uint8_t* def = moves + (uint64_t)mv * ORC_STATE_STORAGE_LEN;
            std::memset(next, 0, sizeof(next));
            for (uint32_t i = 0; i < state_len; ++i) next[i] = cur[def[i]];
            std::memcpy(cur, next, sizeof(cur));
            last = mv;
        }
        std::memcpy(states + (uint64_t)sample * ORC_STATE_STORAGE_LEN, cur, ORC_STATE_STORAGE_LEN);
        labels[sample] = (float)depth;
        meta[sample].depth = depth;
        meta[sample].last_move = last;
        meta[sample].rng_counter = rng;
    }
    return ORC_OK;
}

void orc_build_cyclic_puzzle(uint32_t state_len, uint32_t move_count, uint32_t max_moves, uint8_t* moves, uint8_t* target) {
    std::memset(moves, 0, (size_t)max_moves * ORC_STATE_STORAGE_LEN);
    std::memset(target, 0, ORC_STATE_STORAGE_LEN);
    for (uint32_t mv = 0; mv < max_moves; ++mv)
        for (uint32_t i = 0; i < state_len; ++i)
            moves[(size_t)mv * ORC_STATE_STORAGE_LEN + i] = (uint8_t)(mv < move_count ? (i + mv + 1) % state_len : i);
    for (uint32_t i = 0; i < state_len; ++i) target[i] = (uint8_t)i;
}

uint64_t orc_mlp_param_count(const orc_mlp_shape_t* shape) {
    if (!shape || !ValidShape(*shape)) return 0;
    return BuildOffsets(*shape).total;
}

int orc_mlp_forward(const orc_mlp_shape_t* shape, const float* weights, const uint8_t* states, uint32_t sample_count, float* outputs) {
    if (!shape || !ValidShape(*shape) || !weights || !states || !outputs || sample_count == 0) return ORC_INVALID_CONFIG;
    const orc_mlp_shape_t& s = *shape;
    const Offsets o = BuildOffsets(s);
    Tape t(s);
    for (uint32_t b = 0; b < sample_count; ++b) {
        const int st = ForwardOne(s, o, weights, states + (uint64_t)b * ORC_STATE_STORAGE_LEN, &t, outputs + (uint64_t)b * s.output_dim);
        if (st != ORC_OK) return st;
    }
    return ORC_OK;
}

int orc_mlp_loss_grad(const orc_mlp_shape_t* shape, const float* w, const uint8_t* states, const float* labels,
                      uint32_t sample_count, float* loss, float* grad) {
    if (!shape || !ValidShape(*shape) || !w || !states || !labels || !loss || !grad || sample_count == 0) return ORC_INVALID_CONFIG;
    const orc_mlp_shape_t& s = *shape;
    const Offsets o = BuildOffsets(s);
    std::fill(grad, grad + o.total, 0.0f);
    *loss = 0.0f;
    Tape t(s);
    const uint32_t H2 = s.hd2;
    std::vector<float> block_inputs((uint64_t)(s.residual_blocks + 1U) * H2), output(s.output_dim), dcur(H2), dprev(H2), dfc1(H2), dzfc2(H2), dzfc1(H2), dz1(s.hd1), da1(s.hd1), dz2(H2);
    const float inv_n = 1.0f / (float)((uint64_t)sample_count * s.output_dim);
    for (uint32_t sample = 0; sample < sample_count; ++sample) {
        const uint8_t* state = states + (uint64_t)sample * ORC_STATE_STORAGE_LEN;
        const int st = ForwardOne(s, o, w, state, &t, output.data());
        if (st != ORC_OK) return st;
        std::copy(t.a2.begin(), t.a2.end(), block_inputs.begin());
        std::vector<float> replay = t.a2;
        for (uint32_t b = 0; b < s.residual_blocks; ++b) {
            for (uint32_t j = 0; j < H2; ++j) replay[j] = Relu(replay[j] + t.rz2[(uint64_t)b * H2 + j]);
            std::copy(replay.begin(), replay.end(), block_inputs.begin() + (uint64_t)(b + 1U) * H2);
        }
        std::fill(dcur.begin(), dcur.end(), 0.0f);
        for (uint32_t out = 0; out < s.output_dim; ++out) {
            const float diff = output[out] - labels[(uint64_t)sample * s.output_dim + out];
            *loss += diff * diff * inv_n;
            const float dy = 2.0f * diff * inv_n;
            grad[o.output_bias + out] += dy;
            for (uint32_t j = 0; j < H2; ++j) {
                const uint64_t wi = o.output_weight + (uint64_t)j * s.output_dim + out;
                grad[wi] += t.rout[j] * dy;
                dcur[j] += w[wi] * dy;
            }
        }
        for (uint32_t rb = s.residual_blocks; rb > 0; --rb) {
            const uint32_t b = rb - 1U;
            const uint64_t base = (uint64_t)b * H2;
            const float* input = block_inputs.data() + base;
            const uint64_t f1w = Fc1W(s, o, b), f1b = Fc1B(s, o, b), f2w = Fc2W(s, o, b), f2b = Fc2B(s, o, b);
            std::fill(dprev.begin(), dprev.end(), 0.0f);
            std::fill(dfc1.begin(), dfc1.end(), 0.0f);
            for (uint32_t j = 0; j < H2; ++j) dzfc2[j] = dcur[j] * ((input[j] + t.rz2[base + j]) > 0.0f ? 1.0f : 0.0f);
            for (uint32_t j = 0; j < H2; ++j) grad[f2b + j] += dzfc2[j];
            for (uint32_t i = 0; i < H2; ++i)
                for (uint32_t j = 0; j < H2; ++j) {
                    grad[f2w + (uint64_t)i * H2 + j] += t.ra1[base + i] * dzfc2[j];
                    dfc1[i] += w[f2w + (uint64_t)i * H2 + j] * dzfc2[j];
                }
            for (uint32_t j = 0; j < H2; ++j) dzfc1[j] = dfc1[j] * (t.rz1[base + j] > 0.0f ? 1.0f : 0.0f);
            for (uint32_t j = 0; j < H2; ++j) grad[f1b + j] += dzfc1[j];
            for (uint32_t i = 0; i < H2; ++i) {
                dprev[i] += dzfc2[i];
                for (uint32_t j = 0; j < H2; ++j) {
                    grad[f1w + (uint64_t)i * H2 + j] += input[i] * dzfc1[j];
                    dprev[i] += w[f1w + (uint64_t)i * H2 + j] * dzfc1[j];
                }
            }
            dcur.swap(dprev);
        }
        for (uint32_t j = 0; j < H2; ++j) {
            dz2[j] = dcur[j] * (t.z2[j] > 0.0f ? 1.0f : 0.0f);
            grad[o.hidden_bias + j] += dz2[j];
        }
        std::fill(da1.begin(), da1.end(), 0.0f);
        for (uint32_t h = 0; h < s.hd1; ++h)
            for (uint32_t j = 0; j < H2; ++j) {
                grad[o.hidden_weight + (uint64_t)h * H2 + j] += t.a1[h] * dz2[j];
                da1[h] += w[o.hidden_weight + (uint64_t)h * H2 + j] * dz2[j];
            }
        for (uint32_t h = 0; h < s.hd1; ++h) {
            dz1[h] = da1[h] * (t.z1[h] > 0.0f ? 1.0f : 0.0f);
            grad[o.input_bias + h] += dz1[h];
        }
        for (uint32_t pos = 0; pos < s.state_len; ++pos) {
            const uint64_t base = o.input_table + ((uint64_t)pos * s.state_value_pad + state[pos]) * s.hd1;
            for (uint32_t h = 0; h < s.hd1; ++h) grad[base + h] += dz1[h];
        }
    }
    return ORC_OK;
}

uint16_t orc_float_to_half_rn(float value) {
    uint32_t x;
    std::memcpy(&x, &value, 4);
    const uint32_t sign = (x >> 16) & 0x8000U;
    const uint32_t absx = x & 0x7fffffffU;
    if (absx >= 0x7f800000U) return (uint16_t)(sign | 0x7c00U | ((absx > 0x7f800000U) ? 0x200U : 0U));
    if (absx >= 0x477ff000U) {  // >= 65520 rounds to inf
        return (uint16_t)(sign | 0x7c00U);
    }
    if (absx < 0x38800000U) {  // below the smallest normal half: denormal result
        if (absx < 0x33000000U) return (uint16_t)sign;  // < 2^-25 rounds to zero (2^-25 itself ties to even = 0)
        const int32_t exp = (int32_t)(absx >> 23);
        const uint32_t mant = (absx & 0x7fffffU) | 0x800000U;
        const uint32_t shift = (uint32_t)(126 - exp);  // 14..24
        const uint32_t q = mant >> shift;
        const uint32_t rem = mant & ((1U << shift) - 1U);
        const uint32_t half = 1U << (shift - 1U);
        uint32_t r = q;
        if (rem > half || (rem == half && (q & 1U))) r += 1U;
        return (uint16_t)(sign | r);
    }
    const uint32_t exp = (absx >> 23) - 112U;
    const uint32_t mant = absx & 0x7fffffU;
    uint32_t h = (exp << 10) | (mant >> 13);
    const uint32_t rem = mant & 0x1fffU;
    if (rem > 0x1000U || (rem == 0x1000U && (h & 1U))) h += 1U;
    return (uint16_t)(sign | h);
}

float orc_half_to_float(uint16_t bits) {
    const uint32_t sign = ((uint32_t)bits & 0x8000U) << 16;
    const uint32_t exp = (bits >> 10) & 0x1fU;
    const uint32_t mant = bits & 0x3ffU;
    uint32_t x;
    if (exp == 0) {
        if (mant == 0) {
            x = sign;
        } else {
            float f = (float)mant * 5.9604644775390625e-08f;  // 2^-24
            std::memcpy(&x, &f, 4);
            x |= sign;
        }
    } else if (exp == 31) {
        x = sign | 0x7f800000U | (mant << 13);
    } else {
        x = sign | ((exp + 112U) << 23) | (mant << 13);
    }
    float out;
    std::memcpy(&out, &x, 4);
    return out;
}

uint16_t orc_export_float_to_fp16(float value) {
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    const uint32_t sign = (bits >> 16U) & 0x8000U;
    int32_t exp = (int32_t)((bits >> 23U) & 0xffU) - 127 + 15;
    uint32_t mant = bits & 0x7fffffU;
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        mant = (mant | 0x800000U) >> (uint32_t)(1 - exp);
        return (uint16_t)(sign | ((mant + 0x1000U) >> 13U));
    }
    if (exp >= 31) return (uint16_t)(sign | 0x7c00U);
    return (uint16_t)(sign | ((uint32_t)exp << 10U) | ((mant + 0x1000U) >> 13U));
}

uint16_t orc_float_to_bf16_rn(float value) {
    uint32_t x;
    std::memcpy(&x, &value, 4);
    if ((x & 0x7fffffffU) > 0x7f800000U) return (uint16_t)((x >> 16) | 0x40U);  // NaN stays NaN
    const uint32_t lsb = (x >> 16) & 1U;
    x += 0x7fffU + lsb;  // round to nearest, ties to even
    return (uint16_t)(x >> 16);
}

float orc_bf16_to_float(uint16_t bits) {
    const uint32_t x = (uint32_t)bits << 16;
    float out;
    std::memcpy(&out, &x, 4);
    return out;
}

namespace {
inline float Q(float x, int fmt) { return fmt == ORC_OPERAND_BF16 ? orc_bf16_to_float(orc_float_to_bf16_rn(x)) : orc_half_to_float(orc_float_to_half_rn(x)); }

// c[m,n] = sum_k a[m,k]*b[k,n], row-major, fp32 accumulate in k order.
void MatMulNN(const float* a, const float* b, float* c, uint32_t m, uint32_t n, uint32_t k) {
    for (uint32_t i = 0; i < m; ++i)
        for (uint32_t j = 0; j < n; ++j) {
            float sum = 0.0f;
            for (uint32_t x = 0; x < k; ++x) sum += a[(uint64_t)i * k + x] * b[(uint64_t)x * n + j];
            c[(uint64_t)i * n + j] = sum;
        }
}
// grad_w[in,out] = sum_b x[b,in]*dz[b,out]
void MatMulTN(const float* x, const float* dz, float* gw, uint32_t samples, uint32_t in_dim, uint32_t out_dim) {
    for (uint32_t i = 0; i < in_dim; ++i)
        for (uint32_t j = 0; j < out_dim; ++j) {
            float sum = 0.0f;
            for (uint32_t b = 0; b < samples; ++b) sum += x[(uint64_t)b * in_dim + i] * dz[(uint64_t)b * out_dim + j];
            gw[(uint64_t)i * out_dim + j] = sum;
        }
}
// dx[b,in] = sum_out dz[b,out]*w[in,out]
void MatMulNT(const float* dz, const float* w, float* dx, uint32_t samples, uint32_t in_dim, uint32_t out_dim) {
    for (uint32_t b = 0; b < samples; ++b)
        for (uint32_t i = 0; i < in_dim; ++i) {
            float sum = 0.0f;
            for (uint32_t j = 0; j < out_dim; ++j) sum += dz[(uint64_t)b * out_dim + j] * w[(uint64_t)i * out_dim + j];
            dx[(uint64_t)b * in_dim + i] = sum;
        }
}
void ColSum(const float* dz, float* out, uint32_t samples, uint32_t cols) {
    for (uint32_t j = 0; j < cols; ++j) {
        float sum = 0.0f;
        for (uint32_t b = 0; b < samples; ++b) sum += dz[(uint64_t)b * cols + j];
        out[j] = sum;
    }
}
std::vector<float> Quantized(const std::vector<float>& v, bool on, int fmt) {
    if (!on) return v;
    std::vector<float> q(v.size());
    for (size_t i = 0; i < v.size(); ++i) q[i] = Q(v[i], fmt);
    return q;
}

// Training-mode batch normalisation of z[B][H] over the batch, column by column:
//   y = gamma * (z - mean) * rstd + beta,  mean/var (biased) of the column, rstd = 1 / sqrt(var + eps).
// Keeps xhat = (z - mean) * rstd and rstd for the backward pass. Sums run over the samples in order, in fp32.
struct BnTape {
    std::vector<float> xhat, rstd, mean, var;
};
void BnForward(const std::vector<float>& z, uint32_t B, uint32_t H, const float* gamma, const float* beta, float eps, std::vector<float>* y, BnTape* t) {
    t->xhat.resize((uint64_t)B * H);
    t->rstd.resize(H);
    t->mean.resize(H);
    t->var.resize(H);
    y->resize((uint64_t)B * H);
    const float inv_b = 1.0f / (float)B;
    for (uint32_t j = 0; j < H; ++j) {
        float s1 = 0.0f, s2 = 0.0f;
        for (uint32_t b = 0; b < B; ++b) {
            const float v = z[(uint64_t)b * H + j];
            s1 += v;
            s2 += v * v;
        }
        const float mean = s1 * inv_b;
        float var = s2 * inv_b - mean * mean;
        if (var < 0.0f) var = 0.0f;
        const float rstd = 1.0f / std::sqrt(var + eps);
        t->mean[j] = mean;
        t->var[j] = var;
        t->rstd[j] = rstd;
        for (uint32_t b = 0; b < B; ++b) {
            const float xh = (z[(uint64_t)b * H + j] - mean) * rstd;
            t->xhat[(uint64_t)b * H + j] = xh;
            (*y)[(uint64_t)b * H + j] = gamma[j] * xh + beta[j];
        }
    }
}
// dy -> dz through the normalisation; dgamma = sum dy * xhat, dbeta = sum dy, dz = gamma * rstd * (dy - mean(dy) - xhat * mean(dy * xhat))
void BnBackward(const std::vector<float>& dy, uint32_t B, uint32_t H, const float* gamma, const BnTape& t, float* dgamma, float* dbeta, std::vector<float>* dz) {
    dz->resize((uint64_t)B * H);
    const float inv_b = 1.0f / (float)B;
    for (uint32_t j = 0; j < H; ++j) {
        float s1 = 0.0f, s2 = 0.0f;
        for (uint32_t b = 0; b < B; ++b) {
            const float g = dy[(uint64_t)b * H + j];
            s1 += g;
            s2 += g * t.xhat[(uint64_t)b * H + j];
        }
        dbeta[j] = s1;
        dgamma[j] = s2;
        const float m1 = s1 * inv_b, m2 = s2 * inv_b, k = gamma[j] * t.rstd[j];
        for (uint32_t b = 0; b < B; ++b) {
            const uint64_t i = (uint64_t)b * H + j;
            (*dz)[i] = k * (dy[i] - m1 - t.xhat[i] * m2);
        }
    }
}
}  // namespace

uint64_t orc_bn_param_count(const orc_mlp_shape_t* shape) {
    if (!shape || !ValidShape(*shape)) return 0;
    return 2ULL * (shape->residual_blocks + 1ULL) * shape->hd2;
}

int orc_mlp_loss_grad_ex(const orc_mlp_shape_t* shape, const float* w, const uint8_t* states, const float* labels, uint32_t B,
                         const orc_train_options_t* opt, float* loss, float* grad, float* bn_batch_stats) {
    if (!shape || !ValidShape(*shape) || !w || !states || !labels || !loss || !grad || !opt || B == 0) return ORC_INVALID_CONFIG;
    const orc_mlp_shape_t& s = *shape;
    const Offsets o = BuildOffsets(s);
    const uint32_t H1 = s.hd1, H2 = s.hd2, R = s.residual_blocks, OUT = s.output_dim;
    const bool hl = opt->half_linear != 0, hi = opt->half_input_grad != 0, bn = opt->batch_norm != 0, ce = opt->loss_kind == ORC_LOSS_CROSS_ENTROPY;
    const int fmt = opt->operand_format;
    if (ce && OUT < 2) return ORC_INVALID_CONFIG;
    // batch-norm scale and shift follow the reference's parameters: layer 0 = hidden layer, layer k + 1 = block k; each gamma[H2], beta[H2]
    const uint64_t bn_base = o.total;
    const uint64_t total = o.total + (bn ? 2ULL * (R + 1ULL) * H2 : 0ULL);
    auto gamma_of = [&](uint32_t layer) { return w + bn_base + 2ULL * layer * H2; };
    auto beta_of = [&](uint32_t layer) { return w + bn_base + 2ULL * layer * H2 + H2; };
    // weights mirror: mlp_backward.cu:1267-1271 / adamw.cu:45
    std::vector<float> wq(o.total);
    for (uint64_t i = 0; i < o.total; ++i) wq[i] = hl ? Q(w[i], fmt) : w[i];
    std::fill(grad, grad + total, 0.0f);

    // embedding forward: mlp_backward.cu:696-832 (mirror table AND mirror bias on the fp16 path)
    std::vector<float> a1((uint64_t)B * H1);
    for (uint32_t b = 0; b < B; ++b) {
        const uint8_t* st = states + (uint64_t)b * ORC_STATE_STORAGE_LEN;
        for (uint32_t h = 0; h < H1; ++h) {
            float acc = wq[o.input_bias + h];
            for (uint32_t pos = 0; pos < s.state_len; ++pos) {
                if (st[pos] >= s.state_value_pad) return ORC_INVALID_CONFIG;
                acc += wq[((uint64_t)pos * s.state_value_pad + st[pos]) * H1 + h];
            }
            a1[(uint64_t)b * H1 + h] = Relu(acc);
        }
    }
    const std::vector<float> a1q = Quantized(a1, hl, fmt);
    // hidden: mlp_backward.cu:1281-1291 (fp32 master bias); with batch norm the pre-activation is normalised before the ReLU
    std::vector<BnTape> tapes(bn ? R + 1U : 0U);
    std::vector<float> x((uint64_t)B * H2), zh;
    MatMulNN(a1q.data(), wq.data() + o.hidden_weight, x.data(), B, H2, H1);
    for (uint32_t b = 0; b < B; ++b)
        for (uint32_t j = 0; j < H2; ++j) x[(uint64_t)b * H2 + j] += w[o.hidden_bias + j];
    if (bn) {
        zh = x;
        BnForward(zh, B, H2, gamma_of(0), beta_of(0), opt->bn_eps, &x, &tapes[0]);
    }
    for (uint64_t i = 0; i < (uint64_t)B * H2; ++i) x[i] = Relu(x[i]);
    std::vector<std::vector<float>> xin(R + 1U), xinq(R + 1U), r1(R), r1q(R), rz2(R);
    xin[0] = x;
    xinq[0] = Quantized(x, hl, fmt);
    // residual blocks: mlp_backward.cu:1294-1323; with batch norm the fc2 output is normalised before it joins the skip path
    for (uint32_t k = 0; k < R; ++k) {
        r1[k].resize((uint64_t)B * H2);
        rz2[k].resize((uint64_t)B * H2);
        MatMulNN(xinq[k].data(), wq.data() + Fc1W(s, o, k), r1[k].data(), B, H2, H2);
        for (uint32_t b = 0; b < B; ++b)
            for (uint32_t j = 0; j < H2; ++j) r1[k][(uint64_t)b * H2 + j] = Relu(r1[k][(uint64_t)b * H2 + j] + w[Fc1B(s, o, k) + j]);
        r1q[k] = Quantized(r1[k], hl, fmt);
        MatMulNN(r1q[k].data(), wq.data() + Fc2W(s, o, k), rz2[k].data(), B, H2, H2);
        for (uint32_t b = 0; b < B; ++b)
            for (uint32_t j = 0; j < H2; ++j) rz2[k][(uint64_t)b * H2 + j] += w[Fc2B(s, o, k) + j];
        if (bn) {
            const std::vector<float> z = rz2[k];
            BnForward(z, B, H2, gamma_of(k + 1U), beta_of(k + 1U), opt->bn_eps, &rz2[k], &tapes[k + 1U]);
        }
        xin[k + 1].resize((uint64_t)B * H2);
        for (uint64_t i = 0; i < (uint64_t)B * H2; ++i) xin[k + 1][i] = Relu(xin[k][i] + rz2[k][i]);
        xinq[k + 1] = Quantized(xin[k + 1], hl, fmt);
    }
    if (bn && bn_batch_stats != nullptr) {
        for (uint32_t l = 0; l <= R; ++l)
            for (uint32_t j = 0; j < H2; ++j) {
                bn_batch_stats[(2ULL * l) * H2 + j] = tapes[l].mean[j];
                bn_batch_stats[(2ULL * l + 1ULL) * H2 + j] = tapes[l].var[j];
            }
    }
    // output head + loss: mlp_backward.cu:1333-1363
    const std::vector<float>& fin = xin[R];
    std::vector<float> dcur((uint64_t)B * H2, 0.0f);
    float loss_acc = 0.0f;
    if (OUT == 1U) {
        const float inv_n = 1.0f / (float)B;
        std::vector<float> dy(B);
        for (uint32_t b = 0; b < B; ++b) {
            float y = w[o.output_bias];
            for (uint32_t j = 0; j < H2; ++j) y += fin[(uint64_t)b * H2 + j] * w[o.output_weight + j];
            const float diff = y - labels[b];
            dy[b] = 2.0f * diff * inv_n;
            loss_acc += diff * diff * inv_n;
            for (uint32_t j = 0; j < H2; ++j) dcur[(uint64_t)b * H2 + j] = w[o.output_weight + j] * dy[b];
        }
        for (uint32_t j = 0; j < H2; ++j) {
            float sum = 0.0f;
            for (uint32_t b = 0; b < B; ++b) sum += fin[(uint64_t)b * H2 + j] * dy[b];
            grad[o.output_weight + j] = sum;
        }
        float sum = 0.0f;
        for (uint32_t b = 0; b < B; ++b) sum += dy[b];
        grad[o.output_bias] = sum;
    } else {
        const uint64_t items = (uint64_t)B * OUT;
        std::vector<float> outv(items), dy(items);
        MatMulNN(xinq[R].data(), wq.data() + o.output_weight, outv.data(), B, OUT, H2);
        if (!ce) {
            const float inv_n = 1.0f / (float)items;
            for (uint64_t i = 0; i < items; ++i) {
                const float y = outv[i] + w[o.output_bias + (i % OUT)];
                const float diff = y - labels[i];
                dy[i] = 2.0f * diff * inv_n;
                loss_acc += diff * diff * inv_n;
            }
        } else {
            // per-depth logits: class = depth - 1 (labels carry the walk depth K in every output slot), mean over the batch of
            // -log softmax(y)[class]; dy = (softmax(y) - onehot(class)) / B
            const float inv_b = 1.0f / (float)B;
            for (uint32_t b = 0; b < B; ++b) {
                const float depth = labels[(uint64_t)b * OUT];
                const int32_t cls = (int32_t)std::lround(depth) - 1;
                if (cls < 0 || cls >= (int32_t)OUT) return ORC_INVALID_CONFIG;
                float mx = -3.0e38f;
                for (uint32_t c = 0; c < OUT; ++c) {
                    outv[(uint64_t)b * OUT + c] += w[o.output_bias + c];
                    mx = std::max(mx, outv[(uint64_t)b * OUT + c]);
                }
                float sum = 0.0f;
                for (uint32_t c = 0; c < OUT; ++c) sum += std::exp(outv[(uint64_t)b * OUT + c] - mx);
                const float log_sum = std::log(sum) + mx;
                loss_acc += (log_sum - outv[(uint64_t)b * OUT + (uint32_t)cls]) * inv_b;
                for (uint32_t c = 0; c < OUT; ++c) {
                    const float p = std::exp(outv[(uint64_t)b * OUT + c] - log_sum);
                    dy[(uint64_t)b * OUT + c] = (p - (c == (uint32_t)cls ? 1.0f : 0.0f)) * inv_b;
                }
            }
        }
        const std::vector<float> dyq = Quantized(dy, hl, fmt);
        MatMulTN(xinq[R].data(), dyq.data(), grad + o.output_weight, B, H2, OUT);
        MatMulNT(dyq.data(), wq.data() + o.output_weight, dcur.data(), B, H2, OUT);
        ColSum(dy.data(), grad + o.output_bias, B, OUT);
    }
    *loss = loss_acc;
    // residual backward: mlp_backward.cu:1367-1413
    std::vector<float> dz2((uint64_t)B * H2), dra1((uint64_t)B * H2), dz1((uint64_t)B * H2), dprev((uint64_t)B * H2), dpre;
    for (uint32_t rb = R; rb > 0; --rb) {
        const uint32_t k = rb - 1U;
        for (uint64_t i = 0; i < (uint64_t)B * H2; ++i) dz2[i] = dcur[i] * ((xin[k][i] + rz2[k][i]) > 0.0f ? 1.0f : 0.0f);
        dpre = dz2;  // gradient w.r.t. the sum entering the ReLU: goes down the skip path unchanged
        if (bn) {
            const std::vector<float> dy = dz2;
            BnBackward(dy, B, H2, gamma_of(k + 1U), tapes[k + 1U], grad + bn_base + 2ULL * (k + 1U) * H2, grad + bn_base + 2ULL * (k + 1U) * H2 + H2, &dz2);
        }
        const std::vector<float> dz2q = Quantized(dz2, hl, fmt);
        MatMulTN(r1q[k].data(), dz2q.data(), grad + Fc2W(s, o, k), B, H2, H2);
        ColSum(dz2.data(), grad + Fc2B(s, o, k), B, H2);
        MatMulNT(dz2q.data(), wq.data() + Fc2W(s, o, k), dra1.data(), B, H2, H2);
        for (uint64_t i = 0; i < (uint64_t)B * H2; ++i) dz1[i] = dra1[i] * (r1[k][i] > 0.0f ? 1.0f : 0.0f);
        const std::vector<float> dz1q = Quantized(dz1, hl, fmt);
        MatMulTN(xinq[k].data(), dz1q.data(), grad + Fc1W(s, o, k), B, H2, H2);
        ColSum(dz1.data(), grad + Fc1B(s, o, k), B, H2);
        MatMulNT(dz1q.data(), wq.data() + Fc1W(s, o, k), dprev.data(), B, H2, H2);
        for (uint64_t i = 0; i < (uint64_t)B * H2; ++i) dprev[i] += dpre[i];
        dcur.swap(dprev);
    }
    // hidden backward: mlp_backward.cu:1417-1438
    std::vector<float> dzh((uint64_t)B * H2);
    for (uint64_t i = 0; i < (uint64_t)B * H2; ++i) dzh[i] = dcur[i] * (xin[0][i] > 0.0f ? 1.0f : 0.0f);
    if (bn) {
        const std::vector<float> dy = dzh;
        BnBackward(dy, B, H2, gamma_of(0), tapes[0], grad + bn_base, grad + bn_base + H2, &dzh);
    }
    const std::vector<float> dzhq = Quantized(dzh, hl, fmt);
    MatMulTN(a1q.data(), dzhq.data(), grad + o.hidden_weight, B, H1, H2);
    ColSum(dzh.data(), grad + o.hidden_bias, B, H2);
    std::vector<float> da1((uint64_t)B * H1);
    MatMulNT(dzhq.data(), wq.data() + o.hidden_weight, da1.data(), B, H1, H2);
    for (uint64_t i = 0; i < (uint64_t)B * H1; ++i) da1[i] = da1[i] * (a1[i] > 0.0f ? 1.0f : 0.0f);
    const std::vector<float> dzin = Quantized(da1, hi, fmt);
    // embedding gradient: mlp_backward.cu:1440-1505 (one-hot^T x dz1 is a scatter-add)
    for (uint32_t b = 0; b < B; ++b) {
        const uint8_t* st = states + (uint64_t)b * ORC_STATE_STORAGE_LEN;
        for (uint32_t pos = 0; pos < s.state_len; ++pos) {
            float* row = grad + ((uint64_t)pos * s.state_value_pad + st[pos]) * H1;
            for (uint32_t h = 0; h < H1; ++h) row[h] += dzin[(uint64_t)b * H1 + h];
        }
    }
    ColSum(da1.data(), grad + o.input_bias, B, H1);
    return ORC_OK;
}

int orc_mlp_loss_grad_mixed(const orc_mlp_shape_t* shape, const float* w, const uint8_t* states, const float* labels,
                            uint32_t B, int half_linear, int half_input_grad, float* loss, float* grad) {
    orc_train_options_t opt{};
    opt.half_linear = half_linear;
    opt.half_input_grad = half_input_grad;
    opt.operand_format = ORC_OPERAND_FP16;
    opt.loss_kind = ORC_LOSS_MSE;
    return orc_mlp_loss_grad_ex(shape, w, states, labels, B, &opt, loss, grad, nullptr);
}

int orc_adamw_step(float* weights, const float* grad, float* m, float* v, uint64_t n, uint64_t step, float lr,
                   float beta1, float beta2, float eps, float wd, uint16_t* half_mirror) {
    if (!weights || !grad || !m || !v || n == 0 || step == 0 || lr <= 0.0f || eps <= 0.0f || beta1 < 0.0f ||
        beta1 >= 1.0f || beta2 < 0.0f || beta2 >= 1.0f || wd < 0.0f) return ORC_INVALID_CONFIG;
    const float bias1 = 1.0f - std::pow(beta1, (float)step);
    const float bias2 = 1.0f - std::pow(beta2, (float)step);
    for (uint64_t i = 0; i < n; ++i) {
        const float g = grad[i] + wd * weights[i];
        m[i] = beta1 * m[i] + (1.0f - beta1) * g;
        v[i] = beta2 * v[i] + (1.0f - beta2) * g * g;
        const float m_hat = m[i] / bias1;
        const float v_hat = v[i] / bias2;
        weights[i] -= lr * m_hat / (std::sqrt(v_hat) + eps);
        if (half_mirror) half_mirror[i] = orc_float_to_half_rn(weights[i]);
    }
    return ORC_OK;
}

void orc_allreduce_average(const float* const* rank_grads, uint32_t world_size, uint64_t count, float* out) {
    const float inv = 1.0f / (float)world_size;
    for (uint64_t i = 0; i < count; ++i) {
        float sum = rank_grads[0][i];
        for (uint32_t r = 1; r < world_size; ++r) sum += rank_grads[r][i];
        out[i] = world_size > 1 ? sum * inv : sum;
    }
}

}  // extern "C"
