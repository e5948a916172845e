// CPU oracle for the decode-step operators around the quantized linears.
// TEST INFRASTRUCTURE ONLY: nothing in the product path may call it.
//
// Restates, in f32 exactly as the reference's host golden does, the operators
// that sit either side of the quantized linears in one Llama decode step.
// Every function cites the reference file:line it follows (paths relative to
// the reference project's root).  Sums run in source order, products and sums
// are rounded separately (the build uses -ffp-contract=off), so each output is
// the value the reference's Rust computes for the same f32 inputs.
//
// Parity status: PINNED — tests/test_oracle_decode_kat.py restates, as data,
// the reference's own known-answer tests for these functions
// (crates/targets/metal/src/cpu_golden.rs:1091-1436 and
// crates/targets/metal/tests/argmax_split_test.rs:24-33).

#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

extern "C" {

// crates/targets/metal/src/cpu_golden.rs:25-37 (`rmsnorm`), applied to `rows`
// rows of `hidden` elements: sum of squares in index order, rms =
// sqrt(sum/n + eps), inv = 1/rms, out = x * inv * w (left to right).
void orc_rmsnorm(const float* input, const float* weight, float* output, int64_t rows, int64_t hidden,
                 float eps) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float* x = input + r * hidden;
        float sum_sq = 0.0f;
        for (int64_t i = 0; i < hidden; ++i) sum_sq += x[i] * x[i];
        const float rms = std::sqrt(sum_sq / float(hidden) + eps);
        const float inv_rms = 1.0f / rms;
        for (int64_t i = 0; i < hidden; ++i) output[r * hidden + i] = x[i] * inv_rms * weight[i];
    }
}

// cpu_golden.rs:171-200 (`fused_add_rmsnorm`): residual += delta in place, the
// sum of squares is taken off the post-add residual, delta receives
// rmsnorm(residual, weight).
//
// `round_residual_bf16` != 0 models a bf16 residual stream: the post-add value
// is rounded to bf16 (RNE) before it is stored and before it is squared, which
// is what "the post-add residual" is when the buffer holds bf16.  With 0 the
// function is the reference's f32 statement unchanged.
static inline float round_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) {
        u |= 0x00400000u;
        u &= 0xFFFF0000u;
    } else {
        u += 0x7FFFu + ((u >> 16) & 1u);
        u &= 0xFFFF0000u;
    }
    float o;
    std::memcpy(&o, &u, 4);
    return o;
}

void orc_fused_add_rmsnorm(float* residual, float* delta, const float* weight, float eps, int64_t rows,
                           int64_t hidden, int round_residual_bf16) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const int64_t base = r * hidden;
        float sum_sq = 0.0f;
        for (int64_t i = 0; i < hidden; ++i) {
            float s = residual[base + i] + delta[base + i];
            if (round_residual_bf16) s = round_bf16(s);
            residual[base + i] = s;
            sum_sq += s * s;
        }
        const float rms = std::sqrt(sum_sq / float(hidden) + eps);
        const float inv_rms = 1.0f / rms;
        for (int64_t i = 0; i < hidden; ++i) delta[base + i] = residual[base + i] * inv_rms * weight[i];
    }
}

// cpu_golden.rs:211-219 (`fused_gate_up_silu_mul`): silu(g) = g / (1 + exp(-g)),
// out = silu(g) * up.
void orc_silu_mul(const float* gate, const float* up, float* out, int64_t count) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        const float g = gate[i];
        const float silu_g = g / (1.0f + std::exp(-g));
        out[i] = silu_g * up[i];
    }
}

// cpu_golden.rs:114-124 (`embed`): out[i] = table[ids[i]].  Returns -1 when an
// id is outside the table (the reference asserts), 0 otherwise.
int orc_embed(const uint32_t* ids, int64_t n_ids, const float* table, int64_t vocab, int64_t hidden,
              float* out) {
    for (int64_t i = 0; i < n_ids; ++i) {
        if (int64_t(ids[i]) >= vocab) return -1;
        std::memcpy(out + i * hidden, table + int64_t(ids[i]) * hidden, size_t(hidden) * 4);
    }
    return 0;
}

// Paged-cache addressing, crates/targets/metal/src/paged_kv_layout.rs:74-115:
// the buffer is [num_blocks, num_kv_heads, block_size, head_dim].
static inline int64_t kv_offset(int64_t block, int64_t kv_head, int64_t slot_in_block, int64_t num_kv_heads,
                                int64_t block_size, int64_t head_dim) {
    return block * (num_kv_heads * block_size * head_dim) + kv_head * (block_size * head_dim) +
           slot_in_block * head_dim;
}

// cpu_golden.rs:289-362 (`rope_append`): NeoX pairing (d with d + head_dim/2);
// cos/sin tables are [max_pos, head_dim] and only the first head_dim/2 columns
// of a row are read; q_out = rotated q; the rotated k and the UNrotated v go to
// global slot slot_mapping[t] (block = slot / block_size, offset = slot % block_size).
void orc_rope_append(const float* q_in, const float* k_in, const float* v_in, const uint32_t* positions,
                     const uint32_t* slot_mapping, const float* cos_table, const float* sin_table,
                     float* q_out, float* kv_cache_k, float* kv_cache_v, int64_t num_tokens,
                     int64_t num_q_heads, int64_t num_kv_heads, int64_t head_dim, int64_t block_size) {
    const int64_t q_dim = num_q_heads * head_dim, kv_dim = num_kv_heads * head_dim, half = head_dim / 2;
    for (int64_t t = 0; t < num_tokens; ++t) {
        const float* cos_row = cos_table + int64_t(positions[t]) * head_dim;
        const float* sin_row = sin_table + int64_t(positions[t]) * head_dim;
        for (int64_t h = 0; h < num_q_heads; ++h) {
            const int64_t base = t * q_dim + h * head_dim;
            for (int64_t d = 0; d < half; ++d) {
                const float x0 = q_in[base + d], x1 = q_in[base + half + d];
                const float c = cos_row[d], s = sin_row[d];
                q_out[base + d] = x0 * c - x1 * s;
                q_out[base + half + d] = x1 * c + x0 * s;
            }
        }
        const int64_t slot = slot_mapping[t];
        for (int64_t h = 0; h < num_kv_heads; ++h) {
            const int64_t kv_base = t * kv_dim + h * head_dim;
            const int64_t cache_base =
                kv_offset(slot / block_size, h, slot % block_size, num_kv_heads, block_size, head_dim);
            for (int64_t d = 0; d < half; ++d) {
                const float x0 = k_in[kv_base + d], x1 = k_in[kv_base + half + d];
                const float c = cos_row[d], s = sin_row[d];
                kv_cache_k[cache_base + d] = x0 * c - x1 * s;
                kv_cache_k[cache_base + half + d] = x1 * c + x0 * s;
            }
            std::memcpy(kv_cache_v + cache_base, v_in + kv_base, size_t(head_dim) * 4);
        }
    }
}

// cpu_golden.rs:386-460 (`attention_via_cache`): one query token per sequence;
// score[t] = dot(q, k_t) * scale with the dot summed over d in order; softmax
// with the maximum subtracted and inv_sum = 1 / (sum_exp + 1e-6); out[d] =
// sum over t, in order, of score[t] * inv_sum * v_t[d].  kv_len == 0 leaves zeros.
void orc_attention_via_cache(const float* q, const float* kv_cache_k, const float* kv_cache_v,
                             const uint32_t* block_table, const uint32_t* seq_used_k, float* output,
                             int64_t batch, int64_t num_q_heads, int64_t num_kv_heads, int64_t head_dim,
                             int64_t block_size, int64_t max_blocks_per_seq, float attn_scale) {
    const int64_t q_dim = num_q_heads * head_dim;
    const int64_t group_ratio = num_q_heads / num_kv_heads;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int64_t seq = 0; seq < batch; ++seq) {
        for (int64_t h = 0; h < num_q_heads; ++h) {
            const int64_t kv_len = seq_used_k[seq];
            const uint32_t* row_blocks = block_table + seq * max_blocks_per_seq;
            const int64_t kv_h = h / group_ratio;
            const int64_t q_off = seq * q_dim + h * head_dim;
            std::vector<float> scores(size_t(kv_len), 0.0f);
            std::vector<int64_t> base(size_t(kv_len), 0);
            for (int64_t t = 0; t < kv_len; ++t) {
                base[size_t(t)] = kv_offset(row_blocks[t / block_size], kv_h, t % block_size, num_kv_heads,
                                            block_size, head_dim);
                float dot = 0.0f;
                for (int64_t d = 0; d < head_dim; ++d) dot += q[q_off + d] * kv_cache_k[base[size_t(t)] + d];
                scores[size_t(t)] = dot * attn_scale;
            }
            float max_logit = -std::numeric_limits<float>::infinity();
            for (float s : scores) max_logit = std::fmax(max_logit, s);
            float sum_exp = 0.0f;
            for (float& s : scores) {
                s = std::exp(s - max_logit);
                sum_exp += s;
            }
            const float inv_sum = 1.0f / (sum_exp + 1e-6f);
            for (int64_t d = 0; d < head_dim; ++d) {
                float acc = 0.0f;
                for (int64_t t = 0; t < kv_len; ++t)
                    acc += scores[size_t(t)] * inv_sum * kv_cache_v[base[size_t(t)] + d];
                output[q_off + d] = acc;
            }
        }
    }
}

// crates/targets/metal/tests/argmax_split_test.rs:24-33 (`argmax_ref`): the id
// of the row's largest value, the smallest id among equal ones, NaN never.
void orc_argmax(const float* logits, int64_t rows, int64_t width, uint32_t* out) {
    for (int64_t r = 0; r < rows; ++r) {
        float best = -std::numeric_limits<float>::infinity();
        uint32_t best_i = 0;
        for (int64_t i = 0; i < width; ++i) {
            const float v = logits[r * width + i];
            if (v > best || (v == best && uint32_t(i) < best_i)) {
                best = v;
                best_i = uint32_t(i);
            }
        }
        out[r] = best_i;
    }
}

}  // extern "C"
