// flat_oracle.cpp — TEST INFRASTRUCTURE, not product code.
//
// CPU restatement (C++17) of FLAT-ATTENTION's deterministic scalar Rust oracle.  Only the
// test-suite, the smoke check and the benchmark's CPU-baseline leg may load this library; the
// CUDA product path never calls it.
//
// Parity status: the reference ships no stored numeric golden vectors and no Rust toolchain is
// available to run it, so this restatement is pinned by the reference's own oracle-only tests
// restated in tests/test_oracle_*.py (cross-oracle bit-exact equalities, invariants, finite
// differences, known-answer page-table cases).  It is not pinned against executed reference
// output: "parity unpinned" in that strict sense.
//
// Bit-fidelity rules followed here: IEEE f32 everywhere, serial loop order exactly as the
// reference writes it, no FMA contraction (build with -ffp-contract=off, no -ffast-math),
// expf/logf/powf/sinf/cosf/fmaxf from glibc (what Rust's std lowers to on Linux), 1.0f/x for
// `recip`, alpha = 0 when the running max is -inf, positions cast to f32 before the multiply.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <functional>
#include <limits>
#include <thread>
#include <vector>

#include "../include/flat_attention_b200.h"

namespace {

thread_local char g_detail[256] = "";

int fail(int status, const char *fmt, const char *tensor, unsigned long long a,
         unsigned long long b) {
    std::snprintf(g_detail, sizeof g_detail, fmt, tensor, a, b);
    return status;
}

using usize = uint64_t;

bool checked_mul(usize a, usize b, usize *out) { return !__builtin_mul_overflow(a, b, out); }
bool checked_add(usize a, usize b, usize *out) { return !__builtin_add_overflow(a, b, out); }

// validate_input (src/lib.rs:428-447): length first, then the first non-finite index.
int validate_input(const char *name, const float *data, usize len, usize expected) {
    if (len != expected)
        return fail(FLAT_ERR_LENGTH_MISMATCH, "tensor %s contains %llu elements, expected %llu",
                    name, len, expected);
    for (usize i = 0; i < len; ++i)
        if (!std::isfinite(data[i]))
            return fail(FLAT_ERR_NON_FINITE_INPUT,
                        "tensor %s contains a non-finite value at index %llu", name, i, 0);
    return FLAT_OK;
}

// FlatAttentionConfig::resolved_scale (src/lib.rs:257-268).
int resolved_scale(int has_scale, float scale_in, usize head_dim, float *out) {
    if (head_dim == 0) return FLAT_ERR_ZERO_DIMENSION;
    float scale = has_scale ? scale_in : 1.0f / std::sqrt((float)head_dim);
    if (!std::isfinite(scale) || scale <= 0.0f) return FLAT_ERR_INVALID_SCALE;
    *out = scale;
    return FLAT_OK;
}

struct Shape {
    usize batch, q_heads, kv_heads, query_len, kv_len, head_dim, query_position_offset;
};

// AsymmetricGroupedAttentionShape::{q_tensor_len,kv_tensor_len,lse_len,validate}
// (src/asymmetric_grouped.rs:37-60,184-207); GroupedAttentionShape::validate
// (src/grouped.rs:54-75) and AttentionShape::validate (src/lib.rs:237-244) are the
// equal-length / equal-head special cases of the same checks.
int shape_lens(const Shape &s, usize *q_len, usize *kv_len, usize *lse_len) {
    usize t;
    if (!checked_mul(s.batch, s.q_heads, &t) || !checked_mul(t, s.query_len, &t)) return FLAT_ERR_SHAPE_OVERFLOW;
    *lse_len = t;
    if (!checked_mul(t, s.head_dim, q_len)) return FLAT_ERR_SHAPE_OVERFLOW;
    if (!checked_mul(s.batch, s.kv_heads, &t) || !checked_mul(t, s.kv_len, &t) ||
        !checked_mul(t, s.head_dim, kv_len))
        return FLAT_ERR_SHAPE_OVERFLOW;
    return FLAT_OK;
}

int validate_shape(const Shape &s) {
    if (s.batch == 0 || s.q_heads == 0 || s.kv_heads == 0 || s.query_len == 0 || s.kv_len == 0 ||
        s.head_dim == 0)
        return FLAT_ERR_ZERO_DIMENSION;
    if (s.q_heads % s.kv_heads != 0)
        return fail(FLAT_ERR_INVALID_HEAD_GROUPING,
                    "%sq_heads (%llu) must be exactly divisible by kv_heads (%llu)", "", s.q_heads,
                    s.kv_heads);
    usize t;
    if (!checked_add(s.query_position_offset, s.query_len - 1, &t)) return FLAT_ERR_SHAPE_OVERFLOW;
    usize a, b, c;
    return shape_lens(s, &a, &b, &c);
}

// RotaryEmbeddingConfig::validate (src/rotary_grouped.rs:21-33).
int validate_rotary(float theta, usize position_offset, usize head_dim, usize seq_len) {
    if (head_dim == 0 || head_dim % 2 != 0) return FLAT_ERR_INVALID_ROTARY_HEAD_DIM;
    if (!std::isfinite(theta) || theta <= 0.0f) return FLAT_ERR_INVALID_ROTARY_THETA;
    usize t;
    if (!checked_add(position_offset, seq_len == 0 ? 0 : seq_len - 1, &t)) return FLAT_ERR_POSITION_OVERFLOW;
    return FLAT_OK;
}

// rotated_pair (src/rotary_grouped.rs:36-50, src/projection_asymmetric.rs:70-84).
inline void rotated_pair(float even, float odd, usize pair, usize head_dim, usize position,
                         float theta, float *re, float *ro) {
    float exponent = -2.0f * (float)pair / (float)head_dim;
    float frequency = powf(theta, exponent);
    float angle = (float)position * frequency;
    float s = sinf(angle), c = cosf(angle);
    *re = even * c - odd * s;
    *ro = even * s + odd * c;
}

struct Rope {
    bool on = false;
    float theta = 0.0f;
    usize q_position = 0;   // absolute rotary position of this query row
    usize kv_offset = 0;    // rotary position of key 0
};

// AttentionBias::score (src/attention_bias.rs:61-97) for one (batch, q_head, query row): dense values of that row,
// or slope * (key_position - query_position) with the difference formed in f64 and rounded to f32.
struct RowBias {
    int mode = 0;                 // 0 none, 1 dense, 2 ALiBi
    const float *dense = nullptr; // [kv_len] values of this row
    float slope = 0.0f;
    usize query_position = 0, kv_offset = 0;
    float at(usize key_pos) const {
        if (mode == 1) return dense[key_pos];
        if (mode == 2) {
            double delta = (double)(kv_offset + key_pos) - (double)query_position;
            return slope * (float)delta;
        }
        return 0.0f;
    }
};

// One query row of the online-softmax update shared by every forward oracle:
// src/lib.rs:478-516, src/grouped.rs:110-147, src/asymmetric_grouped.rs:260-298,
// src/rotary_grouped.rs:92-150, src/projection_asymmetric.rs:120-232.
// q_row/out_row address head_dim contiguous floats; key j lives at k0 + j*kv_stride.
void attend_row(const float *q_row, const float *k0, const float *v0, usize kv_stride,
                usize key_count, usize head_dim, float scale, const Rope &rope, float *out_row,
                float *lse_out, const RowBias *bias = nullptr) {
    float running_max = -std::numeric_limits<float>::infinity();
    float running_sum = 0.0f;
    for (usize d = 0; d < head_dim; ++d) out_row[d] = 0.0f;
    for (usize key_pos = 0; key_pos < key_count; ++key_pos) {
        const float *k_row = k0 + key_pos * kv_stride;
        const float *v_row = v0 + key_pos * kv_stride;
        float dot = 0.0f;
        if (rope.on) {
            usize key_position = rope.kv_offset + key_pos;
            for (usize pair = 0; pair < head_dim / 2; ++pair) {
                usize dim = 2 * pair;
                float qe, qo, ke, ko;
                rotated_pair(q_row[dim], q_row[dim + 1], pair, head_dim, rope.q_position,
                             rope.theta, &qe, &qo);
                rotated_pair(k_row[dim], k_row[dim + 1], pair, head_dim, key_position, rope.theta,
                             &ke, &ko);
                dot += qe * ke;
                dot += qo * ko;
            }
        } else {
            for (usize d = 0; d < head_dim; ++d) dot += q_row[d] * k_row[d];
        }
        float score = dot * scale;
        if (bias) score = dot * scale + bias->at(key_pos);  // src/attention_bias.rs:282-283
        float new_max = fmaxf(running_max, score);
        float alpha = std::isinf(running_max) ? 0.0f : expf(running_max - new_max);
        float p = expf(score - new_max);
        for (usize d = 0; d < head_dim; ++d) out_row[d] = out_row[d] * alpha + p * v_row[d];
        running_sum = running_sum * alpha + p;
        running_max = new_max;
    }
    float inv_sum = 1.0f / running_sum;
    for (usize d = 0; d < head_dim; ++d) out_row[d] *= inv_sum;
    *lse_out = running_max + logf(running_sum);
}

// Element offset of (batch, head, position, dim 0).
inline usize row_base(int layout, usize batch, usize head, usize pos, usize heads, usize seq,
                      usize head_dim) {
    if (layout == FLAT_LAYOUT_HEAD_MAJOR) return ((batch * heads + head) * seq + pos) * head_dim;
    return ((batch * seq + pos) * heads + head) * head_dim;  // projection_index, src/projection_asymmetric.rs:46-68
}

struct ForwardArgs {
    const float *q, *k, *v;
    Shape s;
    int layout;
    int causal;
    float scale;
    bool rope;
    float theta;
    usize q_rope_offset, kv_rope_offset;
};

inline void forward_one(const ForwardArgs &a, usize batch, usize q_head, usize query_pos,
                        usize active_kv, usize causal_offset, float *out_row, float *lse_out) {
    const Shape &s = a.s;
    usize group = s.q_heads / s.kv_heads;
    usize kv_head = q_head / group;
    usize kv_stride = a.layout == FLAT_LAYOUT_HEAD_MAJOR ? s.head_dim : s.kv_heads * s.head_dim;
    usize absolute = causal_offset + query_pos;
    usize key_count = active_kv;
    if (a.causal && absolute + 1 < key_count) key_count = absolute + 1;  // `break` at key_pos > query position
    Rope rope;
    rope.on = a.rope;
    rope.theta = a.theta;
    rope.q_position = a.q_rope_offset + query_pos;
    rope.kv_offset = a.kv_rope_offset;
    const float *q_row = a.q + row_base(a.layout, batch, q_head, query_pos, s.q_heads, s.query_len, s.head_dim);
    const float *k0 = a.k + row_base(a.layout, batch, kv_head, 0, s.kv_heads, s.kv_len, s.head_dim);
    const float *v0 = a.v + row_base(a.layout, batch, kv_head, 0, s.kv_heads, s.kv_len, s.head_dim);
    attend_row(q_row, k0, v0, kv_stride, key_count, s.head_dim, a.scale, rope, out_row, lse_out);
}

void run_parallel(usize items, int threads, const std::function<void(usize)> &body) {
    if (threads <= 1 || items <= 1) {
        for (usize i = 0; i < items; ++i) body(i);
        return;
    }
    std::atomic<usize> next{0};
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t)
        pool.emplace_back([&] {
            for (;;) {
                usize i = next.fetch_add(1);
                if (i >= items) break;
                body(i);
            }
        });
    for (auto &th : pool) th.join();
}

int forward_full(const ForwardArgs &a, float *out, float *lse) {
    const Shape &s = a.s;
    for (usize batch = 0; batch < s.batch; ++batch)
        for (usize q_head = 0; q_head < s.q_heads; ++q_head)
            for (usize query_pos = 0; query_pos < s.query_len; ++query_pos) {
                float *out_row = out + row_base(a.layout, batch, q_head, query_pos, s.q_heads, s.query_len, s.head_dim);
                float *lse_out = lse + (batch * s.q_heads + q_head) * s.query_len + query_pos;
                forward_one(a, batch, q_head, query_pos, s.kv_len, s.query_position_offset, out_row, lse_out);
            }
    return FLAT_OK;
}

int prepare(const Shape &s, const float *q, usize q_n, const float *k, usize k_n, const float *v,
            usize v_n, const flat_attention_config *cfg, bool rope, float theta, usize q_rope_off,
            usize kv_rope_off, float *scale) {
    int st = validate_shape(s);
    if (st) return st;
    if (rope) {
        if ((st = validate_rotary(theta, q_rope_off, s.head_dim, s.query_len))) return st;
        if ((st = validate_rotary(theta, kv_rope_off, s.head_dim, s.kv_len))) return st;
    }
    usize ql, kl, ll;
    if ((st = shape_lens(s, &ql, &kl, &ll))) return st;
    if ((st = validate_input("Q", q, q_n, ql))) return st;
    if ((st = validate_input("K", k, k_n, kl))) return st;
    if ((st = validate_input("V", v, v_n, kl))) return st;
    return resolved_scale(cfg->has_softmax_scale, cfg->softmax_scale, s.head_dim, scale);
}

Shape to_shape(const flat_attention_shape *p) {
    return Shape{p->batch, p->q_heads, p->kv_heads, p->query_len, p->kv_len, p->head_dim,
                 p->query_position_offset};
}

}  // namespace

extern "C" {

const char *flat_oracle_last_error(void) { return g_detail; }

// forward_reference (src/lib.rs:454-521): MHA, head-major, equal length.
int32_t flat_oracle_forward_reference(const float *q, uint64_t q_n, const float *k, uint64_t k_n,
                                      const float *v, uint64_t v_n, uint64_t batch, uint64_t heads,
                                      uint64_t seq_len, uint64_t head_dim,
                                      const flat_attention_config *cfg, float *out, float *lse) {
    Shape s{batch, heads, heads, seq_len, seq_len, head_dim, 0};
    float scale;
    int st = prepare(s, q, q_n, k, k_n, v, v_n, cfg, false, 0, 0, 0, &scale);
    if (st) return st;
    ForwardArgs a{q, k, v, s, FLAT_LAYOUT_HEAD_MAJOR, cfg->causal, scale, false, 0, 0, 0};
    return forward_full(a, out, lse);
}

// forward_reference_grouped (src/grouped.rs:81-153) when query_len == kv_len and offset == 0;
// forward_reference_grouped_asymmetric (src/asymmetric_grouped.rs:230-304) in general.
int32_t flat_oracle_forward_grouped_asymmetric(const float *q, uint64_t q_n, const float *k,
                                               uint64_t k_n, const float *v, uint64_t v_n,
                                               const flat_attention_shape *shape,
                                               const flat_attention_config *cfg, float *out,
                                               float *lse) {
    Shape s = to_shape(shape);
    float scale;
    int st = prepare(s, q, q_n, k, k_n, v, v_n, cfg, false, 0, 0, 0, &scale);
    if (st) return st;
    ForwardArgs a{q, k, v, s, FLAT_LAYOUT_HEAD_MAJOR, cfg->causal, scale, false, 0, 0, 0};
    return forward_full(a, out, lse);
}

// forward_reference_grouped_rope (src/rotary_grouped.rs:57-156): head-major, fused RoPE,
// one position offset for Q and K.
int32_t flat_oracle_forward_grouped_rope(const float *q, uint64_t q_n, const float *k, uint64_t k_n,
                                         const float *v, uint64_t v_n,
                                         const flat_attention_shape *shape,
                                         const flat_attention_config *cfg, float theta,
                                         uint64_t position_offset, float *out, float *lse) {
    Shape s = to_shape(shape);
    float scale;
    int st = prepare(s, q, q_n, k, k_n, v, v_n, cfg, true, theta, position_offset, position_offset, &scale);
    if (st) return st;
    ForwardArgs a{q, k, v, s, FLAT_LAYOUT_HEAD_MAJOR, cfg->causal, scale, true, theta, position_offset, position_offset};
    return forward_full(a, out, lse);
}

// forward_reference_projection_grouped_rope (src/projection_grouped.rs:62-164) when the shape
// is square with equal offsets; forward_reference_projection_grouped_rope_asymmetric
// (src/projection_asymmetric.rs:97-238) in general.
int32_t flat_oracle_forward_projection_rope_asymmetric(
    const float *q, uint64_t q_n, const float *k, uint64_t k_n, const float *v, uint64_t v_n,
    const flat_attention_shape *shape, const flat_attention_config *cfg, float theta,
    uint64_t query_rope_offset, uint64_t kv_rope_offset, float *out, float *lse) {
    Shape s = to_shape(shape);
    float scale;
    int st = prepare(s, q, q_n, k, k_n, v, v_n, cfg, true, theta, query_rope_offset, kv_rope_offset, &scale);
    if (st) return st;
    ForwardArgs a{q, k, v, s, FLAT_LAYOUT_PROJECTION, cfg->causal, scale, true, theta, query_rope_offset, kv_rope_offset};
    return forward_full(a, out, lse);
}

// forward_reference_projection_grouped_rope_asymmetric_biased (src/attention_bias.rs:193-339).
// bias_mode 0: none; 1: dense [batch, q_heads, query_len, kv_len] in `bias` (bias_n elements);
// 2: ALiBi, `bias` holds q_heads slopes, positions start at bias_q_offset / bias_kv_offset.
int32_t flat_oracle_forward_projection_rope_asymmetric_biased(
    const float *q, uint64_t q_n, const float *k, uint64_t k_n, const float *v, uint64_t v_n,
    const flat_attention_shape *shape, const flat_attention_config *cfg, float theta,
    uint64_t query_rope_offset, uint64_t kv_rope_offset, int32_t bias_mode, const float *bias, uint64_t bias_n,
    uint64_t bias_q_offset, uint64_t bias_kv_offset, float *out, float *lse) {
    Shape s = to_shape(shape);
    int st = validate_shape(s);
    if (st) return st;
    if ((st = validate_rotary(theta, query_rope_offset, s.head_dim, s.query_len))) return st;
    if ((st = validate_rotary(theta, kv_rope_offset, s.head_dim, s.kv_len))) return st;
    // AttentionBias::validate (src/attention_bias.rs:31-58) comes before the tensors are looked at
    if (bias_mode == 1) {
        usize expected;
        if (!checked_mul(s.batch, s.q_heads, &expected) || !checked_mul(expected, s.query_len, &expected) ||
            !checked_mul(expected, s.kv_len, &expected))
            return FLAT_ERR_SHAPE_OVERFLOW;
        if ((st = validate_input("attention bias", bias, bias_n, expected))) return st;
    } else if (bias_mode == 2) {
        if ((st = validate_input("ALiBi slopes", bias, bias_n, s.q_heads))) return st;
        usize t;
        if (!checked_add(bias_q_offset, s.query_len - 1, &t) || !checked_add(bias_kv_offset, s.kv_len - 1, &t))
            return FLAT_ERR_POSITION_OVERFLOW;
    }
    float scale;
    if ((st = prepare(s, q, q_n, k, k_n, v, v_n, cfg, true, theta, query_rope_offset, kv_rope_offset, &scale))) return st;
    const usize group = s.q_heads / s.kv_heads, kv_stride = s.kv_heads * s.head_dim;
    for (usize batch = 0; batch < s.batch; ++batch)
        for (usize q_head = 0; q_head < s.q_heads; ++q_head)
            for (usize query_pos = 0; query_pos < s.query_len; ++query_pos) {
                usize kv_head = q_head / group;
                usize key_count = s.kv_len, absolute = s.query_position_offset + query_pos;
                if (cfg->causal && absolute + 1 < key_count) key_count = absolute + 1;
                Rope rope;
                rope.on = true;
                rope.theta = theta;
                rope.q_position = query_rope_offset + query_pos;
                rope.kv_offset = kv_rope_offset;
                RowBias rb;
                rb.mode = bias_mode;
                if (bias_mode == 1) rb.dense = bias + ((batch * s.q_heads + q_head) * s.query_len + query_pos) * s.kv_len;
                if (bias_mode == 2) {
                    rb.slope = bias[q_head];
                    rb.query_position = bias_q_offset + query_pos;
                    rb.kv_offset = bias_kv_offset;
                }
                const float *q_row = q + row_base(FLAT_LAYOUT_PROJECTION, batch, q_head, query_pos, s.q_heads, s.query_len, s.head_dim);
                const float *k0 = k + row_base(FLAT_LAYOUT_PROJECTION, batch, kv_head, 0, s.kv_heads, s.kv_len, s.head_dim);
                const float *v0 = v + row_base(FLAT_LAYOUT_PROJECTION, batch, kv_head, 0, s.kv_heads, s.kv_len, s.head_dim);
                float *out_row = out + row_base(FLAT_LAYOUT_PROJECTION, batch, q_head, query_pos, s.q_heads, s.query_len, s.head_dim);
                float *lse_out = lse + (batch * s.q_heads + q_head) * s.query_len + query_pos;
                attend_row(q_row, k0, v0, kv_stride, key_count, s.head_dim, scale, rope, out_row, lse_out,
                           bias_mode ? &rb : nullptr);
            }
    return FLAT_OK;
}

// AsymmetricGroupedAttentionShape::forward_reference_variable_lengths
// (src/asymmetric_grouped.rs:77-182): head-major padded batch, `active` holds
// (active_q, active_kv, query_position_offset) per batch element.
int32_t flat_oracle_forward_variable_lengths(const float *q, uint64_t q_n, const float *k,
                                             uint64_t k_n, const float *v, uint64_t v_n,
                                             const flat_attention_shape *shape,
                                             const uint64_t *active, uint64_t active_count,
                                             const flat_attention_config *cfg, float *out,
                                             float *lse) {
    Shape s = to_shape(shape);
    int st = validate_shape(s);
    if (st) return st;
    usize ql, kl, ll;
    if ((st = shape_lens(s, &ql, &kl, &ll))) return st;
    if ((st = validate_input("Q", q, q_n, ql))) return st;
    if ((st = validate_input("K", k, k_n, kl))) return st;
    if ((st = validate_input("V", v, v_n, kl))) return st;
    if (active_count != s.batch)
        return fail(FLAT_ERR_LENGTH_MISMATCH, "tensor %s contains %llu elements, expected %llu",
                    "active sequence metadata", active_count, s.batch);
    float scale;
    if ((st = resolved_scale(cfg->has_softmax_scale, cfg->softmax_scale, s.head_dim, &scale))) return st;
    for (usize i = 0; i < ql; ++i) out[i] = 0.0f;
    for (usize i = 0; i < ll; ++i) lse[i] = -std::numeric_limits<float>::infinity();
    ForwardArgs a{q, k, v, s, FLAT_LAYOUT_HEAD_MAJOR, cfg->causal, scale, false, 0, 0, 0};
    for (usize batch = 0; batch < s.batch; ++batch) {
        usize aq = active[3 * batch], akv = active[3 * batch + 1], off = active[3 * batch + 2];
        if (aq == 0 || akv == 0) return FLAT_ERR_ZERO_DIMENSION;
        if (aq > s.query_len)
            return fail(FLAT_ERR_LENGTH_MISMATCH, "tensor %s contains %llu elements, expected %llu",
                        "active query length", aq, s.query_len);
        if (akv > s.kv_len)
            return fail(FLAT_ERR_LENGTH_MISMATCH, "tensor %s contains %llu elements, expected %llu",
                        "active KV length", akv, s.kv_len);
        usize t;
        if (!checked_add(off, aq - 1, &t)) return FLAT_ERR_POSITION_OVERFLOW;
        for (usize q_head = 0; q_head < s.q_heads; ++q_head)
            for (usize query_pos = 0; query_pos < aq; ++query_pos) {
                float *out_row = out + row_base(a.layout, batch, q_head, query_pos, s.q_heads, s.query_len, s.head_dim);
                float *lse_out = lse + (batch * s.q_heads + q_head) * s.query_len + query_pos;
                forward_one(a, batch, q_head, query_pos, akv, off, out_row, lse_out);
            }
    }
    return FLAT_OK;
}

// forward_reference_projection_grouped_rope_chunked_prefill
// (src/chunked_projection_prefill.rs:63-169): Q chunks compacted per batch, evaluated by the
// asymmetric projection oracle with kv_len = seq_len, then scattered back.
int32_t flat_oracle_chunked_prefill(const float *q, uint64_t q_n, const float *k, uint64_t k_n,
                                    const float *v, uint64_t v_n, const flat_attention_shape *shape,
                                    const flat_attention_config *cfg, float theta,
                                    uint64_t position_offset, uint64_t query_chunk_size, float *out,
                                    float *lse) {
    if (query_chunk_size == 0) return FLAT_ERR_ZERO_QUERY_CHUNK_SIZE;
    Shape s = to_shape(shape);
    int st = validate_shape(s);
    if (st) return st;
    if ((st = validate_rotary(theta, position_offset, s.head_dim, s.query_len))) return st;
    usize ql, kl, ll;
    if ((st = shape_lens(s, &ql, &kl, &ll))) return st;
    if ((st = validate_input("Q", q, q_n, ql))) return st;
    if ((st = validate_input("K", k, k_n, kl))) return st;
    if ((st = validate_input("V", v, v_n, kl))) return st;
    usize seq_len = s.query_len;
    usize q_width = s.q_heads * s.head_dim;
    usize query_start = 0;
    while (query_start < seq_len) {
        usize chunk_len = std::min<usize>(query_chunk_size, seq_len - query_start);
        std::vector<float> chunk_q;
        chunk_q.reserve(s.batch * chunk_len * q_width);
        for (usize batch = 0; batch < s.batch; ++batch) {
            usize row_start = (batch * seq_len + query_start) * q_width;
            chunk_q.insert(chunk_q.end(), q + row_start, q + row_start + chunk_len * q_width);
        }
        flat_attention_shape cs{s.batch, s.q_heads, s.kv_heads, chunk_len, seq_len, s.head_dim, query_start};
        usize q_rope;
        if (!checked_add(position_offset, query_start, &q_rope)) return FLAT_ERR_POSITION_OVERFLOW;
        std::vector<float> c_out(chunk_q.size()), c_lse(s.batch * s.q_heads * chunk_len);
        st = flat_oracle_forward_projection_rope_asymmetric(chunk_q.data(), chunk_q.size(), k, k_n, v,
                                                            v_n, &cs, cfg, theta, q_rope,
                                                            position_offset, c_out.data(), c_lse.data());
        if (st) return st;
        for (usize batch = 0; batch < s.batch; ++batch) {
            usize chunk_row_base = batch * chunk_len * q_width;
            usize full_row_base = (batch * seq_len + query_start) * q_width;
            std::memcpy(out + full_row_base, c_out.data() + chunk_row_base, chunk_len * q_width * sizeof(float));
            for (usize q_head = 0; q_head < s.q_heads; ++q_head) {
                usize chunk_lse_base = (batch * s.q_heads + q_head) * chunk_len;
                usize full_lse_base = (batch * s.q_heads + q_head) * seq_len + query_start;
                std::memcpy(lse + full_lse_base, c_lse.data() + chunk_lse_base, chunk_len * sizeof(float));
            }
        }
        query_start += chunk_len;
    }
    return FLAT_OK;
}

// backward_reference_grouped (src/backward_grouped.rs:17-93); with q_heads == kv_heads it is
// backward_reference (src/backward.rs:27-98), which the reference proves bitwise equal
// (src/backward_grouped.rs:208-237).
int32_t flat_oracle_backward_grouped(const float *q, uint64_t q_n, const float *k, uint64_t k_n,
                                     const float *v, uint64_t v_n, const float *d_out,
                                     uint64_t d_out_n, const float *fwd_out, uint64_t fwd_out_n,
                                     const float *fwd_lse, uint64_t fwd_lse_n, uint64_t batch,
                                     uint64_t q_heads, uint64_t kv_heads, uint64_t seq_len,
                                     uint64_t head_dim, const flat_attention_config *cfg, float *dq,
                                     float *dk, float *dv) {
    Shape s{batch, q_heads, kv_heads, seq_len, seq_len, head_dim, 0};
    int st = validate_shape(s);
    if (st) return st;
    usize ql, kl, ll;
    if ((st = shape_lens(s, &ql, &kl, &ll))) return st;
    if ((st = validate_input("Q", q, q_n, ql))) return st;
    if ((st = validate_input("K", k, k_n, kl))) return st;
    if ((st = validate_input("V", v, v_n, kl))) return st;
    if ((st = validate_input("dO", d_out, d_out_n, ql))) return st;
    if ((st = validate_input("O", fwd_out, fwd_out_n, ql))) return st;
    if ((st = validate_input("LSE", fwd_lse, fwd_lse_n, ll))) return st;
    float scale;
    if ((st = resolved_scale(cfg->has_softmax_scale, cfg->softmax_scale, head_dim, &scale))) return st;
    usize group_size = q_heads / kv_heads;
    usize head_stride = seq_len * head_dim;
    for (usize i = 0; i < ql; ++i) dq[i] = 0.0f;
    for (usize i = 0; i < kl; ++i) dk[i] = 0.0f, dv[i] = 0.0f;
    for (usize b = 0; b < batch; ++b)
        for (usize q_head = 0; q_head < q_heads; ++q_head) {
            usize kv_head = q_head / group_size;
            usize q_bh = b * q_heads + q_head, kv_bh = b * kv_heads + kv_head;
            usize q_head_base = q_bh * head_stride, kv_head_base = kv_bh * head_stride;
            usize lse_base = q_bh * seq_len;
            for (usize query_pos = 0; query_pos < seq_len; ++query_pos) {
                usize q_base = q_head_base + query_pos * head_dim;
                float lse = fwd_lse[lse_base + query_pos];
                float delta = 0.0f;
                for (usize d = 0; d < head_dim; ++d) delta += d_out[q_base + d] * fwd_out[q_base + d];
                usize key_limit = cfg->causal ? query_pos + 1 : seq_len;
                for (usize key_pos = 0; key_pos < key_limit; ++key_pos) {
                    usize kv_base = kv_head_base + key_pos * head_dim;
                    float dot_qk = 0.0f, d_probability = 0.0f;
                    for (usize d = 0; d < head_dim; ++d) {
                        dot_qk += q[q_base + d] * k[kv_base + d];
                        d_probability += d_out[q_base + d] * v[kv_base + d];
                    }
                    float score = dot_qk * scale;
                    float probability = expf(score - lse);
                    float d_score = probability * (d_probability - delta);
                    float d_dot = d_score * scale;
                    for (usize d = 0; d < head_dim; ++d) {
                        dq[q_base + d] += d_dot * k[kv_base + d];
                        dk[kv_base + d] += d_dot * q[q_base + d];
                        dv[kv_base + d] += probability * d_out[q_base + d];
                    }
                }
            }
        }
    return FLAT_OK;
}

// ---- sampled evaluation for the large configurations -----------------------------------------
// Each oracle query row is independent (src/lib.rs:478-516), so the large configurations are
// checked on sampled (batch, q_head, query_pos) rows.  rows holds `row_count` triples; outputs are
// compact [row_count, head_dim] and [row_count].  No RoPE inside: callers materialise the rotation
// first (flat_oracle_rotate_rows), which tests/rotary_grouped.rs:48-143 proves bit-identical to the
// fused oracle.  `threads` > 1 spreads rows over host threads (each row keeps its serial order).
int32_t flat_oracle_forward_rows(const float *q, const float *k, const float *v,
                                 const flat_attention_shape *shape, int32_t layout,
                                 const flat_attention_config *cfg, const uint64_t *rows,
                                 uint64_t row_count, int32_t threads, float *out_rows,
                                 float *lse_rows) {
    Shape s = to_shape(shape);
    int st = validate_shape(s);
    if (st) return st;
    float scale;
    if ((st = resolved_scale(cfg->has_softmax_scale, cfg->softmax_scale, s.head_dim, &scale))) return st;
    ForwardArgs a{q, k, v, s, layout, cfg->causal, scale, false, 0, 0, 0};
    run_parallel(row_count, threads, [&](usize i) {
        forward_one(a, rows[3 * i], rows[3 * i + 1], rows[3 * i + 2], s.kv_len,
                    s.query_position_offset, out_rows + i * s.head_dim, lse_rows + i);
    });
    return FLAT_OK;
}

// The same row sampling with an ALiBi score bias (AttentionBias::Alibi, src/attention_bias.rs:82-95): slopes holds
// one f32 per query head, bias positions start at bias_q_offset / bias_kv_offset.  No RoPE here either: with the
// rotation materialised first the rows are bit-identical to flat_oracle_forward_projection_rope_asymmetric_biased.
int32_t flat_oracle_forward_rows_alibi(const float *q, const float *k, const float *v,
                                       const flat_attention_shape *shape, int32_t layout,
                                       const flat_attention_config *cfg, const float *slopes,
                                       uint64_t bias_q_offset, uint64_t bias_kv_offset, const uint64_t *rows,
                                       uint64_t row_count, int32_t threads, float *out_rows, float *lse_rows) {
    Shape s = to_shape(shape);
    int st = validate_shape(s);
    if (st) return st;
    float scale;
    if ((st = resolved_scale(cfg->has_softmax_scale, cfg->softmax_scale, s.head_dim, &scale))) return st;
    const usize group = s.q_heads / s.kv_heads;
    const usize kv_stride = layout == FLAT_LAYOUT_HEAD_MAJOR ? s.head_dim : s.kv_heads * s.head_dim;
    run_parallel(row_count, threads, [&](usize i) {
        const usize batch = rows[3 * i], q_head = rows[3 * i + 1], query_pos = rows[3 * i + 2];
        const usize kv_head = q_head / group;
        usize key_count = s.kv_len, absolute = s.query_position_offset + query_pos;
        if (cfg->causal && absolute + 1 < key_count) key_count = absolute + 1;
        Rope rope;
        rope.on = false;
        RowBias rb;
        rb.mode = 2;
        rb.slope = slopes[q_head];
        rb.query_position = bias_q_offset + query_pos;
        rb.kv_offset = bias_kv_offset;
        const float *q_row = q + row_base(layout, batch, q_head, query_pos, s.q_heads, s.query_len, s.head_dim);
        const float *k0 = k + row_base(layout, batch, kv_head, 0, s.kv_heads, s.kv_len, s.head_dim);
        const float *v0 = v + row_base(layout, batch, kv_head, 0, s.kv_heads, s.kv_len, s.head_dim);
        attend_row(q_row, k0, v0, kv_stride, key_count, s.head_dim, scale, rope, out_rows + i * s.head_dim, lse_rows + i, &rb);
    });
    return FLAT_OK;
}

// Backward for whole (batch, kv_head) units: dK/dV need every query row of the unit.  units holds
// `unit_count` (batch, kv_head) pairs; dq_units is [unit_count, group, seq_len, head_dim], dk/dv
// are [unit_count, seq_len, head_dim].  Loop order inside a unit is the reference's
// (q_head ascending, then query_pos, then key_pos), so each unit's sums are bit-identical to the
// same elements of flat_oracle_backward_grouped.
int32_t flat_oracle_backward_units(const float *q, const float *k, const float *v,
                                   const float *d_out, const float *fwd_out, const float *fwd_lse,
                                   uint64_t batch, uint64_t q_heads, uint64_t kv_heads,
                                   uint64_t seq_len, uint64_t head_dim,
                                   const flat_attention_config *cfg, const uint64_t *units,
                                   uint64_t unit_count, int32_t threads, float *dq_units,
                                   float *dk_units, float *dv_units) {
    Shape s{batch, q_heads, kv_heads, seq_len, seq_len, head_dim, 0};
    int st = validate_shape(s);
    if (st) return st;
    float scale;
    if ((st = resolved_scale(cfg->has_softmax_scale, cfg->softmax_scale, head_dim, &scale))) return st;
    usize group = q_heads / kv_heads;
    usize head_stride = seq_len * head_dim;
    run_parallel(unit_count, threads, [&](usize u) {
        usize b = units[2 * u], kv_head = units[2 * u + 1];
        float *dqu = dq_units + u * group * head_stride;
        float *dku = dk_units + u * head_stride;
        float *dvu = dv_units + u * head_stride;
        for (usize i = 0; i < group * head_stride; ++i) dqu[i] = 0.0f;
        for (usize i = 0; i < head_stride; ++i) dku[i] = 0.0f, dvu[i] = 0.0f;
        usize kv_head_base = (b * kv_heads + kv_head) * head_stride;
        for (usize g = 0; g < group; ++g) {
            usize q_head = kv_head * group + g;
            usize q_bh = b * q_heads + q_head;
            usize q_head_base = q_bh * head_stride;
            for (usize query_pos = 0; query_pos < seq_len; ++query_pos) {
                usize q_base = q_head_base + query_pos * head_dim;
                float *dq_row = dqu + (g * seq_len + query_pos) * head_dim;
                float lse = fwd_lse[q_bh * seq_len + query_pos];
                float delta = 0.0f;
                for (usize d = 0; d < head_dim; ++d) delta += d_out[q_base + d] * fwd_out[q_base + d];
                usize key_limit = cfg->causal ? query_pos + 1 : seq_len;
                for (usize key_pos = 0; key_pos < key_limit; ++key_pos) {
                    usize kv_base = kv_head_base + key_pos * head_dim;
                    float dot_qk = 0.0f, d_probability = 0.0f;
                    for (usize d = 0; d < head_dim; ++d) {
                        dot_qk += q[q_base + d] * k[kv_base + d];
                        d_probability += d_out[q_base + d] * v[kv_base + d];
                    }
                    float score = dot_qk * scale;
                    float probability = expf(score - lse);
                    float d_score = probability * (d_probability - delta);
                    float d_dot = d_score * scale;
                    for (usize d = 0; d < head_dim; ++d) {
                        dq_row[d] += d_dot * k[kv_base + d];
                        dku[key_pos * head_dim + d] += d_dot * q[q_base + d];
                        dvu[key_pos * head_dim + d] += probability * d_out[q_base + d];
                    }
                }
            }
        }
    });
    return FLAT_OK;
}

// Backward on sampled output rows for the large configurations.  dq_rows holds (batch, q_head, query)
// triples, dkv_rows holds (batch, kv_head, key) triples.  Every output element is accumulated in the
// order the reference visits its contributions (src/backward_grouped.rs:44-88: q_head ascending, then
// query ascending for dK/dV; key ascending for dQ), so a row equals the same row of
// flat_oracle_backward_grouped bit for bit.
int32_t flat_oracle_backward_rows(const float *q, const float *k, const float *v, const float *d_out,
                                  const float *fwd_out, const float *fwd_lse, uint64_t batch, uint64_t q_heads,
                                  uint64_t kv_heads, uint64_t seq_len, uint64_t head_dim,
                                  const flat_attention_config *cfg, const uint64_t *dq_rows, uint64_t n_dq,
                                  const uint64_t *dkv_rows, uint64_t n_dkv, int32_t threads, float *dq_out,
                                  float *dk_out, float *dv_out) {
    Shape s{batch, q_heads, kv_heads, seq_len, seq_len, head_dim, 0};
    int st = validate_shape(s);
    if (st) return st;
    float scale;
    if ((st = resolved_scale(cfg->has_softmax_scale, cfg->softmax_scale, head_dim, &scale))) return st;
    const usize group = q_heads / kv_heads, D = head_dim, N = seq_len;
    auto pair_terms = [&](usize b, usize q_head, usize query_pos, usize key_pos, float delta, float *prob, float *d_dot) {
        const usize kv_head = q_head / group;
        const usize q_base = ((b * q_heads + q_head) * N + query_pos) * D;
        const usize kv_base = ((b * kv_heads + kv_head) * N + key_pos) * D;
        float dot_qk = 0.0f, d_probability = 0.0f;
        for (usize d = 0; d < D; ++d) {
            dot_qk += q[q_base + d] * k[kv_base + d];
            d_probability += d_out[q_base + d] * v[kv_base + d];
        }
        const float score = dot_qk * scale;
        *prob = expf(score - fwd_lse[(b * q_heads + q_head) * N + query_pos]);
        const float d_score = *prob * (d_probability - delta);
        *d_dot = d_score * scale;
    };
    auto delta_of = [&](usize b, usize q_head, usize query_pos) {
        const usize q_base = ((b * q_heads + q_head) * N + query_pos) * D;
        float delta = 0.0f;
        for (usize d = 0; d < D; ++d) delta += d_out[q_base + d] * fwd_out[q_base + d];
        return delta;
    };
    run_parallel(n_dq, threads, [&](usize i) {
        const usize b = dq_rows[3 * i], q_head = dq_rows[3 * i + 1], query_pos = dq_rows[3 * i + 2];
        const usize kv_head = q_head / group;
        float *out = dq_out + i * D;
        for (usize d = 0; d < D; ++d) out[d] = 0.0f;
        const float delta = delta_of(b, q_head, query_pos);
        const usize key_limit = cfg->causal ? query_pos + 1 : N;
        for (usize key_pos = 0; key_pos < key_limit; ++key_pos) {
            float prob, d_dot;
            pair_terms(b, q_head, query_pos, key_pos, delta, &prob, &d_dot);
            const usize kv_base = ((b * kv_heads + kv_head) * N + key_pos) * D;
            for (usize d = 0; d < D; ++d) out[d] += d_dot * k[kv_base + d];
        }
    });
    run_parallel(n_dkv, threads, [&](usize i) {
        const usize b = dkv_rows[3 * i], kv_head = dkv_rows[3 * i + 1], key_pos = dkv_rows[3 * i + 2];
        float *ok = dk_out + i * D, *ov = dv_out + i * D;
        for (usize d = 0; d < D; ++d) ok[d] = 0.0f, ov[d] = 0.0f;
        for (usize g = 0; g < group; ++g) {
            const usize q_head = kv_head * group + g;
            for (usize query_pos = cfg->causal ? key_pos : 0; query_pos < N; ++query_pos) {
                const float delta = delta_of(b, q_head, query_pos);
                float prob, d_dot;
                pair_terms(b, q_head, query_pos, key_pos, delta, &prob, &d_dot);
                const usize q_base = ((b * q_heads + q_head) * N + query_pos) * D;
                for (usize d = 0; d < D; ++d) {
                    ok[d] += d_dot * q[q_base + d];
                    ov[d] += prob * d_out[q_base + d];
                }
            }
        }
    });
    return FLAT_OK;
}

// Materialised RoPE, the helper of tests/rotary_grouped.rs:15-47 generalised to a list of rows:
// row r (head_dim contiguous floats at src + r*head_dim) is rotated at positions[r].
void flat_oracle_rotate_rows(const float *src, float *dst, uint64_t row_count, uint64_t head_dim,
                             const uint64_t *positions, float theta) {
    for (usize r = 0; r < row_count; ++r)
        for (usize pair = 0; pair < head_dim / 2; ++pair) {
            usize i = r * head_dim + 2 * pair;
            float e = src[i], o = src[i + 1], re, ro;
            rotated_pair(e, o, pair, head_dim, positions[r], theta, &re, &ro);
            dst[i] = re;
            dst[i + 1] = ro;
        }
}

// The frequency table theta^(-2j/D) exactly as rotated_pair computes it (f32 powf).
void flat_oracle_rope_frequencies(float theta, uint64_t head_dim, float *out) {
    for (usize pair = 0; pair < head_dim / 2; ++pair)
        out[pair] = powf(theta, -2.0f * (float)pair / (float)head_dim);
}

// Closed-form test fixtures of the reference tests: sin(x)*a + cos(x*c)*b with x = i*step + phase
// in f32 libm arithmetic (tests/grouped.rs:6-13, tests/rotary_grouped.rs:6-13, ...).
// F16::from_f32 (src/f16.rs:26-82): IEEE binary16, round to nearest, ties to even, written out on the bit fields.
static uint16_t f16_from_f32_bits(float value) {
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    const uint16_t sign = (uint16_t)((bits >> 16) & 0x8000);
    const int32_t exponent = (int32_t)((bits >> 23) & 0xff);
    uint32_t mantissa = bits & 0x007fffffu;
    if (exponent == 0xff) {
        if (mantissa == 0) return sign | 0x7c00;
        uint16_t payload = (uint16_t)(mantissa >> 13);
        if (payload == 0) payload = 1;
        return sign | 0x7c00 | payload;
    }
    int32_t half_exponent = exponent - 127 + 15;
    if (half_exponent >= 31) return sign | 0x7c00;
    if (half_exponent <= 0) {
        if (half_exponent < -10) return sign;
        mantissa |= 0x00800000u;
        const uint32_t shift = (uint32_t)(14 - half_exponent);
        uint32_t half_mantissa = mantissa >> shift;
        const uint32_t remainder = mantissa & ((1u << shift) - 1);
        const uint32_t halfway = 1u << (shift - 1);
        if (remainder > halfway || (remainder == halfway && (half_mantissa & 1))) half_mantissa += 1;
        return sign | (uint16_t)half_mantissa;
    }
    uint32_t half_mantissa = mantissa >> 13;
    const uint32_t remainder = mantissa & 0x1fff;
    if (remainder > 0x1000 || (remainder == 0x1000 && (half_mantissa & 1))) {
        half_mantissa += 1;
        if (half_mantissa == 0x400) {
            half_mantissa = 0;
            half_exponent += 1;
            if (half_exponent >= 31) return sign | 0x7c00;
        }
    }
    return sign | (uint16_t)(half_exponent << 10) | (uint16_t)half_mantissa;
}

// F16::to_f32 (src/f16.rs:85-110): exact.
static float f16_to_f32_bits(uint16_t bits) {
    const uint32_t sign = (uint32_t)(bits & 0x8000) << 16;
    const uint32_t exponent = (bits >> 10) & 0x1f;
    const uint32_t mantissa = bits & 0x03ff;
    uint32_t out;
    if (exponent == 0) {
        if (mantissa == 0) {
            out = sign;
        } else {
            uint32_t normalized = mantissa;
            uint32_t exponent32 = 127 - 14;
            while ((normalized & 0x400) == 0) {
                normalized <<= 1;
                exponent32 -= 1;
            }
            normalized &= 0x03ff;
            out = sign | (exponent32 << 23) | (normalized << 13);
        }
    } else if (exponent == 0x1f) {
        out = sign | 0x7f800000u | (mantissa << 13);
    } else {
        out = sign | ((exponent + (127 - 15)) << 23) | (mantissa << 13);
    }
    float f;
    std::memcpy(&f, &out, 4);
    return f;
}

void flat_oracle_f16_from_f32(const float *src, uint64_t n, uint16_t *dst) {
    for (uint64_t i = 0; i < n; ++i) dst[i] = f16_from_f32_bits(src[i]);
}
void flat_oracle_f16_to_f32(const uint16_t *src, uint64_t n, float *dst) {
    for (uint64_t i = 0; i < n; ++i) dst[i] = f16_to_f32_bits(src[i]);
}

void flat_oracle_fixture(float *out, uint64_t len, float step, float phase, float a, float c,
                         float b) {
    for (usize i = 0; i < len; ++i) {
        float x = (float)i * step + phase;
        out[i] = b == 0.0f ? sinf(x) * a : sinf(x) * a + cosf(x * c) * b;
    }
}

// ---- PagedKvTable (src/paged_kv.rs:75-188) ----------------------------------------------------
struct flat_oracle_paged_table {
    usize page_size, physical_pages;
    usize live_tokens = 0;
    uint64_t generation = 0;
    std::vector<std::pair<usize, uint64_t>> logical_pages;  // (physical_page, generation)
    std::vector<usize> free_pages;
};

int32_t flat_oracle_paged_table_new(uint64_t page_size, uint64_t physical_pages,
                                    flat_oracle_paged_table **out) {
    if (page_size == 0 || physical_pages == 0) return FLAT_ERR_ZERO_DIMENSION;
    usize cap;
    if (!checked_mul(page_size, physical_pages, &cap)) return FLAT_ERR_CAPACITY_OVERFLOW;
    auto *t = new flat_oracle_paged_table;
    t->page_size = page_size;
    t->physical_pages = physical_pages;
    for (usize p = physical_pages; p-- > 0;) t->free_pages.push_back(p);  // (0..pages).rev()
    *out = t;
    return FLAT_OK;
}
void flat_oracle_paged_table_free(flat_oracle_paged_table *t) { delete t; }

int32_t flat_oracle_paged_table_append(flat_oracle_paged_table *t, uint64_t tokens) {
    if (tokens == 0) return FLAT_OK;
    usize new_len;
    if (!checked_add(t->live_tokens, tokens, &new_len)) return FLAT_ERR_CAPACITY_OVERFLOW;
    usize capacity = t->page_size * t->physical_pages;
    if (new_len > capacity)
        return fail(FLAT_ERR_CAPACITY_EXCEEDED, "%spaged KV append requires %llu tokens, capacity is %llu", "", new_len, capacity);
    usize required_pages = (new_len + t->page_size - 1) / t->page_size;
    while (t->logical_pages.size() < required_pages) {
        usize page = t->free_pages.back();
        t->free_pages.pop_back();
        t->logical_pages.emplace_back(page, t->generation);
    }
    t->live_tokens = new_len;
    return FLAT_OK;
}

// returns 1 and fills out[3] = (physical_page, offset_in_page, generation), or 0 for None.
int32_t flat_oracle_paged_table_address(const flat_oracle_paged_table *t, uint64_t logical_token,
                                        uint64_t *out) {
    if (logical_token >= t->live_tokens) return 0;
    usize logical_page = logical_token / t->page_size;
    if (logical_page >= t->logical_pages.size()) return 0;
    auto e = t->logical_pages[logical_page];
    if (e.second != t->generation) return 0;
    out[0] = e.first;
    out[1] = logical_token % t->page_size;
    out[2] = e.second;
    return 1;
}

// out[6] = live_tokens, capacity_tokens, mapped_pages, free_pages, internal_fragmentation, generation
void flat_oracle_paged_table_telemetry(const flat_oracle_paged_table *t, uint64_t *out) {
    out[0] = t->live_tokens;
    out[1] = t->page_size * t->physical_pages;
    out[2] = t->logical_pages.size();
    out[3] = t->free_pages.size();
    out[4] = t->logical_pages.size() * t->page_size - t->live_tokens;
    out[5] = t->generation;
}

int32_t flat_oracle_paged_table_reset(flat_oracle_paged_table *t) {
    if (t->generation == std::numeric_limits<uint64_t>::max()) return FLAT_ERR_GENERATION_OVERFLOW;
    t->generation += 1;
    t->live_tokens = 0;
    t->logical_pages.clear();
    t->free_pages.clear();
    for (usize p = t->physical_pages; p-- > 0;) t->free_pages.push_back(p);
    return FLAT_OK;
}

}  // extern "C"
