// TEST INFRASTRUCTURE ONLY — never linked into, imported by or executed from the
// product library.  Only tests/, the smoke check and bench.py's CPU-baseline legs
// may load this file's shared object.
//
// CPU restatement ("port") of the reference's decoder-layer hot path, written from
// the reference's behaviour, one C-ABI function per reference function.  Every
// function names the reference file:line whose arithmetic and ordering it follows.
// Parity pin: tests/test_oracle.py checks each function here against the reference
// itself (oracle/_ref/libsfref.so, built from the unmodified sources) and against
// the golden fixtures under tests/golden/ that were generated from it.
//
// Built with -ffp-contract=off: every `a += b * c` below is a multiply rounded to
// float followed by an add rounded to float, in source order.  Where the reference
// uses explicit FMA intrinsics, std::fmaf is used here.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <numeric>
#include <thread>
#include <vector>

namespace {

constexpr float kNegInf = -std::numeric_limits<float>::infinity();

int host_threads() { return static_cast<int>(std::max(1U, std::thread::hardware_concurrency())); }

// Static row partition over host threads (test-speed only; no arithmetic depends on it).
template <class F>
void parallel_rows(long long rows, int threads, F&& body) {
    threads = static_cast<int>(std::clamp<long long>(threads <= 0 ? host_threads() : threads, 1,
                                                     std::max<long long>(1, rows)));
    if (threads == 1) { body(0LL, rows); return; }
    std::vector<std::thread> pool;
    const long long chunk = (rows + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        const long long begin = t * chunk, end = std::min(rows, begin + chunk);
        if (begin < end) pool.emplace_back([=, &body] { body(begin, end); });
    }
    for (auto& thread : pool) thread.join();
}

// 8-lane FMA dot product with the lane sums folded in lane order, then a scalar
// tail: the rounding sequence of dot_product, src/attention_compiler.cpp:74-94
// when AVX2+FMA are enabled.
float dot8(const float* a, const float* b, int n) {
    float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int i = 0;
    for (; i + 8 <= n; i += 8)
        for (int l = 0; l < 8; ++l) lanes[l] = std::fmaf(a[i + l], b[i + l], lanes[l]);
    float sum = 0.0F;
    for (int l = 0; l < 8; ++l) sum += lanes[l];
    for (; i < n; ++i) sum += a[i] * b[i];
    return sum;
}

// out[d] = fma(w, v[d], out[d]) on full 8-groups, mul+add on the tail:
// accumulate_value, src/attention_compiler.cpp:114-130.
void axpy8(float* out, const float* v, float w, int n) {
    int d = 0;
    for (; d + 8 <= n; d += 8)
        for (int l = 0; l < 8; ++l) out[d + l] = std::fmaf(w, v[d + l], out[d + l]);
    for (; d < n; ++d) out[d] += w * v[d];
}

float silu(float x) { return x / (1.0F + std::exp(-x)); }  // src/moe_compiler.cpp:51

}  // namespace

extern "C" {

struct orp_decoder_config {
    int batch, sequence, hidden, intermediate, query_heads, kv_heads, head_dim;
    float rms_epsilon, rope_theta;
    int causal, ffn_moe, experts, top_k, context_sequence;
};

struct orp_decoder_data {
    const float* input;
    const float* rms1_weight;
    const float* query_weight;
    const float* key_weight;
    const float* value_weight;
    const float* output_weight;
    const float* rms2_weight;
    const float* gate_weight;
    const float* up_weight;
    const float* down_weight;
    const float* router_weight;
    const float* w1;
    const float* w3;
    const float* w2;
    const float* cached_key;
    const float* cached_value;
    const int* trace_expert_ids;
    const float* trace_expert_weights;
    const int* trace_counts;
};

struct orp_attention_config {
    int batch, query_heads, kv_heads, sequence_query, sequence_kv, head_dim, head_dim_value;
    int causal;
    float scale;
};

struct orp_moe_config {
    int tokens, hidden, intermediate, experts, top_k;
};

int orp_hardware_threads() { return host_threads(); }

// Round-to-nearest-even float -> bf16 -> float, bit trick `bits + 0x7FFF + lsb`:
// convert_to_bf16 / convert_from_bf16, src/compiler.cpp:34-52.
void orp_round_bf16(float* values, long long count) {
    for (long long i = 0; i < count; ++i) {
        std::uint32_t bits;
        std::memcpy(&bits, &values[i], 4);
        bits = (bits + 0x7FFFU + ((bits >> 16) & 1U)) & 0xFFFF0000U;
        std::memcpy(&values[i], &bits, 4);
    }
}

// RMSNorm with the sum of squares in double: rms_norm, src/decoder_compiler.cpp:41-62.
void orp_rms_norm(const float* input, const float* weight, int rows, int width, float epsilon,
                  float* output) {
    for (int r = 0; r < rows; ++r) {
        const float* x = input + static_cast<std::size_t>(r) * width;
        double ss = 0.0;
        for (int c = 0; c < width; ++c) ss += static_cast<double>(x[c]) * x[c];
        const float inv = 1.0F / std::sqrt(static_cast<float>(ss / static_cast<double>(width)) + epsilon);
        for (int c = 0; c < width; ++c)
            output[static_cast<std::size_t>(r) * width + c] = x[c] * inv * weight[c];
    }
}

// C[m,n] = A[m,k] . B[k,n], row-major, one accumulator per output over ascending k.
// fma == 0: multiply then add, scalar_matmul, src/decoder_compiler.cpp:64-75.
// fma != 0: the native GEMM's arithmetic: the first floor(n/8)*8 columns are AVX2 register
//           kernels = one single-rounding FMA chain per output (src/runtime.cpp:278-370, hot
//           loop :332-347; src/moe_compiler.cpp:77-101), the remaining n%8 tail columns are
//           a scalar multiply-then-add loop (src/runtime.cpp:420-432; src/moe_compiler.cpp:105-117).
void orp_matmul(const float* a, const float* b, float* c, int m, int n, int k, int fma,
                int threads) {
    const int n_fma = fma ? n / 8 * 8 : 0;
    parallel_rows(m, threads, [&](long long begin, long long end) {
        std::vector<float> acc(static_cast<std::size_t>(n));
        for (long long i = begin; i < end; ++i) {
            std::fill(acc.begin(), acc.end(), 0.0F);
            for (int r = 0; r < k; ++r) {
                const float x = a[i * k + r];
                const float* brow = b + static_cast<std::size_t>(r) * n;
                for (int j = 0; j < n_fma; ++j) acc[j] = std::fmaf(x, brow[j], acc[j]);
                for (int j = n_fma; j < n; ++j) acc[j] += x * brow[j];
            }
            std::memcpy(c + i * n, acc.data(), static_cast<std::size_t>(n) * 4);
        }
    });
}

// Interleaved-pair rotary embedding on a head-major [batch, heads, sequence, dim]
// tensor; positions restart at 0 for each batch element:
// apply_rope, src/decoder_compiler.cpp:96-114.
void orp_apply_rope(float* tensor, int batch, int heads, int sequence, int dim, float theta) {
    for (int b = 0; b < batch; ++b)
        for (int h = 0; h < heads; ++h)
            for (int t = 0; t < sequence; ++t)
                for (int d = 0; d + 1 < dim; d += 2) {
                    const float freq = std::pow(theta, -static_cast<float>(d) / static_cast<float>(dim));
                    const float angle = static_cast<float>(t) * freq;
                    const float co = std::cos(angle), si = std::sin(angle);
                    float* p = tensor + ((static_cast<std::size_t>(b) * heads + h) * sequence + t) * dim + d;
                    const float even = p[0], odd = p[1];
                    p[0] = even * co - odd * si;
                    p[1] = even * si + odd * co;
                }
}

// Fused [T, H + 2*kv] projection -> head-major Q [B,Hq,S,D], K and V [B,Hkv,S,D],
// RoPE on Q and K only: split_qkv, src/decoder_compiler.cpp:116-148.
void orp_split_qkv_rope(const orp_decoder_config* c, const float* fused, float* q, float* k,
                        float* v) {
    const int kvw = c->kv_heads * c->head_dim, total = c->hidden + 2 * kvw, d = c->head_dim;
    for (int b = 0; b < c->batch; ++b)
        for (int t = 0; t < c->sequence; ++t) {
            const float* row = fused + static_cast<std::size_t>(b * c->sequence + t) * total;
            for (int h = 0; h < c->query_heads; ++h)
                std::memcpy(q + ((static_cast<std::size_t>(b) * c->query_heads + h) * c->sequence + t) * d,
                            row + h * d, static_cast<std::size_t>(d) * 4);
            for (int h = 0; h < c->kv_heads; ++h) {
                const std::size_t dst = ((static_cast<std::size_t>(b) * c->kv_heads + h) * c->sequence + t) * d;
                std::memcpy(k + dst, row + c->hidden + h * d, static_cast<std::size_t>(d) * 4);
                std::memcpy(v + dst, row + c->hidden + kvw + h * d, static_cast<std::size_t>(d) * 4);
            }
        }
    orp_apply_rope(q, c->batch, c->query_heads, c->sequence, d, c->rope_theta);
    orp_apply_rope(k, c->batch, c->kv_heads, c->sequence, d, c->rope_theta);
}

// [B,Hq,S,D] -> [T, Hq*D]: merge_attention, src/decoder_compiler.cpp:150-174.
void orp_merge_heads(const orp_decoder_config* c, const float* attention, float* merged) {
    const int d = c->head_dim;
    for (int b = 0; b < c->batch; ++b)
        for (int h = 0; h < c->query_heads; ++h)
            for (int t = 0; t < c->sequence; ++t)
                std::memcpy(merged + static_cast<std::size_t>(b * c->sequence + t) * c->hidden + h * d,
                            attention + ((static_cast<std::size_t>(b) * c->query_heads + h) * c->sequence + t) * d,
                            static_cast<std::size_t>(d) * 4);
}

// gate = first I columns, up = last I columns: swiglu, src/decoder_compiler.cpp:183-194.
void orp_swiglu(const float* gate_up, int rows, int intermediate, float* output) {
    for (int r = 0; r < rows; ++r)
        for (int j = 0; j < intermediate; ++j) {
            const float g = gate_up[static_cast<std::size_t>(r) * 2 * intermediate + j];
            const float u = gate_up[static_cast<std::size_t>(r) * 2 * intermediate + intermediate + j];
            output[static_cast<std::size_t>(r) * intermediate + j] = g / (1.0F + std::exp(-g)) * u;
        }
}

// ---- attention --------------------------------------------------------------------

static float scale_of(const orp_attention_config* c) {  // src/attention_compiler.cpp:43-46
    return c->scale > 0.0F ? c->scale : 1.0F / std::sqrt(static_cast<float>(c->head_dim));
}

static bool visible(const orp_attention_config* c, int q, int key) {  // :68-72
    return !c->causal || key <= c->sequence_kv - c->sequence_query + q;
}

// Exact two-pass softmax attention, GQA head map kv = head*Hkv/Hq:
// reference_attention, src/attention_compiler.cpp:742-781.
void orp_attention_reference(const orp_attention_config* c, const float* q, const float* k,
                             const float* v, float* out, int threads) {
    const int Sq = c->sequence_query, Sk = c->sequence_kv, D = c->head_dim, Dv = c->head_dim_value;
    const float scale = scale_of(c);
    const long long rows = static_cast<long long>(c->batch) * c->query_heads * Sq;
    parallel_rows(rows, threads, [&](long long begin, long long end) {
        for (long long row = begin; row < end; ++row) {
            const int qt = static_cast<int>(row % Sq);
            const int head = static_cast<int>((row / Sq) % c->query_heads);
            const int b = static_cast<int>(row / Sq / c->query_heads);
            const int kvh = head * c->kv_heads / c->query_heads;
            const float* qrow = q + row * D;
            const float* kbase = k + (static_cast<std::size_t>(b) * c->kv_heads + kvh) * Sk * D;
            const float* vbase = v + (static_cast<std::size_t>(b) * c->kv_heads + kvh) * Sk * Dv;
            float* o = out + row * Dv;
            std::fill(o, o + Dv, 0.0F);
            float mx = kNegInf;
            for (int key = 0; key < Sk; ++key)
                if (visible(c, qt, key)) mx = std::max(mx, dot8(qrow, kbase + static_cast<std::size_t>(key) * D, D) * scale);
            float den = 0.0F;
            for (int key = 0; key < Sk; ++key) {
                if (!visible(c, qt, key)) continue;
                const float p = std::exp(dot8(qrow, kbase + static_cast<std::size_t>(key) * D, D) * scale - mx);
                den += p;
                axpy8(o, vbase + static_cast<std::size_t>(key) * Dv, p, Dv);
            }
            for (int d = 0; d < Dv; ++d) o[d] /= den;
        }
    });
}

// Materialized strategy: full score matrix, row max, probabilities normalised by the
// row sum BEFORE the PV product (plain multiply-add): execute_materialized,
// src/attention_compiler.cpp:170-237.
void orp_attention_materialized(const orp_attention_config* c, const float* q, const float* k,
                                const float* v, float* out) {
    const int Sq = c->sequence_query, Sk = c->sequence_kv, D = c->head_dim, Dv = c->head_dim_value;
    const float scale = scale_of(c);
    std::vector<float> scores(Sk), probs(Sk);
    for (int b = 0; b < c->batch; ++b)
        for (int head = 0; head < c->query_heads; ++head) {
            const int kvh = head * c->kv_heads / c->query_heads;
            const float* kbase = k + (static_cast<std::size_t>(b) * c->kv_heads + kvh) * Sk * D;
            const float* vbase = v + (static_cast<std::size_t>(b) * c->kv_heads + kvh) * Sk * Dv;
            for (int qt = 0; qt < Sq; ++qt) {
                const std::size_t row = (static_cast<std::size_t>(b) * c->query_heads + head) * Sq + qt;
                float mx = kNegInf;
                for (int key = 0; key < Sk; ++key) {
                    scores[key] = visible(c, qt, key)
                        ? dot8(q + row * D, kbase + static_cast<std::size_t>(key) * D, D) * scale : kNegInf;
                    mx = std::max(mx, scores[key]);
                }
                float den = 0.0F;
                for (int key = 0; key < Sk; ++key) {
                    probs[key] = std::isfinite(scores[key]) ? std::exp(scores[key] - mx) : 0.0F;
                    den += probs[key];
                }
                float* o = out + row * Dv;
                std::fill(o, o + Dv, 0.0F);
                for (int key = 0; key < Sk; ++key) {
                    const float pr = probs[key] / den;
                    for (int d = 0; d < Dv; ++d) o[d] += pr * vbase[static_cast<std::size_t>(key) * Dv + d];
                }
            }
        }
}

// IO-aware tiled online softmax (per query tile x key tile, causal tile skip, rows
// whose tile is fully masked skipped): execute_streaming, IO-aware branch,
// src/attention_compiler.cpp:286-376.
void orp_attention_io_aware(const orp_attention_config* c, int query_tile, int kv_tile,
                            const float* q, const float* k, const float* v, float* out,
                            int threads) {
    const int Sq = c->sequence_query, Sk = c->sequence_kv, D = c->head_dim, Dv = c->head_dim_value;
    query_tile = std::clamp(query_tile, 1, Sq);
    kv_tile = std::clamp(kv_tile, 1, Sk);
    const int qblocks = (Sq + query_tile - 1) / query_tile;
    const float scale = scale_of(c);
    const long long tasks = static_cast<long long>(c->batch) * c->query_heads * qblocks;
    parallel_rows(tasks, threads, [&](long long begin, long long end) {
        std::vector<float> mx, den, num, scores;
        for (long long task = begin; task < end; ++task) {
            const int qb = static_cast<int>(task % qblocks);
            const int head = static_cast<int>((task / qblocks) % c->query_heads);
            const int b = static_cast<int>(task / qblocks / c->query_heads);
            const int q0 = qb * query_tile, q1 = std::min(q0 + query_tile, Sq), nq = q1 - q0;
            const int kvh = head * c->kv_heads / c->query_heads;
            const float* kbase = k + (static_cast<std::size_t>(b) * c->kv_heads + kvh) * Sk * D;
            const float* vbase = v + (static_cast<std::size_t>(b) * c->kv_heads + kvh) * Sk * Dv;
            mx.assign(nq, kNegInf);
            den.assign(nq, 0.0F);
            num.assign(static_cast<std::size_t>(nq) * Dv, 0.0F);
            scores.assign(static_cast<std::size_t>(nq) * kv_tile, 0.0F);
            for (int k0 = 0; k0 < Sk; k0 += kv_tile) {
                if (c->causal && k0 > Sk - Sq + q1 - 1) break;
                const int nk = std::min(k0 + kv_tile, Sk) - k0;
                for (int lq = 0; lq < nq; ++lq) {
                    const int qt = q0 + lq;
                    const float* qrow = q + ((static_cast<std::size_t>(b) * c->query_heads + head) * Sq + qt) * D;
                    float bmax = kNegInf;
                    for (int lk = 0; lk < nk; ++lk) {
                        float s = kNegInf;
                        if (visible(c, qt, k0 + lk))
                            s = dot8(qrow, kbase + static_cast<std::size_t>(k0 + lk) * D, D) * scale;
                        scores[static_cast<std::size_t>(lq) * kv_tile + lk] = s;
                        bmax = std::max(bmax, s);
                    }
                    if (!std::isfinite(bmax)) continue;
                    const float nmax = std::max(mx[lq], bmax);
                    const float old = std::isfinite(mx[lq]) ? std::exp(mx[lq] - nmax) : 0.0F;
                    den[lq] *= old;
                    float* o = num.data() + static_cast<std::size_t>(lq) * Dv;
                    for (int d = 0; d < Dv; ++d) o[d] *= old;
                    for (int lk = 0; lk < nk; ++lk) {
                        const float s = scores[static_cast<std::size_t>(lq) * kv_tile + lk];
                        if (!std::isfinite(s)) continue;
                        const float p = std::exp(s - nmax);
                        den[lq] += p;
                        axpy8(o, vbase + static_cast<std::size_t>(k0 + lk) * Dv, p, Dv);
                    }
                    mx[lq] = nmax;
                }
            }
            for (int lq = 0; lq < nq; ++lq)
                for (int d = 0; d < Dv; ++d)
                    out[((static_cast<std::size_t>(b) * c->query_heads + head) * Sq + q0 + lq) * Dv + d] =
                        num[static_cast<std::size_t>(lq) * Dv + d] / den[lq];
        }
    });
}

namespace {
struct Online {
    float mx = kNegInf, den = 0.0F;
    std::vector<float> num;
};
}  // namespace

// Split-KV decode: per (row, split) a per-key online-softmax partial over keys
// [Sk*s/n, Sk*(s+1)/n), then an exact log-sum-exp merge in split order with empty
// splits skipped: execute_streaming split-KV branch, src/attention_compiler.cpp:244-285,
// compute_range :147-168, update_online :102-112, merge_online :132-145.
void orp_attention_split_kv(const orp_attention_config* c, int splits, int kv_tile,
                            const float* q, const float* k, const float* v, float* out,
                            int threads) {
    const int Sq = c->sequence_query, Sk = c->sequence_kv, D = c->head_dim, Dv = c->head_dim_value;
    splits = std::max(1, splits);
    kv_tile = std::max(1, kv_tile);
    const float scale = scale_of(c);
    const long long rows = static_cast<long long>(c->batch) * c->query_heads * Sq;
    parallel_rows(rows, threads, [&](long long begin, long long end) {
        for (long long row = begin; row < end; ++row) {
            const int qt = static_cast<int>(row % Sq);
            const int head = static_cast<int>((row / Sq) % c->query_heads);
            const int b = static_cast<int>(row / Sq / c->query_heads);
            const int kvh = head * c->kv_heads / c->query_heads;
            const float* qrow = q + row * D;
            const float* kbase = k + (static_cast<std::size_t>(b) * c->kv_heads + kvh) * Sk * D;
            const float* vbase = v + (static_cast<std::size_t>(b) * c->kv_heads + kvh) * Sk * Dv;
            std::vector<Online> parts(splits);
            for (int s = 0; s < splits; ++s) {
                Online& st = parts[s];
                st.num.assign(Dv, 0.0F);
                const int kb = static_cast<int>(static_cast<long long>(Sk) * s / splits);
                const int ke = static_cast<int>(static_cast<long long>(Sk) * (s + 1) / splits);
                for (int k0 = kb; k0 < ke; k0 += kv_tile) {
                    if (c->causal && k0 > Sk - Sq + qt) break;
                    for (int key = k0; key < std::min(k0 + kv_tile, ke); ++key) {
                        if (!visible(c, qt, key)) continue;
                        const float score = dot8(qrow, kbase + static_cast<std::size_t>(key) * D, D) * scale;
                        const float nmax = std::max(st.mx, score);
                        const float old = std::isfinite(st.mx) ? std::exp(st.mx - nmax) : 0.0F;
                        const float p = std::exp(score - nmax);
                        st.den = st.den * old + p;
                        const float* vrow = vbase + static_cast<std::size_t>(key) * Dv;
                        for (int d = 0; d < Dv; ++d) st.num[d] = st.num[d] * old + p * vrow[d];
                        st.mx = nmax;
                    }
                }
            }
            Online acc = parts[0];
            for (int s = 1; s < splits; ++s) {
                const Online& rhs = parts[s];
                if (!std::isfinite(acc.mx)) { acc = rhs; continue; }
                if (!std::isfinite(rhs.mx)) continue;
                Online merged;
                merged.mx = std::max(acc.mx, rhs.mx);
                const float ls = std::exp(acc.mx - merged.mx), rs = std::exp(rhs.mx - merged.mx);
                merged.den = acc.den * ls + rhs.den * rs;
                merged.num.resize(Dv);
                for (int d = 0; d < Dv; ++d) merged.num[d] = acc.num[d] * ls + rhs.num[d] * rs;
                acc = std::move(merged);
            }
            for (int d = 0; d < Dv; ++d) out[row * Dv + d] = acc.num[d] / acc.den;
        }
    });
}

// ---- paged KV cache -----------------------------------------------------------------
// Storage keys[(((page*B + b)*Hkv + h)*P + t)*D + d] (src/next_milestones.cpp:29-33); one
// page table and one length for the whole batch; pages are taken from the BACK of the
// free list (make_paged_kv_cache :472-484, append_paged_kv :486-524, release :526-538,
// truncate :540-550, gather :552-581).

struct orp_paged {
    int batch, kv_heads, dim, dim_v, page_tokens, capacity, length;
    std::vector<int> table, free_pages;
    std::vector<float> keys, values;
    std::size_t at(int page, int b, int h, int t, int width) const {
        return (((static_cast<std::size_t>(page) * batch + b) * kv_heads + h) * page_tokens + t) * width;
    }
    int pages() const { return (capacity + page_tokens - 1) / page_tokens; }
};

orp_paged* orp_paged_create(int batch, int kv_heads, int dim, int dim_v, int page_tokens,
                            int capacity) {
    if (batch <= 0 || kv_heads <= 0 || dim <= 0 || dim_v <= 0 || page_tokens <= 0 || capacity <= 0)
        return nullptr;  // "invalid paged KV configuration", :23-27
    auto* p = new orp_paged{batch, kv_heads, dim, dim_v, page_tokens, capacity, 0, {}, {}, {}, {}};
    p->free_pages.resize(p->pages());
    std::iota(p->free_pages.begin(), p->free_pages.end(), 0);
    const std::size_t page_rows = static_cast<std::size_t>(batch) * kv_heads * page_tokens;
    p->keys.assign(p->pages() * page_rows * dim, 0.0F);
    p->values.assign(p->pages() * page_rows * dim_v, 0.0F);
    return p;
}

void orp_paged_destroy(orp_paged* p) { delete p; }

void orp_paged_set_free_pages(orp_paged* p, const int* pages, int count) {
    p->free_pages.assign(pages, pages + count);
}

// Returns 0, 1 (invalid argument: capacity exceeded) or 2 (allocator exhausted).
// keys/values are [batch][kv_head][tokens][dim].
int orp_paged_append(orp_paged* p, const float* keys, const float* values, int tokens) {
    if (tokens <= 0 || p->length + tokens > p->capacity) return 1;
    const int last_page = (p->length + tokens - 1) / p->page_tokens;
    while (static_cast<int>(p->table.size()) <= last_page) {
        if (p->free_pages.empty()) return 2;
        p->table.push_back(p->free_pages.back());
        p->free_pages.pop_back();
    }
    for (int t = 0; t < tokens; ++t) {
        const int logical = p->length + t;
        const int page = p->table[logical / p->page_tokens], slot = logical % p->page_tokens;
        for (int b = 0; b < p->batch; ++b)
            for (int h = 0; h < p->kv_heads; ++h) {
                const std::size_t src = (static_cast<std::size_t>(b) * p->kv_heads + h) * tokens + t;
                std::memcpy(&p->keys[p->at(page, b, h, slot, p->dim)], keys + src * p->dim,
                            static_cast<std::size_t>(p->dim) * 4);
                std::memcpy(&p->values[p->at(page, b, h, slot, p->dim_v)], values + src * p->dim_v,
                            static_cast<std::size_t>(p->dim_v) * 4);
            }
    }
    p->length += tokens;
    return 0;
}

int orp_paged_truncate(orp_paged* p, int new_length) {
    if (new_length < 0 || new_length > p->length) return 1;
    const int keep = new_length == 0 ? 0 : (new_length + p->page_tokens - 1) / p->page_tokens;
    while (static_cast<int>(p->table.size()) > keep) {
        p->free_pages.push_back(p->table.back());
        p->table.pop_back();
    }
    p->length = new_length;
    return 0;
}

int orp_paged_release(orp_paged* p, const int* pages, int count) {
    for (int i = 0; i < count; ++i) {
        const int page = pages[i];
        if (page < 0 || page >= p->pages()) return 1;
        if (std::find(p->table.begin(), p->table.end(), page) != p->table.end()) return 1;
        if (std::find(p->free_pages.begin(), p->free_pages.end(), page) == p->free_pages.end())
            p->free_pages.push_back(page);
    }
    return 0;
}

void orp_paged_info(const orp_paged* p, int* info, int* table, int table_capacity,
                    int* free_pages, int free_capacity) {
    info[0] = p->length;
    info[1] = static_cast<int>(p->table.size());
    info[2] = static_cast<int>(p->free_pages.size());
    info[3] = p->pages();
    for (int i = 0; i < info[1] && i < table_capacity; ++i) table[i] = p->table[i];
    for (int i = 0; i < info[2] && i < free_capacity; ++i) free_pages[i] = p->free_pages[i];
}

void orp_paged_storage(const orp_paged* p, float* keys, float* values) {
    std::memcpy(keys, p->keys.data(), p->keys.size() * 4);
    std::memcpy(values, p->values.data(), p->values.size() * 4);
}

// -> [batch][kv_head][length][dim]; returns 1 when the cache is empty.
int orp_paged_gather(const orp_paged* p, float* keys, float* values) {
    if (p->length <= 0) return 1;
    for (int t = 0; t < p->length; ++t) {
        const int page = p->table[t / p->page_tokens], slot = t % p->page_tokens;
        for (int b = 0; b < p->batch; ++b)
            for (int h = 0; h < p->kv_heads; ++h) {
                const std::size_t dst = (static_cast<std::size_t>(b) * p->kv_heads + h) * p->length + t;
                std::memcpy(keys + dst * p->dim, &p->keys[p->at(page, b, h, slot, p->dim)],
                            static_cast<std::size_t>(p->dim) * 4);
                std::memcpy(values + dst * p->dim_v, &p->values[p->at(page, b, h, slot, p->dim_v)],
                            static_cast<std::size_t>(p->dim_v) * 4);
            }
    }
    return 0;
}

// Direct paged decode, per-key online softmax in logical key order with a plain
// scalar dot product (two_pass == 0: paged_attention_online,
// src/next_milestones.cpp:137-184; two_pass != 0: paged_attention_reference :186-231).
// Guards of validate_paged_attention (:98-120) return 1.
int orp_paged_decode(const orp_paged* p, const orp_attention_config* c, const float* query,
                     float* out, int two_pass) {
    if (p->length <= 0 || p->length > c->sequence_kv) return 1;
    if (c->causal && c->sequence_query > p->length) return 1;
    if (p->batch != c->batch || p->kv_heads != c->kv_heads || p->dim != c->head_dim ||
        p->dim_v != c->head_dim_value || c->query_heads % c->kv_heads != 0)
        return 1;
    if (static_cast<int>(p->table.size()) < (p->length + p->page_tokens - 1) / p->page_tokens) return 1;
    const int Sq = c->sequence_query, D = c->head_dim, Dv = c->head_dim_value;
    const float scale = scale_of(c);
    const auto sdot = [&](const float* a, const float* b) {
        float r = 0.0F;
        for (int i = 0; i < D; ++i) r += a[i] * b[i];
        return r;
    };
    const auto kptr = [&](int b, int h, int t) {
        return &p->keys[p->at(p->table[t / p->page_tokens], b, h, t % p->page_tokens, D)];
    };
    const auto vptr = [&](int b, int h, int t) {
        return &p->values[p->at(p->table[t / p->page_tokens], b, h, t % p->page_tokens, Dv)];
    };
    std::vector<float> num(Dv);
    for (int b = 0; b < c->batch; ++b)
        for (int head = 0; head < c->query_heads; ++head) {
            const int kvh = head * c->kv_heads / c->query_heads;
            for (int qt = 0; qt < Sq; ++qt) {
                const std::size_t row = (static_cast<std::size_t>(b) * c->query_heads + head) * Sq + qt;
                const float* qrow = query + row * D;
                const int frontier = p->length - Sq + qt;
                float* o = out + row * Dv;
                if (!two_pass) {
                    float mx = kNegInf, den = 0.0F;
                    std::fill(num.begin(), num.end(), 0.0F);
                    for (int key = 0; key < p->length; ++key) {
                        if (c->causal && key > frontier) continue;
                        const float score = sdot(qrow, kptr(b, kvh, key)) * scale;
                        const float nmax = std::max(mx, score);
                        const float old = std::isfinite(mx) ? std::exp(mx - nmax) : 0.0F;
                        const float pr = std::exp(score - nmax);
                        den = den * old + pr;
                        const float* vrow = vptr(b, kvh, key);
                        for (int d = 0; d < Dv; ++d) num[d] = num[d] * old + pr * vrow[d];
                        mx = nmax;
                    }
                    for (int d = 0; d < Dv; ++d) o[d] = num[d] / den;
                } else {
                    float mx = kNegInf;
                    for (int key = 0; key < p->length; ++key)
                        if (!(c->causal && key > frontier))
                            mx = std::max(mx, sdot(qrow, kptr(b, kvh, key)) * scale);
                    float den = 0.0F;
                    std::fill(o, o + Dv, 0.0F);
                    for (int key = 0; key < p->length; ++key) {
                        if (c->causal && key > frontier) continue;
                        const float pr = std::exp(sdot(qrow, kptr(b, kvh, key)) * scale - mx);
                        den += pr;
                        const float* vrow = vptr(b, kvh, key);
                        for (int d = 0; d < Dv; ++d) o[d] += pr * vrow[d];
                    }
                    for (int d = 0; d < Dv; ++d) o[d] /= den;
                }
            }
        }
    return 0;
}

// ---- MoE ----------------------------------------------------------------------------

// Router logits as a sequential float sum over features (multiply, then add), softmax
// numerators p = exp(logit - max), top-k by partial_sort on p descending over an index
// vector that is iota ONCE and then carried (already permuted) from token to token, gate
// weights (p/den)/sum_selected(p/den), histogram in the same loop:
// route_topk, src/moe_compiler.cpp:412-455.
// `bias` (may be null) adds one term `+ bias[e]` after the feature sum; the reference has
// no such term, so results with a bias are a restatement without a reference pin.
// tie_tokens (may be null) receives the number of tokens for which two experts on either
// side of a selection boundary have bit-identical p (order then depends on history).
void orp_route_topk(const orp_moe_config* c, const float* input, int tokens,
                    const float* router_weight, const float* bias, int* expert_ids,
                    float* expert_weights, int* counts, int* tie_tokens) {
    const int H = c->hidden, E = c->experts, K = c->top_k;
    std::fill(counts, counts + E, 0);
    std::vector<float> p(E);
    std::vector<int> order(E);
    std::iota(order.begin(), order.end(), 0);
    int ties = 0;
    for (int t = 0; t < tokens; ++t) {
        float mx = kNegInf;
        for (int e = 0; e < E; ++e) {
            float logit = 0.0F;
            for (int f = 0; f < H; ++f)
                logit += input[static_cast<std::size_t>(t) * H + f] * router_weight[static_cast<std::size_t>(f) * E + e];
            if (bias) logit += bias[e];
            p[e] = logit;
            mx = std::max(mx, logit);
        }
        float den = 0.0F;
        for (float& value : p) { value = std::exp(value - mx); den += value; }
        std::partial_sort(order.begin(), order.begin() + K, order.end(),
                          [&](int l, int r) { return p[l] > p[r]; });
        bool tie = false;
        for (int s = 0; s < K && !tie; ++s)
            for (int e = 0; e < E; ++e) {
                bool later = true;
                for (int s2 = 0; s2 <= s; ++s2) later = later && order[s2] != e;
                if (later && p[e] == p[order[s]]) { tie = true; break; }
            }
        ties += tie;
        float selected = 0.0F;
        for (int s = 0; s < K; ++s) selected += p[order[s]] / den;
        for (int s = 0; s < K; ++s) {
            const int e = order[s];
            expert_ids[static_cast<std::size_t>(t) * K + s] = e;
            expert_weights[static_cast<std::size_t>(t) * K + s] = (p[e] / den) / selected;
            ++counts[e];
        }
    }
    if (tie_tokens) *tie_tokens = ties;
}

// offsets[0] = 0, offsets[e+1] = offsets[e] + counts[e]: src/moe_compiler.cpp:504-507.
void orp_prefix_sum(const int* counts, int experts, int* offsets) {
    offsets[0] = 0;
    for (int e = 0; e < experts; ++e) offsets[e + 1] = offsets[e] + counts[e];
}

// Stable counting-sort scatter in (token, slot) order, dest = cursor[expert]++:
// dispatch_tokens, src/moe_compiler.cpp:496-528.  `values` may be null.
void orp_dispatch_tokens(const orp_moe_config* c, const float* input, int tokens,
                         const int* expert_ids, const float* expert_weights, const int* counts,
                         float* values, int* offsets, int* token_ids, int* route_slots,
                         float* routing_weights) {
    const int H = c->hidden, E = c->experts, K = c->top_k;
    orp_prefix_sum(counts, E, offsets);
    std::vector<int> cursor(offsets, offsets + E);
    for (int t = 0; t < tokens; ++t)
        for (int s = 0; s < K; ++s) {
            const std::size_t r = static_cast<std::size_t>(t) * K + s;
            const int dst = cursor[expert_ids[r]]++;
            if (values)
                std::memcpy(values + static_cast<std::size_t>(dst) * H, input + static_cast<std::size_t>(t) * H,
                            static_cast<std::size_t>(H) * 4);
            token_ids[dst] = t;
            route_slots[dst] = s;
            routing_weights[dst] = expert_weights[r];
        }
}

// Token-bucket task table: default buckets {4,16,64} plus T, LoadAwareSplit chunks of
// split_threshold rows, big-first stable sort: plan_moe_tasks,
// src/moe_compiler.cpp:530-558; bucket_for :53-56; bucket sanitising :766-772.
// tasks rows = (expert, begin, end, bucket).
int orp_plan_moe_tasks(const orp_moe_config* c, const int* counts, int split_threshold,
                       int* tasks, int capacity) {
    std::vector<int> buckets = {4, 16, 64};
    if (buckets.back() < c->tokens) buckets.push_back(c->tokens);
    if (split_threshold <= 0) split_threshold = 32;
    struct Task { int expert, begin, end, bucket; };
    std::vector<Task> planned;
    int offset = 0;
    for (int e = 0; e < c->experts; ++e) {
        const int count = counts[e], begin0 = offset, end0 = offset + count;
        offset = end0;
        if (count == 0) continue;
        const int chunk = count > split_threshold ? std::max(1, split_threshold) : count;
        for (int b = begin0; b < end0; b += chunk) {
            const int en = std::min(b + chunk, end0);
            int bucket = std::max(en - b, buckets.back());
            for (const int candidate : buckets) if (en - b <= candidate) { bucket = candidate; break; }
            planned.push_back({e, b, en, bucket});
        }
    }
    std::stable_sort(planned.begin(), planned.end(), [](const Task& l, const Task& r) {
        return l.end - l.begin > r.end - r.begin;
    });
    for (std::size_t i = 0; i < planned.size() && static_cast<int>(i) < capacity; ++i) {
        tasks[4 * i] = planned[i].expert;
        tasks[4 * i + 1] = planned[i].begin;
        tasks[4 * i + 2] = planned[i].end;
        tasks[4 * i + 3] = planned[i].bucket;
    }
    return static_cast<int>(planned.size());
}

// Scalar MoE reference per (token, slot): h = x.W1[e], g = silu(x.W3[e]),
// y = (h*g).W2[e], out[token] += w*y in slot order: reference_moe,
// src/moe_compiler.cpp:645-682.  Weights w1,w3 [E,H,I], w2 [E,I,H].
void orp_moe_reference(const orp_moe_config* c, const float* input, int tokens, const float* w1,
                       const float* w3, const float* w2, const int* expert_ids,
                       const float* expert_weights, float* out, int threads) {
    const int H = c->hidden, I = c->intermediate, K = c->top_k;
    std::fill(out, out + static_cast<std::size_t>(tokens) * H, 0.0F);
    parallel_rows(tokens, threads, [&](long long begin, long long end) {
        std::vector<float> first(I), third(I), value(H);
        for (long long t = begin; t < end; ++t)
            for (int s = 0; s < K; ++s) {
                const int e = expert_ids[t * K + s];
                const float w = expert_weights[t * K + s];
                const float* x = input + t * H;
                std::fill(first.begin(), first.end(), 0.0F);
                std::fill(third.begin(), third.end(), 0.0F);
                for (int f = 0; f < H; ++f) {
                    const float* r1 = w1 + (static_cast<std::size_t>(e) * H + f) * I;
                    const float* r3 = w3 + (static_cast<std::size_t>(e) * H + f) * I;
                    for (int i = 0; i < I; ++i) { first[i] += x[f] * r1[i]; third[i] += x[f] * r3[i]; }
                }
                for (int i = 0; i < I; ++i) third[i] = silu(third[i]);
                std::fill(value.begin(), value.end(), 0.0F);
                for (int i = 0; i < I; ++i) {
                    const float* r2 = w2 + (static_cast<std::size_t>(e) * I + i) * H;
                    const float hg = first[i] * third[i];
                    for (int f = 0; f < H; ++f) value[f] += hg * r2[f];
                }
                for (int f = 0; f < H; ++f) out[t * H + f] += w * value[f];
            }
    });
}

// Native grouped path: dispatch, per expert segment FMA-chain GEMMs
// (h = X.W1, g = X.W3, h *= silu(g), y = h.W2), then the weighted combine in
// dispatched (expert-major) order into a zeroed output: execute_once,
// src/moe_compiler.cpp:157-242 with compute_task :121-155 and the combine :219-226.
void orp_moe_grouped(const orp_moe_config* c, const float* input, int tokens, const float* w1,
                     const float* w3, const float* w2, const int* expert_ids,
                     const float* expert_weights, const int* counts, float* out, int threads) {
    const int H = c->hidden, I = c->intermediate, E = c->experts, K = c->top_k;
    const std::size_t assignments = static_cast<std::size_t>(tokens) * K;
    std::vector<float> x(assignments * H), h(assignments * I), g(assignments * I), y(assignments * H);
    std::vector<int> offsets(E + 1), token_ids(assignments), slots(assignments);
    std::vector<float> weights(assignments);
    orp_dispatch_tokens(c, input, tokens, expert_ids, expert_weights, counts, x.data(),
                        offsets.data(), token_ids.data(), slots.data(), weights.data());
    for (int e = 0; e < E; ++e) {
        const int rows = offsets[e + 1] - offsets[e];
        if (rows == 0) continue;
        const std::size_t r0 = offsets[e];
        orp_matmul(x.data() + r0 * H, w1 + static_cast<std::size_t>(e) * H * I, h.data() + r0 * I, rows, I, H, 1, threads);
        orp_matmul(x.data() + r0 * H, w3 + static_cast<std::size_t>(e) * H * I, g.data() + r0 * I, rows, I, H, 1, threads);
        for (std::size_t i = r0 * I; i < (r0 + rows) * I; ++i) h[i] *= silu(g[i]);
        orp_matmul(h.data() + r0 * I, w2 + static_cast<std::size_t>(e) * I * H, y.data() + r0 * H, rows, H, I, 1, threads);
    }
    std::fill(out, out + static_cast<std::size_t>(tokens) * H, 0.0F);
    for (std::size_t a = 0; a < assignments; ++a)
        for (int f = 0; f < H; ++f)
            out[static_cast<std::size_t>(token_ids[a]) * H + f] += weights[a] * y[a * H + f];
}

// ---- whole decoder layer ----------------------------------------------------------------
// native == 0: the scalar layer reference (scalar GEMMs, two-pass attention, scalar MoE):
//              reference_decoder_layer, src/decoder_compiler.cpp:622-673.
// native != 0: the executed path (FMA-chain GEMMs, IO-aware or split-KV attention, grouped
//              MoE): execute_once, src/decoder_compiler.cpp:218-304.
// Decode (context_sequence > 0) attends over cached_key/value only; the new token's K/V
// are computed and dropped, and RoPE sees position 0 (:238-241, :640-645).
// normalized2_out (may be null) receives the FFN RMSNorm output [T,H].
void orp_decoder_layer(const orp_decoder_config* c, const orp_decoder_data* d, int native,
                       int threads, float* output, float* normalized2_out) {
    const int T = c->batch * c->sequence, H = c->hidden, I = c->intermediate;
    const int kvw = c->kv_heads * c->head_dim, QKV = H + 2 * kvw;
    std::vector<float> n1(static_cast<std::size_t>(T) * H);
    orp_rms_norm(d->input, d->rms1_weight, T, H, c->rms_epsilon, n1.data());
    std::vector<float> wqkv(static_cast<std::size_t>(H) * QKV);
    for (int r = 0; r < H; ++r) {  // concatenate_columns, :77-94
        std::memcpy(&wqkv[static_cast<std::size_t>(r) * QKV], d->query_weight + static_cast<std::size_t>(r) * H, static_cast<std::size_t>(H) * 4);
        std::memcpy(&wqkv[static_cast<std::size_t>(r) * QKV + H], d->key_weight + static_cast<std::size_t>(r) * kvw, static_cast<std::size_t>(kvw) * 4);
        std::memcpy(&wqkv[static_cast<std::size_t>(r) * QKV + H + kvw], d->value_weight + static_cast<std::size_t>(r) * kvw, static_cast<std::size_t>(kvw) * 4);
    }
    std::vector<float> qkv(static_cast<std::size_t>(T) * QKV);
    orp_matmul(n1.data(), wqkv.data(), qkv.data(), T, QKV, H, native, threads);
    const std::size_t qn = static_cast<std::size_t>(T) * H, kn = static_cast<std::size_t>(T) * kvw;
    std::vector<float> q(qn), k(kn), v(kn), attended(qn);
    orp_split_qkv_rope(c, qkv.data(), q.data(), k.data(), v.data());
    const int Sk = c->context_sequence > 0 ? c->context_sequence : c->sequence;
    orp_attention_config ac{c->batch, c->query_heads, c->kv_heads, c->sequence, Sk, c->head_dim,
                            c->head_dim, c->causal, 0.0F};
    const float* keys = c->context_sequence > 0 ? d->cached_key : k.data();
    const float* values = c->context_sequence > 0 ? d->cached_value : v.data();
    if (!native) {
        orp_attention_reference(&ac, q.data(), keys, values, attended.data(), threads);
    } else if (c->sequence <= 2) {  // select_attention_plan, src/attention_compiler.cpp:573-580
        const int t = threads <= 0 ? host_threads() : threads;
        const int splits = t > 1 ? std::clamp(std::max(2, Sk / 128), 2, t) : 1;
        orp_attention_split_kv(&ac, splits, Sk >= 1024 ? 128 : 64, q.data(), keys, values,
                               attended.data(), threads);
    } else if (c->sequence <= 16 && Sk <= 64) {  // :581-584
        orp_attention_materialized(&ac, q.data(), keys, values, attended.data());
    } else {  // :585-594 with the reference's default 1 MiB L2 figure
        const int query_tile = c->head_dim >= 128 ? 16 : 32;
        const std::size_t pair_bytes = static_cast<std::size_t>(c->head_dim * 3 + 1) * 4;
        int kv_tile = static_cast<int>(std::clamp<std::size_t>(
            (1024 * 1024) / (pair_bytes * query_tile), 16, 128));
        kv_tile = std::max(16, kv_tile / 16 * 16);
        orp_attention_io_aware(&ac, query_tile, kv_tile, q.data(), keys, values,
                               attended.data(), threads);
    }
    std::vector<float> merged(qn), r1(qn), n2(qn);
    orp_merge_heads(c, attended.data(), merged.data());
    orp_matmul(merged.data(), d->output_weight, r1.data(), T, H, H, native, threads);
    for (std::size_t i = 0; i < qn; ++i) r1[i] = r1[i] + d->input[i];  // add, :176-181
    orp_rms_norm(r1.data(), d->rms2_weight, T, H, c->rms_epsilon, n2.data());
    if (normalized2_out) std::memcpy(normalized2_out, n2.data(), qn * 4);
    std::vector<float> ffn(qn);
    if (!c->ffn_moe) {
        std::vector<float> wgu(static_cast<std::size_t>(H) * 2 * I);
        for (int r = 0; r < H; ++r) {
            std::memcpy(&wgu[static_cast<std::size_t>(r) * 2 * I], d->gate_weight + static_cast<std::size_t>(r) * I, static_cast<std::size_t>(I) * 4);
            std::memcpy(&wgu[static_cast<std::size_t>(r) * 2 * I + I], d->up_weight + static_cast<std::size_t>(r) * I, static_cast<std::size_t>(I) * 4);
        }
        std::vector<float> gu(static_cast<std::size_t>(T) * 2 * I), act(static_cast<std::size_t>(T) * I);
        orp_matmul(n2.data(), wgu.data(), gu.data(), T, 2 * I, H, native, threads);
        orp_swiglu(gu.data(), T, I, act.data());
        orp_matmul(act.data(), d->down_weight, ffn.data(), T, H, I, native, threads);
    } else {
        orp_moe_config mc{T, H, I, c->experts, c->top_k};
        std::vector<int> ids(static_cast<std::size_t>(T) * c->top_k), counts(c->experts);
        std::vector<float> weights(ids.size());
        if (d->trace_expert_ids && d->trace_expert_weights && d->trace_counts) {
            std::copy_n(d->trace_expert_ids, ids.size(), ids.begin());
            std::copy_n(d->trace_expert_weights, ids.size(), weights.begin());
            std::copy_n(d->trace_counts, counts.size(), counts.begin());
        } else {
            orp_route_topk(&mc, n2.data(), T, d->router_weight, nullptr, ids.data(), weights.data(),
                           counts.data(), nullptr);
        }
        if (native)
            orp_moe_grouped(&mc, n2.data(), T, d->w1, d->w3, d->w2, ids.data(), weights.data(),
                            counts.data(), ffn.data(), threads);
        else
            orp_moe_reference(&mc, n2.data(), T, d->w1, d->w3, d->w2, ids.data(), weights.data(),
                              ffn.data(), threads);
    }
    for (std::size_t i = 0; i < qn; ++i) output[i] = r1[i] + ffn[i];
}

}  // extern "C"
