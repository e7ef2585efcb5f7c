/*
 * attention_oracle.c -- CPU restatement of the f32 attention-side shaders that sit between the
 * qkv and o projections of a decoder layer: rotary embedding, scaled-dot-product attention,
 * attention over a contiguous KV cache, the cache append, and attention over a paged KV cache.
 *
 * TEST INFRASTRUCTURE ONLY, like qmatmul_oracle.c: nothing in the shipped library links or calls it.
 * PARITY UNPINNED: luxcpp/webgpu never dispatches these shaders and holds no test vector for them,
 * so the functions follow the shader text; each cites its lines (paths inside luxcpp/webgpu).
 * tests/test_oracle_attention.py checks them against an independent float64 softmax attention.
 * Built without contraction, so "a += b * c" is two roundings.
 *
 * Where the shader text and its evident intent part, the intent is restated and the place says so:
 *   - steel/attention/paged.wgsl reduces the workgroup's max and sum through partial_max[tid / 32]
 *     written only by the lanes with tid % 32 == 0 and with the warp-level step left empty
 *     (:112-131, :141-157), so 248 of the 256 threads' partial sums never reach the total, and
 *     it declares workgroup variables inside the function, which WGSL does not accept.  The
 *     restatement is the softmax over the whole context that the surrounding comments describe.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>

#define WG 256
#define NEG_INF_F (-3.402823e+38f)

/* exp(clamp(x, -88, 88)): gpu/scaled_dot_product_attention.wgsl:68-70, steel/attention/flash.wgsl:54-56 */
static float safe_exp(float x) {
    if (x < -88.0f) x = -88.0f;
    if (x > 88.0f) x = 88.0f;
    return expf(x);
}

/* ---- rotary embedding: gpu/rope.wgsl --------------------------------------------------------- */

/* compute_freq, rope.wgsl:56-60: pow(theta_base, -2 i / head_dim) with the exponent formed in f32.
 * The power itself is taken in double and rounded once, i.e. a correctly rounded f32 pow. */
float orc_rope_freq(uint32_t dim_pair, uint32_t head_dim, float theta_base) {
    const float exponent = -2.0f * (float)dim_pair / (float)head_dim;
    return (float)pow((double)theta_base, (double)exponent);
}

/* rope_precompute_cache, rope.wgsl:269-291: cos/sin[pos, head_dim/2] of f32(pos) * freq */
int orc_rope_precompute_cache(uint32_t max_seq_len, uint32_t head_dim, float theta_base, float* cos_out, float* sin_out) {
    if (head_dim == 0 || head_dim % 2) return -1;
    const uint32_t half = head_dim / 2;
    for (uint32_t pos = 0; pos < max_seq_len; pos++)
        for (uint32_t i = 0; i < half; i++) {
            const float angle = (float)pos * orc_rope_freq(i, head_dim, theta_base);
            cos_out[(size_t)pos * half + i] = cosf(angle);
            sin_out[(size_t)pos * half + i] = sinf(angle);
        }
    return 0;
}

/*
 * The rotation of rope_forward (:67-111), rope_forward_no_cache (:118-160), rope_inplace
 * (:167-203, out == in), rope_backward (:214-252), rope_ntk_scaled (:312-353),
 * rope_custom_positions (:359-397) and rope_qk_fused (:406-448, called once per tensor):
 *   x [batch, seq, heads, head_dim]; pairs are ADJACENT elements (2i, 2i + 1);
 *   position = position_ids[b * seq + s] if given, else position_offset + s;
 *   cos/sin from the cache at [position * head_dim/2 + i] if given, else of f32(position) * freq;
 *   forward:  out0 = x0 cos - x1 sin, out1 = x0 sin + x1 cos
 *   backward: out0 = x0 cos + x1 sin, out1 = -x0 sin + x1 cos
 * ntk_scale > 0: theta = theta_base * pow(ntk_scale, head_dim / (head_dim - 2)) and, as in the
 * shader, the angle uses the index in the sequence without the offset.
 */
int orc_rope(const float* x, float* out, const float* cos_cache, const float* sin_cache, const uint32_t* position_ids,
             uint32_t batch, uint32_t seq, uint32_t heads, uint32_t head_dim, float theta_base, uint32_t position_offset,
             float ntk_scale, int backward) {
    if (head_dim == 0 || head_dim % 2) return -1;
    const uint32_t half = head_dim / 2;
    float theta = theta_base;
    if (ntk_scale > 0.0f) theta = theta_base * powf(ntk_scale, (float)head_dim / ((float)head_dim - 2.0f));
    for (uint32_t b = 0; b < batch; b++)
        for (uint32_t s = 0; s < seq; s++) {
            uint32_t position = position_ids ? position_ids[(size_t)b * seq + s] : position_offset + s;
            if (ntk_scale > 0.0f) position = s;
            for (uint32_t h = 0; h < heads; h++)
                for (uint32_t i = 0; i < half; i++) {
                    float c, sn;
                    if (cos_cache && sin_cache) {
                        c = cos_cache[(size_t)position * half + i];
                        sn = sin_cache[(size_t)position * half + i];
                    } else {
                        const float angle = (float)position * orc_rope_freq(i, head_dim, theta);
                        c = cosf(angle);
                        sn = sinf(angle);
                    }
                    const size_t i0 = (((size_t)b * seq + s) * heads + h) * head_dim + 2 * (size_t)i;
                    const float x0 = x[i0], x1 = x[i0 + 1];
                    if (!backward) {
                        out[i0] = x0 * c - x1 * sn;
                        out[i0 + 1] = x0 * sn + x1 * c;
                    } else {
                        out[i0] = x0 * c + x1 * sn;
                        out[i0 + 1] = -x0 * sn + x1 * c;
                    }
                }
        }
    return 0;
}

/* ---- one attention row in the order of the 256-thread shaders -------------------------------- */

/* scores[t] = (sum_d q[d] * key_t[d]) * scale for t < n; the max and the sum of safe_exp are
 * reduced as the shaders do: thread t takes keys t, t + 256, ..., then a binary tree over the
 * 256 partials (stride 128 ... 1).  Returns max; *sum_out the denominator. */
static float row_softmax_stats(const float* scores, uint32_t n, float* sum_out) {
    float part[WG];
    for (uint32_t t = 0; t < WG; t++) {
        float m = NEG_INF_F;
        for (uint32_t i = t; i < n; i += WG) m = fmaxf(m, scores[i]);
        part[t] = m;
    }
    for (uint32_t s = WG / 2; s > 0; s >>= 1)
        for (uint32_t t = 0; t < s; t++) part[t] = fmaxf(part[t], part[t + s]);
    const float mx = part[0];
    for (uint32_t t = 0; t < WG; t++) {
        float a = 0.0f;
        for (uint32_t i = t; i < n; i += WG) a += safe_exp(scores[i] - mx);
        part[t] = a;
    }
    for (uint32_t s = WG / 2; s > 0; s >>= 1)
        for (uint32_t t = 0; t < s; t++) part[t] += part[t + s];
    *sum_out = part[0];
    return mx;
}

/*
 * sdpa_basic, gpu/scaled_dot_product_attention.wgsl:81-199 (one workgroup per batch, head and
 * query position), with the K/V head of sdpa_mqa (:539-637, one shared head) and of sdpa_kv_cache
 * (:386-489, kv_head = head / (num_heads / num_kv_heads)) as a parameter:
 *   q, out [batch, heads, seq_q, head_dim]; k, v [batch, kv_heads, seq_kv, head_dim]
 *   causal: query i sees keys 0 .. min(i + 1, seq_kv) - 1                      (:104-107)
 *   weight_t = safe_exp(score_t - max) * inv_sum, inv_sum = sum > 0 ? 1 / sum : 0  (:177, :189)
 *   out[d] = sum_t weight_t * v[t, d], keys in order                            (:182-194)
 * lse (may be NULL) [batch, heads, seq_q] = max + log(sum), -3.402823e38 for an empty row
 * (flash_attention_forward, steel/attention/flash.wgsl:233-239).
 */
int orc_sdpa(const float* q, const float* k, const float* v, float* out, float* lse, uint32_t batch, uint32_t heads,
             uint32_t kv_heads, uint32_t seq_q, uint32_t seq_kv, uint32_t head_dim, float scale, int causal) {
    if (kv_heads == 0 || heads % kv_heads) return -1;
    const uint32_t group = heads / kv_heads;
    float* sc = (float*)malloc(((size_t)seq_kv + 1) * sizeof(float));
    if (!sc) return -2;
    for (uint32_t b = 0; b < batch; b++)
        for (uint32_t h = 0; h < heads; h++)
            for (uint32_t i = 0; i < seq_q; i++) {
                const float* qr = q + (((size_t)b * heads + h) * seq_q + i) * head_dim;
                const float* kb = k + ((size_t)b * kv_heads + h / group) * seq_kv * head_dim;
                const float* vb = v + ((size_t)b * kv_heads + h / group) * seq_kv * head_dim;
                float* o = out + (((size_t)b * heads + h) * seq_q + i) * head_dim;
                uint32_t n = seq_kv;
                if (causal && i + 1 < n) n = i + 1;
                for (uint32_t t = 0; t < n; t++) {
                    float dot = 0.0f;
                    for (uint32_t d = 0; d < head_dim; d++) dot += qr[d] * kb[(size_t)t * head_dim + d];
                    sc[t] = dot * scale;
                }
                float sum;
                const float mx = row_softmax_stats(sc, n, &sum);
                const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
                for (uint32_t d = 0; d < head_dim; d++) {
                    float acc = 0.0f;
                    for (uint32_t t = 0; t < n; t++) acc += safe_exp(sc[t] - mx) * inv * vb[(size_t)t * head_dim + d];
                    o[d] = acc;
                }
                if (lse) lse[((size_t)b * heads + h) * seq_q + i] = sum > 0.0f ? mx + logf(sum) : NEG_INF_F;
            }
    free(sc);
    return 0;
}

/*
 * sdpa_kv_cache, gpu/scaled_dot_product_attention.wgsl:386-489:
 *   q, out [batch, heads, seq_q, head_dim]; caches [batch, kv_heads, max_cache_len, head_dim];
 *   the keys are cache positions 0 .. cache_len + seq_q - 1 (the new tokens are already appended).
 * The shader evaluates the FIRST query row of each head only (q_base has no query index, :413)
 * and applies no mask.  causal_append = 0 restates that for every row i (row 0 is the shader's
 * row); causal_append = 1 limits row i to cache_len + i + 1 keys, which is what a multi-token
 * append needs and equals the shader for seq_q = 1.
 */
int orc_sdpa_kv_cache(const float* q, const float* k_cache, const float* v_cache, float* out, uint32_t batch, uint32_t heads,
                      uint32_t kv_heads, uint32_t seq_q, uint32_t cache_len, uint32_t max_cache_len, uint32_t head_dim,
                      float scale, int causal_append) {
    if (kv_heads == 0 || heads % kv_heads) return -1;
    if ((uint64_t)cache_len + seq_q > max_cache_len) return -1;
    const uint32_t group = heads / kv_heads, total = cache_len + seq_q;
    float* sc = (float*)malloc(((size_t)total + 1) * sizeof(float));
    if (!sc) return -2;
    for (uint32_t b = 0; b < batch; b++)
        for (uint32_t h = 0; h < heads; h++)
            for (uint32_t i = 0; i < seq_q; i++) {
                const float* qr = q + (((size_t)b * heads + h) * seq_q + i) * head_dim;
                const size_t base = ((size_t)b * kv_heads + h / group) * max_cache_len * head_dim;
                float* o = out + (((size_t)b * heads + h) * seq_q + i) * head_dim;
                const uint32_t n = causal_append ? cache_len + i + 1 : total;
                for (uint32_t t = 0; t < n; t++) {
                    float dot = 0.0f;
                    for (uint32_t d = 0; d < head_dim; d++) dot += qr[d] * k_cache[base + (size_t)t * head_dim + d];
                    sc[t] = dot * scale;
                }
                float sum;
                const float mx = row_softmax_stats(sc, n, &sum);
                const float inv = 1.0f / sum;                                   /* :463, no guard */
                for (uint32_t d = 0; d < head_dim; d++) {
                    float acc = 0.0f;
                    for (uint32_t t = 0; t < n; t++) acc += safe_exp(sc[t] - mx) * inv * v_cache[base + (size_t)t * head_dim + d];
                    o[d] = acc;
                }
            }
    free(sc);
    return 0;
}

/* update_kv_cache, gpu/scaled_dot_product_attention.wgsl:496-533: new k, v
 * [batch, kv_heads, seq_q, head_dim] go to cache positions cache_len + s; positions at or past
 * max_cache_len are dropped without an error (:523-525). */
int orc_update_kv_cache(const float* k, const float* v, float* k_cache, float* v_cache, uint32_t batch, uint32_t kv_heads,
                        uint32_t seq_q, uint32_t cache_len, uint32_t max_cache_len, uint32_t head_dim) {
    for (uint32_t b = 0; b < batch; b++)
        for (uint32_t h = 0; h < kv_heads; h++)
            for (uint32_t s = 0; s < seq_q; s++) {
                const uint64_t pos = (uint64_t)cache_len + s;
                if (pos >= max_cache_len) continue;
                const size_t src = (((size_t)b * kv_heads + h) * seq_q + s) * head_dim;
                const size_t dst = (((size_t)b * kv_heads + h) * max_cache_len + pos) * head_dim;
                for (uint32_t d = 0; d < head_dim; d++) {
                    k_cache[dst + d] = k[src + d];
                    v_cache[dst + d] = v[src + d];
                }
            }
    return 0;
}

/* ---- paged KV cache: steel/attention/paged.wgsl ------------------------------------------------ */

static size_t paged_row(const int32_t* table, uint32_t token, uint32_t block_size, uint32_t kv_heads, uint32_t kv_head,
                        uint32_t head_dim) {
    /* :87-93: physical block from the table, then [block, kv_head, offset in block, head_dim] */
    const uint32_t logical = token / block_size, off = token % block_size;
    const uint32_t physical = (uint32_t)table[logical];
    return ((size_t)physical * kv_heads + kv_head) * block_size * head_dim + (size_t)off * head_dim;
}

/*
 * One partition [start, end) of one (sequence, head): scores, exp(score - max) with PLAIN exp
 * (:136, :297), the partition's max and sum, and part_out[d] = sum_t (e_t * (1 / sum)) * v[t, d]
 * (:160-180, :320-344).  The max and the sum run over the whole partition (see the file header).
 */
static void paged_partition(const float* qr, const float* kc, const float* vc, const int32_t* table, uint32_t start, uint32_t end,
                            uint32_t block_size, uint32_t kv_heads, uint32_t kv_head, uint32_t head_dim, float scale, float* sc,
                            float* part_out, float* max_out, float* sum_out) {
    const uint32_t n = end - start;
    float mx = NEG_INF_F;
    for (uint32_t i = 0; i < n; i++) {
        const size_t ko = paged_row(table, start + i, block_size, kv_heads, kv_head, head_dim);
        float dot = 0.0f;
        for (uint32_t d = 0; d < head_dim; d++) dot += qr[d] * kc[ko + d];
        sc[i] = dot * scale;
        mx = fmaxf(mx, sc[i]);
    }
    float sum = 0.0f;
    for (uint32_t i = 0; i < n; i++) {
        sc[i] = expf(sc[i] - mx);
        sum += sc[i];
    }
    const float inv = 1.0f / sum;
    for (uint32_t i = 0; i < n; i++) sc[i] *= inv;
    for (uint32_t d = 0; d < head_dim; d++) {
        float acc = 0.0f;
        for (uint32_t i = 0; i < n; i++) acc += sc[i] * vc[paged_row(table, start + i, block_size, kv_heads, kv_head, head_dim) + d];
        part_out[d] = acc;
    }
    *max_out = mx;
    *sum_out = sum;
}

/*
 * paged_attention_v1 (:55-181) when partition_size == 0, else paged_attention_v2_partial
 * (:209-345) + paged_attention_v2_reduce (:351-405):
 *   q, out [num_seqs, heads, head_dim]; caches [num_blocks, kv_heads, block_size, head_dim];
 *   block_tables [num_seqs, max_blocks_per_seq] (i32); context_lens [num_seqs] (i32).
 * A sequence with context_len <= 0 leaves its output rows untouched (:66-67, :221-222).
 */
int orc_paged_attention(const float* q, const float* k_cache, const float* v_cache, const int32_t* block_tables,
                        const int32_t* context_lens, float* out, uint32_t num_seqs, uint32_t heads, uint32_t kv_heads,
                        uint32_t head_dim, uint32_t block_size, uint32_t max_blocks_per_seq, float scale, uint32_t partition_size) {
    if (kv_heads == 0 || heads % kv_heads || block_size == 0) return -1;
    const uint32_t group = heads / kv_heads;
    for (uint32_t s = 0; s < num_seqs; s++) {
        const int32_t len = context_lens[s];
        if (len <= 0) continue;
        if ((uint64_t)len > (uint64_t)max_blocks_per_seq * block_size) return -1;
        const int32_t* table = block_tables + (size_t)s * max_blocks_per_seq;
        const uint32_t psize = partition_size ? partition_size : (uint32_t)len;
        const uint32_t parts = ((uint32_t)len + psize - 1) / psize;
        float* sc = (float*)malloc((size_t)psize * sizeof(float));
        float* po = (float*)malloc((size_t)parts * head_dim * sizeof(float));
        float* pm = (float*)malloc((size_t)parts * sizeof(float));
        float* ps = (float*)malloc((size_t)parts * sizeof(float));
        if (!sc || !po || !pm || !ps) { free(sc); free(po); free(pm); free(ps); return -2; }
        for (uint32_t h = 0; h < heads; h++) {
            const float* qr = q + ((size_t)s * heads + h) * head_dim;
            float* o = out + ((size_t)s * heads + h) * head_dim;
            for (uint32_t p = 0; p < parts; p++) {
                const uint32_t start = p * psize;
                const uint32_t end = start + psize < (uint32_t)len ? start + psize : (uint32_t)len;
                paged_partition(qr, k_cache, v_cache, table, start, end, block_size, kv_heads, h / group, head_dim, scale, sc,
                                po + (size_t)p * head_dim, pm + p, ps + p);
            }
            if (!partition_size) {
                for (uint32_t d = 0; d < head_dim; d++) o[d] = po[d];
                continue;
            }
            /* reduce, :366-404 */
            float gmax = NEG_INF_F;
            for (uint32_t p = 0; p < parts; p++) gmax = fmaxf(gmax, pm[p]);
            float gsum = 0.0f;
            for (uint32_t p = 0; p < parts; p++)
                if (pm[p] > NEG_INF_F) gsum += ps[p] * expf(pm[p] - gmax);
            for (uint32_t d = 0; d < head_dim; d++) {
                float acc = 0.0f;
                for (uint32_t p = 0; p < parts; p++)
                    if (pm[p] > NEG_INF_F) acc += ps[p] * expf(pm[p] - gmax) / gsum * po[(size_t)p * head_dim + d];
                o[d] = acc;
            }
        }
        free(sc); free(po); free(pm); free(ps);
    }
    return 0;
}
