/*
 * lux/gpu/attention_ext.h -- the f32 attention-side operators of a decoder layer, exported by
 * libluxgpu_backend_cuda.so BESIDE the backend vtable: rotary embedding, scaled-dot-product
 * attention, attention over a contiguous KV cache with its append, and attention over a paged KV
 * cache.  They sit between the qkv and the o projection that lux/gpu/qmatmul_ext.h serves.
 *
 * luxcpp/webgpu carries these operators as WGSL that its plugin never dispatches (no vtable slot,
 * no pipeline: src/webgpu_plugin.cpp:4022-4123 has no attention entry), so there is no host-side
 * signature to mirror; the arguments below are the fields of each shader's uniform block, in the
 * shader's order, and every tensor has the shader's layout:
 *   kernels/wgsl/gpu/rope.wgsl                          RoPEParams :28-37, CacheParams :258-263
 *   kernels/wgsl/gpu/scaled_dot_product_attention.wgsl  SDPAParams :31-40, SDPAKVCacheParams :370-379
 *   kernels/wgsl/steel/attention/paged.wgsl             PagedAttentionParams :20-29
 *   kernels/wgsl/steel/attention/flash.wgsl             FlashAttentionParams :21-30 (same math as
 *                                                       sdpa_basic, plus the log-sum-exp output)
 *
 * Same conventions as qmatmul_ext.h: LuxBackendBuffer operands created through the vtable (or
 * lux_cuda_buffer_wrap), arguments validated before anything is launched, a LuxBackendError
 * comes back, nothing throws.  `flags` takes LUX_QMATMUL_FLAG_NO_SYNC (enqueue and return) and
 * the LUX_ATTN_* bits below.  All data is f32; head_dim is any positive value (multiples of 4 up
 * to 256 take the streaming kernel, the rest a plain one).
 *
 * Arithmetic: scores = (q . k) * scale; weights = softmax over the keys a row sees; out =
 * weights . v, all in f32.  Sums are taken in a different order than the one-workgroup-per-row
 * shaders take them (keys are split over warps and, for long contexts, over thread blocks, and
 * merged with the running-maximum rule of sdpa_flash, scaled_dot_product_attention.wgsl:217-362),
 * so results agree with the shaders to rounding, not bit for bit.  The shaders' safe_exp clamps
 * the exponent to [-88, 88] (:68-70); a key more than 88 below the row maximum therefore keeps a
 * weight of e^-88 there and gets 0 here, a difference below 1e-38 of the row's total.
 */
#ifndef LUX_GPU_ATTENTION_EXT_H
#define LUX_GPU_ATTENTION_EXT_H

#include "lux/gpu/qmatmul_ext.h"

#ifdef __cplusplus
extern "C" {
#endif

enum {
    /* Query i sees keys 0 .. i (sdpa: SDPAParams.causal, FlashAttentionParams.is_causal); with a
     * KV cache, query i of the appended tokens sees the cache_len cached keys and appended keys
     * 0 .. i.  Without the bit a KV-cache call lets every query see all cache_len + seq_len_q
     * keys, which for seq_len_q = 1 is the same thing and is what sdpa_kv_cache computes. */
    LUX_ATTN_FLAG_CAUSAL   = 1u << 4,
    /* lux_cuda_rope_f32: rotate by the opposite angle (rope_backward, rope.wgsl:214-252). */
    LUX_ROPE_FLAG_BACKWARD = 1u << 5
};

/* rope_precompute_cache (rope.wgsl:269-291): cos_out, sin_out [max_seq_len, head_dim / 2] of
 * f32(pos) * theta_base^(-2 i / head_dim).  head_dim even. */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_rope_precompute_cache_f32(
    LuxBackendContext* ctx, LuxBackendBuffer* cos_out, LuxBackendBuffer* sin_out,
    uint32_t max_seq_len, uint32_t head_dim, float theta_base, uint32_t flags);

/*
 * The rotation of rope_forward (:67-111), rope_forward_no_cache (:118-160), rope_inplace (:167-203,
 * pass out == x), rope_backward (:214-252), rope_ntk_scaled (:312-353) and rope_custom_positions
 * (:359-397) in one entry point.  x, out [batch, seq_len, num_heads, head_dim]; pairs are the
 * ADJACENT elements (2i, 2i + 1).
 *   cos_cache, sin_cache  both given: angles come from the cache at [position, i]; both NULL:
 *                         formed on the fly from theta_base.  With a cache the result is
 *                         bit-identical to the shader arithmetic (two products, one sum, no
 *                         contraction).
 *   position_ids          NULL: position = position_offset + index in the sequence; else u32
 *                         [batch, seq_len].  A position outside the cache leaves its pair unwritten
 *                         and sets the context's device status.
 *   ntk_scale             > 0 (no cache only): theta_base * ntk_scale^(head_dim / (head_dim - 2)),
 *                         and, as in the shader, the angle uses the index in the sequence alone.
 */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_rope_f32(
    LuxBackendContext* ctx, LuxBackendBuffer* x, LuxBackendBuffer* out,
    LuxBackendBuffer* cos_cache, LuxBackendBuffer* sin_cache, LuxBackendBuffer* position_ids,
    uint32_t batch_size, uint32_t seq_len, uint32_t num_heads, uint32_t head_dim,
    float theta_base, uint32_t position_offset, float ntk_scale, uint32_t flags);

/* rope_qk_fused (:406-448): q [batch, seq_len, num_heads, head_dim] and k [batch, seq_len,
 * num_kv_heads, head_dim] rotated in place by the cached angles, one launch.  The shader gives
 * both tensors num_heads heads; pass num_kv_heads = num_heads for that. */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_rope_qk_f32(
    LuxBackendContext* ctx, LuxBackendBuffer* q, LuxBackendBuffer* k,
    LuxBackendBuffer* cos_cache, LuxBackendBuffer* sin_cache,
    uint32_t batch_size, uint32_t seq_len, uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_dim,
    uint32_t position_offset, uint32_t flags);

/*
 * sdpa_basic / sdpa_flash / flash_attention_forward (one key/value head per query head) and
 * sdpa_mqa (num_kv_heads = 1); any num_kv_heads that divides num_heads is taken, query head h
 * reading key/value head h / (num_heads / num_kv_heads) as sdpa_kv_cache does (:404-406).
 *   q, out [batch, num_heads, seq_len_q, head_dim]; k, v [batch, num_kv_heads, seq_len_kv, head_dim]
 *   lse    NULL or [batch, num_heads, seq_len_q]: max + log(sum), -3.402823e38 for a row that sees
 *          no key (flash.wgsl:233-239)
 * seq_len_kv = 0 writes zeros (the shaders' inv_sum = 0 rule, :177).  dropout_p of SDPAParams is not
 * taken: the shaders never read it.
 */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_sdpa_f32(
    LuxBackendContext* ctx, LuxBackendBuffer* q, LuxBackendBuffer* k, LuxBackendBuffer* v,
    LuxBackendBuffer* out, LuxBackendBuffer* lse,
    uint32_t batch_size, uint32_t num_heads, uint32_t num_kv_heads, uint32_t seq_len_q, uint32_t seq_len_kv,
    uint32_t head_dim, float scale, uint32_t flags);

/* update_kv_cache (:496-533): k, v [batch, num_kv_heads, seq_len_q, head_dim] are written to
 * positions cache_len .. cache_len + seq_len_q - 1 of the caches [batch, num_kv_heads,
 * max_cache_len, head_dim]; positions at or past max_cache_len are dropped without an error, as
 * the shader drops them (:523-525). */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_update_kv_cache_f32(
    LuxBackendContext* ctx, LuxBackendBuffer* k, LuxBackendBuffer* v,
    LuxBackendBuffer* k_cache, LuxBackendBuffer* v_cache,
    uint32_t batch_size, uint32_t num_kv_heads, uint32_t seq_len_q, uint32_t cache_len, uint32_t max_cache_len,
    uint32_t head_dim, uint32_t flags);

/*
 * sdpa_kv_cache (:386-489): attention of the appended tokens' queries over cache positions
 * 0 .. cache_len + seq_len_q - 1 (call lux_cuda_update_kv_cache_f32 first).  q, out [batch,
 * num_heads, seq_len_q, head_dim].  The shader evaluates the first query row of a head only
 * (:413); here every row is evaluated, row 0 being the shader's, and LUX_ATTN_FLAG_CAUSAL limits
 * row i to cache_len + i + 1 keys.  cache_len + seq_len_q must not exceed max_cache_len.
 */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_sdpa_kv_cache_f32(
    LuxBackendContext* ctx, LuxBackendBuffer* q, LuxBackendBuffer* k_cache, LuxBackendBuffer* v_cache,
    LuxBackendBuffer* out,
    uint32_t batch_size, uint32_t num_heads, uint32_t num_kv_heads, uint32_t seq_len_q, uint32_t cache_len,
    uint32_t max_cache_len, uint32_t head_dim, float scale, uint32_t flags);

/*
 * paged_attention_v1 and paged_attention_v2_partial + _reduce (paged.wgsl:55-181, 209-405) behind
 * one entry point; how a context is partitioned is chosen here and the partition buffers of v2
 * (exp_sums, max_logits, partition_output) are the context's own scratch.
 *   q, out        [num_seqs, num_heads, head_dim]
 *   k/v_cache     [num_blocks, num_kv_heads, block_size, head_dim]
 *   block_tables  i32 [num_seqs, max_blocks_per_seq], physical block of each logical block
 *   context_lens  i32 [num_seqs]; a sequence with context_len <= 0 leaves its output rows
 *                 untouched (:66-67)
 * A context_len above max_blocks_per_seq * block_size is cut there.  The shader text reduces the
 * maximum and the sum through the first lane of each warp only (:112-131, :141-157); the softmax
 * over the whole context that its comments describe is what is computed here.
 */
LUX_GPU_PLUGIN_EXPORT LuxBackendError lux_cuda_paged_attention_f32(
    LuxBackendContext* ctx, LuxBackendBuffer* q, LuxBackendBuffer* k_cache, LuxBackendBuffer* v_cache,
    LuxBackendBuffer* block_tables, LuxBackendBuffer* context_lens, LuxBackendBuffer* out,
    uint32_t num_seqs, uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_dim,
    uint32_t block_size, uint32_t max_blocks_per_seq, float scale, uint32_t flags);

#ifdef __cplusplus
}
#endif
#endif /* LUX_GPU_ATTENTION_EXT_H */
