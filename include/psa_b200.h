/* C ABI of the B200 (sm_100a) Pyramid-Sparse-Attention kernels.
 *
 * Every entry point takes raw device pointers, sizes and a cudaStream_t (passed as void*), enqueues
 * its kernels on that stream and returns a status code without synchronising.  Nothing here allocates
 * device memory unless the comment of the entry point says otherwise: outputs and scratch are the
 * caller's.  All tensors are contiguous; "[BH, S, D]" means batch*heads major, token, channel.
 * dtype codes: 0 = float32, 1 = float16, 2 = bfloat16.
 *
 * Each declaration cites the part of ziplab/Pyramid-Sparse-Attention it stands in for
 * (paths relative to that project).
 */
#ifndef PSA_B200_H_
#define PSA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PSA_OK 0
#define PSA_ERR_ARG 1          /* bad argument (shape, alignment, null pointer) */
#define PSA_ERR_UNSUPPORTED 2  /* valid request this build has no kernel for */
#define PSA_ERR_CUDA 3         /* a CUDA runtime/driver call or launch failed */
#define PSA_ERR_TIMEOUT 4      /* a bounded device-side wait expired (reported through a status word) */

#define PSA_F32 0
#define PSA_F16 1
#define PSA_BF16 2

#define PSA_MAX_LEVELS 8

/* Text of the last error raised on the calling thread ("" if none). */
const char* psa_last_error_string(void);

/* Library version / build info string. */
const char* psa_build_info(void);

/* Pyramid K/V builder.  Replaces pad_to_multiple + pooling chain,
 * src/psa_triton/kernels/psa_kernel.py:318-349 and its call site :381-388 (legacy twin
 * src/psa_triton/kernels/psa_kernel_legacy.py:806-834, 868-875).
 * k, v: [BH, S, D].  Outputs x2/x4/x8: [BH, S_pad/l, D] with S_pad = ceil(S/block_n)*block_n; tokens past
 * S replicate token S-1; each level is the pairwise mean of the previous ROUNDED level (fp32 add, one
 * rounding to dtype).  One pass over K and V; the never-read level 16 is not built. */
int psa_pyramid_kv(const void* k, const void* v, void* k2, void* k4, void* k8, void* v2, void* v4, void* v8,
                   int64_t bh, int64_t seq, int head_dim, int block_n, int dtype, void* stream);

/* Pyramid K/V builder, tile-image form (f16/bf16, head_dim 64/128, block_n a multiple of 64).  Same source lines of
 * the reference as psa_pyramid_kv; the output LAYOUT is this library's own: per operand one buffer of
 * psa_kv_image_bytes() bytes (16-byte aligned) holding levels 1, 2, 4, 8 one after the other, each level as
 * [BH][8-row group][64-channel slab][8 rows][128 B] with the 16-byte chunks of a row XOR-ed by (row & 7) - the image
 * of the 128-byte-swizzled shared-memory tile the tensor cores read, so that a block of pooled rows is one contiguous
 * range.  Values are those of psa_pyramid_kv (level 1 = the input rows, tail rows replicate the last token). */
size_t psa_kv_image_bytes(int64_t bh, int64_t seq, int head_dim, int block_n);
int psa_pyramid_kv_images(const void* k, const void* v, void* kimg, void* vimg, int64_t bh, int64_t seq, int head_dim,
                          int block_n, int dtype, void* stream);

/* Block-importance scores.  Replaces _random_sample_tokens' gather + replicate padding
 * (src/psa_triton/attention.py:128-137, 195-196, 214-215), attn_with_pooling_optimized
 * (src/psa_triton/kernels/attn_pooling_kernel.py:119-431) and the slice at attention.py:223.
 * q: [BH, seq_q, D], k: [BH, seq_k, D]; idx_q: [BH, block_m/4], idx_k: [BH, block_n/4] int32 = the
 * in-block token offsets drawn by topk(rand) on the host side.  po: [BH, ceil(seq_q/block_m),
 * ceil(seq_k/block_n)] in dtype.  scratch: psa_block_scores_scratch_bytes() bytes, 256-byte aligned.
 * impl: 0 = pick (tensor-core kernel for f16/bf16, else scalar), 1 = scalar fp32 kernel, 2 = tcgen05 kernel. */
size_t psa_block_scores_scratch_bytes(int64_t bh, int64_t seq_q, int64_t seq_k, int block_m, int block_n, int dtype);
int psa_block_scores(const void* q, const void* k, const int32_t* idx_q, const int32_t* idx_k, void* po,
                     void* scratch, size_t scratch_bytes, int64_t bh, int64_t seq_q, int64_t seq_k, int head_dim,
                     int block_m, int block_n, int dtype, int impl, void* stream);

/* Block-importance scores for callers that cannot allocate device memory.  (No counterpart in the reference, which
 * allocates its R / Po buffers with torch on every call.)
 * Same arguments, result and kernels as psa_block_scores, minus the scratch pointer: the scratch is a built-in
 * device array of PSA_STATIC_SCRATCH_BYTES (64 MiB) that every GPU loading this library holds until the process
 * exits.  The entry point calls no cudaMalloc/cudaFree and no allocating library routine; the caller still owns
 * q, k, idx_q, idx_k and po.  A call that needs more scratch than the array holds is rejected with PSA_ERR_ARG and a
 * message naming both sizes (split it over fewer heads); the need is computed for the call's own head_dim, so it is
 * at most psa_block_scores_scratch_bytes(), which is sized for head_dim 128.
 * The first call on a device resolves the array's device address (cudaGetSymbolAddress, with that device current);
 * make that first call outside any stream capture.  All calls on a device share the one array, which keeps the last
 * call's contents: every element a call reads it has written before, so nothing needs clearing, but two calls that
 * overlap on the GPU (different streams, or threads) race on it - serialise them.  The resolved address is cached per
 * device for the life of the process: after a cudaDeviceReset the library must be reloaded. */
#define PSA_STATIC_SCRATCH_BYTES (64u << 20)
size_t psa_block_scores_static_capacity(void);
int psa_block_scores_static(const void* q, const void* k, const int32_t* idx_q, const int32_t* idx_k, void* po,
                            int64_t bh, int64_t seq_q, int64_t seq_k, int head_dim, int block_m, int block_n, int dtype,
                            int impl, void* stream);

/* Level assignment.  Replaces transfer_attn_to_mask, all four modes,
 * src/psa_triton/utils/transfer_attn_to_mask.py:6-507.
 * po: [rows, nk] scores in dtype (rows = B*H*Mq).  mask: int32 [rows, nk + n_levels] (newtype) or [rows, nk].
 * Sort is descending with equal scores in ascending index order.
 * threshold_mode 0 (topk*): starts/ends[n_levels] are the rank intervals, computed by the caller with the
 *   reference's Python arithmetic (:63-120 / :282-351); an empty interval has start == end.
 * threshold_mode 1 (thresholdbound*): levels must be in ascending end_ratio order; thresholds[i] is
 *   end_ratio+1e-6 already rounded to dtype; aligns[i] = ceil(level/(block_n/tile_n)); min_index =
 *   min(nk, int(nk*min_full_attn_ratio)+1) applies to level 1 (:225-232, :454-461).
 * text_blocks > 0 (old format only): the last text_blocks columns are forced to 1 (:40-45).
 * level_values/starts/ends/thresholds/aligns are HOST arrays of n_levels <= PSA_MAX_LEVELS entries. */
int psa_assign_levels(const void* po, int32_t* mask, int64_t rows, int nk, int dtype, int threshold_mode,
                      int newtype, int n_levels, const int32_t* level_values, const int32_t* starts,
                      const int32_t* ends, const float* thresholds, const int32_t* aligns, int min_index,
                      int text_blocks, void* stream);

/* Mask density.  Replaces calc_density_newtype / calc_density,
 * src/psa_triton/utils/transfer_attn_to_mask.py:510-622.  per_bh: float32 [BH], the mean density of
 * each (batch, head); no host synchronisation. */
int psa_density(const int32_t* mask, float* per_bh, int64_t bh, int64_t mq, int width, int newtype, void* stream);

/* K-similarity cap.  Replaces calc_k_similarity_triton, src/psa_triton/kernels/calc_ksim_kernel.py:6-225
 * (and its PyTorch twin :227-265) together with the replicate padding at src/psa_triton/attention.py:196.
 * k: [BH, seq, D]; out: int32 [BH, ceil(seq/block_n)] in {1,2,4,8}. */
int psa_ksim(const void* k, int32_t* out, int64_t bh, int64_t seq, int head_dim, int block_n, float t2, float t4,
             float t8, int dtype, void* stream);

/* Multi-level block-sparse attention forward on the separator-format mask.  Replaces _fwd_kernel /
 * _forward, src/psa_triton/kernels/psa_kernel.py:24-316, 351-432 (pyramid tensors come from
 * psa_pyramid_kv).  q/out: [BH, seq_q, D]; k, v: [BH, seq_k, D]; k2..v8 as produced by psa_pyramid_kv;
 * mask: int32 [BH, ceil(seq_q/block_m), mask_width], per row: level-1 block indices, -1, level-2, -1,
 * level-4, -1, level-8, -1, rest ignored.  compat_quirk != 0 reproduces the reference's handling of levels
 * whose pooled block is narrower than half a tile (:261-278): each merged pair also attends pooled tokens
 * [2P, tile_n) of that level.  impl: 0 = pick, 1 = scalar kernel, 2 = tcgen05 kernel (f16/bf16, block_m 128).
 * status: device int32 word, written non-zero if a bounded wait inside the kernel expired (may be NULL).
 * The tcgen05 kernel is persistent: its CTAs claim query blocks from a counter.  The counters are a ring of 256 device
 * words inside the library (one per launch, zeroed on the launching stream right before the kernel); the first
 * tcgen05 launch on a device resolves the ring's address (cudaGetSymbolAddress) - make it outside any stream capture -
 * and more than 256 launches of this family in flight at once on one device would share counters (a captured graph pins
 * its slot for every replay: do not replay such graphs while more than 255 other launches overlap them).  This holds
 * for every psa_fwd* / psa_legacy_fwd_images* entry point.
 * bf16 without the causal rule is TWO launches of the tcgen05 kernel.  The first takes the probabilities of a query row
 * relative to the maximum of the row's first tile instead of a running maximum (same result: the factor cancels against
 * the row sum; bf16 probabilities and the fp32 sum have the exponent range for it), which saves the maximum pass and
 * the rescaling; a row whose sum leaves the safe range sets a guard word (another slot of the counter ring).  The
 * second launch is the running-maximum kernel: it reads the guard word, returns at once if it is zero and recomputes
 * the call otherwise.  Both are ordered on `stream`; nothing is read back by the host.  fp16 calls and the causal
 * variants are one launch of the running-maximum kernel.  A bf16 call therefore takes THREE words of the ring (two row
 * counters and the guard word): about 85 such calls may be in flight on one device before words are shared. */
int psa_fwd(const void* q, const void* k, const void* v, const void* k2, const void* k4, const void* k8,
            const void* v2, const void* v4, const void* v8, const int32_t* mask, void* out, int64_t bh,
            int64_t seq_q, int64_t seq_k, int head_dim, int block_m, int block_n, int tile_n, int mask_width,
            float sm_scale, int compat_quirk, int impl, int dtype, int32_t* status, void* stream);

/* The same forward (tcgen05 kernel only) reading K/V from the tile images of psa_pyramid_kv_images: every selected
 * block is fetched with one linear bulk copy per operand instead of one tensor-map TMA operation per 64-channel
 * slab.  Replaces the same reference code as psa_fwd. */
int psa_fwd_images(const void* q, const void* kimg, const void* vimg, const int32_t* mask, void* out, int64_t bh,
                   int64_t seq_q, int64_t seq_k, int head_dim, int block_m, int block_n, int tile_n, int mask_width,
                   float sm_scale, int compat_quirk, int dtype, int32_t* status, void* stream);

/* Token reordering folded into the kernels.  Replaces GilbertRearranger.rearrange / rearrange_single / reversed_rearrange,
 * src/psa_triton/utils/rearranger.py:69-132 (three index_select copies of q, k, v before the attention and one of the
 * output after it; the text tokens move from the front of the sequence to its end and back).
 * perm: int32 [seq], a permutation of 0..seq-1 shared by all heads: token t of the sequence the attention works on is
 * row perm[t] of the tensor as stored.  k, v and the sampled quarter of q are read through perm by the kernels that
 * read them anyway; the forward stores output row t at row out_perm[t], so with out_perm == perm the output is back
 * in the stored order; only q needs a reordered copy (psa_gather_rows), because the forward fetches query tiles with
 * bulk tensor copies.  Results are bit-identical to reordering q, k, v first, running psa_pyramid_kv_images /
 * psa_block_scores / psa_fwd_images, and reordering the output back.
 *   psa_gather_rows:            dst[bh][t][:] = src[bh][perm[t]][:]   (rows a multiple of 16 bytes; not in place)
 *   psa_pyramid_kv_images_perm: psa_pyramid_kv_images of the reordered k, v
 *   psa_block_scores_perm:      psa_block_scores (tcgen05 path, f16/bf16) of the reordered q, k
 *   psa_fwd_images_perm:        psa_fwd_images with q already reordered and the output rows stored through out_perm */
int psa_gather_rows(const void* src, const int32_t* perm, void* dst, int64_t bh, int64_t seq, int head_dim, int elem_bytes,
                    void* stream);
int psa_pyramid_kv_images_perm(const void* k, const void* v, const int32_t* perm, void* kimg, void* vimg, int64_t bh,
                               int64_t seq, int head_dim, int block_n, int dtype, void* stream);
int psa_block_scores_perm(const void* q, const void* k, const int32_t* perm_q, const int32_t* perm_k, const int32_t* idx_q,
                          const int32_t* idx_k, void* po, void* scratch, size_t scratch_bytes, int64_t bh, int64_t seq_q,
                          int64_t seq_k, int head_dim, int block_m, int block_n, int dtype, void* stream);
int psa_fwd_images_perm(const void* q, const void* kimg, const void* vimg, const int32_t* mask, void* out,
                        const int32_t* out_perm, int64_t bh, int64_t seq_q, int64_t seq_k, int head_dim, int block_m,
                        int block_n, int tile_n, int mask_width, float sm_scale, int compat_quirk, int dtype, int32_t* status,
                        void* stream);
/* The same for the presets with the old mask format and the similarity cap (every shipped `attn_impl: old_mask_type`
 * preset reorders too, src/psa_triton/pyramid_sparse_attention.py:340-406):
 *   psa_ksim_perm:               psa_ksim of the reordered k (calc_k_similarity_triton after rearrange)
 *   psa_legacy_fwd_images_perm:  psa_legacy_fwd_images (not causal, no lse) with q already reordered, kimg/vimg from
 *                                psa_pyramid_kv_images_perm(block_n = 128), output row t stored at row out_perm[t] */
int psa_ksim_perm(const void* k, const int32_t* perm, int32_t* out, int64_t bh, int64_t seq, int head_dim, int block_n, float t2,
                  float t4, float t8, int dtype, void* stream);
int psa_legacy_fwd_images_perm(const void* q, const void* kimg, const void* vimg, const int32_t* mask, int32_t* index_scratch,
                               void* out, const int32_t* out_perm, int64_t bh, int64_t seq, int head_dim, int mask_cols,
                               float sm_scale, int dtype, int32_t* status, void* stream);

/* Token-major tensors.  Replaces the three transpose(1, 2) of q, k, v in front of the attention call and the
 * transpose(1, 2).flatten(2, 3) behind it in the diffusers processors, modify_diffusers.py:302-307 and :357-371 (each
 * becomes a full copy when the reference makes the tensors contiguous, src/psa_triton/attention.py:302-306), optionally
 * together with the token reordering above.
 * q, k, v, out: one batch element, [seq][heads][head_dim] as the projection layers produce / consume them.  perm
 * (may be NULL): int32 [seq], token t of the attention's sequence is stored token perm[t].  The score and tile-image
 * kernels read the rows where they lie, the forward stores output row t into out[perm[t]][head]; q alone is regrouped
 * by head (psa_gather_heads), because the forward fetches query tiles with bulk tensor copies.  Bit-identical to the
 * head-major calls on transposed (and reordered) copies.
 *   psa_gather_heads:          dst[h][t][:] = src[perm ? perm[t] : t][h][:]
 *   psa_pyramid_kv_images_tm:  psa_pyramid_kv_images      psa_block_scores_tm: psa_block_scores (tcgen05 path, f16/bf16)
 *   psa_fwd_images_tm:         psa_fwd_images, q head-major [heads][seq][head_dim], out token-major */
int psa_gather_heads(const void* src, const int32_t* perm, void* dst, int heads, int64_t seq, int head_dim, int elem_bytes,
                     void* stream);
int psa_pyramid_kv_images_tm(const void* k, const void* v, const int32_t* perm, void* kimg, void* vimg, int heads, int64_t seq,
                             int head_dim, int block_n, int dtype, void* stream);
int psa_block_scores_tm(const void* q, const void* k, const int32_t* perm, const int32_t* idx_q, const int32_t* idx_k, void* po,
                        void* scratch, size_t scratch_bytes, int heads, int64_t seq, int head_dim, int block_m, int block_n,
                        int dtype, void* stream);
int psa_fwd_images_tm(const void* q, const void* kimg, const void* vimg, const int32_t* mask, void* out, const int32_t* out_perm,
                      int heads, int64_t seq, int head_dim, int block_m, int block_n, int tile_n, int mask_width, float sm_scale,
                      int compat_quirk, int dtype, int32_t* status, void* stream);

/* The same three loads with the rotary embedding of the diffusion transformers applied on the way, so that the
 * processors (modify_diffusers.py:260-281 Wan, :363-369 CogVideoX) need not write rotated copies of q and k: every
 * kernel that touches a q or k row rotates it as it reads it.  rope_a, rope_b: fp32 device tables [seq - rope_first]
 * [head_dim], 16-byte aligned; stored token s >= rope_first uses table row s - rope_first (CogVideoX leaves its leading
 * text tokens alone), tokens before it pass unchanged.  Channel pair (x0, x1) becomes
 *     (x0*a[even] - x1*b[even],  x1*a[odd] + x0*b[odd]),
 * each product and sum rounded to fp32 separately and the result rounded once to the element type: bit for bit the
 * element-wise formulation of both processors (Wan: a = cos at the even entries, b = sin at the odd entries, both
 * repeated over the pair; CogVideoX: a = cos, b = sin).  Values are never rotated. */
int psa_gather_heads_rope(const void* src, const int32_t* perm, const float* rope_a, const float* rope_b, int64_t rope_first,
                          void* dst, int heads, int64_t seq, int head_dim, int dtype, void* stream);
int psa_pyramid_kv_images_tm_rope(const void* k, const void* v, const int32_t* perm, const float* rope_a, const float* rope_b,
                                  int64_t rope_first, void* kimg, void* vimg, int heads, int64_t seq, int head_dim, int block_n,
                                  int dtype, void* stream);
int psa_block_scores_tm_rope(const void* q, const void* k, const int32_t* perm, const float* rope_a, const float* rope_b,
                             int64_t rope_first, const int32_t* idx_q, const int32_t* idx_k, void* po, void* scratch,
                             size_t scratch_bytes, int heads, int64_t seq, int head_dim, int block_m, int block_n, int dtype,
                             void* stream);
/* The same for head-major tensors [bh][seq][head_dim] (what the CogVideoX processor holds after its per-head norms,
 * modify_diffusers.py:357-369): psa_gather_rows / psa_pyramid_kv_images_perm / psa_block_scores_perm with the rows
 * rotated as they are read.  perm may be NULL (stored order); self-attention (one length, one table pair). */
int psa_gather_rows_rope(const void* src, const int32_t* perm, const float* rope_a, const float* rope_b, int64_t rope_first,
                         void* dst, int64_t bh, int64_t seq, int head_dim, int dtype, void* stream);
int psa_pyramid_kv_images_perm_rope(const void* k, const void* v, const int32_t* perm, const float* rope_a, const float* rope_b,
                                    int64_t rope_first, void* kimg, void* vimg, int64_t bh, int64_t seq, int head_dim, int block_n,
                                    int dtype, void* stream);
int psa_block_scores_perm_rope(const void* q, const void* k, const int32_t* perm, const float* rope_a, const float* rope_b,
                               int64_t rope_first, const int32_t* idx_q, const int32_t* idx_k, void* po, void* scratch,
                               size_t scratch_bytes, int64_t bh, int64_t seq, int head_dim, int block_m, int block_n, int dtype,
                               void* stream);

/* Antidiagonal block-importance estimate of the causal (vision-language) call site.  Replaces estimate_block_importance
 * with select_mode "inverse", softmax, kdb 1 - and its Triton kernels flat_group_gemm_fuse_reshape /
 * softmax_fuse_block_sum - qwen2.5-vl-example/src/attention/PSA_casual/utils/block_importance.py:282-562,
 * kernels/block_importance_kernels.py:7-117, 256-325.
 * q, k: [BH, seq, D] (f16/bf16, equal lengths, D 64/128).  Tokens are zero-padded to a multiple of chunk_size and taken
 * in groups of `stride`; logit(i, j) = sum_s q[i*stride + stride-1-s] . k[j*stride + s] / sqrt(D) / stride; causal: group
 * i sees groups j <= i, else all groups of the padded length; out [BH, nb, nb] (dtype), nb = ceil(seq/block_size) =
 * softmax mass per (query block, key block).  block_size/stride must be a power of two in 2..32.
 * scratch: psa_antidiag_scratch_bytes() bytes (the fp32 logits), 16-byte aligned.
 * psa_antidiag_scores_impl: impl 0 = pick (the tcgen05 kernel when seq is a multiple of stride, else the warp-level
 * mma.sync kernel), 2 = tcgen05 (PSA_ERR_UNSUPPORTED otherwise), 3 = mma.sync; status (may be NULL): device word that
 * receives PSA_ERR_TIMEOUT if a bounded wait of the tcgen05 kernel expires (the output is then incomplete). */
size_t psa_antidiag_scratch_bytes(int64_t bh, int64_t seq, int head_dim, int block_size, int stride, int chunk_size);
int psa_antidiag_scores(const void* q, const void* k, void* out, void* scratch, size_t scratch_bytes, int64_t bh, int64_t seq,
                        int head_dim, int block_size, int stride, int chunk_size, int causal, int dtype, void* stream);
int psa_antidiag_scores_impl(const void* q, const void* k, void* out, void* scratch, size_t scratch_bytes, int64_t bh, int64_t seq,
                             int head_dim, int block_size, int stride, int chunk_size, int causal, int dtype, int impl,
                             int32_t* status, void* stream);

/* Level assignment of the causal call site.  Replaces transfer_attn_to_mask,
 * qwen2.5-vl-example/src/attention/PSA_casual/PyramidAdaptiveBlockSparseAttn.py:85-168.
 * attn: [BH, n, n] scores (dtype); mask: int32 [BH, n, n] in {0,1,2,4,8}.  Rows are sorted descending, equal scores in
 * ascending column order.  energy_mode 0 ("topk"): level i takes ranks [int(len*start_ratios[i]), int(len*end_ratios[i]))
 * with len = row+1 (causal) or n, products in fp32; energy_mode 1 ("energybound"): level i takes the ranks whose
 * cumulative share e of the row sum satisfies lower_bounds[i] < e <= upper_bounds[i] (bounds already rounded to dtype by
 * the caller, lower = max(start, previous end)).  Later levels overwrite earlier ones.  Then: the last special_blocks
 * columns and rows are 1, entries above the diagonal 0 (causal), the diagonal and column 0 are 1.
 * level_values, ratios and bounds are HOST arrays of n_levels <= PSA_MAX_LEVELS entries. */
int psa_assign_levels_causal(const void* attn, int32_t* mask, int64_t bh, int n, int dtype, int energy_mode, int causal,
                             int n_levels, const int32_t* level_values, const float* start_ratios, const float* end_ratios,
                             const float* lower_bounds, const float* upper_bounds, int special_blocks, void* stream);

/* Legacy forward on the dense old-format mask, optional causal.  Replaces _fwd_kernel / _forward,
 * src/psa_triton/kernels/psa_kernel_legacy.py:415-799, 837-938 (block sizes fixed 128/32/128, :1333-1351).
 * mask: int32 [BH, ceil(seq/128), mask_cols] in {0,1,2,4,8}; lse: float32 [BH, seq] = M + ln(max(L,1e-8))
 * (:931), may be NULL. */
int psa_legacy_fwd(const void* q, const void* k, const void* v, const void* k2, const void* k4, const void* k8,
                   const void* v2, const void* v4, const void* v8, const int32_t* mask, void* out, float* lse,
                   int64_t bh, int64_t seq, int head_dim, int mask_cols, float sm_scale, int causal, int dtype,
                   void* stream);

/* The same legacy forward on the tcgen05 kernel: the dense level row is regrouped into an index row
 * (index_scratch: psa_legacy_index_bytes(bh, seq) bytes of device memory) and the tile-image forward runs with block 128
 * and no compatibility extras; lse (may be NULL) and the "no visible key -> 0, lse = -inf" rule follow the legacy kernel
 * (psa_kernel_legacy.py:931).  kimg/vimg: psa_pyramid_kv_images(..., block_n = 128).  f16/bf16 only. */
size_t psa_legacy_index_bytes(int64_t bh, int64_t seq);
int psa_legacy_fwd_images(const void* q, const void* kimg, const void* vimg, const int32_t* mask, int32_t* index_scratch,
                          void* out, float* lse, int64_t bh, int64_t seq, int head_dim, int mask_cols, float sm_scale,
                          int causal, int dtype, int32_t* status, void* stream);

/* Legacy backward.  Replaces _sparse_attention.backward and its kernels/helpers,
 * src/psa_triton/kernels/psa_kernel_legacy.py:947-1320.  dq/dk/dv: [BH, seq, D] in dtype; delta: float32
 * [BH, seq] scratch.  Gradients follow the reference's rule (causality on original key positions of the
 * repeat-expanded pooled K/V, :1139-1150). */
int psa_legacy_bwd(const void* q, const void* k, const void* v, const void* k2, const void* k4, const void* k8,
                   const void* v2, const void* v4, const void* v8, const int32_t* mask, const void* out,
                   const float* lse, const void* dout, void* dq, void* dk, void* dv, float* delta, int64_t bh,
                   int64_t seq, int head_dim, int mask_cols, float sm_scale, int causal, int dtype, void* stream);

/* The same backward on tensor cores (warp-level mma, f16/bf16 operands, fp32 accumulation; f16/bf16 only).  Same
 * arguments and reference code as psa_legacy_bwd; the products ds*c and p*c (c = visible copies of a pooled token) are
 * rounded to the element type once more where c is 3, 5, 6 or 7 (causal diagonal, replicate-padded tail). */
int psa_legacy_bwd_tc(const void* q, const void* k, const void* v, const void* k2, const void* k4, const void* k8,
                      const void* v2, const void* v4, const void* v8, const int32_t* mask, const void* out,
                      const float* lse, const void* dout, void* dq, void* dk, void* dv, float* delta, int64_t bh,
                      int64_t seq, int head_dim, int mask_cols, float sm_scale, int causal, int dtype, void* stream);

/* The same backward on tcgen05 tensor cores with TMEM accumulators (f16/bf16, head_dim 64/128): the kernel of a training
 * step.  Same reference code as psa_legacy_bwd (psa_kernel_legacy.py:947-1320: driver :947-1069, dQ :1085-1156, dK/dV
 * :1159-1234, pool/fold :1298-1320) and the same rounding rule as psa_legacy_bwd_tc.
 * kimg/vimg: psa_pyramid_kv_images(k, v, block_n = 128), the buffers the forward psa_legacy_fwd_images read.  out/lse:
 * the forward's results.  scratch: psa_legacy_bwd_scratch_bytes() bytes, 256-byte aligned (row statistics, the fp32 sums
 * of the pooled rows of every level, work lists, two work counters); nothing in it needs initialising.
 * Launches: row statistics, work list, dQ (one persistent CTA per SM: per query block the selected key blocks of all
 * levels packed into 128-token tiles), dK/dV (per level and 128 pooled key rows: every query block that selected them),
 * fold (pooled sums -> original positions, replicate-padded tail into the last token, one rounding).
 * status: device int32 word, written non-zero if a bounded wait inside a kernel expired (may be NULL). */
size_t psa_legacy_bwd_scratch_bytes(int64_t bh, int64_t seq, int head_dim);
int psa_legacy_bwd_tcgen05(const void* q, const void* kimg, const void* vimg, const int32_t* mask, const void* out,
                           const float* lse, const void* dout, void* dq, void* dk, void* dv, void* scratch,
                           size_t scratch_bytes, int64_t bh, int64_t seq, int head_dim, int mask_cols, float sm_scale,
                           int causal, int dtype, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * Head sharding over the GPUs of one node, by peer memory instead of an all-to-all collective.  No counterpart in the
 * reference (it runs on one GPU); these calls sit where a sequence-parallel host model would otherwise call
 * all_to_all before and after the attention layer.
 *
 * psa_peer_alloc: cudaMalloc + IPC handle (64 bytes) for an exchange buffer; psa_peer_open maps a peer's handle into
 * this process (peer access is enabled on demand); psa_peer_close / psa_peer_free undo them.  Set-up calls, not for
 * the hot path.
 *
 * psa_pull_heads: dst [heads_local][n_peers*tokens_per_rank][head_dim] <- rows of heads [head0, head0+heads_local)
 * read straight from the peers' buffers peer_src[r] = [tokens_per_rank][heads_total][head_dim] (token t lives on
 * rank t / tokens_per_rank).  peer_src is a HOST array of n_peers device-accessible pointers (own buffer included).
 * The caller orders it after the peers have written their buffers (a barrier between steps); the kernel itself never
 * waits on a peer.  max_blocks caps the grid (0 = whole GPU): a copy that runs under compute kernels should stay
 * small, since each of its resident CTAs keeps a compute CTA off that SM.  self_rank (0..n_peers-1) only rotates the
 * order in which the peers are visited, so that the ranks of a node do not all read from the same GPU at once.
 *
 * psa_fwd_images_scatter: psa_fwd_images whose output rows go to the rank that owns the token:
 * peer_out[t / tokens_per_rank] laid out [tokens_per_rank][heads_total][head_dim], this rank writing heads
 * [head0, head0+bh).  peer_out is a HOST array of n_peers device-accessible pointers.
 *
 * psa_block_scores_peers / psa_pyramid_kv_images_peers: psa_block_scores (tcgen05 path) and psa_pyramid_kv_images whose
 * row-major inputs are read straight from the peers' buffers (same layout and pointer arrays as psa_pull_heads), so
 * k and v never need a local row-major copy: the score kernels touch only the sampled quarter of the q/k rows, and the
 * image builder reads every k/v element exactly once, over NVLink.  seq = n_peers * tokens_per_rank. */
int psa_block_scores_peers(const void* const* peer_q, const void* const* peer_k, int n_peers, int64_t tokens_per_rank,
                           int heads_total, int head0, const int32_t* idx_q, const int32_t* idx_k, void* po, void* scratch,
                           size_t scratch_bytes, int64_t heads_local, int head_dim, int block_m, int block_n, int dtype,
                           void* stream);
int psa_pyramid_kv_images_peers(const void* const* peer_k, const void* const* peer_v, int n_peers, int64_t tokens_per_rank,
                                int heads_total, int head0, void* kimg, void* vimg, int64_t heads_local, int head_dim,
                                int block_n, int dtype, int max_blocks, void* stream);
int psa_peer_alloc(size_t bytes, void** ptr, void* handle64);
int psa_peer_open(const void* handle64, void** ptr);
int psa_peer_close(void* ptr);
int psa_peer_free(void* ptr);
int psa_pull_heads(const void* const* peer_src, int n_peers, void* dst, int64_t tokens_per_rank, int heads_total, int head0,
                   int heads_local, int head_dim, int elem_bytes, int max_blocks, int self_rank, void* stream);
/* The same exchange in the other direction: this rank's rows src [tokens_per_rank][heads_total][head_dim] are stored into
 * the peers' head-sharded buffers peer_dst[r] = [heads_total/n_peers][n_peers*tokens_per_rank][head_dim] (rank r owns
 * heads [r*hp, (r+1)*hp)).  One sequential pass over local memory, posted stores over NVLink.  The receivers may read
 * their buffers after a barrier that follows this call on every rank. */
int psa_push_heads(const void* src, void* const* peer_dst, int n_peers, int64_t tokens_per_rank, int heads_total, int head_dim,
                   int elem_bytes, int self_rank, int max_blocks, void* stream);
/* Sampled rows first: psa_push_samples sends only the rows the block-score stage reads (a quarter of q and of k) into
 * the head owners' compacted sample matrices (peer_dst[r] = [heads_total/n_peers][n_out][head_dim]; idx = the sample
 * offsets of ALL heads, [heads_total][keep]; geometry from psa_sample_rows), and psa_block_scores_samples computes the
 * block scores from such matrices, skipping the gather of psa_block_scores.  The full rows can then travel while the
 * scores are computed. */
int psa_sample_rows(int64_t seq_q, int64_t seq_k, int block_m, int block_n, int64_t* nq, int64_t* nk_valid, int64_t* nk);
int psa_push_samples(const void* src, const int32_t* idx, void* const* peer_dst, int n_peers, int64_t tokens_per_rank,
                     int heads_total, int head_dim, int elem_bytes, int block, int keep, int64_t n_valid, int64_t n_out,
                     int self_rank, void* stream);
int psa_block_scores_samples(const void* qs, const void* ks, void* po, void* scratch, size_t scratch_bytes, int64_t bh,
                             int64_t seq_q, int64_t seq_k, int head_dim, int block_m, int block_n, int dtype, void* stream);
int psa_fwd_images_scatter(const void* q, const void* kimg, const void* vimg, const int32_t* mask, void* const* peer_out,
                           int n_peers, int64_t tokens_per_rank, int heads_total, int head0, int64_t bh, int64_t seq_q,
                           int64_t seq_k, int head_dim, int block_m, int block_n, int tile_n, int mask_width, float sm_scale,
                           int compat_quirk, int dtype, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PSA_B200_H_ */
