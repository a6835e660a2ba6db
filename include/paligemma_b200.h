/*
 * paligemma_b200.h -- C ABI of libpaligemma_b200.so: the sm_100a kernels behind the PaliGemma inference hot path.
 *
 * The reference (prtk1729/Paligemma-MultiModal-System) has no FFI: its boundary is the Python module API
 * (modeling_paligemma.py:257-307 forward, modeling_gemma.py:8-64 KVCache, inference.py:29-106 loop).  The host side of
 * this repo keeps that API in Python (paligemma_multimodal_system_b200/*.py) and reaches the GPU only through the
 * entry points below (ctypes).  Every function:
 *   - takes raw DEVICE pointers, sizes and a cudaStream_t (as void*); no torch types;
 *   - is asynchronous on `stream`; returns PG_OK or a negative PG_ERR_* code (never throws, never falls back to CPU);
 *   - cites the reference call site(s) it replaces.
 * Tensors are row-major; "ld" arguments are row pitches in ELEMENTS.
 */
#ifndef PALIGEMMA_B200_H
#define PALIGEMMA_B200_H

#ifdef __cplusplus
extern "C" {
#endif

#define PG_OK 0
#define PG_ERR_ARG (-1)    /* bad shape / alignment / enum */
#define PG_ERR_CUDA (-2)   /* launch or attribute failure (cudaGetLastError) */
#define PG_ERR_DRIVER (-3) /* cuTensorMapEncodeTiled entry point not found */
#define PG_ERR_TMAP (-4)   /* tensor-map encode rejected the geometry */
#define PG_ERR_ARCH (-5)   /* device is not sm_100 */

/* GEMM epilogues */
#define PG_EPI_BF16 0       /* out_bf16[t,f] = act((acc + bias[f]) * scale)                */
#define PG_EPI_F32 1        /* out_f32[t,f]  = (acc + bias[f]) * scale + resid_f32[t,f]    */
#define PG_EPI_ATOMIC_F32 2 /* out_f32[t,f] += (acc + bias[f]) * scale   (split-K, red.add) */
#define PG_EPI_GEGLU 3      /* out_bf16[t,g] = gelu_tanh(gate[t,g]) * up[t,g]; weight rows packed [64 gate | 64 up] */

/* Library / device info.  Returns the ABI version (>0) or PG_ERR_ARCH when the current device is not sm_100. */
int pg_abi_version(void);
int pg_check_device(void);
/* Streaming multiprocessors of the current device (the host side sizes split-K factors and persistent grids with it). */
int pg_num_sms(void);
/* Number of kernel launches this library has issued in the calling process (host-side counter). */
long long pg_launch_count(void);
/* Programmatic dependent launch for the decode-step kernels (default on): the next kernel's prologue and weight
 * prefetch overlap the running kernel; every such kernel executes griddepcontrol.wait before dependent accesses. */
int pg_set_pdl(int on);
/* Profiling aid: when non-NULL, CTA 0 of launch i writes 6 clock64 stamps to buffer[8*(i%64) ..] (device). */
int pg_debug_set_gemm_trace(long long* device_buffer);
int pg_debug_set_rmsnorm_early_trigger(int on); /* A/B runs: the decode RMSNorm triggers its dependents before / after its own dependency wait */
int pg_debug_set_gemm_pair(int mode, int min_tiles); /* A/B runs: mode bit 0 = CTA-pair (cta_group::2) prefill GEMM allowed, bit 1 = banded tile raster OFF, bits 2-3 = epilogue warps of the pair kernel (1 = eight, 2 = four, 0 = automatic) (default mode 1); min_tiles > 0 sets the pair kernel's tile-count threshold */
int pg_debug_set_attn_prefill_trace(long long* device_buffer); /* profiling aid: clock64 stamps of CTA (0,0,0) of the tcgen05 prefill attention, 3 roles x 32 tiles x 8 events */
int pg_debug_set_attn_prefill(int force_qt, int stagger_clk); /* tuning sweeps of the prefill attention: force_qt bits 0-1 = query tiles per CTA for dh <= 128, bits 4-5 = softmax warps per TMEM lane quadrant of the one-tile variant (0 = automatic); stagger_clk >= 0 = start offset of the second softmax group */
int pg_debug_set_gemm_bn(int bn); /* tuning sweeps: force the N tile (64 / 128 / 256) of the token-major GEMM, 0 = automatic */
int pg_debug_set_topp_bracket(int half_width_bins); /* > 0 overrides the estimated-bracket half width of pg_sample_top_p */
int pg_debug_topp_trace(long long* host_out16); /* clock64 stamps of CTA 0 after each phase of the last pg_sample_top_p */
int pg_debug_topp_retries(void); /* rows whose estimated top-p bracket failed verification (second full pass), cumulative */
int pg_debug_set_sampler_cluster(int ctas_per_row); /* tuning sweeps: cluster size of pg_sample_top_p_stats (1/2/4/8), 0 = automatic */
int pg_debug_set_sampler_cluster(int ctas_per_row); /* tuning sweeps: cluster size of pg_sample_top_p_stats (1/2/4/8), 0 = automatic */
int pg_debug_set_attn_trace(long long* device_buffer); /* same for pg_attention_decode_fused (8 stamps per launch) */

/*
 * acc[t,f] = sum_k x[t,k] * w[f,k]  (bf16 in, fp32 accumulate on tcgen05 tensor cores, accumulator in TMEM).
 * Replaces every nn.Linear on the path: modeling_siglip.py:59-62,71-75,156,177-185; modeling_paligemma.py:57,64;
 * modeling_gemma.py:205-218,255-259,274-278,356,484,523; and nn.Conv2d (modeling_siglip.py:258-263) after pg_im2col.
 *   swap:   0 = tokens on the UMMA M axis (prefill), 1 = features on the M axis (decode, tokens <= 128), -1 = auto
 *   split_k: >1 only with PG_EPI_ATOMIC_F32
 */
int pg_gemm_bf16(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo,
                 const float* bias, const float* resid, long long ldr, int tokens, int features, int K, int mode,
                 int act_gelu /* 0 none, 1 gelu(tanh), 2 relu(x)^2: bf16 epilogue */, float scale, int swap, int split_k, void* stream);

/*
 * pg_gemm_bf16 with per-call-site extras; `fusion` may be NULL (= pg_gemm_bf16).  zero_buf and stats belong to the swap-AB
 * (tokens <= 128, decode) kernels, resid_row_mod to the token-major (prefill) kernels.
 *
 *  - zero_buf / zero_count: zero-filled (fp32, count % 4 == 0, 16-byte aligned) after the dependency wait; o_proj uses it to
 *    reset the split-K accumulator of the q/k/v projection once the attention kernel has consumed it.
 *  - stats (PG_EPI_F32 only, no resid / split-K): the lm_head of a decode step (modeling_gemma.py:523-525) also emits, for
 *    every token t and every 32-row vocabulary segment g (g = f / 32), stats[g * stats_ld + t] = (m, s) with
 *    m = max logit of the segment and s = sum exp2((logit - m) * stat_c), stat_c = inv_temperature * log2(e) -- temperature
 *    scaling and the max / partition-function passes of softmax + top-p (inference.py:63-66,90-106) folded into the GEMM
 *    epilogue; consumed by pg_sample_top_p_stats / pg_argmax_stats.  float2 [4 * ceil(features / 128)][stats_ld >= tokens].
 *  - resid_row_mod > 0 (token-major kernels, PG_EPI_F32 with resid): the residual row of token t is t % resid_row_mod, i.e.
 *    resid is a [resid_row_mod, features] table broadcast over the batch -- the position-embedding add of the SigLIP patch
 *    embedding (modeling_siglip.py:289-298) folded into the patch GEMM's epilogue.
 *  - out_row_map (token-major kernels, PG_EPI_F32 without resid): token t is written to output row out_row_map[t] -- the
 *    multimodal projector (modeling_paligemma.py:57-65) scattering its rows, times `scale`, straight to the `<image>` positions of
 *    the merged embedding sequence (masked_scatter of _merge_input_ids_with_image_features, :201-251); map from pg_merge_scan.
 *  - PG_EPI_GEGLU takes the kind of gated unit from act_gelu: 0 / 1 gelu_tanh(g) * u, 3 silu(g) * u, 4 the clamped form
 *    g' = min(g, c), u' = clamp(u, -c, c), g' * sigmoid(glu_alpha * g') * (u' + 1) with c = `scale` (glu_alpha 0 reads as 1).  In this
 *    mode `bias` (fp32 [features]) is in the packed row order of the weight ([64 gate | 64 up] per 128 rows) and is added before
 *    the gated unit.
 */
typedef struct PgGemmFusion {
  float* zero_buf;
  long long zero_count;
  void* stats;
  long long stats_ld;
  float stat_c;
  int resid_row_mod;
  const int* out_row_map;
  float glu_alpha;
} PgGemmFusion;
int pg_gemm_bf16_fused(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo,
                       const float* bias, const float* resid, long long ldr, int tokens, int features, int K, int mode,
                       int act_gelu, float scale, int swap, int split_k, const PgGemmFusion* fusion, void* stream);

/*
 * Prefill q/k/v projection with RoPE and the KV-cache append in the GEMM epilogue (modeling_gemma.py:274-302 + KVCache.update
 * :18-57): qkv_out[t, :] = bf16 of [rope(q heads) | rope(k heads) | v heads] of x[t, :] @ w^T, w = [q_proj; k_proj; v_proj]
 * ([(Hq + 2 Hkv) * dh, K] bf16), rotate-half with angle pos[t] * inv_freq[i]; k / v rows are also written into their cache
 * pages (page = page_table[b * max_pages + slot / 64], slot = slot_base[b] + (t - b * tokens_per_seq); k_pages == NULL: no
 * cache).  One head per UMMA N tile: dh in {64, 256}.  The prefill attention reads q / k / v straight out of qkv_out through
 * strided tensor maps, so no separate RoPE / append launch and no second copy of the projections exists.
 */
int pg_gemm_qkv_rope(const void* x, long long ldx, const void* w, long long ldw, void* qkv_out, long long ldo, int tokens, int K,
                     int Hq, int Hkv, int dh, const int* pos, const float* inv_freq, void* k_pages, void* v_pages,
                     const int* page_table, const int* slot_base, int tokens_per_seq, int page_size, int max_pages, void* stream);

/* Packs gate_proj / up_proj [F,K] bf16 into the [64 gate | 64 up] row-interleaved [2F,K] layout PG_EPI_GEGLU expects.
 * (modeling_gemma.py:205-206 weights; F % 64 == 0) */
int pg_pack_gate_up(const void* gate, const void* up, void* packed, int F, int K, void* stream);

/* fp32 -> bf16 cast (weight packing, pixel staging). */
int pg_cast_f32_bf16(const float* src, void* dst, long long n, void* stream);

/* nn.LayerNorm (modeling_siglip.py:199-204,310,319): x fp32 [rows, D] -> y bf16 (and/or fp32 if y_f32 != NULL). */
int pg_layernorm(const float* x, const float* gamma, const float* beta, void* y_bf16, float* y_f32, int rows, int D,
                 float eps, void* stream);

/* GemmaRMSNorm (modeling_gemma.py:157-182): y = x * rsqrt(mean(x^2) + eps) * (1 + w); x fp32 -> y bf16.  (Prefill, and the
 * decode norms.) */
int pg_rmsnorm(const float* x, const float* w, void* y_bf16, int rows, int D, float eps, void* stream);

/*
 * Image path of PaliGemmaProcessor (processing_paligemma.py:13-73) on the GPU, bit-exact with the reference's CPU path:
 * Pillow's 8-bit bicubic resize as two separable fixed-point passes, then rescale / normalise / HWC->CHW.
 *   pg_resample_h_u8:      src uint8 [H, W, 3] -> dst uint8 [H, S, 3]     (image.resize, horizontal pass, :17-19)
 *   pg_resample_v_u8_norm: src uint8 [H, Wd, 3] -> out fp32 [3, S, Wd]    (vertical pass + lut[256] = the reference's
 *                          (u * 1/255).astype(float32), (x - 0.5) / 0.5 of :21-33, + the transpose of :71)
 * kk int32 [S, ksize] 22-bit fixed-point weights and bounds int32 [S, 2] = (first input index, count) are built by the
 * host exactly as Pillow's precompute_coeffs / normalize_coeffs_8bpc do (image_preprocess.py).
 */
int pg_resample_h_u8(const void* src, void* dst, int H, int W, int S, const int* kk, const int* bounds, int ksize, void* stream);
int pg_resample_v_u8_norm(const void* src, float* out, int H, int Wd, int S, const int* kk, const int* bounds, int ksize,
                          const float* lut, void* stream);

/* SiglipVisionEmbeddings im2col (modeling_siglip.py:258-263,285-297): pixel fp32 [B,C,H,W] -> patches bf16
 * [B*(H/P)*(W/P), Kpad], column order (c, py, px) = Conv2d weight order, zero padded to Kpad. */
int pg_im2col(const float* pixels, void* patches, int B, int C, int H, int W, int P, int Kpad, void* stream);

/*
 * Non-causal softmax(Q K^T * scale) V, flash style (modeling_siglip.py:96-136; modeling_gemma.py:307-339 prefill
 * with the all-zero mask of modeling_paligemma.py:154-156).  bf16 in/out, fp32 softmax.
 * Row r of batch b, head h:  q + b*q_bs + (r / group)*q_ts + (r % group)*q_hs + h*q_head_off  (same for o);
 * K/V rows: k + b*kv_bs + n*kv_ts + h*kv_head_off.  `group` > 1 stacks the query heads of one KV head as consecutive
 * rows (MQA/GQA, replaces repeat_kv modeling_gemma.py:185-196).  All strides in elements.  dh in {64, 72, 256}.
 */
int pg_attention_prefill(const void* q, const void* k, const void* v, void* o, int B, int H, int rows, int keys, int dh,
                         int group, long long q_bs, long long q_ts, long long q_hs, long long q_head_off,
                         long long kv_bs, long long kv_ts, long long kv_head_off, long long o_bs, long long o_ts,
                         long long o_hs, long long o_head_off, float scale, void* stream);

/*
 * pg_attention_prefill for a ragged batch (prompts of different lengths in one prefill; the reference
 * runs B = 1, inference.py:69, and never masks padding, modeling_paligemma.py:154-156): problem b attends only to its first
 * key_lens[b] keys (int32 [B] on the device, clamped to [1, keys]).  Rows past a problem's length are computed and must be
 * ignored by the caller; K/V rows in [key_lens[b], keys) must hold finite values.  tcgen05 kernel only (dh 64 / 72 / 256,
 * 128 % group == 0, 16-byte aligned strides): other shapes return PG_ERR_ARG.
 */
int pg_attention_prefill_varlen(const void* q, const void* k, const void* v, void* o, const int* key_lens, int B, int H,
                                int rows, int keys, int dh, int group, long long q_bs, long long q_ts, long long q_hs,
                                long long q_head_off, long long kv_bs, long long kv_ts, long long kv_head_off,
                                long long o_bs, long long o_ts, long long o_hs, long long o_head_off, float scale,
                                void* stream);

/*
 * RoPE + KV append (modeling_gemma.py:116-151,285-302 and KVCache.update :18-57): reads qkv [T, (Hq+2Hkv)*dh]
 * (bf16, or fp32 when qkv_is_f32), rotates q and k (rotate-half, fp32 angle = pos[t] * inv_freq[i], inv_freq fp32 [dh/2] built by the host exactly as
 * GemmaRotaryEmbedding.__init__ does), writes q_out bf16
 * [T, Hq*dh], optional k_out/v_out bf16 [T, Hkv*dh] (dense, for prefill attention) and appends k/v into the paged
 * cache: page = page_table[b*max_pages + slot/page_size], slot = slot_base[b] + (t - b*tokens_per_seq).
 */
int pg_rope_kv_append(const void* qkv, int qkv_is_f32, const int* pos, void* q_out, void* k_out, void* v_out,
                      void* k_pages, void* v_pages, const int* page_table, const int* slot_base, int B,
                      int tokens_per_seq, int Hq, int Hkv, int dh, int page_size, int max_pages,
                      const float* inv_freq, void* stream);

/*
 * Decode-step attention in ONE launch (modeling_gemma.py:285-339 at q_len == 1 + KVCache.update :18-57): rotates q and
 * the new k (fp32 qkv [B, (Hq+2Hkv)*dh] straight from the split-K QKV GEMM), appends k/v to the paged cache at slot
 * kv_len[b]-1 and attends over kv_len[b] keys.  One thread-block cluster per (sequence, kv head): each rank streams a
 * contiguous range of 64-key pages (TMA tensor loads into 128B-swizzled shared memory) and the ranks merge through
 * distributed shared memory.  num_pages = pages in the pool (k_pages / v_pages are [num_pages, 64, Hkv*dh] bf16).
 * GQA group Hq/Hkv <= 8, dh in {64, 256}.
 */
int pg_attention_decode_fused(const float* qkv, const int* pos, const int* kv_len, const float* inv_freq, void* k_pages,
                              void* v_pages, const int* page_table, void* out, int B, int Hq, int Hkv, int dh,
                              int page_size, int num_pages, int max_pages, float scale, void* stream);

/* Gathers the dense K or V of one layer, [B, Hkv, len, dh] bf16, from the paged cache (KVCache.k_cache / v_cache
 * views, modeling_gemma.py:8-64). */
int pg_kv_gather(const void* pages, const int* page_table, void* dense, int B, int len, int Hkv, int dh, int page_size,
                 int max_pages, void* stream);

/*
 * Embedding gather + image-feature merge (+ position ids)
 * (modeling_paligemma.py:93-128,195,288 and the *sqrt(hidden) of modeling_gemma.py:510-511):
 *   text token : h[b,s,:] = embed[id,:] * text_scale      image token (j-th in row b): h = img[b,j,:] * img_scale
 *   pad token  : 0                                         pos[b,s] = cumsum(mask)[s], 1 where mask == 0
 * embed bf16 [V,D]; img fp32 [B,N,D]; h fp32 [B,S,D]; src_scratch int32 [B,S].  err_flag[0] is set to 1 when a row
 * does not hold exactly N image tokens (the reference leaves this unchecked, modeling_paligemma.py:120-121).
 */
int pg_merge_embeddings(const long long* input_ids, const long long* attn_mask, const void* embed, const float* img,
                        float* h, int* pos, int* src_scratch, int* err_flag, int B, int S, int D, int N,
                        long long image_token, long long pad_token, float text_scale, float img_scale, void* stream);

/*
 * The same merge as two halves around the projector GEMM, so that the image features never take a round trip of their own:
 *   pg_merge_scan  -> pos[b,s], src_scratch[b,s] (j >= 0: j-th image token | -1 text | -2 pad), err_flag, and (dst_row != NULL)
 *                     dst_row[b*N + j] = b*S + s: the merged row of image feature j, the out_row_map of the projector GEMM;
 *   pg_merge_text  -> fills the text / pad rows of h (embedding gather * text_scale, zeros) and leaves the image rows alone.
 */
int pg_merge_scan(const long long* input_ids, const long long* attn_mask, int* pos, int* src_scratch, int* dst_row, int* err_flag,
                  int B, int S, int N, long long image_token, long long pad_token, void* stream);
int pg_merge_text(const long long* input_ids, const int* src_scratch, const void* embed, float* h, int B, int S, int D, int N,
                  float text_scale, void* stream);

/* Decode-step embedding with the same merge rules at q_len = 1; tokens are int32 on the device; img may be NULL. */
int pg_embed_tokens(const int* tokens, const void* embed, const float* img, float* h, int B, int D, int N,
                    float text_scale, float img_scale, long long pad_token, long long image_token, void* stream);

/* Greedy argmax over fp32 logits [B, V] (inference.py:68); ties -> lowest index.  out int32 [B]. */
int pg_argmax(const float* logits, long long ld, int* out, int B, int V, void* stream);

/*
 * Top-p sampling (inference.py:65,90-106) from fp32 logits [B, V]: probs = softmax(logits * inv_temperature);
 * keep every token whose strictly-greater probability mass is <= top_p (= the reference's exclusive-cumsum rule; tied
 * probabilities are kept or dropped together); sample from the renormalised kept set by inverse CDF in vocabulary
 * order with a counter-based RNG keyed by (seed, *step_ptr, row).  out int32 [B]; kept_count optional int32 [B].
 */
int pg_sample_top_p(const float* logits, long long ld, int* out, int* kept_count, int B, int V, float inv_temperature,
                    float top_p, unsigned long long seed, const int* step_ptr, void* stream);

/*
 * The same two samplers fed by the segment statistics the lm_head epilogue emits (PgGemmFusion.stats: per 32-token vocabulary
 * segment, max logit and sum exp2((x - max) * inv_temperature * log2 e)): row maximum, partition function and the segment
 * masses of the inverse-CDF draw come from 8 bytes per segment instead of passes over the fp32 row; only the top-p
 * verification pass (mass of strictly more probable tokens <= top_p, inference.py:96-100) still reads the logits.
 * stats: float2 [ceil(V / 32) or more segment rows][stats_ld >= B]; the statistics must have been produced with the SAME
 * inv_temperature.  seed_ptr (device, optional) overrides `seed`, so that a captured CUDA graph serves every seed.
 * A row whose 64 candidates are all rejected (top_p far below the largest probability) yields its most probable token.
 */
int pg_argmax_stats(const float* logits, long long ld, const void* stats, long long stats_ld, int* out, int B, int V,
                    void* stream);
int pg_sample_top_p_stats(const float* logits, long long ld, const void* stats, long long stats_ld, int* out, int B, int V,
                          float inv_temperature, float top_p, unsigned long long seed, const unsigned long long* seed_ptr,
                          const int* step_ptr, void* stream);

/* After sampling (device-side loop state, CUDA-graph friendly): tok_hist[step*B + b] = next[b]; cur_tok[b] = next[b];
 * counters[c*B + b] += 1 for c < n_counters (position ids, KV write slots, KV lengths); step += 1.  B <= 1024. */
int pg_advance_decode(const int* next, int* tok_hist, int* cur_tok, int* counters, int n_counters, int* step, int B,
                      void* stream);

/* pg_advance_decode for continuous batching (the inference.py:45-79 loop state of B independent requests, one per slot):
 * tok_ring[(step % ring)*B + b] = next[b]; cur_tok[b] = next[b]; the three counters of slot b (int32 [3, B]: position id, KV
 * write slot, KV length) advance only while counters[2][b] < kv_limit[b] -- a slot that has used its budget (finished or
 * idle) is frozen until the host re-arms it; step += 1. */
int pg_advance_decode_slots(const int* next, int* tok_ring, int ring, int* cur_tok, int* counters, const int* kv_limit,
                            int* step, int B, void* stream);

/* Decode chain, no reference counterpart (the reference's nn.Linear weights sit in host caches): asks the bulk-copy engine to
 * pull the contiguous range [ptr, ptr + bytes) -- the weights of a LATER GEMM of the decode step (modeling_gemma.py:205-218
 * gate/up/down projections) -- into L2 and returns at once.  Meant for a forked branch of the step's CUDA graph, while the
 * attention block leaves the HBM idle.  `ctas` (0 = one per SM) paces the stream: every CTA keeps one SM's bulk-copy engine busy
 * (~80 GB/s), so a small grid is a background stream that leaves HBM bandwidth to the critical-path loads.  evict_last != 0
 * tags the lines L2::evict_last (measured: no benefit for the gate/up weights, kept for experiments).  ptr 16-byte aligned,
 * bytes >= 16 (rounded down to a multiple of 16).  Never changes results. */
int pg_prefetch_l2(const void* ptr, long long bytes, int ctas, int evict_last, void* stream);

/* ---------------------------------------------------------------------------------------------------------------------
 * Token-sequence decoders (models/registry: text-only designs served through a ragged step).  A step's rows are the new
 * tokens of several requests ("entries"): entry e owns rows [entry_row0[e], entry_row0[e] + entry_n[e]) and continues a
 * sequence of entry_ctx[e] tokens that already sit in the paged cache / the recurrent state.  "act" tensors are bf16
 * (act_f32 = 0) or fp32 (act_f32 = 1); norms, scores, probabilities, states and residual sums are always fp32.
 * ------------------------------------------------------------------------------------------------------------------- */

/* out[t, f] = sum_k x[t, k] w[f, k] with plain fp32 FMAs (no tensor-core mode): the exact-precision matrix product of
 * the fp32 serving mode, and the bf16 product for shapes the TMA kernels cannot take (K or a pitch not a multiple of 8).
 * in_f32: x and w are fp32 (else bf16); out_f32: out is fp32 (else bf16). */
int pg_gemm_simt(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo, int tokens, int features,
                 int K, int in_f32, int out_f32, void* stream);

/* pg_layernorm_shift: rows of x (fp32 [rows, D]) through one or two layer norms that share the row's mean and variance:
 *   a = (x - mean) / sqrt(var + eps) * w1 + b1 -> out1, the same with (w2, b2) -> out2 (out2 NULL: one norm).
 * shift != NULL (fp32 [D]): out1[t] = a[t] + (a[t-1] - a[t]) * shift, where a[t-1] belongs to the previous token of the SAME
 * sequence: zeros at position 0, the row before inside an entry, and for an entry's first row the fp32 state slot
 * state[entry_slot[e], 0:D], which afterwards holds a of the entry's last row.  out1 / out2: bf16, or fp32 when out_f32.
 * pg_glu: out[t, f] from gu[t, f] (gate) and gu[t, F + f] (up): kind 1 silu(g) * u; kind 2 g' = min(g, limit),
 *   u' = clamp(u, -limit, limit), g' * sigmoid(alpha * g') * (u' + 1). */
int pg_layernorm_shift(const float* x, const float* w1, const float* b1, const float* shift, const float* w2, const float* b2, void* out1,
                       void* out2, float* state, const int* pos, const int* row_entry, const int* entry_row0, const int* entry_n,
                       const int* entry_slot, int rows, int D, float eps, int out_f32, void* stream);
int pg_glu(const void* gu, long long ldgu, void* out, long long ldo, int rows, int F, int kind, float limit, float alpha, int act_f32,
           void* stream);

/* The same product with out[t, f] = (sum + bias[f]) * scale (bias fp32 [features] or NULL) + (accumulate != 0 ? out[t, f] : 0):
 * projections with biases and projections that add into the fp32 residual stream (scale: a residual multiplier). */
int pg_gemm_simt_bias(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo, const float* bias,
                      int accumulate, float scale, int tokens, int features, int K, int in_f32, int out_f32, void* stream);

/* ---- normalised residual read through a short causal convolution; polynomial-of-norms activation ------------------------------
 * pg_rmsnorm_conv: h[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w (w: fp32 [D], or ONE number when w_scalar != 0); out_h[t] = h[t];
 *   out_conv[t, c] = h[t, c] + sum_{j < taps} conv_w[j * D + c] * h[t - taps + 1 + j, c] (conv_w tap-major: fp32 [taps, D]), where rows before the sequence's
 *   start are zeros and rows before this step come from state (fp32 [slots, taps - 1, D]: the last taps - 1 rows h of the
 *   sequence in slot entry_slot[e], oldest first; ignored when entry_ctx[e] == 0; rewritten here).  conv_w NULL: no convolution,
 *   no state (a bare norm; out_conv, when given, equals out_h).  Either output may be NULL.  taps <= 8.  entries = number of entries
 *   of the step (0: unknown; steps of thousands of rows then stay on the one-CTA-per-row kernel).
 * pg_polynorm: out[t, f] = a N(z)[f] + b N(z^2)[f] + c N(z^3)[f] + e with (a, b, c, e) = coef[0..3] (fp32, device), powers taken
 *   element by element and N(v) = v / sqrt(mean_f(v^2) + eps); z and out in the activation type, statistics fp32.
 * pg_sigmoid_gate_mul: y[t, c] *= sigmoid(gate[t, c]) for c < n (both in the activation type, pitches ldy / ldg). */
int pg_rmsnorm_conv(const float* x, const float* w, int w_scalar, const float* conv_w, int taps, float* state, void* out_h, void* out_conv,
                    const int* row_entry, const int* entry_row0, const int* entry_n, const int* entry_ctx, const int* entry_slot, int rows, int entries,
                    int D, float eps, int out_f32, void* stream);
int pg_polynorm(const void* z, long long ldz, const float* coef, void* out, long long ldo, int rows, int F, float eps, int act_f32, void* stream);
int pg_sigmoid_gate_mul(void* y, long long ldy, const void* gate, long long ldg, int rows, int n, int act_f32, void* stream);

/* grid.z = batch independent products out_b = x_b w_b^T; operand b starts batch_* elements after operand b - 1 (per-head
 * projections: x a column slice per head, w one matrix per head). */
int pg_gemm_simt_batched(const void* x, long long ldx, long long batch_x, const void* w, long long ldw, long long batch_w, void* out,
                         long long ldo, long long batch_out, int tokens, int features, int K, int batch, int in_f32, int out_f32,
                         void* stream);

/* out[t, 0:D] (fp32) = table[tokens[t], col0 : col0 + D] * scale  (embedding lookup; table bf16 or fp32, pitch ld). */
int pg_embed_rows(const int* tokens, const void* table, long long ld, int col0, float* out, int rows, int D, float scale,
                  int table_f32, void* stream);

/* Grouped RMS norm folded into the residual add: r = gnorm(y[t, :]) * w, where the row is cut into `groups` equal
 * consecutive parts and each part is divided by sqrt(mean(part^2) + eps).  x != NULL: x[t, :] += r in place (fp32 residual
 * stream); x == NULL: the bare norm.  out_act != NULL also receives the result (new residual or bare norm) in the activation
 * type -- the operand of the next matrix product. */
int pg_group_rmsnorm_add(const float* y, long long ldy, const float* w, float* x, void* out_act, int rows, int D, int groups,
                         float eps, int out_f32, void* stream);

/* out[t, :] = o[t, :] / sqrt(mean(o[t, :]^2) + eps) * w * sigmoid(gate[t, :])   (o fp32 [rows, D]; gate / out: act type). */
int pg_rmsnorm_gate(const float* o, const float* w, const void* gate, long long ldg, void* out, int rows, int D, float eps,
                    int act_f32, void* stream);

/* out[t, f] = gelu_tanh(gu[t, f]) * gu[t, F + f]: the gate || up product when it is not fused into the GEMM epilogue. */
int pg_geglu(const void* gu, long long ldgu, void* out, long long ldo, int rows, int F, int act_f32, void* stream);

/* x[t, f] <- relu(x[t, f])^2 in place (rows x F, pitch ld): the activation when it is not fused into the GEMM epilogue. */
int pg_relu2(void* x, long long ld, int rows, int F, int act_f32, void* stream);

/* out[t, j] = gelu_tanh(z[t, j]) * table[tokens[t], col0 + j] for j < n, 0 for n <= j < n_pad (per-token side input: a
 * gate projection of the residual, fp32, times the token's own low-dimensional embedding slice). */
int pg_side_gate(const float* z, long long ldz, const int* tokens, const void* table, long long ldt, int col0, void* out,
                 long long ldo, int rows, int n, int n_pad, int act_f32, void* stream);

/* Softmax-attention front end on the fused projection rows qkv[t] = [q heads | k heads | v heads | ...] (pitch ld):
 * q and k heads are RMS-normalised over dim with the shared weights q_norm / k_norm, then the first rot_dims dimensions are
 * rotated in interleaved pairs (2i, 2i+1) by pos[t] * freq[i] (freq: double [rot_dims / 2]); v heads are divided by their
 * root mean square over vdim.  q goes to q_out [rows, H * dim]; k and v go to cache row
 * page_table[row_entry[t] * max_pages + pos[t] / page] * page + pos[t] % page of k_pages [.., G * dim] / v_pages [.., G * vdim].
 * norm_qk == 0 / norm_v == 0 leave out the q/k norm / the value norm; q_norm, k_norm NULL: a norm without a weight; k_pages and
 * v_pages both NULL: the row holds queries only (a layer that attends over another layer's cache).  v_from_k != 0: the row is
 * [q heads | k heads | ...] and value head g is key head g as projected, before norm and rotation (vdim == dim). */
int pg_attn_prepare(const void* qkv, long long ld, const int* pos, const int* row_entry, const int* page_table, int max_pages,
                    int page, const double* freq, const float* q_norm, const float* k_norm, void* q_out, void* k_pages,
                    void* v_pages, int rows, int H, int G, int dim, int vdim, int rot_dims, float eps, int norm_qk, int norm_v, int v_from_k,
                    int act_f32, void* stream);

/* Optional parts of a softmax attention's score and mask, read by pg_attn_ragged, pg_attn_ragged_mma, pg_attn_decode and
 * pg_attn_decode_merge (a NULL pointer or an all-zero struct: plain causal attention).  With i the query's position and j a key's:
 *   window > 0      j is visible only when i - j < window, or j < keep_first (the first keys of a sequence stay visible; they
 *                   keep their true positions);
 *   sink            [H] fp32: exp(sink[h]) joins the softmax denominator once, with no key, no value and no scale;
 *   dist_a, dist_b  [H] fp32 each: the score loses dist_a[h] * log(1 + dist_b[h] * (i - j));
 *   head_scale      [H] fp32: the scaled dot product is multiplied by head_scale[h] (before the distance term is taken off). */
typedef struct PgAttnScore {
  int window;
  int keep_first;
  const float* sink;
  const float* dist_a;
  const float* dist_b;
  const float* head_scale;
} PgAttnScore;

/* Causal attention of every entry's new rows over its cached keys / values (query head h reads k/v head h / (H / G)):
 * s = (q . k) * scale, s <- softcap * tanh(s / softcap) when softcap > 0, softmax over keys 0 .. position, times V; the
 * result is multiplied by sigmoid(gate[t, h * vdim + c]) when gate != NULL and written to out [rows, H * vdim].
 * page_table: int32 [entries, max_pages]; max_n = the largest entry_n (sizes the grid).  skip_single != 0 leaves entries with
 * entry_n == 1 to pg_attn_decode.
 * pg_attn_decode handles ONLY entries with entry_n == 1 (decoded tokens): nsplit CTAs per (entry, k/v head) share the keys,
 * every warp streams its own 32-key tiles from the pages; with nsplit > 1 the partial (max, sum, accumulator) triples go
 * through `partial` (fp32 [entries, H, nsplit, vdim + 2]) and a merge launch.
 * krow / vrow: elements between consecutive cache rows of k_pages / v_pages (<= 0: G * dim, G * vdim).  A cache that keeps one
 * row per token serving as key AND value (latent attention: G = 1, v_pages == k_pages, vrow == krow, the value is the first
 * vdim columns of the key row) is staged once per tile.  gate_per_head != 0: one gate scalar per head, gate[t * ldg + h]. */
int pg_attn_ragged(const void* q, const void* k_pages, const void* v_pages, const void* gate, long long ldg, void* out,
                   const int* entry_row0, const int* entry_n, const int* entry_ctx, const int* page_table, int max_pages, int page,
                   int entries, int max_n, int H, int G, int dim, int vdim, float scale, float softcap, int skip_single, int act_f32,
                   long long krow, long long vrow, int gate_per_head, const PgAttnScore* score, void* stream);
/* pg_attn_ragged for bf16 activations on the tensor cores (mma.sync m16n8k16): S = Q K^T from the bf16 operands with fp32
 * accumulation; the fp32 probabilities are cut into three bf16 terms each and P V runs as three passes over the bf16 values,
 * so no probability is rounded to bf16.  Head sizes (dim, vdim) in {(32,32), (64,64), (128,128), (64,128), (128,64), (96,64),
 * (192,128)}; anything else returns PG_ERR_ARG and belongs to pg_attn_ragged. */
int pg_attn_ragged_mma(const void* q, const void* k_pages, const void* v_pages, const void* gate, long long ldg, void* out,
                       const int* entry_row0, const int* entry_n, const int* entry_ctx, const int* page_table, int max_pages, int page,
                       int entries, int max_n, int H, int G, int dim, int vdim, float scale, float softcap, int skip_single,
                       int gate_per_head, const PgAttnScore* score, void* stream);
int pg_attn_decode(const void* q, const void* k_pages, const void* v_pages, const void* gate, long long ldg, void* out, float* partial,
                   const int* entry_row0, const int* entry_n, const int* entry_ctx, const int* page_table, int max_pages, int page,
                   int entries, int nsplit, int H, int G, int dim, int vdim, float scale, float softcap, int act_f32, long long krow,
                   long long vrow, int gate_per_head, const PgAttnScore* score, void* stream);

/* The merge launch of pg_attn_decode on its own: rows of single-token entries from `partial` (fp32 [entries, H, nsplit, vdim + 2]:
 * running max in natural-log units, sum, unnormalised accumulator), times the gate, to out [rows, H * vdim]. */
int pg_attn_decode_merge(const float* partial, const void* gate, long long ldg, void* out, const int* entry_row0, const int* entry_n,
                         int entries, int nsplit, int H, int vdim, int gate_per_head, int act_f32, const PgAttnScore* score, void* stream);
/* Single-token entries of a latent-attention layer (absorbed form) on the tensor cores, bf16: q [rows, H, dim] against the
 * one-row-per-token cache `pages` [.., page, dim] whose first vdim columns are the values; all heads of a token share one key
 * tile (mma.sync, fp32 probabilities as three bf16 terms, values read from the key tile with ldmatrix.trans).  gate: one scalar
 * per head (gate[t * ldg + h]) or NULL.  nsplit > 1: partial triples in the layout above, to be finished by pg_attn_decode_merge.
 * window > 0: a token at position i reads keys i - window + 1 .. i only (0: all keys).
 * (dim, vdim) in {(96,64), (160,128), (192,128), (288,256), (544,512), (576,512)}; anything else returns PG_ERR_ARG and belongs to pg_attn_decode. */
int pg_attn_latent_decode_mma(const void* q, const void* pages, const void* gate, long long ldg, void* out, float* partial,
                              const int* entry_row0, const int* entry_n, const int* entry_ctx, const int* page_table, int max_pages,
                              int page, int entries, int nsplit, int H, int dim, int vdim, float scale, int window, void* stream);

/* Decayed linear attention on qkv[t] = [q heads | k heads | v heads | ...] (q, k: H x dim, v: H x vdim; silu applied here):
 * per head S <- decay[h] * S + k v^T, out[t, h * vdim + :] = S^T q (fp32).  state: fp32 [slots, H, dim, vdim]; entry e
 * continues state[entry_slot[e]] (from zero when entry_ctx[e] == 0) and leaves its new state there.
 * pg_linear_attn_scan steps token by token; pg_linear_attn_chunked advances in blocks of 32 tokens (same results up to
 * fp32 summation order) and is meant for prompt portions. */
int pg_linear_attn_scan(const void* qkv, long long ld, float* state, const float* decay, float* out, const int* entry_row0,
                        const int* entry_n, const int* entry_ctx, const int* entry_slot, int entries, int H, int dim, int vdim,
                        int act_f32, void* stream);
int pg_linear_attn_chunked(const void* qkv, long long ld, float* state, const float* decay, float* out, const int* entry_row0,
                           const int* entry_n, const int* entry_ctx, const int* entry_slot, int entries, int H, int dim, int vdim,
                           int act_f32, void* stream);

/* ---- multi-stream residual ("hyper-connections"): xs fp32 [rows, S, D], S <= 16 ------------------------------------------------
 * pg_embed_streams: xs[t, s, :] = table[tokens[t], 0:D] * scale for every stream s.
 * pg_stream_mix_norm, per row, in this order:
 *   y != NULL:         x_to <- sum_s mix[s * S + to] x_s + write_coef[to] * y[t, :]   (all streams from the old ones, in place)
 *   read_coef != NULL: u = sum_s read_coef[s] x_s;  out_act[t, :] = u / sqrt(mean(u^2) + eps) * norm_w  (norm_w NULL: no weight)
 * y, mix, write_coef come together; read_coef and out_act come together. */
int pg_embed_streams(const int* tokens, const void* table, long long ld, float* xs, int rows, int S, int D, float scale, int table_f32,
                     void* stream);
int pg_stream_mix_norm(float* xs, const float* y, long long ldy, const float* mix, const float* write_coef, const float* read_coef,
                       const float* norm_w, void* out_act, int rows, int S, int D, float eps, int out_f32, void* stream);

/* ---- latent attention: the cache keeps one row [c (rank) | r (rot)] per token ---------------------------------------------------
 * pg_latent_prepare: proj[t] = [q latent (q_rank) | kv latent (rank) | key part (rot) | ...] (pitch ld).  cq_out[t, :] =
 *   rms(q latent) * q_norm (skipped when q_rank == 0); cache row of position pos[t] <- [rms(kv latent) * c_norm | key part with
 *   its first rot_dims dimensions rotated in interleaved pairs by pos[t] * freq[i]].  pages: [.., page, rank + rot].
 *   rot_gain multiplies the cosines and sines (1: a pure rotation).  pages NULL (q_rank > 0): only cq_out is made -- a layer that
 *   reads another layer's cached rows; proj then holds [q latent | ...].
 * pg_rotate_heads: for every row and head, n elements at src[t * ld_src + h * head_stride_src ..] are copied to
 *   dst[t * ld_dst + h * head_stride_dst ..] with the first rot_dims rotated the same way.
 * pg_latent_gather: lat[dense_row0[e] + j, 0:rank] <- cached row j of entry e, j < ctx + n (width = elements per cache row).
 *   Entries with n == 1 are skipped here and in pg_latent_pack_kv (they own no dense rows).
 * pg_latent_pack_kv: up[row] = [H x dim plain key parts | H x vdim values] (pitch ld_up) of the gathered rows ->
 *   k_out[row, h, :] = [plain (dim) | cached rotated part (rot)], v_out[row, h, :]. */
int pg_latent_prepare(const void* proj, long long ld, const int* pos, const int* row_entry, const int* page_table, int max_pages,
                      int page, const double* freq, const float* q_norm, const float* c_norm, void* cq_out, void* pages, int rows,
                      int q_rank, int rank, int rot, int rot_dims, float eps, float rot_gain, int act_f32, void* stream);
int pg_rotate_heads(const void* src, long long ld_src, long long head_stride_src, void* dst, long long ld_dst, long long head_stride_dst,
                    const int* pos, const double* freq, int rows, int H, int n, int rot_dims, float rot_gain, int act_f32, void* stream);
int pg_latent_gather(const void* pages, const int* page_table, int max_pages, int page, const int* dense_row0, const int* entry_n,
                     const int* entry_ctx, void* lat, int entries, int max_len, int rank, int width, int act_f32, void* stream);
int pg_latent_pack_kv(const void* up, long long ld_up, const void* pages, const int* page_table, int max_pages, int page,
                      const int* dense_row0, const int* entry_n, const int* entry_ctx, void* k_out, void* v_out, int entries, int max_len,
                      int H, int dim, int rot, int vdim, int rank, int act_f32, void* stream);

/* ---- routed feed-forward (mixture of experts), everything on the device ---------------------------------------------------------
 * pg_moe_route: logits fp32 [tokens, n_all] (pitch ld).  p = softmax(logits); choice = p + correction (NULL: none); with
 *   group_count > 1 the outputs form group_count equal runs of neighbours and only the group_keep runs with the largest best
 *   choice stay eligible; ids[t, 0:top] = the largest choices (descending), weights[t, k] = p[ids] / (sum + 1e-20) * scale.
 *   Outputs >= n_real are identity experts.  counts[e] (e < n_real) = pairs routed to expert e (zeroed here).
 * pg_moe_plan: offsets[0..n_real] (exclusive scan of counts), plan[0] = tiles, plan[4 + 3i ..] = (expert, first sorted row, rows)
 *   of tile i (pg_moe_tile_rows() rows at most; max_tiles >= ceil(pairs / tile) + n_real), sorted_pair[row] = pair t * top + k,
 *   pair_row[pair] = its sorted row (-1: identity expert).  fill: int32 [n_real] scratch.
 * pg_moe_gemm: out[row, f] = act(sum_k x[src(row), k] * w[expert(row)][f, k]) for the rows of every tile; src(row) =
 *   sorted_pair[row] / src_div when src_div > 0, else row.  w: [n_real] matrices [F, K] (pitch ldw, expert_stride elements apart).
 *   act: 0 none, 2 relu(x)^2, 3 gated silu -- the rows of w alternate gate / up (F even) and out has F / 2 columns:
 *   out[row, f] = silu(acc[2f]) * acc[2f + 1].  x_expert_off / out_expert_off: elements added to x / out per expert index (0 for routed
 *   experts).  With a host-made plan of (batch index, first row, rows) tiles over the SAME rows for every index this is a batched
 *   product whose operands are column slices: out[:, b, :] = x[:, b, :] w[b]^T (per-head projections on the tensor cores).
 * pg_moe_combine: y[t, :] = sum_k weights[t, k] * (pair_row[t, k] < 0 ? h[t, :] : expert_out[pair_row[t, k], :]) + shared_out[t, :]
 *   (shared_out may be NULL); shared_gate != NULL: the shared term is multiplied by sigmoid(shared_gate[t * ldsg]);
 *   accumulate != 0: y[t, :] += instead of = (y is the fp32 residual stream).
 * pg_moe_route's logit_bias (fp32 [n_all] or NULL) is added to the logits before the softmax. */
int pg_moe_route(const float* logits, long long ld, const float* correction, int* ids, float* weights, int* counts, int tokens, int n_all,
                 int n_real, int top, int group_count, int group_keep, float scale, const float* logit_bias, void* stream);
int pg_moe_tile_rows(void);
int pg_moe_plan(const int* counts, const int* ids, int* offsets, int* fill, int* plan, int* sorted_pair, int* pair_row, int pairs,
                int n_real, int max_tiles, void* stream);
int pg_moe_gemm(const void* x, long long ldx, const int* sorted_pair, int src_div, const void* w, long long expert_stride, long long ldw,
                void* out, long long ldo, const int* plan, int max_tiles, int F, int K, int act, int in_f32, int out_f32,
                long long x_expert_off, long long out_expert_off, void* stream);
/* xg[row, 0:D] = x[sorted_pair[row] / top, 0:D] for row < *total_rows (device: offsets[n_real] of pg_moe_plan): the tokens of
 * every expert as one contiguous run of rows, for per-expert dense products. */
int pg_moe_gather_rows(const void* x, long long ldx, const int* sorted_pair, const int* total_rows, int top, void* xg, long long ldg,
                       int max_rows, int D, int act_f32, void* stream);
/* Per-expert dense products over the gathered runs: expert e owns the next counts_host[e] rows (host array, n_real entries);
 * mid[rows, F] = relu(xg W_up[e]^T)^2 in bf16, eo[rows, D] = mid W_down[e]^T in fp32, both through pg_gemm_bf16.  bf16 only;
 * D, F and the pitches multiples of 8.  glu != 0: w_up holds [n_real, 2F, D] with gate and up rows in blocks of 64
 * ([64 gate | 64 up], F a multiple of 64) and mid = silu(gate) * up comes from the product's gated epilogue. */
int pg_moe_dense_runs(const void* xg, long long ldx, const void* w_up, const void* w_down, void* mid, long long ldm, float* eo, long long ldo,
                      const int* counts_host, int n_real, int D, int F, int glu, void* stream);
int pg_moe_combine(const float* expert_out, long long ldy, const int* pair_row, const int* ids, const float* weights, const void* h,
                   long long ldh, const float* shared_out, long long lds, float* y, int tokens, int D, int top, int act_f32,
                   const float* shared_gate, long long ldsg, int accumulate, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PALIGEMMA_B200_H */
