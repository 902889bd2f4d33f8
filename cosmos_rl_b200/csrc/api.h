// C ABI of the sm_100a kernel library (libb200rl). Every launcher takes raw device pointers and a
// stream, allocates nothing unless stated, and returns 0 or a negative B200_ERR_* code. Kernels
// that can wait (tensor-core pipelines, peer flags) also take a device `status` word that stays 0
// on success and receives a b200::ST_* code when a bounded wait ran out.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define B200_ERR_ARG (-1)
#define B200_ERR_TENSORMAP (-2)
#define B200_ERR_LAUNCH (-3)
#define B200_ERR_TOO_LARGE (-4)
#define B200_ERR_RUNTIME (-5)

#ifdef __cplusplus
extern "C" {
#endif

// ---- tensor-core GEMMs ---------------------------------------------------------------------------
int b200_gemm_bf16_nt(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                      long long ldc, int out_fp32, int accumulate, uint32_t* status, int num_sms,
                      cudaStream_t stream);
// General form: a_mn / b_mn = 1 when the operand is stored with the contraction index as the ROW index
// ([K, M] / [K, N] row-major). Covers forward (0,0), dgrad (0,1) and wgrad (1,1) without transposed copies.
int b200_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                   long long ldc, int a_mn, int b_mn, int out_fp32, int accumulate, uint32_t* status, int num_sms,
                   cudaStream_t stream);

// Same with the epilogues of the CTA-pair kernel (256 x 256 tiles over two SMs, TMA-store epilogue):
//   bias      [N] added to every row (nullable; bf16 when bias_bf16 else fp32)
//   epilogue  0: C[M, N] = A B^T (+ bias);  1: SwiGLU, C[M, N/2] = silu(A Bg^T) * (A Bu^T) where Bg = B[0 : N/2] and
//             Bu = B[up_row0 : up_row0 + N/2] (the fused gate_up weight: up_row0 = intermediate size)
//   path      0: choose (pairs when M > 128 and C is 16-byte aligned), 1: single-CTA kernel, 2: CTA pairs
int b200_gemm_bf16_ex(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                      long long ldc, int a_mn, int b_mn, int out_fp32, int accumulate, const void* bias,
                      int bias_bf16, int epilogue, int up_row0, int path, uint32_t* status, int num_sms,
                      cudaStream_t stream);

// Weight-streaming GEMM for decode-sized batches (M <= 256) and the reductions that finish a decode-layer step
// (gemm_skinny.cu). x [M, K] bf16, W [rows, K] bf16. ws == NULL: out (bf16) = x W^T (+ bias), splits = 1; swiglu: W is a
// fused gate/up weight with up rows at up_row0 and out = silu(x Wg^T) * (x Wu^T) of N columns. ws != NULL: fp32
// partial results [splits, M, N] for one of the reduce kernels.
int b200_gemm_skinny_splits(int M, int N, int K, int swiglu, int num_sms);
int b200_gemm_skinny(const void* x, const void* W, void* out, float* ws, int M, int N, int K, long long ldx,
                     long long ldw, long long ldo, const void* bias, int bias_bf16, int swiglu, int up_row0,
                     int splits, uint32_t* status, int num_sms, cudaStream_t stream);
int b200_splitk_reduce(const float* ws, int splits, int M, int N, const void* bias, int bias_bf16, void* out,
                       long long ldo, cudaStream_t stream);
// res_out = sum(ws) (+ res_in);  y = rmsnorm(res_out) * w   (bf16 rows of H <= 8192 values)
int b200_splitk_reduce_residual_rmsnorm(const float* ws, int splits, int M, int H, const void* res_in, const void* w,
                                        float eps, void* res_out, void* y, cudaStream_t stream);
// q_out [M, hq * d] = rope(sum(ws) + bias); K and V rows go to cache [pages, 2, hkv, page_size, d] at slot_mapping[r]
// (V slabs [d, page_size] when v_transposed; slot < 0 skips the write).
int b200_splitk_reduce_qkv_rope_append(const float* ws, int splits, int M, int hq, int hkv, int d, const void* bias,
                                       int bias_bf16, const long long* positions, const int* slot_mapping,
                                       float theta, void* q_out, void* cache, int page_size, int v_transposed,
                                       cudaStream_t stream);

int b200_last_tmap_error(void);

// Fused lm_head GEMM + per-token log-prob statistics, never materialising [T, V] logits.
//   hidden [T, H] bf16, weight [V, H] bf16, labels [T] int64 (label < 0: row ignored)
//   partial [T, nsplit, 4] fp32 scratch: (max, sumexp, label_logit, sum p_unnorm*logit)
// followed by b200_logprob_combine -> logprob [T], lse [T], entropy [T] (fp32).
int b200_lmhead_logprob_partial(const void* hidden, const void* weight, const long long* labels, float* partial,
                                int T, int V, int H, long long ldh, long long ldw, float inv_temperature,
                                int nsplit, uint32_t* status, int num_sms, cudaStream_t stream);
int b200_logprob_combine(const float* partial, const long long* labels, float* logprob, float* lse, float* entropy,
                         int T, int nsplit, cudaStream_t stream);
// Backward helper: dlogits[T, Vc] (bf16) = (softmax(logits/temp) * (g_lp_total) - onehot * g_lp) * inv_temp for a vocab
// chunk [v0, v0+Vc), recomputing the logits tile on the tensor cores.
int b200_lmhead_dlogits(const void* hidden, const void* weight, const long long* labels, const float* lse,
                        const float* g_logprob, const float* g_entropy, const float* entropy, void* dlogits, int T,
                        int V, int H, long long ldh, long long ldw, int v0, int Vc, long long ldd,
                        float inv_temperature, uint32_t* status, int num_sms, cudaStream_t stream);

// ---- mixture of experts ----------------------------------------------------------------------------------
// Router: logits [T, E] fp32 -> softmax -> top-k (k <= 8, E <= 256) -> probs [T, k] (renormalised when renorm),
// idx [T, k], and the per-expert histogram counts [E] (must be zeroed by the caller; may be null).
int b200_moe_route_topk(const float* logits, int T, int E, int k, int renorm, float* probs, int* idx, int* counts,
                        cudaStream_t stream);
// counts [E] -> offsets [E+1] (every expert block padded to 128 rows), tile_expert [max_tiles], n_tiles [1];
// cursor [E] is cleared for the permute kernel.
int b200_moe_offsets(const int* counts, int E, int* offsets, int* tile_expert, int* n_tiles, int* cursor,
                     int max_tiles, cudaStream_t stream);
int b200_moe_permute(const void* x, const int* idx, const int* offsets, int* cursor, int* row_map, void* xp, int T,
                     int k, int H, cudaStream_t stream);
int b200_moe_scatter_scaled(const void* src, const float* probs, const int* row_map, void* dst, int T, int k, int H,
                            cudaStream_t stream);
int b200_moe_combine(const void* y, const float* probs, const int* row_map, void* out, int T, int k, int H,
                     cudaStream_t stream);
int b200_moe_combine_dprob(const void* dout, const void* y, const int* row_map, float* dprob, int T, int k, int H,
                           cudaStream_t stream);
// Grouped GEMMs over the padded, expert-sorted token buffer (see grouped_gemm.cu for the three forms).
int b200_grouped_gemm(const void* X, const void* W, void* Y, int max_rows, int N, int K, int num_experts,
                      long long ldx, long long ldy, const int* tile_expert, const int* n_tiles, int mode,
                      int accumulate, uint32_t* status, int num_sms, cudaStream_t stream);
int b200_grouped_wgrad(const void* dY, const void* X, void* dW, int max_rows, int N, int K, int num_experts,
                       long long lddy, long long ldx, const int* expert_offsets, int out_fp32, int accumulate,
                       uint32_t* status, int num_sms, cudaStream_t stream);

// ---- normalisation / activation / rotary ------------------------------------------------------------
int b200_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* residual_out, float* rstd,
                     int T, int H, float eps, cudaStream_t stream);
int b200_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                     float* dw_partial, int n_partial, int T, int H, cudaStream_t stream);
int b200_rmsnorm_bwd2(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                      float* dw_accum, long long T, int H, cudaStream_t stream);
int b200_colsum_f32(const float* partial, float* out, int rows, int cols, int accumulate, cudaStream_t stream);
int b200_rope_inplace(void* q, void* k, const long long* positions, int T, int hq, int hkv, int d, long long q_stride,
                      long long k_stride, float theta, int backward, cudaStream_t stream);
int b200_swiglu_fwd(const void* gate_up, void* out, long long T, int I, cudaStream_t stream);
int b200_swiglu_bwd(const void* dout, const void* gate_up, void* dgate_up, long long T, int I, cudaStream_t stream);

// ---- optimizer -----------------------------------------------------------------------------------------
// Flat fused AdamW on fp32 master weights with bf16 (or fp32) grads; writes the bf16 compute copy.
// grad_scale_dev: device scalar multiplied into every gradient (clip coefficient), may be null.
int b200_adamw(float* master, float* m, float* v, const void* grad, int grad_fp32, void* param_bf16, long long n,
               float lr, float beta1, float beta2, float eps, float weight_decay, float bias1, float bias2,
               const float* grad_scale_dev, cudaStream_t stream);
int b200_sumsq(const void* x, int is_fp32, long long n, float* out_accum, cudaStream_t stream);
int b200_clip_coef(const float* sumsq, float max_norm, float* coef_out, float* norm_out, cudaStream_t stream);

// Fused per-token GRPO objective (grpo_loss.cu). per_tok/dlp/kl_out are [n] fp32, stats is [3] fp32
// {clipped-token count, sum of ratios, sum of kl*mask}. ref_lp / roll_lp / mask may be null.
int b200_grpo_loss(const float* lp, const float* old_lp, const float* ref_lp, const float* roll_lp,
                   const float* adv, const float* mask, int n, float eps_lo, float eps_hi, float lower_bound,
                   int use_dual_clip, float kl_beta, int unbiased_kl, int use_aipo, float aipo_rho, int decoupled,
                   int use_cap, float behav_cap, float* per_tok, float* dlp, float* kl_out, float* stats,
                   cudaStream_t stream);

// Data-parallel step over peer memory (n_ranks <= 8): gradient reduce-scatter + sum of squares, and AdamW whose
// bf16 store goes to every rank's parameter buffer. Pointers are device addresses valid in this process
// (own buffer or IPC-mapped peers); lo and n are multiples of 8 elements.
int b200_reduce_scatter_sumsq(void* const* grads, int n_ranks, long long lo, long long n, float* out_shard,
                              float* sumsq_accum, float scale, cudaStream_t stream);
int b200_adamw_publish(float* master, float* m, float* v, const float* grad_shard, void* const* params, int n_ranks,
                       long long lo, long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                       float bias1, float bias2, const float* grad_scale_dev, cudaStream_t stream);

// ---- sampling --------------------------------------------------------------------------------------------
// logits [B, V] (fp32 or bf16), per-row temperature/top_p/top_k; writes token [B] (int64) and its log-prob
// under softmax(logits / temperature). offset_dev (nullable) is a device counter added to `offset`.
int b200_sample(const void* logits, int logits_bf16, long long ld, int B, int V, const float* temperature,
                const float* top_p, const int* top_k, unsigned long long seed, unsigned long long offset,
                const unsigned long long* offset_dev, long long* tokens, float* logprobs, cudaStream_t stream);

// ---- attention ----------------------------------------------------------------------------------------------
// Paged KV cache layout: [num_pages, 2 (k,v), hkv, page_size, d] bf16.
int b200_kv_append(const void* k, const void* v, void* cache, const int* slot_mapping, int T, int hkv, int d,
                   long long k_stride, long long v_stride, int page_size, cudaStream_t stream);
int b200_paged_decode(const void* q, const void* cache, const int* block_table, const int* seq_lens, void* out,
                      float* scratch, int B, int hq, int hkv, int d, int page_size, int max_pages, int nsplit,
                      float scale, cudaStream_t stream);
// Tensor-core (tcgen05 + TMA) decode attention. Requires d == 128, page_size == 128 and the cache layout
// [pages, 2, hkv, 128 x 128] with K slabs as [token, d] and V slabs transposed as [d, token]
// (written by b200_kv_append_vt). hq / hkv <= 8.
int b200_kv_append_vt(const void* k, const void* v, void* cache, const int* slot_mapping, int T, int hkv, int d,
                      long long k_stride, long long v_stride, int page_size, cudaStream_t stream);
int b200_paged_decode_tc(const void* q, const void* cache, long long num_pages, const int* block_table,
                         const int* seq_lens, void* out, float* scratch, int B, int hq, int hkv, int d, int page_size,
                         int max_pages, int nsplit, float scale, uint32_t* status, int num_sms, cudaStream_t stream);
// Same with a shared-prefix pass: prefix_pages[b] leading pages of sequence b are shared by the `group` consecutive
// sequences of its group and are read once per group (scratch: B * hq * (max_shared + nsplit) * (d + 2) floats).
int b200_paged_decode_prefix_tc(const void* q, const void* cache, long long num_pages, const int* block_table,
                                const int* seq_lens, void* out, float* scratch, int B, int hq, int hkv, int d,
                                int page_size, int max_pages, int nsplit, float scale, const int* prefix_pages,
                                int group, int max_shared, uint32_t* status, int num_sms, cudaStream_t stream);
// Decode attention for callers that cannot allocate device memory (a host that gave the whole device to
// weights and KV cache at start-up, or plain-C callers without a device allocator). Same computation and
// arguments as b200_paged_decode, minus `scratch`: the split-merge scratch is a 16 MiB array inside the
// library, held by every GPU that loads it until exit. Limit: B * hq * nsplit * (d + 2) <= 4 Mi floats,
// otherwise B200_ERR_TOO_LARGE. The first call on a device resolves the array's device address and should
// come before any stream capture; calls that overlap on the GPU race on the shared array. Allocates
// nothing. This entry point has no counterpart in the reference.
int b200_paged_decode_static(const void* q, const void* cache, const int* block_table, const int* seq_lens,
                             void* out, int B, int hq, int hkv, int d, int page_size, int max_pages, int nsplit,
                             float scale, cudaStream_t stream);
// Varlen causal flash attention forward on tcgen05 (flash_fwd.cu): packed sequences, GQA, head_dim 128.
// q [Tq,hq,d], k/v [Tk,hkv,d] with token strides; out [Tq,hq,d]; lse [hq,Tq] fp32; queries are aligned to the
// end of their sequence's keys.
int b200_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_q,
                   const int* cu_k, int B, int Tq, int Tk, int hq, int hkv, int d, long long ldq, long long ldk,
                   long long ldv, long long ldo, int max_q, int causal, float scale, uint32_t* status,
                   cudaStream_t stream);

// Gradients of b200_flash_fwd (flash_bwd.cu). dq_accum [Tq,hq,d] fp32 must be zero on entry; dk/dv are overwritten;
// delta [hq,Tq] fp32 is scratch.
int b200_flash_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                   float* dq_accum, void* dk, void* dv, float* delta, const int* cu_q, const int* cu_k, int B, int Tq,
                   int Tk, int hq, int hkv, int d, long long ldq, long long ldk, long long ldv, long long ldo,
                   long long lddo, long long lddk, long long lddv, int max_k, int causal, float scale,
                   uint32_t* status, cudaStream_t stream);

// ---- quantisation ----------------------------------------------------------------------------------------------
// bf16 [R, C] -> e4m3 [R, C] with one fp32 scale per 128 x 128 block (weights) or per 1 x 128 (activations).
int b200_quant_fp8_block(const void* src, long long ld_src, void* dst, long long ld_dst, float* scales, int R, int C,
                         int block_rows, cudaStream_t stream);

// bf16 [R, C] <-> microscaling fp4 (E2M1 elements, one E8M0 scale per 32 elements; mxfp4.cu). swizzle = 1 stores the
// scales in the 128 x 4 tile interleaving block-scaled tensor-core MMA reads.
int b200_quant_mxfp4(const void* x, long long ldx, void* q, void* sf, int R, int C, int swizzle, cudaStream_t stream);
int b200_dequant_mxfp4(const void* q, const void* sf, void* out, long long ldo, int R, int C, int swizzle,
                       cudaStream_t stream);

// ---- peer-memory weight sync -------------------------------------------------------------------------------------
// One descriptor = copy a [rows, cols] bf16 rectangle from (possibly another GPU's) memory into a local
// destination, optionally quantising to block-scaled fp8 on the way.
struct B200CopyDesc {
  const void* src;      // peer or local pointer
  void* dst;            // local pointer (bf16 or e4m3)
  float* dst_scale;     // fp8 only: scale for this rectangle's 128x128 blocks, row-major [ceil(rows/128), ld_scale]
  long long src_ld;     // elements
  long long dst_ld;     // elements
  int rows, cols;
  int ld_scale;
  int quant;            // 0: bf16 copy, 1: fp8 e4m3 128x128 block-scaled (rows/cols of dst start on block boundaries)
};
int b200_reshard_pull(const B200CopyDesc* descs_dev, const int* tile_prefix_dev, int n_desc, int total_tiles,
                      uint32_t* status, cudaStream_t stream);

// In-place averaging all-reduce of a flat bf16 buffer over peer memory (fsdp_fused.cu): this rank reduces and
// republishes [lo, lo + n).
int b200_peer_all_reduce(void* const* bufs, int n_ranks, long long lo, long long n, float scale, cudaStream_t stream);

// All-to-all-v of rows over peer memory (a2av.cu): push the rows owed to every rank into its receive buffer and add
// the delivered row count to its arrival counter.
int b200_a2av_push(const void* src, long long src_ld_bytes, int row_bytes, int ep, const int* send_off,
                   void* const* dst_ptrs, const long long* dst_row, long long dst_ld_bytes, void* const* flag_ptrs,
                   cudaStream_t stream);

// Expert-parallel MoE forward over peer memory (ep_gemm.cu): device-side layout from the all-gathered counts, token
// dispatch fused into the first grouped GEMM, combine push.
int b200_ep_layout(const int* counts, int ep, int E, int rank, int max_tiles, int* send_off, int* dst_base,
                   int* ret_base, int* block_start, int* tile_expert, int* block_target, int* n_tiles,
                   cudaStream_t stream);
int b200_ep_dispatch_gemm(const void* x, long long ldx, const void* W, void* Y, long long ldy, int max_rows, int N,
                          int H, int E, int ep, int rank, const int* send_off, const int* dst_base,
                          void* const* recv_ptrs, void* const* flag_ptrs, const int* tile_expert,
                          const int* block_target, const int* n_tiles, unsigned long long wait_ns, uint32_t* status,
                          int num_sms, cudaStream_t stream);
int b200_ep_combine_push(const void* y, int H, int E, int ep, int rank, const int* counts, const int* block_start,
                         const int* ret_base, void* const* ret_ptrs, void* const* flag_ptrs, cudaStream_t stream);

// Block-scaled fp8 GEMM (gemm_fp8_block.cu): A [M,K] e4m3 + sa [M, ldsa] (1 x 128 blocks), B [N,K] e4m3 +
// sb [ceil(N/128), ldsb] (128 x 128 blocks), C [M,N] bf16.
int b200_gemm_fp8_block(const void* A, const float* sa, const void* B, const float* sb, void* C, int M, int N, int K,
                        long long lda, long long ldb, long long ldc, int ldsa, int ldsb, uint32_t* status, int num_sms,
                        cudaStream_t stream);

// Column-parallel GEMM fused with the tensor-parallel all-gather of its input rows (ag_gemm.cu).
int b200_ag_gemm(const void* x, const void* W, void* out, int M, int N, int K, long long ldx, long long ldw,
                 long long ldc, void* const* gathered_ptrs, void* const* flag_ptrs, uint32_t* ctrl, int tp, int rank,
                 long long set_elems, int max_blocks, unsigned long long wait_ns, uint32_t* status, int num_sms,
                 cudaStream_t stream);

// Row-parallel GEMM fused with the tensor-parallel all-reduce (mode 0) or reduce-scatter over rows (mode 1)
// through peer-mapped staging slots and arrival counters (tp_gemm.cu). ctrl: two local uint32 words.
int b200_tp_gemm(const void* A, const void* W, void* out, const void* residual, int M, int N, int K, long long lda,
                 long long ldw, long long ldo, long long ldr, void* const* stage_ptrs, void* const* flag_ptrs,
                 uint32_t* ctrl, int tp, int rank, int mode, long long slot_elems, int max_tiles,
                 unsigned long long wait_ns, uint32_t* status, int num_sms, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
