/*
 * fast_route_sm100.h - C ABI of libfastroute_sm100.so, the sm_100a (B200) implementation of
 * the fused-routing Mixture-of-Experts layer.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*,
 * the value of a cudaStream_t), launches asynchronously on that stream, allocates nothing
 * and keeps no pointer after it returns.  Return value: 0 = ok, negative = argument
 * rejected on the host (see fr_error_string), positive = a cudaError_t.
 * Device-side problems (an id out of range, a bounded wait that expired) never trap: they
 * are recorded in a device status block read with fr_check_status().
 *
 * Each declaration names the interface of the reference (hgl71964/fast-route, paths inside
 * that project) that it stands in for.
 */
#ifndef FAST_ROUTE_SM100_H_
#define FAST_ROUTE_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of activations / weights / logits */
enum { FR_F16 = 0, FR_BF16 = 1, FR_F32 = 2 };

/* host-side argument errors */
enum {
  FR_OK = 0,
  FR_ERR_ARG = -1,         /* null pointer, negative size, k > E ... */
  FR_ERR_UNSUPPORTED = -2, /* a size or layout outside what the kernels cover */
  FR_ERR_ALIGN = -3,       /* pointer or stride not 16-byte aligned where TMA needs it */
  FR_ERR_WORKSPACE = -4,   /* workspace too small */
  FR_ERR_DRIVER = -5       /* the CUDA driver entry point for tensor maps is unavailable */
};

/* alignment block of the expert GEMMs: the reference passes its Triton BLOCK_SIZE_M
 * (fast_route/fast_route/layers/stable_route.py:82-83); here it is the MMA tile height. */
#define FR_GEMM_BLOCK_M 128

int fr_version(void);
const char* fr_error_string(int code);

/* Synchronous read (and clear) of the device status block of the current device:
 * out4[0] = first error code (0 ok, 1 wait timeout, 2 expert id out of range,
 * 3 bad sorted id, 4 expert-parallel receive capacity exceeded), out4[1] = detail, out4[2] = block, out4[3] = count.
 * No counterpart in the reference, whose kernels have no error reporting. */
int fr_check_status(unsigned int* out4);

/* Router from logits: stable descending top-k (ties -> lower expert id) and softmax over
 * the selected k.  Stands in for the epilogue of route_kernel,
 * fast_route/fast_route/ops/stable_route.py:91-121, and for stable_argsort,
 * ops/stable_argsort.py:96-114.  logits[M,E] with element strides; weights fp32 and ids
 * int32 are written at [row*stride + j].  fill_rest != 0 reproduces what the reference
 * leaves in [M,E] buffers (ids: the full argsort; weights: zeros past k).
 * renormalize == 0 divides by the sum over all E columns instead. */
int fr_topk_softmax(const void* logits, int dtype, int64_t M, int E, int64_t stride_m, int64_t stride_e,
                    int topk, int renormalize, float* weights, int64_t w_stride, int32_t* ids,
                    int64_t id_stride, int fill_rest, void* stream);

/* Softmax over all E columns followed by top-k on the probabilities (ties -> lower expert id):
 * the routing of the reference's baseline layer, fast_route/fast_route/layers/vllm_route.py:72-84,
 * i.e. vllm._moe_C.topk_softmax of vLLM 0.4.0 plus the optional renormalisation at :83-84.
 * weights fp32 / ids int32 / source_rows int32 (may be NULL; entry [t,j] = j*M + t, the op's
 * token_expert_indicies) are written at [row*stride + j].  renormalize != 0 divides the k
 * probabilities by their sum.  Limits: E <= 256, topk <= 8, else FR_ERR_UNSUPPORTED. */
int fr_softmax_topk(const void* logits, int dtype, int64_t M, int E, int64_t stride_m, int64_t stride_e,
                    int topk, int renormalize, float* weights, int64_t w_stride, int32_t* ids,
                    int64_t id_stride, int32_t* source_rows, int64_t src_stride, void* stream);

/* Stable counting sort of the n = M*topk flattened routing ids by expert, every expert's
 * segment padded to a multiple of block_size with the sentinel n.  Stands in for
 * moe_align_block_size, fast_route/fast_route/ops/fused_moe.py:133-175 (the vLLM 0.4.0 CUDA
 * op it calls plus the fill_ of the wrapper).  sorted_ids has sorted_len entries
 * (>= n + E*(block_size-1)), expert_ids has expert_ids_len entries; entries past the valid
 * prefix are set to n / -1.  Optional outputs (may be NULL): counts[E] tokens per expert,
 * inv_pos[n] position of every flat assignment in sorted_ids (-1 for an id outside [0, E), which
 * is reported through fr_check_status and left out of the sort).
 * workspace (may be NULL): fr_align_workspace_bytes(E) bytes of scratch, 16-byte aligned, that
 * lets batches of >= 8192 assignments run as one cooperative launch over all SMs instead of one
 * 8-CTA cluster.  Its first 16 bytes are control words (grid-barrier count and generation, a
 * completion counter, and the barrier's poll budget: 0 = the default, about a second): ZERO THE
 * BUFFER ONCE before its first use (and again after fr_check_status has reported an expired
 * wait); completed calls leave it ready for the next one.  One workspace serves one stream at
 * a time. */
size_t fr_align_workspace_bytes(int E);
int fr_align(const int32_t* topk_ids, int64_t n, int E, int block_size, int32_t* sorted_ids,
             int64_t sorted_len, int32_t* expert_ids, int64_t expert_ids_len, int32_t* num_tokens_post_pad,
             int32_t* counts, int32_t* inv_pos, void* workspace, size_t workspace_bytes, void* stream);

/* fr_align for callers that cannot hand over scratch memory of their own: code that runs where
 * cudaMalloc is off limits (inside a caller-managed memory pool or arena with nothing left to
 * carve, from a plugin whose host forbids device allocation after start-up, or on a hot path
 * that must never reach the allocator).  It has no counterpart in the reference.  It runs the
 * same whole-GPU cooperative kernel as fr_align, with the histogram and barrier words kept in a
 * 262,400-byte (256.25 KB) array that the library itself owns on every GPU that loads it, until
 * the process exits.  It calls no cudaMalloc / cudaFree and no allocating library routine.
 * Limits: E <= FR_ALIGN_NOALLOC_MAX_EXPERTS and 1 <= n <= 8192 * (number of SMs); anything
 * larger returns FR_ERR_UNSUPPORTED (use fr_align with a workspace).  Outputs are identical
 * to fr_align's.
 * The first call on each device looks up the array's device address (make that call with the
 * device current, before any stream capture starts; a first call made while the stream is being
 * captured returns FR_ERR_UNSUPPORTED).  All calls on a device share the one
 * array: calls whose kernels could overlap on the GPU (different streams) race on it and must
 * be serialised by the caller.  The barrier words are cleared at the start of every call. */
#define FR_ALIGN_NOALLOC_MAX_EXPERTS 256
int fr_align_noalloc(const int32_t* topk_ids, int64_t n, int E, int block_size, int32_t* sorted_ids,
                     int64_t sorted_len, int32_t* expert_ids, int64_t expert_ids_len,
                     int32_t* num_tokens_post_pad, int32_t* counts, int32_t* inv_pos, void* stream);

/* fr_topk_softmax followed by fr_align on its compact [M,topk] ids: the routing/align
 * latency path (logits -> the five routing outputs), two launches on the stream.  The
 * workspace follows the contract of fr_align. */
int fr_route_align(const void* logits, int dtype, int64_t M, int E, int64_t stride_m, int64_t stride_e,
                   int topk, float* weights, int32_t* ids, int block_size, int32_t* sorted_ids,
                   int64_t sorted_len, int32_t* expert_ids, int64_t expert_ids_len,
                   int32_t* num_tokens_post_pad, void* workspace, size_t workspace_bytes, void* stream);

/* Fused router: logits = X[M,H] . G[H,E] on the tensor cores with the top-k / softmax
 * epilogue in registers.  Stands in for fused_route + route_kernel,
 * fast_route/fast_route/ops/stable_route.py:32-178.  x is row-major with row pitch ldx
 * elements; gate element (h,e) is at gate[h*gate_stride_h + e*gate_stride_e] (the layer
 * passes W_g[E,H].t(), i.e. gate_stride_h = 1; a row-major [H,E] gate is transposed into
 * the workspace first).  weights/ids are compact [M,topk].  logits_out (may be NULL)
 * receives the fp32 logits [M,E].  dtype is FR_F16 or FR_BF16. */
size_t fr_route_fused_workspace_bytes(int64_t M, int H, int E, int topk);
int fr_route_fused(const void* x, int dtype, int64_t M, int H, int64_t ldx, const void* gate,
                   int64_t gate_stride_h, int64_t gate_stride_e, int E, int topk, int renormalize,
                   float* weights, int32_t* ids, float* logits_out, void* workspace, size_t workspace_bytes,
                   void* stream);

/* Gathers token rows into expert-sorted order: dst[p,:] = src[sorted_ids[p] / topk, :] for
 * p < num_tokens_post_pad (zeros for padding entries).  Stands in for the gathered A loads
 * of fused_moe_kernel, fast_route/fast_route/ops/fused_moe.py:82-89. */
int fr_permute_rows(const void* src, int dtype, int H, int64_t ld_src, const int32_t* sorted_ids,
                    const int32_t* num_tokens_post_pad, int64_t n, int topk, int64_t max_rows, void* dst,
                    int64_t ld_dst, void* stream);

/* Grouped expert GEMM 1 with the SiLU-and-multiply epilogue, on expert-sorted rows:
 * act[p, j] = silu(a[p,:] . w1[e, j, :]) * (a[p,:] . w1[e, I + j, :]),  e = expert_ids[p / 128].
 * Stands in for invoke_fused_moe_kernel(..., mul_routed_weight=False)
 * (fast_route/fast_route/ops/fused_moe.py:10-130, 178-214) followed by ops.silu_and_mul
 * (fast_route/fast_route/layers/stable_route.py:85-90).  a_sorted[max_rows, H] (pitch lda),
 * w1[E, 2I, H] contiguous, act[max_rows, I] (pitch ld_act), max_rows a multiple of 128.
 * split_k > 1 (few rows, many K slices: the small-batch path) sums fp32 partial tiles in
 * slice order; it needs sorted_ids, the number n of real assignments and a workspace of
 * fr_gemm_splitk_workspace_bytes(n, 2*I, split_k) bytes.  sorted_ids may be NULL otherwise. */
size_t fr_gemm_splitk_workspace_bytes(int64_t n, int64_t n_cols, int split_k);
int fr_gemm1_silu(const void* a_sorted, int64_t lda, const void* w1, int dtype, int64_t max_rows, int H, int I,
                  int E, const int32_t* expert_ids, const int32_t* num_tokens_post_pad, const int32_t* sorted_ids,
                  int64_t n, void* act, int64_t ld_act, int split_k, void* workspace, size_t workspace_bytes,
                  void* stream);

/* Grouped expert GEMM 2 with the routed weight applied in fp32 before rounding:
 * y[p, h] = topk_weights[sorted_ids[p]] * (act[p,:] . w2[e, h, :]).
 * Stands in for invoke_fused_moe_kernel(..., mul_routed_weight=True, top_k=1)
 * (fast_route/fast_route/ops/fused_moe.py:117-121, layers/stable_route.py:92-95).
 * Output rows stay in expert-sorted order; fr_combine gathers them per token.
 * topk_weights (flat [n], indexed by sorted id) may be NULL (weight 1).  split_k as above
 * with fr_gemm_splitk_workspace_bytes(n, H, split_k). */
int fr_gemm2(const void* act, int64_t ld_act, const void* w2, int dtype, int64_t max_rows, int H, int I, int E,
             const int32_t* expert_ids, const int32_t* num_tokens_post_pad, const int32_t* sorted_ids,
             const float* topk_weights, int64_t n, void* y, int64_t ld_y, int split_k, void* workspace,
             size_t workspace_bytes, void* stream);

/* Combine: out[t,:] = sum_j y[inv_pos[t*topk + j], :], accumulated in fp32 in slot order and
 * rounded once; positions outside [0, max_rows) are skipped.
 * Stands in for torch.sum(intermediate_cache3, dim=1),
 * fast_route/fast_route/layers/stable_route.py:97-102. */
int fr_combine(const void* y, int64_t ld_y, int dtype, const int32_t* inv_pos, int64_t M, int topk, int H,
               int64_t max_rows, void* out, int64_t ld_out, void* stream);

/* The whole layer on one stream: route -> align -> permute -> GEMM1+SiLU -> GEMM2 -> combine.
 * Stands in for fused_moe, fast_route/fast_route/layers/stable_route.py:10-102.
 * x[M,H], gate as in fr_route_fused, w1[E,2I,H], w2[E,H,I], out[M,H] (may alias x: the
 * reference's inplace=True).  topk_weights_out / topk_ids_out (may be NULL) receive the
 * compact routing.  The workspace (1024-byte aligned) holds every intermediate; zero it once
 * before its first use (it contains the align stage's grid-barrier words, see fr_align). */
size_t fr_moe_workspace_bytes(int64_t M, int H, int I, int E, int topk);
int fr_moe_layer(const void* x, const void* gate, int64_t gate_stride_h, int64_t gate_stride_e, const void* w1,
                 const void* w2, int dtype, int64_t M, int H, int I, int E, int topk, int renormalize, void* out,
                 float* topk_weights_out, int32_t* topk_ids_out, void* workspace, size_t workspace_bytes,
                 void* stream);

/* Transformer-block glue around the layer (the reference's block is h = attn(x) + x; fused_moe(h),
 * benchmarks/fused_route/transformerLayer_bench.py:66-79; Mixtral adds an RMSNorm and a second residual).
 * fr_add_rmsnorm: h = a (+ b);  x = h * rsqrt(mean(h^2) + eps) * gamma, one pass over the rows.
 * b, gamma, h_out, x_out are optional (without gamma x_out = h).  H <= 16384.
 * fr_moe_block:  h = attn_out (+ x);  u = gamma ? rmsnorm(h) * gamma : h;
 *                out = (add_residual ? h : 0) + moe(u)
 * as one launch sequence: the add and the norm are one kernel, the second residual is added inside
 * the combine kernel (fp32, one rounding).  out may alias attn_out or x. */
int fr_add_rmsnorm(const void* a, int64_t ld_a, const void* b, int64_t ld_b, const void* gamma, float eps, int dtype,
                   int64_t M, int H, void* h_out, int64_t ld_h, void* x_out, int64_t ld_x, void* stream);
size_t fr_moe_block_workspace_bytes(int64_t M, int H, int I, int E, int topk);
int fr_moe_block(const void* attn_out, const void* x, const void* gamma, float eps, const void* gate,
                 int64_t gate_stride_h, int64_t gate_stride_e, const void* w1, const void* w2, int dtype, int64_t M,
                 int H, int I, int E, int topk, int renormalize, int add_residual, void* out, void* workspace,
                 size_t workspace_bytes, void* stream);

/* The layer with 8-bit floating-point (E4M3) expert weights: w1_q[E,2I,H] and w2_q[E,H,I] hold E4M3
 * bytes, w1_scale[E*2I] / w2_scale[E*H] one fp32 scale per weight row (weight = byte value * scale).
 * Activations stay in `dtype` (FR_F16 / FR_BF16) at the interface; each row is quantised to E4M3 with
 * its own scale (absmax / 448) while it is gathered, and again between the two GEMMs; both GEMMs run as
 * tcgen05 kind::f8f6f4 MMAs with fp32 accumulation and the scales are applied in the epilogue.  Router,
 * align and combine are those of fr_moe_layer.  H and I must be multiples of 16 and at most 16384.
 * The reference only hints at this (commented-out "good config for fp8 inputs" autotune entries,
 * fast_route/fast_route/ops/stable_route.py:20-28); it halves the weight bytes a small batch streams. */
size_t fr_moe_fp8_workspace_bytes(int64_t M, int H, int I, int E, int topk);
int fr_moe_layer_fp8(const void* x, const void* gate, int64_t gate_stride_h, int64_t gate_stride_e, const void* w1_q,
                     const float* w1_scale, const void* w2_q, const float* w2_scale, int dtype, int64_t M, int H, int I,
                     int E, int topk, int renormalize, void* out, float* topk_weights_out, int32_t* topk_ids_out,
                     void* workspace, size_t workspace_bytes, void* stream);

/* The layer for a routing computed elsewhere: align -> permute -> GEMM1+SiLU -> GEMM2 -> combine with
 * the caller's compact topk_ids[M,topk] (int32) and topk_weights[M,topk] (fp32, may be NULL = 1).
 * Stands in for the vLLM-style signature fused_moe(hidden_states, w1, w2, topk_weights, topk_ids)
 * that the reference benchmarks against (benchmarks/swizzle_moe/v0_moe_fused.py:219-224,
 * benchmarks/swizzle_moe/perf_test_moe.py:48-58).  Workspace as fr_moe_layer. */
int fr_moe_layer_routed(const void* x, const int32_t* topk_ids, const float* topk_weights, const void* w1,
                        const void* w2, int dtype, int64_t M, int H, int I, int E, int topk, void* out,
                        void* workspace, size_t workspace_bytes, void* stream);

/* Expert-parallel building blocks (no counterpart in the reference, which is single-GPU).
 * fr_moe_experts: the expert part of the layer for rows that already carry an expert id
 * (tokens received from other ranks): align by local expert -> permute -> GEMM1+SiLU ->
 * GEMM2 -> rows returned in the order they came in.  rows[R,H], row_expert[R] in
 * [0, E_local), row_weight[R] (may be NULL), y[R,H].  Workspace contract as fr_moe_layer. */
size_t fr_moe_experts_workspace_bytes(int64_t R, int H, int I, int E_local);
int fr_moe_experts(const void* rows, const int32_t* row_expert, const float* row_weight, const void* w1,
                   const void* w2, int dtype, int64_t R, int H, int I, int E_local, void* y, void* workspace,
                   size_t workspace_bytes, void* stream);

/* Expert parallelism over peer memory with no host in the loop (no counterpart in the reference, which
 * is single-GPU; the sharded layer is fast_route/fast_route/layers/stable_route.py:10-102).
 * Rank r of `world` owns experts [r*E/world, (r+1)*E/world) and brings its own tokens.  Every rank keeps a
 * region of identical layout that all GPUs of the node can read (symmetric memory); peer_base is a DEVICE
 * array of `world` region base pointers (entry `rank` may be the local one).  Inside a region, at byte offsets:
 *   x_off       x[peer_rows, H]   the rank's tokens (row pitch ld_x elements)
 *   sorted_off  int32[n_per_rank] its flat assignment ids ordered by expert (fr_align with block_size 1)
 *   tw_off      float[n_per_rank] its routing weights by flat assignment id
 *   y_off       y[y_rows, H]      the results of the rank's OWN experts in expert-sorted order
 * all_counts[world][E] (device, e.g. from one all-gather of every rank's fr_align counts) is the only
 * metadata that travels.  From it each rank derives on the device where every (local expert, source rank)
 * segment sits in its operand and, as token owner, in which row of the expert owner's y each of its
 * assignments ends up, so no sizes reach the host and no position list is sent back.
 * fr_ep_experts ("pack"): plan -> gather of the token rows from their owners (16-byte NVLink loads) into the
 *   expert-sorted operand -> GEMM1+SiLU -> GEMM2 x routing weight -> y_sorted (= this rank's y, y_rows rows,
 *   a multiple of 128; fr_moe_experts_rows_cap(world * n_per_rank, E / world) always suffices; more rows than
 *   that capacity are dropped and reported as status 4).  comb_base[E] is written for fr_ep_combine.
 *   n_per_rank is the capacity of sorted / tw (and the row count the tile order is tuned for).  stages is a
 *   mask: 1 = plan + gather, 2 = GEMM1, 4 = GEMM2 (7 = all; a caller timing the stages issues them one by one).
 * fr_ep_combine ("unpack"): out[t,:] = sum_j y of the owner of topk_ids[t,j], row comb_base[e] + inv_pos[t*k+j],
 *   fp32 in slot order; inv_pos is the one fr_align(block_size 1) returned on this rank.
 * The caller orders the ranks with two small collectives: every region's x / sorted / tw complete before any
 * fr_ep_experts (the all-gather of the counts does that), every y complete before any fr_ep_combine.
 * The workspace is fr_ep_workspace_bytes(y_rows, ...) bytes, 1024-byte aligned. */
int64_t fr_moe_experts_rows_cap(int64_t R, int E_local);
size_t fr_ep_workspace_bytes(int64_t cap_rows, int H, int I, int E);
int fr_ep_experts(const void* const* peer_base, int world, int rank, int64_t x_off, int64_t ld_x, int64_t peer_rows,
                  int64_t sorted_off, int64_t tw_off, int64_t n_per_rank, int topk, const int32_t* all_counts,
                  const void* w1, const void* w2, int dtype, int H, int I, int E, void* y_sorted, int64_t y_rows,
                  int32_t* comb_base, int stages, void* workspace, size_t workspace_bytes, void* stream);
int fr_ep_combine(const void* const* peer_base, int world, int64_t y_off, int64_t ld_y, int64_t y_rows, int dtype,
                  const int32_t* topk_ids, const int32_t* inv_pos, const int32_t* comb_base, int64_t M, int topk, int H,
                  int E, void* out, int64_t ld_out, void* stream);

/* Gather rows by index: dst[i,:] = src[idx[i],:] (idx < 0 writes zeros); 16-byte vectors. */
int fr_gather_rows(const void* src, int64_t ld_src, const int32_t* idx, int64_t rows, int row_bytes, void* dst,
                   int64_t ld_dst, void* stream);

/* W4A16 small-batch GEMM with split-K: c[m,n] = a[m,k] . dequant(qweight)[k,n].  Stands in for
 * matmul_split_k and its Triton kernel, benchmarks/splitk_gemm/splitk.py:26-103 and :178-216.
 * a fp16 [m,k] (row pitch lda elements), qweight int32 [k/8, n] (nibble j of word [kk,n] is row
 * 8*kk+j), scales fp16 [k/groupsize, n], qzeros int32 [k/groupsize, n/8] (nibble j of word [g,nn]
 * is column 8*nn+j), all dense row-major; c fp16 [m,n] (row pitch ldc).
 * w = fp16(q)*s - fp16(z+1)*s with every operation rounded to fp16 (:83-87); fp32 accumulation.
 * The K slices are reduced in a fixed order inside one kernel (the reference adds them with fp16
 * atomics, :103), so the result is deterministic.  split_k: 0 = choose, or 1, 2, 4, 8.
 * Requirements: n % 8 == 0, k % 64 == 0, groupsize % 64 == 0, k % groupsize == 0, lda % 8 == 0.
 * Batches above 128 rows run as consecutive launches of 128 rows. */
int fr_w4a16_gemm(const void* a, int64_t lda, const int32_t* qweight, const void* scales, const int32_t* qzeros,
                  int64_t m, int n, int k, int groupsize, void* c, int64_t ldc, int split_k, void* stream);

/* The dense fp16 weight matrix w[k,n] (row pitch ldw) that fr_w4a16_gemm multiplies with, produced with
 * the same arithmetic (benchmarks/splitk_gemm/splitk.py:83-87). */
int fr_w4a16_dequant(const int32_t* qweight, const void* scales, const int32_t* qzeros, int n, int k,
                     int groupsize, void* w, int64_t ldw, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FAST_ROUTE_SM100_H_ */
