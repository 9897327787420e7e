// Router from logits (stable top-k + softmax over the selected k) and the align stage
// (stable counting sort of routing ids by expert with per-expert padding).
//
// Semantics follow the reference's route_kernel epilogue
// (fast_route/fast_route/ops/stable_route.py:91-121), its stable argsort tie rule
// (ops/stable_argsort.py:37-50: equal values keep the lower expert id first) and the
// contract of moe_align_block_size (ops/fused_moe.py:133-175).
#include <cooperative_groups.h>

#include "fr_common.cuh"

namespace cg = cooperative_groups;

namespace fr {

// ----------------------------------------------------------------------------------
// top-k from logits, register path: a group of L lanes owns one row, each lane holds VPL
// consecutive columns.  k selection rounds; each round is a local scan plus an
// L-lane butterfly on (value, column) where the larger value wins and equal values go
// to the lower column.
// ----------------------------------------------------------------------------------
constexpr int KMAX = 8;

// packed-key top-k for 16-bit logits and the cooperative route+align kernel (fr_route_coop.cu)
template <typename T>
int launch_topk16(const void* logits, int64_t M, int E, int64_t stride_m, int64_t stride_e, int k, float* weights,
                  int64_t w_stride, int32_t* ids, int64_t id_stride, cudaStream_t st);
int align_coop_dispatch(const int32_t* ids_in, int64_t n, int E, int bs, int32_t* sorted_ids, int64_t sorted_len,
                        int32_t* expert_ids, int64_t expert_ids_len, int32_t* num_post, int32_t* counts,
                        int32_t* inv_pos, void* workspace, size_t workspace_bytes, cudaStream_t st,
                        int64_t min_n = 8192);

// (bitwise on purpose: evaluated without short-circuit branches, which cost dearly inside unrolled selection loops)
__device__ __forceinline__ bool beats(float v, int c, float bv, int bc) {
  return static_cast<bool>(static_cast<int>(v > bv) | (static_cast<int>(v == bv) & static_cast<int>(c < bc)));
}

template <typename T, int L, int VPL>
__global__ void __launch_bounds__(256) topk_softmax_kernel(const T* __restrict__ logits, int64_t M, int E,
                                                           int64_t stride_m, int64_t stride_e, int k,
                                                           int renormalize, float* __restrict__ weights,
                                                           int64_t w_stride, int32_t* __restrict__ ids,
                                                           int64_t id_stride, int vec_ok) {
  const int64_t gthread = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t row = gthread / L;
  const int sub = static_cast<int>(gthread % L);
  const bool row_ok = row < M;
  const int64_t r = row_ok ? row : (M - 1);

  float v[VPL];
  const int c0 = sub * VPL;
  const T* src = logits + r * stride_m;
  if (vec_ok && (sizeof(T) * VPL) % 16 == 0) {
    // contiguous, 16-byte aligned rows with E == L*VPL: 16-byte loads
    constexpr int NV = (sizeof(T) * VPL) / 16 > 0 ? (sizeof(T) * VPL) / 16 : 1;
    uint4 raw[NV];
    const uint4* p = reinterpret_cast<const uint4*>(src + c0);
#pragma unroll
    for (int i = 0; i < NV; ++i) raw[i] = __ldg(p + i);
    const T* tv = reinterpret_cast<const T*>(raw);
#pragma unroll
    for (int i = 0; i < VPL; ++i) v[i] = to_f32<T>(tv[i]);
  } else {
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = c0 + i;
      v[i] = (c < E) ? to_f32<T>(src[static_cast<int64_t>(c) * stride_e]) : -INFINITY;
    }
  }
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    if (v[i] != v[i]) v[i] = -INFINITY;  // NaN is outside the contract; rank it last
    if (c0 + i >= E) v[i] = -INFINITY;
  }

  float sel_v[KMAX];
  int sel_c[KMAX];
  uint32_t taken = 0;
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    sel_v[j] = -INFINITY;
    sel_c[j] = 0;
    if (j < k) {
      float bv = -INFINITY;
      int bc = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const bool free_slot = !((taken >> i) & 1u) && (c0 + i < E);
        if (free_slot && beats(v[i], c0 + i, bv, bc)) {
          bv = v[i];
          bc = c0 + i;
        }
      }
#pragma unroll
      for (int off = L / 2; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
        const int oc = __shfl_xor_sync(0xffffffffu, bc, off);
        if (beats(ov, oc, bv, bc)) {
          bv = ov;
          bc = oc;
        }
      }
      if (bc >= c0 && bc < c0 + VPL) taken |= 1u << (bc - c0);
      sel_v[j] = bv;
      sel_c[j] = bc;
    }
  }

  // softmax over the selected k (recipe shared with the CPU checker)
  float e[KMAX];
  float s = 0.0f;
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    e[j] = 0.0f;
    if (j < k) {
      e[j] = exp_recipe(__fsub_rn(sel_v[j], sel_v[0]));
      s = (j == 0) ? e[0] : __fadd_rn(s, e[j]);
    }
  }
  if (!renormalize) {
    float part = 0.0f;
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      if (c0 + i < E) part += exp_recipe(__fsub_rn(v[i], sel_v[0]));
#pragma unroll
    for (int off = L / 2; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
    s = part;
  }
  if (row_ok) {
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      if (j < k && (j % L) == sub) {
        weights[row * w_stride + j] = __fdiv_rn(e[j], s);
        ids[row * id_stride + j] = sel_c[j];
      }
    }
  }
}

// ----------------------------------------------------------------------------------
// general path: one warp per row, rank by counting (any E <= 2048, any k <= E, optional
// fill of all E columns).  rank(c) = #{c' : v[c'] > v[c] or (v[c'] == v[c] and c' < c)}.
// ----------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) topk_rank_kernel(const T* __restrict__ logits, int64_t M, int E,
                                                        int64_t stride_m, int64_t stride_e, int k,
                                                        int renormalize, float* __restrict__ weights,
                                                        int64_t w_stride, int32_t* __restrict__ ids,
                                                        int64_t id_stride, int fill_rest) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + warp;
  float* val = sm + static_cast<size_t>(warp) * (2 * E);  // [E] values, then [E] values by rank
  float* byrank = val + E;
  if (row >= M) return;
  const T* src = logits + row * stride_m;
  for (int c = lane; c < E; c += 32) {
    float x = to_f32<T>(src[static_cast<int64_t>(c) * stride_e]);
    if (x != x) x = -INFINITY;
    val[c] = x;
  }
  __syncwarp();
  const int nout = fill_rest ? E : k;
  for (int c = lane; c < E; c += 32) {
    const float x = val[c];
    int rank = 0;
    for (int o = 0; o < E; ++o) rank += beats(val[o], o, x, c) ? 1 : 0;
    byrank[rank] = x;
    if (rank < nout) ids[row * id_stride + rank] = c;
  }
  __syncwarp();
  const float top = byrank[0];
  float s;
  if (renormalize) {
    s = 0.0f;
    for (int j = 0; j < k; ++j) {
      const float ej = exp_recipe(__fsub_rn(byrank[j], top));
      s = (j == 0) ? ej : __fadd_rn(s, ej);
    }
  } else {
    float part = 0.0f;
    for (int c = lane; c < E; c += 32) part += exp_recipe(__fsub_rn(val[c], top));
    for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
    s = part;
  }
  for (int j = lane; j < nout; j += 32)
    weights[row * w_stride + j] = (j < k) ? __fdiv_rn(exp_recipe(__fsub_rn(byrank[j], top)), s) : 0.0f;
}

template <typename T>
static int launch_topk(const void* logits, int64_t M, int E, int64_t stride_m, int64_t stride_e, int k,
                       int renormalize, float* weights, int64_t w_stride, int32_t* ids, int64_t id_stride,
                       int fill_rest, cudaStream_t st) {
  const T* lp = static_cast<const T*>(logits);
  const bool reg_path = !fill_rest && k <= KMAX && E <= 256;
  if constexpr (sizeof(T) == 2) {
    if (reg_path && renormalize)
      return launch_topk16<T>(logits, M, E, stride_m, stride_e, k, weights, w_stride, ids, id_stride, st);
  }
  if (reg_path) {
    const int threads = 256;
#define FR_LAUNCH_TOPK(L_, VPL_)                                                                            \
  do {                                                                                                      \
    const int vec_ok = (stride_e == 1) && (E == (L_) * (VPL_)) && ((stride_m * sizeof(T)) % 16 == 0) &&     \
                       ((reinterpret_cast<uintptr_t>(lp) & 15) == 0);                                       \
    const int64_t total = M * (L_);                                                                         \
    const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);                         \
    topk_softmax_kernel<T, L_, VPL_><<<blocks, threads, 0, st>>>(lp, M, E, stride_m, stride_e, k,           \
                                                                 renormalize, weights, w_stride, ids,       \
                                                                 id_stride, vec_ok);                        \
  } while (0)
    if (E <= 8) FR_LAUNCH_TOPK(1, 8);
    else if (E <= 16) FR_LAUNCH_TOPK(2, 8);
    else if (E <= 32) FR_LAUNCH_TOPK(4, 8);
    else if (E <= 64) FR_LAUNCH_TOPK(8, 8);
    else if (E <= 128) FR_LAUNCH_TOPK(16, 8);
    else FR_LAUNCH_TOPK(32, 8);
#undef FR_LAUNCH_TOPK
  } else {
    if (E > 2048) return FR_ERR_UNSUPPORTED;
    const int warps = 4;
    const size_t smem = static_cast<size_t>(warps) * 2 * E * sizeof(float);
    const unsigned blocks = static_cast<unsigned>((M + warps - 1) / warps);
    topk_rank_kernel<T><<<blocks, warps * 32, smem, st>>>(lp, M, E, stride_m, stride_e, k, renormalize,
                                                          weights, w_stride, ids, id_stride, fill_rest);
  }
  return static_cast<int>(cudaGetLastError());
}

int topk_softmax_dispatch(const void* logits, int dtype, int64_t M, int E, int64_t stride_m, int64_t stride_e,
                          int k, int renormalize, float* weights, int64_t w_stride, int32_t* ids,
                          int64_t id_stride, int fill_rest, cudaStream_t st) {
  if (!logits || !weights || !ids || M < 0 || E <= 0 || k <= 0 || k > E) return FR_ERR_ARG;
  if (M == 0) return FR_OK;
  switch (dtype) {
    case FR_F16:
      return launch_topk<__half>(logits, M, E, stride_m, stride_e, k, renormalize, weights, w_stride, ids,
                                 id_stride, fill_rest, st);
    case FR_BF16:
      return launch_topk<__nv_bfloat16>(logits, M, E, stride_m, stride_e, k, renormalize, weights, w_stride,
                                        ids, id_stride, fill_rest, st);
    case FR_F32:
      return launch_topk<float>(logits, M, E, stride_m, stride_e, k, renormalize, weights, w_stride, ids,
                                id_stride, fill_rest, st);
    default:
      return FR_ERR_ARG;
  }
}

// ----------------------------------------------------------------------------------
// Softmax over ALL E columns, then top-k on the probabilities: the routing of the reference's
// baseline layer (fast_route/fast_route/layers/vllm_route.py:72-84), whose topk_softmax op comes from
// vLLM 0.4.0 (csrc/moe/topk_softmax_kernels.cu there: softmax in fp32, k rounds of arg-max where
// equal probabilities go to the lower expert id, source row = j*M + token).
// Recipe, made of single IEEE fp32 operations so that a CPU checker can follow it bit by bit:
//   e_c = exp_recipe(l_c - max_c l_c);  s = sums of 8 consecutive columns (ascending), combined by a
//   balanced binary tree over adjacent blocks (E padded to a power of two >= 8 with exact zeros);
//   p_c = e_c * (1 / s);  selection on p_c;  renormalize: w_j = p_j / ((p_0 + p_1) + ...).
// ----------------------------------------------------------------------------------
template <typename T, int L>
__global__ void __launch_bounds__(256) softmax_topk_kernel(const T* __restrict__ logits, int64_t M, int E,
                                                           int64_t stride_m, int64_t stride_e, int k,
                                                           int renormalize, float* __restrict__ weights,
                                                           int64_t w_stride, int32_t* __restrict__ ids,
                                                           int64_t id_stride, int32_t* __restrict__ source_rows,
                                                           int64_t src_stride) {
  constexpr int VPL = 8;
  const int64_t gthread = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t row = gthread / L;
  const int sub = static_cast<int>(gthread % L);
  const bool row_ok = row < M;
  const int64_t r = row_ok ? row : (M - 1);
  const int c0 = sub * VPL;
  const T* src = logits + r * stride_m;

  float v[VPL];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = c0 + i;
    float x = (c < E) ? to_f32<T>(src[static_cast<int64_t>(c) * stride_e]) : -INFINITY;
    if (x != x) x = -INFINITY;  // NaN is outside the contract; rank it last
    v[i] = x;
    mx = fmaxf(mx, x);
  }
#pragma unroll
  for (int off = 1; off < L; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));

  float part = 0.0f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    v[i] = (c0 + i < E) ? exp_recipe(__fsub_rn(v[i], mx)) : 0.0f;
    part = (i == 0) ? v[0] : __fadd_rn(part, v[i]);
  }
#pragma unroll
  for (int off = 1; off < L; off <<= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, off));
  const float inv = __fdiv_rn(1.0f, part);
#pragma unroll
  for (int i = 0; i < VPL; ++i) v[i] = (c0 + i < E) ? __fmul_rn(v[i], inv) : -INFINITY;

  float sel_v[KMAX];
  int sel_c[KMAX];
  uint32_t taken = 0;
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    sel_v[j] = 0.0f;
    sel_c[j] = 0;
    if (j < k) {
      float bv = -INFINITY;
      int bc = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const bool free_slot = !((taken >> i) & 1u) && (c0 + i < E);
        if (free_slot && beats(v[i], c0 + i, bv, bc)) {
          bv = v[i];
          bc = c0 + i;
        }
      }
#pragma unroll
      for (int off = L / 2; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
        const int oc = __shfl_xor_sync(0xffffffffu, bc, off);
        if (beats(ov, oc, bv, bc)) {
          bv = ov;
          bc = oc;
        }
      }
      if (bc >= c0 && bc < c0 + VPL) taken |= 1u << (bc - c0);
      sel_v[j] = bv;
      sel_c[j] = bc;
    }
  }
  float s = 1.0f;
  if (renormalize) {
#pragma unroll
    for (int j = 0; j < KMAX; ++j)
      if (j < k) s = (j == 0) ? sel_v[0] : __fadd_rn(s, sel_v[j]);
  }
  if (row_ok) {
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      if (j < k && (j % L) == sub) {
        weights[row * w_stride + j] = renormalize ? __fdiv_rn(sel_v[j], s) : sel_v[j];
        ids[row * id_stride + j] = sel_c[j];
        if (source_rows) source_rows[row * src_stride + j] = static_cast<int32_t>(j * M + row);
      }
    }
  }
}

template <typename T>
static int launch_softmax_topk(const void* logits, int64_t M, int E, int64_t stride_m, int64_t stride_e, int k,
                               int renormalize, float* weights, int64_t w_stride, int32_t* ids, int64_t id_stride,
                               int32_t* source_rows, int64_t src_stride, cudaStream_t st) {
  const T* lp = static_cast<const T*>(logits);
  const int threads = 256;
#define FR_LAUNCH_SMTOPK(L_)                                                                                   \
  do {                                                                                                        \
    const int64_t total = M * (L_);                                                                           \
    const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);                           \
    softmax_topk_kernel<T, L_><<<blocks, threads, 0, st>>>(lp, M, E, stride_m, stride_e, k, renormalize,      \
                                                           weights, w_stride, ids, id_stride, source_rows,    \
                                                           src_stride);                                       \
  } while (0)
  if (E <= 8) FR_LAUNCH_SMTOPK(1);
  else if (E <= 16) FR_LAUNCH_SMTOPK(2);
  else if (E <= 32) FR_LAUNCH_SMTOPK(4);
  else if (E <= 64) FR_LAUNCH_SMTOPK(8);
  else if (E <= 128) FR_LAUNCH_SMTOPK(16);
  else FR_LAUNCH_SMTOPK(32);
#undef FR_LAUNCH_SMTOPK
  return static_cast<int>(cudaGetLastError());
}

int softmax_topk_dispatch(const void* logits, int dtype, int64_t M, int E, int64_t stride_m, int64_t stride_e,
                          int k, int renormalize, float* weights, int64_t w_stride, int32_t* ids,
                          int64_t id_stride, int32_t* source_rows, int64_t src_stride, cudaStream_t st) {
  if (!logits || !weights || !ids || M < 0 || E <= 0 || k <= 0 || k > E) return FR_ERR_ARG;
  if (E > 256 || k > KMAX || static_cast<int64_t>(k) * M > 0x7fffffffLL) return FR_ERR_UNSUPPORTED;
  if (M == 0) return FR_OK;
  switch (dtype) {
    case FR_F16:
      return launch_softmax_topk<__half>(logits, M, E, stride_m, stride_e, k, renormalize, weights, w_stride, ids,
                                         id_stride, source_rows, src_stride, st);
    case FR_BF16:
      return launch_softmax_topk<__nv_bfloat16>(logits, M, E, stride_m, stride_e, k, renormalize, weights,
                                                w_stride, ids, id_stride, source_rows, src_stride, st);
    case FR_F32:
      return launch_softmax_topk<float>(logits, M, E, stride_m, stride_e, k, renormalize, weights, w_stride, ids,
                                        id_stride, source_rows, src_stride, st);
    default:
      return FR_ERR_ARG;
  }
}

// ----------------------------------------------------------------------------------
// align: one thread-block cluster (1..8 CTAs) sorts all n ids.  Warp g of the cluster owns
// the contiguous slice [g*seg, (g+1)*seg) of the flat ids, so (cta, warp, row-of-32, lane)
// order is flat-index order and the sort is stable by construction.
//   pass 1: per-warp per-expert counts (groups of lanes with equal ids, one writer per group)
//   exchange: CTA totals through distributed shared memory; every CTA derives the padded
//             expert starts and its own base offsets
//   pass 2: each id gets base[warp][e] + rank inside its match group
// ----------------------------------------------------------------------------------
// Lanes of the warp holding the same expert id (0 for lanes without a valid id).  One ballot
// per id bit: constant cost, whereas the hardware match instruction slows down with the
// number of distinct values in the warp (up to 32 with many experts).
__device__ __forceinline__ unsigned same_expert_lanes(int e, int nbits) {
  unsigned peers = __ballot_sync(0xffffffffu, e >= 0);
  for (int b = 0; b < nbits; ++b) {
    const bool bit = (e >> b) & 1;
    const unsigned bal = __ballot_sync(0xffffffffu, bit);
    peers &= bit ? bal : ~bal;
  }
  return e >= 0 ? peers : 0u;
}

struct AlignParams {
  const int32_t* ids;
  int64_t n;
  int E;
  int bs;
  int32_t* sorted;
  int64_t sorted_len;
  int32_t* expert_ids;
  int64_t expert_ids_len;
  int32_t* num_post;
  int32_t* counts;
  int32_t* inv_pos;
  int64_t seg;  // ids per warp, multiple of 32
  int nbits;    // bits needed for an expert id
};

// ITERS > 0: a warp's slice is at most ITERS rows of 32 ids and is loaded once into
// registers (all loads in flight together); ITERS == 0: any length, ids re-read per pass.
template <int ITERS>
__global__ void __launch_bounds__(1024) align_cluster_kernel(AlignParams p) {
  extern __shared__ int sm_i[];
  cg::cluster_group cluster = cg::this_cluster();
  const int C = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  const int nwarps = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int E = p.E;

  int* cnt = sm_i;                 // [nwarps][E]  counts, then running write positions
  int* cta_tot = cnt + nwarps * E; // [E]   this CTA's totals (read by the other CTAs)
  int* total = cta_tot + E;        // [E]   cluster-wide totals
  int* start = total + E;          // [E+1] padded starts
  int* before = start + E + 1;     // [E]   totals of lower-ranked CTAs

  for (int i = threadIdx.x; i < nwarps * E; i += blockDim.x) cnt[i] = 0;
  __syncthreads();

  const int64_t g = static_cast<int64_t>(rank) * nwarps + warp;
  const int64_t lo = g * p.seg;
  const int64_t hi = (lo + p.seg < p.n) ? lo + p.seg : p.n;
  int* my = cnt + warp * E;

  constexpr int NREG = ITERS > 0 ? ITERS : 1;
  int held[NREG];
  if constexpr (ITERS > 0) {
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int64_t i = lo + it * 32 + lane;
      held[it] = (i < hi) ? __ldg(p.ids + i) : -1;
    }
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int64_t i = lo + it * 32 + lane;
      if (i < hi && (held[it] < 0 || held[it] >= E)) {
        report(ST_BAD_EXPERT_ID, static_cast<unsigned int>(held[it]));
        held[it] = -1;
      }
    }
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      if (lo + it * 32 < hi) {
        const int e = held[it];
        const unsigned grp = same_expert_lanes(e, p.nbits);
        if (e >= 0 && lane == (__ffs(grp) - 1)) my[e] += __popc(grp);
        __syncwarp();
      }
    }
  } else {
    for (int64_t b = lo; b < hi; b += 32) {
      const int64_t i = b + lane;
      int e = -1;
      if (i < hi) {
        e = __ldg(p.ids + i);
        if (e < 0 || e >= E) {
          report(ST_BAD_EXPERT_ID, static_cast<unsigned int>(e));
          e = -1;
        }
      }
      const unsigned grp = same_expert_lanes(e, p.nbits);
      if (e >= 0 && lane == (__ffs(grp) - 1)) my[e] += __popc(grp);
      __syncwarp();
    }
  }
  __syncthreads();

  // exclusive prefix over the warps of this CTA, CTA totals
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < nwarps; ++w) {
      const int c = cnt[w * E + e];
      cnt[w * E + e] = run;
      run += c;
    }
    cta_tot[e] = run;
  }
  cluster.sync();
  // gather every CTA's totals (one remote load per thread, all in flight), then reduce locally
  int* gathered = before + E;  // [C][E]
  for (int i = threadIdx.x; i < C * E; i += blockDim.x) {
    const int c = i / E, e = i - c * E;
    gathered[i] = cluster.map_shared_rank(cta_tot, c)[e];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0, bfr = 0;
    for (int c = 0; c < C; ++c) {
      const int v = gathered[c * E + e];
      if (c < rank) bfr += v;
      t += v;
    }
    total[e] = t;
    before[e] = bfr;
  }
  cluster.sync();  // nobody reads remote shared memory after this point

  // exclusive scan of padded sizes over experts (warp 0; each lane owns a contiguous chunk)
  if (warp == 0) {
    const int chunk = (E + 31) / 32;
    const int e0 = lane * chunk;
    int sum = 0;
    for (int e = e0; e < e0 + chunk && e < E; ++e) sum += (total[e] + p.bs - 1) / p.bs * p.bs;
    int incl = sum;
    for (int off = 1; off < 32; off <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += o;
    }
    int run = incl - sum;
    for (int e = e0; e < e0 + chunk && e < E; ++e) {
      start[e] = run;
      run += (total[e] + p.bs - 1) / p.bs * p.bs;
    }
    if (lane == 31) start[E] = incl;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nwarps * E; i += blockDim.x) {
    const int e = i % E;
    cnt[i] += start[e] + before[e];
  }
  __syncthreads();

  // pass 2: scatter
  auto place = [&](int64_t i, int e) {
    const unsigned grp = same_expert_lanes(e, p.nbits);
    int pos = 0;
    if (e >= 0) pos = my[e] + __popc(grp & ((1u << lane) - 1u));
    __syncwarp();
    if (e >= 0) {
      if (lane == (__ffs(grp) - 1)) my[e] += __popc(grp);
      if (pos < p.sorted_len) p.sorted[pos] = static_cast<int32_t>(i);
      if (p.inv_pos) p.inv_pos[i] = pos;
    } else if (i < hi && p.inv_pos) {
      p.inv_pos[i] = -1;   // rejected id: the combine must not pick up a stale position
    }
    __syncwarp();
  };
  if constexpr (ITERS > 0) {
#pragma unroll
    for (int it = 0; it < ITERS; ++it)
      if (lo + it * 32 < hi) place(lo + it * 32 + lane, held[it]);
  } else {
    for (int64_t b = lo; b < hi; b += 32) {
      const int64_t i = b + lane;
      int e = -1;
      if (i < hi) {
        e = __ldg(p.ids + i);
        if (e < 0 || e >= E) e = -1;
      }
      place(i, e);
    }
  }

  // padding entries, block -> expert table, tails; spread over the cluster
  const int num_post = start[E];
  const int gwarp = rank * nwarps + warp;
  const int gwarps = C * nwarps;
  for (int e = gwarp; e < E; e += gwarps) {
    const int s = start[e], t = total[e], pe = start[e + 1];
    for (int q = s + t + lane; q < pe; q += 32)
      if (q < p.sorted_len) p.sorted[q] = static_cast<int32_t>(p.n);
    for (int blk = s / p.bs + lane; blk < pe / p.bs; blk += 32)
      if (blk < p.expert_ids_len) p.expert_ids[blk] = e;
    if (p.counts && lane == 0) p.counts[e] = t;
  }
  const int64_t gthread = static_cast<int64_t>(rank) * blockDim.x + threadIdx.x;
  const int64_t gthreads = static_cast<int64_t>(C) * blockDim.x;
  for (int64_t q = num_post + gthread; q < p.sorted_len; q += gthreads) p.sorted[q] = static_cast<int32_t>(p.n);
  for (int64_t blk = num_post / p.bs + gthread; blk < p.expert_ids_len; blk += gthreads) p.expert_ids[blk] = -1;
  if (rank == 0 && threadIdx.x == 0) *p.num_post = num_post;
}

int align_dispatch(const int32_t* topk_ids, int64_t n, int E, int bs, int32_t* sorted_ids, int64_t sorted_len,
                   int32_t* expert_ids, int64_t expert_ids_len, int32_t* num_post, int32_t* counts,
                   int32_t* inv_pos, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (!sorted_ids || !expert_ids || !num_post || n < 0 || E <= 0 || bs <= 0) return FR_ERR_ARG;
  if (n > 0 && !topk_ids) return FR_ERR_ARG;
  if (n >= (1ll << 30) || E > 2048) return FR_ERR_UNSUPPORTED;
  // every possible layout must fit: the reference allocates exactly these sizes
  if (sorted_len < n + static_cast<int64_t>(E) * (bs - 1)) return FR_ERR_ARG;
  if (expert_ids_len < (n + static_cast<int64_t>(E) * (bs - 1)) / bs) return FR_ERR_ARG;

  // many assignments and a scratch buffer: spread over the whole GPU (one cooperative launch)
  {
    const int rc = align_coop_dispatch(topk_ids, n, E, bs, sorted_ids, sorted_len, expert_ids, expert_ids_len,
                                       num_post, counts, inv_pos, workspace, workspace_bytes, st);
    if (rc <= 0 && rc != FR_ERR_UNSUPPORTED) return rc;
    // a launch the device refused (cooperative grid too large for a partitioned GPU, ...) is not
    // fatal: clear the error and let the cluster kernel take the call
    if (rc > 0) (void)cudaGetLastError();
  }

  int threads = 1024;
  if (E > 1024) threads = 256;
  else if (E > 512) threads = 512;
  int C = 1;
  while (C < 8 && static_cast<int64_t>(C) * 4096 < n) C <<= 1;
  const int nwarps = threads / 32;
  const int64_t total_warps = static_cast<int64_t>(C) * nwarps;
  int64_t seg = (n + total_warps - 1) / total_warps;
  seg = (seg + 31) / 32 * 32;
  if (seg == 0) seg = 32;

  AlignParams p{topk_ids, n, E, bs, sorted_ids, sorted_len, expert_ids, expert_ids_len, num_post, counts, inv_pos, seg, 0};
  while ((1 << p.nbits) < E) ++p.nbits;
  const size_t smem = (static_cast<size_t>(nwarps) * E + (4 + static_cast<size_t>(C)) * E + 1) * sizeof(int);
  if (smem > 200 * 1024) return FR_ERR_UNSUPPORTED;
  const int64_t rows_per_warp = seg / 32;
  void (*kern)(AlignParams) = rows_per_warp <= 4    ? align_cluster_kernel<4>
                              : rows_per_warp <= 16 ? align_cluster_kernel<16>
                                                    : align_cluster_kernel<0>;
  if (smem > 48 * 1024)
    FR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(C);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = C;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FR_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p));
  return FR_OK;
}

}  // namespace fr
