// C ABI of libfastroute_sm100.so: argument checks, workspace carving, the memory-bound
// helper kernels (row permute / gather, combine, gate transpose) and the whole-layer
// launch sequence.  See include/fast_route_sm100.h for the contract of every entry point.
#include <cuda_fp8.h>

#include "fr_common.cuh"

namespace fr {

int topk_softmax_dispatch(const void* logits, int dtype, int64_t M, int E, int64_t stride_m, int64_t stride_e,
                          int k, int renormalize, float* weights, int64_t w_stride, int32_t* ids,
                          int64_t id_stride, int fill_rest, cudaStream_t st);
int align_dispatch(const int32_t* topk_ids, int64_t n, int E, int bs, int32_t* sorted_ids, int64_t sorted_len,
                   int32_t* expert_ids, int64_t expert_ids_len, int32_t* num_post, int32_t* counts,
                   int32_t* inv_pos, void* workspace, size_t workspace_bytes, cudaStream_t st);
size_t coop_workspace_bytes(int E);
int align_noalloc_dispatch(const int32_t* topk_ids, int64_t n, int E, int bs, int32_t* sorted_ids,
                           int64_t sorted_len, int32_t* expert_ids, int64_t expert_ids_len, int32_t* num_post,
                           int32_t* counts, int32_t* inv_pos, cudaStream_t st);
int gemm_grouped_dispatch(int which, const void* a, int64_t lda, const void* w, int dtype, int64_t max_rows,
                          int K, int n_out, int E, int b_rows_per_expert, const int32_t* expert_ids,
                          const int32_t* num_post, const int32_t* sorted_ids, const float* topk_w, int64_t n_valid,
                          void* out, int64_t ldo, int split_k, void* workspace, size_t workspace_bytes,
                          cudaStream_t st, int* deferred_split, const QuantArgs* quant, int64_t rows_hint);
int combine_partial_dispatch(const void* workspace, int split_k, int64_t n_valid, int n_out, int64_t partial_cols,
                             const float* topk_w, const int32_t* inv_pos, int64_t M, int topk, int dtype,
                             const void* residual, int64_t ld_res, void* out, int64_t ld_out, cudaStream_t st);
int gemm_tokenn_dispatch(int which, const void* a, int64_t lda, const void* w, int dtype, int64_t max_rows, int K,
                         int n_out, int E, int w_rows_per_expert, const int32_t* counts, const int32_t* num_post,
                         const int32_t* sorted_ids, const float* topk_w, int64_t n_valid, void* out, int64_t ldo,
                         int split_k, void* workspace, size_t workspace_bytes, cudaStream_t st, int* deferred_split,
                         const QuantArgs* quant);
int router_gemm_dispatch(const void* x, int dtype, int64_t M, int H, int64_t ldx, const void* gate_km,
                         int64_t ld_gate, int E, int topk, int renormalize, int do_topk, float* weights,
                         int32_t* ids, float* logits_out, cudaStream_t st);
int choose_split_k(int64_t est_tiles, int KB, int sm_count, bool few_rows = false);

constexpr int kBlockM = FR_GEMM_BLOCK_M;
constexpr int kTileN = 256;
constexpr int kTileK = 64;

// ----------------------------------------------------------------------------------
// memory-bound helpers
// ----------------------------------------------------------------------------------
// dst[p,:] = src[sorted_ids[p] / topk, :] for p < num_post; padding entries become zeros.
__global__ void __launch_bounds__(256) permute_rows_kernel(const uint4* __restrict__ src, int64_t ld_src_v,
                                                           const int32_t* __restrict__ sorted_ids,
                                                           const int32_t* __restrict__ num_post, int64_t n, int topk,
                                                           uint4* __restrict__ dst, int64_t ld_dst_v, int row_v) {
  const int64_t row = blockIdx.x;
  if (num_post && row >= __ldg(num_post)) return;
  const int32_t sid = __ldg(sorted_ids + row);
  uint4* d = dst + row * ld_dst_v;
  if (sid >= 0 && sid < n) {
    const uint4* s = src + static_cast<int64_t>(sid / topk) * ld_src_v;
    for (int v = threadIdx.x; v < row_v; v += blockDim.x) d[v] = __ldg(s + v);
  } else {
    for (int v = threadIdx.x; v < row_v; v += blockDim.x) d[v] = make_uint4(0, 0, 0, 0);
  }
}

// dst[i,:] = src[idx[i],:]; idx < 0 -> zeros
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ src, int64_t ld_src_v,
                                                          const int32_t* __restrict__ idx, uint4* __restrict__ dst,
                                                          int64_t ld_dst_v, int row_v) {
  const int64_t row = blockIdx.x;
  const int32_t s = __ldg(idx + row);
  uint4* d = dst + row * ld_dst_v;
  if (s >= 0) {
    const uint4* sp = src + static_cast<int64_t>(s) * ld_src_v;
    for (int v = threadIdx.x; v < row_v; v += blockDim.x) d[v] = __ldg(sp + v);
  } else {
    for (int v = threadIdx.x; v < row_v; v += blockDim.x) d[v] = make_uint4(0, 0, 0, 0);
  }
}

// out[t,:] = (residual[t,:] +) sum_j y[inv_pos[t*topk+j], :], fp32 accumulation in slot order, one
// rounding.  out may alias residual (each thread reads its residual vector before storing it).
template <bool BF16>
__global__ void __launch_bounds__(256) combine_kernel(const uint4* __restrict__ y, int64_t ld_y_v,
                                                      const int32_t* __restrict__ inv_pos, int topk, int row_v,
                                                      int64_t max_rows, const uint4* residual, int64_t ld_res_v,
                                                      uint4* out, int64_t ld_out_v) {
  const int64_t t = blockIdx.x;
  for (int v = threadIdx.x; v < row_v; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    if (residual) {
      const uint4 raw = residual[t * ld_res_v + v];
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack2<BF16>(w[i]);
        acc[2 * i] = f.x;
        acc[2 * i + 1] = f.y;
      }
    }
    for (int j = 0; j < topk; ++j) {
      const int32_t pos = __ldg(inv_pos + t * topk + j);
      if (pos < 0 || pos >= max_rows) continue;
      const uint4 raw = __ldg(y + static_cast<int64_t>(pos) * ld_y_v + v);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack2<BF16>(w[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
    out[t * ld_out_v + v] = make_uint4(pack2<BF16>(acc[0], acc[1]), pack2<BF16>(acc[2], acc[3]),
                                       pack2<BF16>(acc[4], acc[5]), pack2<BF16>(acc[6], acc[7]));
  }
}

// gate[h*sh + e*se] (two-byte elements) -> gate_km[e*ld + h]
__global__ void transpose_gate_kernel(const uint16_t* __restrict__ gate, int64_t sh, int64_t se, int H, int E,
                                      uint16_t* __restrict__ out, int64_t ld) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<int64_t>(E) * ld) return;
  const int e = static_cast<int>(i / ld);
  const int h = static_cast<int>(i % ld);
  out[i] = h < H ? gate[h * sh + e * se] : static_cast<uint16_t>(0);
}

// Residual add and RMSNorm in one pass over the rows: h = a (+ b); x = h * rsqrt(mean(h^2) + eps) * gamma.
// One CTA per row, 16-byte vectors, the row is held in registers between the two phases (H <= 16384).
// h is rounded to the element type first and the norm is taken of the rounded values, as a framework
// that materialises h would do.  h_out and x_out are optional; without gamma, x_out = h.
template <bool BF16>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const uint4* __restrict__ a, int64_t ld_a_v,
                                                          const uint4* __restrict__ b, int64_t ld_b_v,
                                                          const uint4* __restrict__ gamma, float eps, int H,
                                                          uint4* __restrict__ h_out, int64_t ld_h_v,
                                                          uint4* __restrict__ x_out, int64_t ld_x_v) {
  constexpr int MAXV = 8;
  __shared__ float red[8];
  const int64_t row = blockIdx.x;
  const int row_v = H / 8;
  uint4 hv[MAXV];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < row_v) {
      uint4 ra = __ldg(a + row * ld_a_v + v);
      uint32_t w[4] = {ra.x, ra.y, ra.z, ra.w};
      if (b) {
        const uint4 rb = __ldg(b + row * ld_b_v + v);
        const uint32_t wb[4] = {rb.x, rb.y, rb.z, rb.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 fa = unpack2<BF16>(w[q]), fb = unpack2<BF16>(wb[q]);
          w[q] = pack2<BF16>(fa.x + fb.x, fa.y + fb.y);
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = unpack2<BF16>(w[q]);
        ss = fmaf(f.x, f.x, ss);
        ss = fmaf(f.y, f.y, ss);
      }
      hv[i] = make_uint4(w[0], w[1], w[2], w[3]);
      if (h_out) h_out[row * ld_h_v + v] = hv[i];
    }
  }
  if (!x_out) return;
  float scale = 1.0f;
  if (gamma) {
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w];
    scale = rsqrtf(tot / static_cast<float>(H) + eps);
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < row_v) {
      uint32_t w[4] = {hv[i].x, hv[i].y, hv[i].z, hv[i].w};
      if (gamma) {
        const uint4 rg = __ldg(gamma + v);
        const uint32_t wg[4] = {rg.x, rg.y, rg.z, rg.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = unpack2<BF16>(w[q]), g = unpack2<BF16>(wg[q]);
          w[q] = pack2<BF16>(f.x * scale * g.x, f.y * scale * g.y);
        }
      }
      x_out[row * ld_x_v + v] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// ----------------------------------------------------------------------------------
// fp8 (E4M3) activations: one scale per row, scale = absmax / 448, value = round(v / scale)
// ----------------------------------------------------------------------------------
__device__ __forceinline__ uint2 quant8_e4m3(const float (&v)[8], float scale) {
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint32_t a = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(v[4 * i], scale), __fdiv_rn(v[4 * i + 1], scale)),
                                                __NV_SATFINITE, __NV_E4M3);
    const uint32_t b = __nv_cvt_float2_to_fp8x2(
        make_float2(__fdiv_rn(v[4 * i + 2], scale), __fdiv_rn(v[4 * i + 3], scale)), __NV_SATFINITE, __NV_E4M3);
    const uint32_t w = a | (b << 16);
    if (i == 0) lo = w; else hi = w;
  }
  return make_uint2(lo, hi);
}

// Shared body: the CTA holds one row (up to 8 vectors of 8 elements per thread), finds its absmax,
// writes the fp8 row and the scale.  src == nullptr writes a zero row with scale 1.
template <bool BF16>
__device__ __forceinline__ void quant_row(const uint4* __restrict__ src, int row_v, uint2* __restrict__ dst,
                                          float* __restrict__ scale_out) {
  constexpr int MAXV = 8;
  __shared__ float red[8];
  float vals[MAXV][8];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < row_v && src) {
      const uint4 raw = __ldg(src + v);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = unpack2<BF16>(w[q]);
        vals[i][2 * q] = f.x;
        vals[i][2 * q + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) vals[i][q] = 0.0f;
    }
  }
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot = fmaxf(tot, red[w]);
  const float scale = tot > 0.0f ? __fdiv_rn(tot, 448.0f) : 1.0f;
  if (threadIdx.x == 0) *scale_out = scale;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < row_v) dst[v] = quant8_e4m3(vals[i], scale);
  }
}

// a_q[p,:] = fp8(x[sorted_ids[p] / topk, :]) with its row scale: the gather of the fp8 layer
template <bool BF16>
__global__ void __launch_bounds__(256) permute_quant_rows_kernel(const uint4* __restrict__ src, int64_t ld_src_v,
                                                                 const int32_t* __restrict__ sorted_ids,
                                                                 const int32_t* __restrict__ num_post, int64_t n,
                                                                 int topk, uint2* __restrict__ dst, int64_t ld_dst_v,
                                                                 float* __restrict__ row_scale, int row_v) {
  const int64_t row = blockIdx.x;
  if (row >= __ldg(num_post)) return;
  const int32_t sid = __ldg(sorted_ids + row);
  const uint4* s = (sid >= 0 && sid < n) ? src + static_cast<int64_t>(sid / topk) * ld_src_v : nullptr;
  quant_row<BF16>(s, row_v, dst + row * ld_dst_v, row_scale + row);
}

// act_q[p,:] = fp8(act[p,:]) with its row scale, for the rows in use
template <bool BF16>
__global__ void __launch_bounds__(256) quant_rows_kernel(const uint4* __restrict__ src, int64_t ld_src_v,
                                                         const int32_t* __restrict__ num_post,
                                                         uint2* __restrict__ dst, int64_t ld_dst_v,
                                                         float* __restrict__ row_scale, int row_v) {
  const int64_t row = blockIdx.x;
  if (row >= __ldg(num_post)) return;
  quant_row<BF16>(src + row * ld_src_v, row_v, dst + row * ld_dst_v, row_scale + row);
}

// Router for a handful of rows (decode-sized batches): one CTA per token, the H-long dot
// products are split over the threads (fp32 FMA, fixed reduction order), then warp 0 ranks
// the E logits by counting (ties -> lower expert id) and writes the top-k and its softmax.
// A 128-row tensor-core tile would leave 147 SMs idle and walk H serially on one.
template <bool BF16>
__device__ __forceinline__ void router_small_body(float* rs, int64_t row, const uint16_t* __restrict__ x, int64_t ldx,
                                                  const uint16_t* __restrict__ gate_km, int64_t ld_gate, int H, int E,
                                                  int topk, int renormalize, float* __restrict__ weights,
                                                  int32_t* __restrict__ ids, float* __restrict__ logits_out) {
  float* part = rs;                 // [H splits][E]
  float* logit = rs + 8 * E;        // [E]
  float* byrank = logit + E;        // [E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint16_t* xr = x + row * ldx;
  // The 8 warps form eg expert groups x hs splits of H (eg * hs = 8): a warp accumulates 8 experts over its share
  // of H, so one pass covers 8 * eg experts (E = 8: all warps split H; E >= 64: every warp walks all of H for its
  // own 8 experts and 64 experts take one pass instead of eight).
  int eg = 1;
  while (eg < 8 && eg * 8 < E) eg <<= 1;
  const int hs = 8 / eg;
  const int g = warp % eg, sidx = warp / eg;
  for (int ec = 0; ec < E; ec += 8 * eg) {
    const int e0 = ec + g * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    if (e0 < E) {
      for (int h = (sidx * 32 + lane) * 8; h < H; h += hs * 32 * 8) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xr + h);
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (e0 + i < E) {
            const uint4 gv = __ldg(reinterpret_cast<const uint4*>(gate_km + static_cast<int64_t>(e0 + i) * ld_gate + h));
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 a = unpack2<BF16>(xw[q]);
              const float2 b = unpack2<BF16>(gw[q]);
              acc[i] = fmaf(a.x, b.x, acc[i]);
              acc[i] = fmaf(a.y, b.y, acc[i]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float v = acc[i];
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      if (lane == 0 && e0 + i < E) part[sidx * E + e0 + i] = v;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += 256) {
    float v = 0.0f;
    for (int w = 0; w < hs; ++w) v += part[w * E + e];
    if (v != v) v = -INFINITY;
    logit[e] = v;
    if (logits_out) logits_out[row * E + e] = v;
  }
  __syncthreads();
  if (warp != 0 || !weights) return;
  for (int c = lane; c < E; c += 32) {
    const float v = logit[c];
    int rank = 0;
    for (int o = 0; o < E; ++o) {
      const float ov = logit[o];
      rank += static_cast<int>(ov > v) | (static_cast<int>(ov == v) & static_cast<int>(o < c));
    }
    byrank[rank] = v;
    if (rank < topk) ids[row * topk + rank] = c;
  }
  __syncwarp();
  const float top = byrank[0];
  float s;
  if (renormalize) {
    s = 0.0f;
    for (int j = 0; j < topk; ++j) {
      const float ej = exp_recipe(__fsub_rn(byrank[j], top));
      s = (j == 0) ? ej : __fadd_rn(s, ej);
    }
  } else {
    float psum = 0.0f;
    for (int c = lane; c < E; c += 32) psum += exp_recipe(__fsub_rn(logit[c], top));
    for (int off = 16; off > 0; off >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, off);
    s = psum;
  }
  for (int j = lane; j < topk; j += 32) weights[row * topk + j] = __fdiv_rn(exp_recipe(__fsub_rn(byrank[j], top)), s);
}

template <bool BF16>
__global__ void __launch_bounds__(256) router_small_kernel(const uint16_t* __restrict__ x, int64_t ldx,
                                                           const uint16_t* __restrict__ gate_km, int64_t ld_gate,
                                                           int H, int E, int topk, int renormalize,
                                                           float* __restrict__ weights, int32_t* __restrict__ ids,
                                                           float* __restrict__ logits_out) {
  extern __shared__ float rs[];
  router_small_body<BF16>(rs, blockIdx.x, x, ldx, gate_km, ld_gate, H, E, topk, renormalize, weights, ids,
                          logits_out);
}

// Logits of a handful of rows against MANY experts: the one-CTA-per-token router walks H once per 64 experts with
// its loads in a serial chain (E = 128, H = 4096: 60 us for one token, whatever the batch).  Here a CTA takes 8
// experts of one token and its 8 warps split H, so a token's experts spread over E / 8 CTAs; the ranking then runs
// as the router-from-logits kernel on the fp32 logits.
template <bool BF16>
__global__ void __launch_bounds__(256) router_logits_small_kernel(const uint16_t* __restrict__ x, int64_t ldx,
                                                                  const uint16_t* __restrict__ gate_km,
                                                                  int64_t ld_gate, int H, int E,
                                                                  float* __restrict__ logits_out) {
  __shared__ float part[8][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e0 = blockIdx.x * 8;
  const int64_t row = blockIdx.y;
  const uint16_t* xr = x + row * ldx;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  for (int h = (warp * 32 + lane) * 8; h < H; h += 8 * 32 * 8) {
    const uint4 xv = *reinterpret_cast<const uint4*>(xr + h);
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
    uint4 gv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      gv[i] = (e0 + i < E) ? __ldg(reinterpret_cast<const uint4*>(gate_km + static_cast<int64_t>(e0 + i) * ld_gate + h))
                           : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t gw[4] = {gv[i].x, gv[i].y, gv[i].z, gv[i].w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 a = unpack2<BF16>(xw[q]);
        const float2 b = unpack2<BF16>(gw[q]);
        acc[i] = fmaf(a.x, b.x, acc[i]);
        acc[i] = fmaf(a.y, b.y, acc[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float v = acc[i];
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if (lane == 0) part[warp][i] = v;
  }
  __syncthreads();
  if (threadIdx.x < 8 && e0 + threadIdx.x < E) {
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) v += part[w][threadIdx.x];   // fixed order
    if (v != v) v = -INFINITY;
    logits_out[row * E + e0 + threadIdx.x] = v;
  }
}

// Decode prologue: router, align (block 16) and the row gather of a batch of at most 16 assignments in ONE launch.
// One CTA per token routes it; the CTA that finishes last (a counter in the zeroed scratch, put back to zero) then
// sorts the handful of assignments by expert and copies the token rows into expert order.  At this size the three
// separate launches cost more in launch gaps than in work (router 5-12, cluster align 7, gather 4 us for 1 token).
// Rows of a_sorted that only pad an expert's segment are left untouched: a padded row is one column of the
// tokens-on-N GEMM tiles and never mixes into another token's results.
constexpr int kPrologueMaxAssign = 16;
struct PrologueParams {
  const uint16_t* x;
  int64_t ldx;
  const uint16_t* gate_km;
  int64_t ld_gate;
  int H, E, topk, renormalize, M, bs;
  float* weights;
  int32_t* ids;
  int32_t* sorted;
  int64_t sorted_len;
  int32_t* expert_ids;
  int64_t expert_ids_len;
  int32_t* num_post;
  int32_t* counts;
  int32_t* inv_pos;
  uint16_t* a_sorted;      // row pitch H
  unsigned int* counter;   // zero before the launch, zero again after it
};

template <bool BF16>
__global__ void __launch_bounds__(256) decode_prologue_kernel(const PrologueParams p) {
  extern __shared__ float rs[];
  __shared__ int s_last;
  __shared__ int s_ids[kPrologueMaxAssign];
  __shared__ int s_pos[kPrologueMaxAssign];
  router_small_body<BF16>(rs, blockIdx.x, p.x, p.ldx, p.gate_km, p.ld_gate, p.H, p.E, p.topk, p.renormalize,
                          p.weights, p.ids, nullptr);
  // publish this token's routing, then find out whether every other token is done
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(p.counter, 1u);
    s_last = (prev == static_cast<unsigned int>(p.M) - 1u) ? 1 : 0;
    if (s_last) *p.counter = 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();

  const int E = p.E, n = p.M * p.topk, bs = p.bs;
  int* cnt = reinterpret_cast<int*>(rs);      // [E] counts, the router's scratch is free now
  int* start = cnt + E;                       // [E+1] padded starts
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    int e = __ldcg(p.ids + i);
    if (e < 0 || e >= E) {
      report(ST_BAD_EXPERT_ID, static_cast<unsigned int>(e));
      e = -1;
    }
    s_ids[i] = e;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int c = 0;
    for (int i = 0; i < n; ++i) c += (s_ids[i] == e) ? 1 : 0;
    cnt[e] = c;
    if (p.counts) p.counts[e] = c;
  }
  __syncthreads();
  if (threadIdx.x < 32) {     // exclusive scan of the padded counts, a chunk of experts per lane
    const int lane = threadIdx.x;
    const int chunk = (E + 31) / 32;
    const int e0 = lane * chunk;
    int sum = 0;
    for (int e = e0; e < e0 + chunk && e < E; ++e) sum += (cnt[e] + bs - 1) / bs * bs;
    int incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += o;
    }
    int run = incl - sum;
    for (int e = e0; e < e0 + chunk && e < E; ++e) {
      start[e] = run;
      run += (cnt[e] + bs - 1) / bs * bs;
    }
    if (lane == 31) start[E] = incl;
  }
  __syncthreads();
  const int num_post = start[E];
  // sentinels and the block -> expert table everywhere, then the valid entries on top
  for (int64_t q = threadIdx.x; q < p.sorted_len; q += blockDim.x) p.sorted[q] = n;
  for (int64_t b = threadIdx.x; b < p.expert_ids_len; b += blockDim.x) p.expert_ids[b] = -1;
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    for (int b = start[e] / bs; b < start[e + 1] / bs; ++b)
      if (b < p.expert_ids_len) p.expert_ids[b] = e;
  if (threadIdx.x < n) {
    const int i = threadIdx.x, e = s_ids[i];
    int pos = -1;
    if (e >= 0) {
      int rank = 0;
      for (int j = 0; j < i; ++j) rank += (s_ids[j] == e) ? 1 : 0;    // stable: earlier flat index first
      pos = start[e] + rank;
      if (pos < p.sorted_len) p.sorted[pos] = i;
    }
    if (p.inv_pos) p.inv_pos[i] = pos;   // -1 for a rejected id: the combine skips it
    s_pos[i] = pos;
  }
  if (threadIdx.x == 0) *p.num_post = num_post;
  __syncthreads();
  // gather: token rows into expert order, 16-byte vectors
  const int row_v = p.H / 8;
  for (int i = 0; i < n; ++i) {
    const int pos = s_pos[i];
    if (pos < 0) continue;
    const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<int64_t>(i / p.topk) * p.ldx);
    uint4* dst = reinterpret_cast<uint4*>(p.a_sorted + static_cast<int64_t>(pos) * p.H);
    for (int v = threadIdx.x; v < row_v; v += blockDim.x) dst[v] = __ldg(src + v);
  }
}

// ----------------------------------------------------------------------------------
// workspace carving
// ----------------------------------------------------------------------------------
struct Carver {
  uint8_t* base;
  size_t off = 0;
  explicit Carver(void* b) : base(static_cast<uint8_t*>(b)) {}
  template <typename T>
  T* take(size_t count) {
    off = (off + 1023) & ~size_t(1023);
    T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += count * sizeof(T);
    return p;
  }
  size_t total() const { return (off + 1023) & ~size_t(1023); }
};

static int64_t round_up(int64_t a, int64_t b) { return (a + b - 1) / b * b; }

static int sm_count_or_default() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) == cudaSuccess &&
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0)
    return sms;
  (void)cudaGetLastError();
  return 148;
}

// Upper bound on padded rows: every expert that can hold a token pads by < kBlockM.
static int64_t rows_cap(int64_t n, int E) {
  const int64_t active = n < E ? n : E;
  return round_up(n + active * (kBlockM - 1), kBlockM);
}

struct SplitPlan {
  int s1 = 1, s2 = 1;
  size_t bytes = 0;
};
static SplitPlan plan_split(int64_t n, int H, int I, int E) {
  SplitPlan sp;
  if (n <= 0) return sp;
  const int sms = sm_count_or_default();
  const int64_t est_mb = (n < E ? n : E) + n / kBlockM;
  const int nb1 = (I + kTileN / 2 - 1) / (kTileN / 2), nb2 = (H + kTileN - 1) / kTileN;
  sp.s1 = choose_split_k(est_mb * nb1, (H + kTileK - 1) / kTileK, sms);
  sp.s2 = choose_split_k(est_mb * nb2, (I + kTileK - 1) / kTileK, sms);
  size_t b1 = sp.s1 > 1 ? static_cast<size_t>(sp.s1) * n * nb1 * kTileN * sizeof(float) : 0;
  size_t b2 = sp.s2 > 1 ? static_cast<size_t>(sp.s2) * n * nb2 * kTileN * sizeof(float) : 0;
  sp.bytes = b1 > b2 ? b1 : b2;
  return sp;
}

// Token-N path (fr_gemm_tokenn.cu): used while an expert sees at most this many tokens on average.
// Its small token operand leaves room for up to 10 pipeline stages of weights (160 KB in flight per
// SM against 128 KB in the row-block kernel), which is what a weight-streaming batch needs; with
// 256-token tiles only a third of the in-flight bytes are weights and the row-block kernel wins.
// (measured on B200, Mixtral-8x7B shape: 3-13 % faster up to 128 tokens per expert, slower from 256)
constexpr int64_t kTokenNMaxTokensPerExpert = 200;   // measured: 160/expert -9 %, 192/expert -5 %, 256/expert +3 %
constexpr int kTokenNMaxExperts = 256;
static bool use_tokenn(int64_t n, int E) { return E <= kTokenNMaxExperts && n <= kTokenNMaxTokensPerExpert * E; }

static SplitPlan plan_split_tokenn(int64_t n, int H, int I, int E) {
  SplitPlan sp;
  if (n <= 0) return sp;
  const int sms = sm_count_or_default();
  const int64_t avg = (n + E - 1) / E;
  int box = 16;
  while (box < 256 && box < 2 * avg) box <<= 1;
  const int64_t est_tt = (n < E ? n : E) + n / box;  // token tiles: one per active expert + full ones
  const int wt1 = (I + 63) / 64, wt2 = (H + 127) / 128;
  const bool few = n <= 32;
  sp.s1 = choose_split_k(est_tt * wt1, (H + kTileK - 1) / kTileK, sms, few);
  sp.s2 = choose_split_k(est_tt * wt2, (I + kTileK - 1) / kTileK, sms, few);
  size_t b1 = sp.s1 > 1 ? static_cast<size_t>(sp.s1) * n * wt1 * 128 * sizeof(float) : 0;
  size_t b2 = sp.s2 > 1 ? static_cast<size_t>(sp.s2) * n * wt2 * 128 * sizeof(float) : 0;
  sp.bytes = b1 > b2 ? b1 : b2;
  return sp;
}

constexpr int kSmallRouterRows = 32;
// The batches the one-CTA-per-token router takes (see route_fused_impl), and among them the ones with enough
// experts that a token's experts are better spread over several CTAs.
static bool small_router_batch(int64_t M, int H, int E) {
  return M <= kSmallRouterRows || static_cast<int64_t>(M) * E * H < (int64_t(1) << 26);
}
static bool small_batch_many_experts(int64_t M, int H, int E) { return E >= 32 && E <= 1024 && small_router_batch(M, H, E); }

struct RouteWs {
  uint16_t* gate_km;
  float* logits;
  int64_t ld_gate;
};
static RouteWs carve_route(Carver& c, int64_t M, int H, int E, int topk) {
  RouteWs r;
  r.ld_gate = round_up(H, 8);
  r.gate_km = c.take<uint16_t>(static_cast<size_t>(E) * r.ld_gate);
  // fp32 logits are kept when the ranking runs as its own kernel: topk > 8, or few rows against many experts
  const bool need_logits = topk > 8 || small_batch_many_experts(M, H, E);
  r.logits = c.take<float>(need_logits ? static_cast<size_t>(M) * E : 0);
  return r;
}

static int route_fused_impl(const void* x, int dtype, int64_t M, int H, int64_t ldx, const void* gate,
                            int64_t gsh, int64_t gse, int E, int topk, int renormalize, float* weights,
                            int32_t* ids, float* logits_out, const RouteWs& ws, cudaStream_t st) {
  const void* gate_km = gate;
  int64_t ld_gate = gse;
  if (gsh != 1 || (gse % 8) != 0 || (reinterpret_cast<uintptr_t>(gate) & 15)) {
    const int64_t total = static_cast<int64_t>(E) * ws.ld_gate;
    transpose_gate_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(
        static_cast<const uint16_t*>(gate), gsh, gse, H, E, ws.gate_km, ws.ld_gate);
    FR_CUDA_OK(cudaGetLastError());
    gate_km = ws.gate_km;
    ld_gate = ws.ld_gate;
  }
  // The tensor-core router walks H serially in every CTA (about 23 us for H = 4096 whatever the batch), so the
  // one-CTA-per-token kernel also takes the mid-size batches for which its M*E*H multiply-adds cost less than that
  // (measured crossover: 2048 tokens at E = 8, H = 4096; 512 tokens at E = 64, H = 2048).  The two kernels add in
  // different orders, so the last bits of a token's logits depend on which one its batch size selects.
  const bool gemv = small_router_batch(M, H, E);
  const bool vec_ok = (H % 8) == 0 && (ldx % 8) == 0 && (ld_gate % 8) == 0 &&
                      (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(gate_km) & 15) == 0;
  if (gemv && vec_ok && small_batch_many_experts(M, H, E) && (logits_out || ws.logits) && M <= 65535) {
    float* lg = logits_out ? logits_out : ws.logits;
    const dim3 grid(static_cast<unsigned>((E + 7) / 8), static_cast<unsigned>(M));
    if (dtype == FR_BF16)
      router_logits_small_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(x), ldx,
                                                             static_cast<const uint16_t*>(gate_km), ld_gate, H, E, lg);
    else
      router_logits_small_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(x), ldx,
                                                              static_cast<const uint16_t*>(gate_km), ld_gate, H, E, lg);
    FR_CUDA_OK(cudaGetLastError());
    if (!weights) return FR_OK;
    return topk_softmax_dispatch(lg, FR_F32, M, E, E, 1, topk, renormalize, weights, topk, ids, topk, 0, st);
  }
  if (gemv && vec_ok && E <= 1024) {
    const size_t smem = static_cast<size_t>(10) * E * sizeof(float);
    if (dtype == FR_BF16)
      router_small_kernel<true><<<static_cast<unsigned>(M), 256, smem, st>>>(
          static_cast<const uint16_t*>(x), ldx, static_cast<const uint16_t*>(gate_km), ld_gate, H, E, topk,
          renormalize, weights, ids, logits_out);
    else
      router_small_kernel<false><<<static_cast<unsigned>(M), 256, smem, st>>>(
          static_cast<const uint16_t*>(x), ldx, static_cast<const uint16_t*>(gate_km), ld_gate, H, E, topk,
          renormalize, weights, ids, logits_out);
    return static_cast<int>(cudaGetLastError());
  }
  if (topk <= 8) {
    return router_gemm_dispatch(x, dtype, M, H, ldx, gate_km, ld_gate, E, topk, renormalize, 1, weights, ids,
                                logits_out, st);
  }
  float* lg = logits_out ? logits_out : ws.logits;
  int rc = router_gemm_dispatch(x, dtype, M, H, ldx, gate_km, ld_gate, E, topk, renormalize, 0, nullptr, nullptr,
                                lg, st);
  if (rc) return rc;
  return topk_softmax_dispatch(lg, FR_F32, M, E, E, 1, topk, renormalize, weights, topk, ids, topk, 0, st);
}

struct ExpertWs {
  int32_t *sorted, *expert_ids, *num_post, *inv_pos, *counts;
  uint16_t *a_sorted, *act, *y_sorted;
  void* split;
  void* align_ws;
  size_t align_ws_bytes;
  int64_t rows, sorted_len, expert_ids_len;
  SplitPlan sp;
};
// The align stage's scratch (grid-barrier words + histogram) must sit at a fixed place of the
// caller's workspace whatever the batch size, because it relies on being zero between calls:
// it is always carved first, at offset 0.
static void carve_align_ws(Carver& c, int E, void** ws, size_t* bytes) {
  *bytes = coop_workspace_bytes(E);
  *ws = c.take<uint8_t>(*bytes);
}

static ExpertWs carve_experts(Carver& c, int64_t n, int H, int I, int E) {
  ExpertWs w;
  w.align_ws = nullptr;
  w.align_ws_bytes = 0;
  w.rows = rows_cap(n, E);
  w.sorted_len = round_up(n + static_cast<int64_t>(E) * (kBlockM - 1), kBlockM);
  w.expert_ids_len = w.sorted_len / 16 + 1;   // block -> expert table, sized for the 16-row alignment
  w.sorted = c.take<int32_t>(w.sorted_len);
  w.expert_ids = c.take<int32_t>(w.expert_ids_len);
  w.num_post = c.take<int32_t>(4);
  w.inv_pos = c.take<int32_t>(n);
  w.counts = c.take<int32_t>(E);
  w.a_sorted = c.take<uint16_t>(static_cast<size_t>(w.rows) * H);
  w.act = c.take<uint16_t>(static_cast<size_t>(w.rows) * I);
  w.y_sorted = c.take<uint16_t>(static_cast<size_t>(w.rows) * H);
  w.sp = use_tokenn(n, E) ? plan_split_tokenn(n, H, I, E) : plan_split(n, H, I, E);
  {  // the scratch also covers the row-block plan (used by the fp8 layer at every batch size)
    const size_t rb = plan_split(n, H, I, E).bytes;
    if (rb > w.sp.bytes) w.sp.bytes = rb;
  }
  w.split = c.take<uint8_t>(w.sp.bytes);
  return w;
}

// Router + align + row gather in one launch for at most kPrologueMaxAssign assignments (see decode_prologue_kernel).
// Returns FR_ERR_UNSUPPORTED when the case does not qualify; the caller then runs the separate stages.
static int decode_prologue_dispatch(const void* x, int dtype, int64_t M, int H, int64_t ldx, const void* gate,
                                    int64_t gsh, int64_t gse, int E, int topk, int renormalize, float* weights,
                                    int32_t* ids, const ExpertWs& w, cudaStream_t st) {
  const int64_t n = M * topk;
  // (with many experts the router inside the prologue, one CTA per token, is the slow part: separate stages then)
  if (n > kPrologueMaxAssign || M < 1 || !use_tokenn(n, E) || E >= 32 || !w.align_ws || w.align_ws_bytes < 16)
    return FR_ERR_UNSUPPORTED;
  if (dtype != FR_F16 && dtype != FR_BF16) return FR_ERR_UNSUPPORTED;
  // the gate must already be K-major (W_g[E,H] viewed as [H,E]); otherwise the transposing path runs
  if (gsh != 1 || (gse % 8) || (H % 8) || (ldx % 8) || (reinterpret_cast<uintptr_t>(gate) & 15) ||
      (reinterpret_cast<uintptr_t>(x) & 15))
    return FR_ERR_UNSUPPORTED;
  PrologueParams p = {};
  p.x = static_cast<const uint16_t*>(x);
  p.ldx = ldx;
  p.gate_km = static_cast<const uint16_t*>(gate);
  p.ld_gate = gse;
  p.H = H;
  p.E = E;
  p.topk = topk;
  p.renormalize = renormalize;
  p.M = static_cast<int>(M);
  p.bs = 16;
  p.weights = weights;
  p.ids = ids;
  p.sorted = w.sorted;
  p.sorted_len = w.sorted_len;
  p.expert_ids = w.expert_ids;
  p.expert_ids_len = w.expert_ids_len;
  p.num_post = w.num_post;
  p.counts = w.counts;
  p.inv_pos = w.inv_pos;
  p.a_sorted = w.a_sorted;
  p.counter = reinterpret_cast<unsigned int*>(w.align_ws) + 2;   // after the two grid-barrier words
  const size_t smem = static_cast<size_t>(10) * E * sizeof(float);
  if (dtype == FR_BF16) decode_prologue_kernel<true><<<static_cast<unsigned>(M), 256, smem, st>>>(p);
  else decode_prologue_kernel<false><<<static_cast<unsigned>(M), 256, smem, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

// align -> permute -> GEMM1+SiLU -> GEMM2 -> combine for n assignments (flat id i belongs to
// token i / topk) whose expert ids are in `ids`.
static int experts_impl(const void* x, int64_t ldx, const int32_t* ids, const float* weights, const void* w1,
                        const void* w2, int dtype, int64_t M, int topk, int H, int I, int E, void* out,
                        int64_t ld_out, const ExpertWs& w, cudaStream_t st, const void* residual = nullptr,
                        int64_t ld_res = 0, bool prologue_done = false) {
  // prologue_done: align outputs and a_sorted were already produced by decode_prologue_dispatch
  const int64_t n = M * topk;
  const bool tokenn = use_tokenn(n, E);
  int rc = FR_OK;
  const int row_v = H / 8;
  if (!prologue_done) {
    rc = align_dispatch(ids, n, E, tokenn ? 16 : kBlockM, w.sorted, w.sorted_len, w.expert_ids, w.expert_ids_len,
                        w.num_post, w.counts, w.inv_pos, w.align_ws, w.align_ws_bytes, st);
    if (rc) return rc;
    permute_rows_kernel<<<static_cast<unsigned>(w.rows), 256, 0, st>>>(
        static_cast<const uint4*>(x), ldx / 8, w.sorted, w.num_post, n, topk, reinterpret_cast<uint4*>(w.a_sorted),
        H / 8, row_v);
    FR_CUDA_OK(cudaGetLastError());
  }
  if (tokenn) {
    // few tokens per expert: tokens on the MMA N axis, experts padded to 16 rows instead of 128
    rc = gemm_tokenn_dispatch(0, w.a_sorted, H, w1, dtype, w.rows, H, I, E, 2 * I, w.counts, w.num_post, w.sorted,
                              nullptr, n, w.act, I, w.sp.s1, w.split, w.sp.bytes, st, nullptr, nullptr);
    if (rc) return rc;
    int deferred = 0;
    rc = gemm_tokenn_dispatch(1, w.act, I, w2, dtype, w.rows, I, H, E, H, w.counts, w.num_post, w.sorted, weights, n,
                              w.y_sorted, H, w.sp.s2, w.split, w.sp.bytes, st, &deferred, nullptr);
    if (rc) return rc;
    if (deferred > 1)
      return combine_partial_dispatch(w.split, deferred, n, H, static_cast<int64_t>((H + 127) / 128) * 128, weights,
                                      w.inv_pos, M, topk, dtype, residual, ld_res, out, ld_out, st);
  } else {
    rc = gemm_grouped_dispatch(0, w.a_sorted, H, w1, dtype, w.rows, H, I, E, 2 * I, w.expert_ids, w.num_post,
                               w.sorted, nullptr, n, w.act, I, w.sp.s1, w.split, w.sp.bytes, st, nullptr, nullptr);
    if (rc) return rc;
    int deferred = 0;
    rc = gemm_grouped_dispatch(1, w.act, I, w2, dtype, w.rows, I, H, E, H, w.expert_ids, w.num_post, w.sorted,
                               weights, n, w.y_sorted, H, w.sp.s2, w.split, w.sp.bytes, st, &deferred, nullptr);
    if (rc) return rc;
    if (deferred > 1)  // split-K GEMM2: its reduction, the routed weights and the sum over slots in one kernel
      return combine_partial_dispatch(w.split, deferred, n, H, static_cast<int64_t>((H + kTileN - 1) / kTileN) * kTileN,
                                      weights, w.inv_pos, M, topk, dtype, residual, ld_res, out, ld_out, st);
  }
  if (dtype == FR_BF16)
    combine_kernel<true><<<static_cast<unsigned>(M), 256, 0, st>>>(
        reinterpret_cast<const uint4*>(w.y_sorted), H / 8, w.inv_pos, topk, row_v, w.rows,
        static_cast<const uint4*>(residual), ld_res / 8, static_cast<uint4*>(out), ld_out / 8);
  else
    combine_kernel<false><<<static_cast<unsigned>(M), 256, 0, st>>>(
        reinterpret_cast<const uint4*>(w.y_sorted), H / 8, w.inv_pos, topk, row_v, w.rows,
        static_cast<const uint4*>(residual), ld_res / 8, static_cast<uint4*>(out), ld_out / 8);
  return static_cast<int>(cudaGetLastError());
}


// ---- expert parallelism over peer memory (kernels in fr_ep.cu) ---------------------------------
struct EpWs {
  int32_t *seg_start, *seg_count, *seg_src_off, *num_post, *expert_ids, *sorted_local;
  float* w_sorted;
  uint16_t *a_sorted, *act;
};
static EpWs carve_ep(Carver& c, int64_t cap_rows, int H, int I, int E) {
  EpWs w;
  const size_t nseg = static_cast<size_t>(E);   // E/W local experts x W sources
  w.seg_start = c.take<int32_t>(nseg + 1);
  w.seg_count = c.take<int32_t>(nseg);
  w.seg_src_off = c.take<int32_t>(nseg);
  w.num_post = c.take<int32_t>(4);
  w.expert_ids = c.take<int32_t>(cap_rows / kBlockM + 1);
  w.sorted_local = c.take<int32_t>(cap_rows);
  w.w_sorted = c.take<float>(cap_rows);
  w.a_sorted = c.take<uint16_t>(static_cast<size_t>(cap_rows) * H);
  w.act = c.take<uint16_t>(static_cast<size_t>(cap_rows) * I);
  return w;
}

}  // namespace fr

using namespace fr;

extern "C" {

int fr_version(void) { return 100; }

const char* fr_error_string(int code) {
  switch (code) {
    case FR_OK: return "ok";
    case FR_ERR_ARG: return "invalid argument";
    case FR_ERR_UNSUPPORTED: return "size, dtype or layout not supported";
    case FR_ERR_ALIGN: return "pointer or stride not 16-byte aligned";
    case FR_ERR_WORKSPACE: return "workspace missing or too small";
    case FR_ERR_DRIVER: return "CUDA driver tensor-map entry point unavailable or rejected the descriptor";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown error";
  }
}

int fr_check_status(unsigned int* out4) {
  if (!out4) return FR_ERR_ARG;
  FR_CUDA_OK(cudaDeviceSynchronize());
  FR_CUDA_OK(cudaMemcpyFromSymbol(out4, g_status, 4 * sizeof(unsigned int)));
  const unsigned int zero[4] = {0, 0, 0, 0};
  FR_CUDA_OK(cudaMemcpyToSymbol(g_status, zero, sizeof(zero)));
  return FR_OK;
}

int fr_topk_softmax(const void* logits, int dtype, int64_t M, int E, int64_t stride_m, int64_t stride_e, int topk,
                    int renormalize, float* weights, int64_t w_stride, int32_t* ids, int64_t id_stride,
                    int fill_rest, void* stream) {
  return topk_softmax_dispatch(logits, dtype, M, E, stride_m, stride_e, topk, renormalize, weights, w_stride, ids,
                               id_stride, fill_rest, static_cast<cudaStream_t>(stream));
}

int fr_w4a16_gemm(const void* a, int64_t lda, const int32_t* qweight, const void* scales, const int32_t* qzeros,
                  int64_t m, int n, int k, int groupsize, void* c, int64_t ldc, int split_k, void* stream) {
  return fr::w4a16_gemm_dispatch(a, lda, qweight, scales, qzeros, m, n, k, groupsize, c, ldc, split_k,
                                 static_cast<cudaStream_t>(stream));
}

int fr_w4a16_dequant(const int32_t* qweight, const void* scales, const int32_t* qzeros, int n, int k, int groupsize,
                     void* w, int64_t ldw, void* stream) {
  return fr::w4a16_dequant_dispatch(qweight, scales, qzeros, n, k, groupsize, w, ldw,
                                    static_cast<cudaStream_t>(stream));
}

int fr_softmax_topk(const void* logits, int dtype, int64_t M, int E, int64_t stride_m, int64_t stride_e, int topk,
                    int renormalize, float* weights, int64_t w_stride, int32_t* ids, int64_t id_stride,
                    int32_t* source_rows, int64_t src_stride, void* stream) {
  return fr::softmax_topk_dispatch(logits, dtype, M, E, stride_m, stride_e, topk, renormalize, weights, w_stride, ids,
                                   id_stride, source_rows, src_stride, static_cast<cudaStream_t>(stream));
}

size_t fr_align_workspace_bytes(int E) { return E > 0 ? coop_workspace_bytes(E) : 0; }

int fr_align(const int32_t* topk_ids, int64_t n, int E, int block_size, int32_t* sorted_ids, int64_t sorted_len,
             int32_t* expert_ids, int64_t expert_ids_len, int32_t* num_tokens_post_pad, int32_t* counts,
             int32_t* inv_pos, void* workspace, size_t workspace_bytes, void* stream) {
  return align_dispatch(topk_ids, n, E, block_size, sorted_ids, sorted_len, expert_ids, expert_ids_len,
                        num_tokens_post_pad, counts, inv_pos, workspace, workspace_bytes,
                        static_cast<cudaStream_t>(stream));
}

int fr_align_noalloc(const int32_t* topk_ids, int64_t n, int E, int block_size, int32_t* sorted_ids,
                     int64_t sorted_len, int32_t* expert_ids, int64_t expert_ids_len, int32_t* num_tokens_post_pad,
                     int32_t* counts, int32_t* inv_pos, void* stream) {
  return align_noalloc_dispatch(topk_ids, n, E, block_size, sorted_ids, sorted_len, expert_ids, expert_ids_len,
                                num_tokens_post_pad, counts, inv_pos, static_cast<cudaStream_t>(stream));
}

int fr_route_align(const void* logits, int dtype, int64_t M, int E, int64_t stride_m, int64_t stride_e, int topk,
                   float* weights, int32_t* ids, int block_size, int32_t* sorted_ids, int64_t sorted_len,
                   int32_t* expert_ids, int64_t expert_ids_len, int32_t* num_tokens_post_pad, void* workspace,
                   size_t workspace_bytes, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!logits || !weights || !ids || !sorted_ids || !expert_ids || !num_tokens_post_pad || M < 0 || E <= 0 ||
      topk <= 0 || topk > E || block_size <= 0)
    return FR_ERR_ARG;
  const int64_t n = M * topk;
  if (sorted_len < n + static_cast<int64_t>(E) * (block_size - 1) ||
      expert_ids_len < (n + static_cast<int64_t>(E) * (block_size - 1)) / block_size)
    return FR_ERR_ARG;
  int rc = topk_softmax_dispatch(logits, dtype, M, E, stride_m, stride_e, topk, 1, weights, topk, ids, topk, 0, st);
  if (rc) return rc;
  return align_dispatch(ids, n, E, block_size, sorted_ids, sorted_len, expert_ids, expert_ids_len,
                        num_tokens_post_pad, nullptr, nullptr, workspace, workspace_bytes, st);
}

size_t fr_route_fused_workspace_bytes(int64_t M, int H, int E, int topk) {
  Carver c(nullptr);
  carve_route(c, M, H, E, topk);
  return c.total();
}

int fr_route_fused(const void* x, int dtype, int64_t M, int H, int64_t ldx, const void* gate, int64_t gate_stride_h,
                   int64_t gate_stride_e, int E, int topk, int renormalize, float* weights, int32_t* ids,
                   float* logits_out, void* workspace, size_t workspace_bytes, void* stream) {
  if (!x || !gate || !weights || !ids || M < 0 || H <= 0 || E <= 0 || topk <= 0 || topk > E) return FR_ERR_ARG;
  if (M == 0) return FR_OK;
  if (!workspace || workspace_bytes < fr_route_fused_workspace_bytes(M, H, E, topk)) return FR_ERR_WORKSPACE;
  Carver c(workspace);
  RouteWs ws = carve_route(c, M, H, E, topk);
  return route_fused_impl(x, dtype, M, H, ldx, gate, gate_stride_h, gate_stride_e, E, topk, renormalize, weights,
                          ids, logits_out, ws, static_cast<cudaStream_t>(stream));
}

int fr_permute_rows(const void* src, int dtype, int H, int64_t ld_src, const int32_t* sorted_ids,
                    const int32_t* num_tokens_post_pad, int64_t n, int topk, int64_t max_rows, void* dst,
                    int64_t ld_dst, void* stream) {
  if (!src || !sorted_ids || !dst || H <= 0 || topk <= 0 || max_rows < 0) return FR_ERR_ARG;
  if (dtype != FR_F16 && dtype != FR_BF16) return FR_ERR_UNSUPPORTED;
  if ((H % 8) || (ld_src % 8) || (ld_dst % 8) || (reinterpret_cast<uintptr_t>(src) & 15) ||
      (reinterpret_cast<uintptr_t>(dst) & 15))
    return FR_ERR_ALIGN;
  if (max_rows == 0) return FR_OK;
  permute_rows_kernel<<<static_cast<unsigned>(max_rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), ld_src / 8, sorted_ids, num_tokens_post_pad, n, topk,
      static_cast<uint4*>(dst), ld_dst / 8, H / 8);
  return static_cast<int>(cudaGetLastError());
}

int64_t fr_moe_experts_rows_cap(int64_t R, int E_local) { return R > 0 && E_local > 0 ? rows_cap(R, E_local) : 0; }

size_t fr_ep_workspace_bytes(int64_t cap_rows, int H, int I, int E) {
  if (cap_rows <= 0 || H <= 0 || I <= 0 || E <= 0) return 0;
  Carver c(nullptr);
  carve_ep(c, cap_rows, H, I, E);
  return c.total();
}

int fr_ep_experts(const void* const* peer_base, int world, int rank, int64_t x_off, int64_t ld_x, int64_t peer_rows,
                  int64_t sorted_off, int64_t tw_off, int64_t n_per_rank, int topk, const int32_t* all_counts,
                  const void* w1, const void* w2, int dtype, int H, int I, int E, void* y_sorted, int64_t y_rows,
                  int32_t* comb_base, int stages, void* workspace, size_t workspace_bytes, void* stream) {
  if (!peer_base || !all_counts || !w1 || !w2 || !y_sorted || !comb_base || world <= 0 || rank < 0 || rank >= world ||
      peer_rows <= 0 || n_per_rank <= 0 || topk <= 0 || H <= 0 || I <= 0 || E <= 0 || y_rows <= 0)
    return FR_ERR_ARG;
  if (E % world || E > kEpMaxExperts) return FR_ERR_UNSUPPORTED;
  if (dtype != FR_F16 && dtype != FR_BF16) return FR_ERR_UNSUPPORTED;
  if ((H % 8) || (I % 8) || (ld_x % 8) || (x_off % 16) || (sorted_off % 4) || (tw_off % 4) || (y_rows % kBlockM) ||
      (reinterpret_cast<uintptr_t>(y_sorted) & 15))
    return FR_ERR_ALIGN;
  if (y_rows >= (int64_t(1) << 31)) return FR_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < fr_ep_workspace_bytes(y_rows, H, I, E)) return FR_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 1023) return FR_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int El = E / world;
  Carver c(workspace);
  EpWs w = carve_ep(c, y_rows, H, I, E);

  EpPlanParams pp = {};
  pp.counts = all_counts;
  pp.W = world;
  pp.E = E;
  pp.El = El;
  pp.rank = rank;
  pp.cap_rows = y_rows;
  pp.seg_start = w.seg_start;
  pp.seg_count = w.seg_count;
  pp.seg_src_off = w.seg_src_off;
  pp.comb_base = comb_base;
  pp.num_post = w.num_post;
  pp.expert_ids = w.expert_ids;
  if (stages & 1) {
    ep_plan_kernel<<<1, 256, 0, st>>>(pp);
    FR_CUDA_OK(cudaGetLastError());
  }

  EpGatherParams gp = {};
  gp.peer_base = reinterpret_cast<const uint8_t* const*>(peer_base);
  gp.x_off = x_off;
  gp.sorted_off = sorted_off;
  gp.tw_off = tw_off;
  gp.ld_x_v = ld_x / 8;
  gp.peer_rows = peer_rows;
  gp.n_per_rank = n_per_rank;
  gp.W = world;
  gp.El = El;
  gp.topk = topk;
  gp.row_v = H / 8;
  gp.seg_start = w.seg_start;
  gp.seg_count = w.seg_count;
  gp.seg_src_off = w.seg_src_off;
  gp.num_post = w.num_post;
  gp.a_sorted = reinterpret_cast<uint4*>(w.a_sorted);
  gp.ld_a_v = H / 8;
  gp.w_sorted = w.w_sorted;
  gp.sorted_local = w.sorted_local;
  gp.cap_rows = y_rows;
  const int64_t want = static_cast<int64_t>(sm_count_or_default()) * 16;
  const unsigned ggrid = static_cast<unsigned>(y_rows < want ? y_rows : want);
  if (stages & 1) {
    ep_gather_kernel<<<ggrid, 256, (static_cast<size_t>(E) + 1) * sizeof(int), st>>>(gp);
    FR_CUDA_OK(cudaGetLastError());
  }

  // Both GEMMs on the rows in use (the count lives on the device; tiles beyond it are never started).  The row
  // count the tile order is tuned for is the balanced share, n_per_rank.  No split-K: its scratch is sized by rows.
  const int64_t rows_hint = n_per_rank;
  int rc = FR_OK;
  if (stages & 2)
    rc = gemm_grouped_dispatch(0, w.a_sorted, H, w1, dtype, y_rows, H, I, El, 2 * I, w.expert_ids, w.num_post,
                               w.sorted_local, nullptr, y_rows, w.act, I, 1, nullptr, 0, st, nullptr, nullptr,
                               rows_hint);
  if (rc) return rc;
  if (stages & 4)
    rc = gemm_grouped_dispatch(1, w.act, I, w2, dtype, y_rows, I, H, El, H, w.expert_ids, w.num_post, w.sorted_local,
                               w.w_sorted, y_rows, y_sorted, H, 1, nullptr, 0, st, nullptr, nullptr, rows_hint);
  return rc;
}

int fr_ep_combine(const void* const* peer_base, int world, int64_t y_off, int64_t ld_y, int64_t y_rows, int dtype,
                  const int32_t* topk_ids, const int32_t* inv_pos, const int32_t* comb_base, int64_t M, int topk, int H,
                  int E, void* out, int64_t ld_out, void* stream) {
  if (!peer_base || !topk_ids || !inv_pos || !comb_base || !out || M < 0 || topk <= 0 || H <= 0 || world <= 0 ||
      E <= 0 || y_rows <= 0)
    return FR_ERR_ARG;
  if (E % world) return FR_ERR_UNSUPPORTED;
  if (dtype != FR_F16 && dtype != FR_BF16) return FR_ERR_UNSUPPORTED;
  if ((H % 8) || (ld_y % 8) || (ld_out % 8) || (y_off % 16) || (reinterpret_cast<uintptr_t>(out) & 15))
    return FR_ERR_ALIGN;
  if (M == 0) return FR_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint8_t* const* pb = reinterpret_cast<const uint8_t* const*>(peer_base);
  if (dtype == FR_BF16)
    ep_combine_kernel<true><<<static_cast<unsigned>(M), 256, 0, st>>>(pb, y_off, ld_y / 8, y_rows, world, E / world, E,
                                                                      topk_ids, inv_pos, comb_base, topk, H / 8,
                                                                      static_cast<uint4*>(out), ld_out / 8);
  else
    ep_combine_kernel<false><<<static_cast<unsigned>(M), 256, 0, st>>>(pb, y_off, ld_y / 8, y_rows, world, E / world,
                                                                       E, topk_ids, inv_pos, comb_base, topk, H / 8,
                                                                       static_cast<uint4*>(out), ld_out / 8);
  return static_cast<int>(cudaGetLastError());
}

int fr_gather_rows(const void* src, int64_t ld_src, const int32_t* idx, int64_t rows, int row_bytes, void* dst,
                   int64_t ld_dst, void* stream) {
  if (!src || !idx || !dst || rows < 0 || row_bytes <= 0) return FR_ERR_ARG;
  if ((row_bytes % 16) || (ld_src % 16) || (ld_dst % 16) || (reinterpret_cast<uintptr_t>(src) & 15) ||
      (reinterpret_cast<uintptr_t>(dst) & 15))
    return FR_ERR_ALIGN;
  if (rows == 0) return FR_OK;
  gather_rows_kernel<<<static_cast<unsigned>(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), ld_src / 16, idx, static_cast<uint4*>(dst), ld_dst / 16, row_bytes / 16);
  return static_cast<int>(cudaGetLastError());
}

size_t fr_gemm_splitk_workspace_bytes(int64_t n_valid, int64_t n_cols, int split_k) {
  if (split_k <= 1) return 0;
  return static_cast<size_t>(split_k) * static_cast<size_t>(n_valid) * round_up(n_cols, kTileN) * sizeof(float);
}

int fr_gemm1_silu(const void* a_sorted, int64_t lda, const void* w1, int dtype, int64_t max_rows, int H, int I,
                  int E, const int32_t* expert_ids, const int32_t* num_tokens_post_pad, const int32_t* sorted_ids,
                  int64_t n, void* act, int64_t ld_act, int split_k, void* workspace, size_t workspace_bytes,
                  void* stream) {
  return gemm_grouped_dispatch(0, a_sorted, lda, w1, dtype, max_rows, H, I, E, 2 * I, expert_ids,
                               num_tokens_post_pad, sorted_ids, nullptr, n, act, ld_act, split_k, workspace,
                               workspace_bytes, static_cast<cudaStream_t>(stream), nullptr, nullptr);
}

int fr_gemm2(const void* act, int64_t ld_act, const void* w2, int dtype, int64_t max_rows, int H, int I, int E,
             const int32_t* expert_ids, const int32_t* num_tokens_post_pad, const int32_t* sorted_ids,
             const float* topk_weights, int64_t n, void* y, int64_t ld_y, int split_k, void* workspace,
             size_t workspace_bytes, void* stream) {
  return gemm_grouped_dispatch(1, act, ld_act, w2, dtype, max_rows, I, H, E, H, expert_ids, num_tokens_post_pad,
                               sorted_ids, topk_weights, n, y, ld_y, split_k, workspace, workspace_bytes,
                               static_cast<cudaStream_t>(stream), nullptr, nullptr);
}

int fr_combine(const void* y, int64_t ld_y, int dtype, const int32_t* inv_pos, int64_t M, int topk, int H,
               int64_t max_rows, void* out, int64_t ld_out, void* stream) {
  if (!y || !inv_pos || !out || M < 0 || topk <= 0 || H <= 0) return FR_ERR_ARG;
  if (dtype != FR_F16 && dtype != FR_BF16) return FR_ERR_UNSUPPORTED;
  if ((H % 8) || (ld_y % 8) || (ld_out % 8) || (reinterpret_cast<uintptr_t>(y) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return FR_ERR_ALIGN;
  if (M == 0) return FR_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == FR_BF16)
    combine_kernel<true><<<static_cast<unsigned>(M), 256, 0, st>>>(static_cast<const uint4*>(y), ld_y / 8, inv_pos,
                                                                   topk, H / 8, max_rows, nullptr, 0,
                                                                   static_cast<uint4*>(out), ld_out / 8);
  else
    combine_kernel<false><<<static_cast<unsigned>(M), 256, 0, st>>>(static_cast<const uint4*>(y), ld_y / 8, inv_pos,
                                                                    topk, H / 8, max_rows, nullptr, 0,
                                                                    static_cast<uint4*>(out), ld_out / 8);
  return static_cast<int>(cudaGetLastError());
}

size_t fr_moe_workspace_bytes(int64_t M, int H, int I, int E, int topk) {
  if (M <= 0 || H <= 0 || I <= 0 || E <= 0 || topk <= 0) return 0;
  Carver c(nullptr);
  void* aws;
  size_t aws_bytes;
  carve_align_ws(c, E, &aws, &aws_bytes);
  carve_route(c, M, H, E, topk);
  c.take<float>(M * topk);
  c.take<int32_t>(M * topk);
  carve_experts(c, M * topk, H, I, E);
  return c.total();
}

int fr_moe_layer(const void* x, const void* gate, int64_t gate_stride_h, int64_t gate_stride_e, const void* w1,
                 const void* w2, int dtype, int64_t M, int H, int I, int E, int topk, int renormalize, void* out,
                 float* topk_weights_out, int32_t* topk_ids_out, void* workspace, size_t workspace_bytes,
                 void* stream) {
  if (!x || !gate || !w1 || !w2 || !out || M < 0 || H <= 0 || I <= 0 || E <= 0 || topk <= 0 || topk > E)
    return FR_ERR_ARG;
  if (dtype != FR_F16 && dtype != FR_BF16) return FR_ERR_UNSUPPORTED;
  if ((H % 8) || (I % 8)) return FR_ERR_ALIGN;
  if (M == 0) return FR_OK;
  if (!workspace || workspace_bytes < fr_moe_workspace_bytes(M, H, I, E, topk)) return FR_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 1023) return FR_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Carver c(workspace);
  void* aws;
  size_t aws_bytes;
  carve_align_ws(c, E, &aws, &aws_bytes);
  RouteWs rws = carve_route(c, M, H, E, topk);
  float* tw = c.take<float>(M * topk);
  int32_t* ti = c.take<int32_t>(M * topk);
  ExpertWs ews = carve_experts(c, M * topk, H, I, E);
  ews.align_ws = aws;
  ews.align_ws_bytes = aws_bytes;
  if (topk_weights_out) tw = topk_weights_out;
  if (topk_ids_out) ti = topk_ids_out;
  int rc = decode_prologue_dispatch(x, dtype, M, H, H, gate, gate_stride_h, gate_stride_e, E, topk, renormalize, tw, ti,
                                    ews, st);
  if (rc == FR_OK) return experts_impl(x, H, ti, tw, w1, w2, dtype, M, topk, H, I, E, out, H, ews, st, nullptr, 0, true);
  if (rc != FR_ERR_UNSUPPORTED) return rc;
  rc = route_fused_impl(x, dtype, M, H, H, gate, gate_stride_h, gate_stride_e, E, topk, renormalize, tw, ti,
                        nullptr, rws, st);
  if (rc) return rc;
  return experts_impl(x, H, ti, tw, w1, w2, dtype, M, topk, H, I, E, out, H, ews, st);
}

int fr_add_rmsnorm(const void* a, int64_t ld_a, const void* b, int64_t ld_b, const void* gamma, float eps, int dtype,
                   int64_t M, int H, void* h_out, int64_t ld_h, void* x_out, int64_t ld_x, void* stream) {
  if (!a || M < 0 || H <= 0 || (!h_out && !x_out)) return FR_ERR_ARG;
  if (dtype != FR_F16 && dtype != FR_BF16) return FR_ERR_UNSUPPORTED;
  if (H > 8 * 8 * 256) return FR_ERR_UNSUPPORTED;
  if ((H % 8) || (ld_a % 8) || (b && (ld_b % 8)) || (h_out && (ld_h % 8)) || (x_out && (ld_x % 8)))
    return FR_ERR_ALIGN;
  for (const void* p : {a, b, gamma, static_cast<const void*>(h_out), static_cast<const void*>(x_out)})
    if (p && (reinterpret_cast<uintptr_t>(p) & 15)) return FR_ERR_ALIGN;
  if (M == 0) return FR_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == FR_BF16)
    add_rmsnorm_kernel<true><<<static_cast<unsigned>(M), 256, 0, st>>>(
        static_cast<const uint4*>(a), ld_a / 8, static_cast<const uint4*>(b), ld_b / 8,
        static_cast<const uint4*>(gamma), eps, H, static_cast<uint4*>(h_out), ld_h / 8, static_cast<uint4*>(x_out),
        ld_x / 8);
  else
    add_rmsnorm_kernel<false><<<static_cast<unsigned>(M), 256, 0, st>>>(
        static_cast<const uint4*>(a), ld_a / 8, static_cast<const uint4*>(b), ld_b / 8,
        static_cast<const uint4*>(gamma), eps, H, static_cast<uint4*>(h_out), ld_h / 8, static_cast<uint4*>(x_out),
        ld_x / 8);
  return static_cast<int>(cudaGetLastError());
}

size_t fr_moe_block_workspace_bytes(int64_t M, int H, int I, int E, int topk) {
  if (M <= 0 || H <= 0) return 0;
  return fr_moe_workspace_bytes(M, H, I, E, topk) + ((static_cast<size_t>(M) * H * 2 + 1023) & ~size_t(1023)) * 2;
}

int fr_moe_block(const void* attn_out, const void* x, const void* gamma, float eps, const void* gate,
                 int64_t gate_stride_h, int64_t gate_stride_e, const void* w1, const void* w2, int dtype, int64_t M,
                 int H, int I, int E, int topk, int renormalize, int add_residual, void* out, void* workspace,
                 size_t workspace_bytes, void* stream) {
  if (!attn_out || !gate || !w1 || !w2 || !out || M < 0 || H <= 0 || I <= 0 || E <= 0 || topk <= 0 || topk > E)
    return FR_ERR_ARG;
  if (M == 0) return FR_OK;
  if (!workspace || workspace_bytes < fr_moe_block_workspace_bytes(M, H, I, E, topk)) return FR_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 1023) return FR_ERR_ALIGN;
  // layer workspace first (its align scratch must stay at offset 0), then h and the normalised input
  const size_t layer_bytes = fr_moe_workspace_bytes(M, H, I, E, topk);
  const size_t row_bytes = (static_cast<size_t>(M) * H * 2 + 1023) & ~size_t(1023);
  uint8_t* base = static_cast<uint8_t*>(workspace);
  void* h = base + layer_bytes;
  void* u = base + layer_bytes + row_bytes;
  const bool need_h = (x != nullptr);   // without x, h is attn_out itself
  const void* moe_in = attn_out;
  const void* res = nullptr;
  if (gamma) {
    int rc = fr_add_rmsnorm(attn_out, H, x, H, gamma, eps, dtype, M, H, need_h ? h : nullptr, H, u, H, stream);
    if (rc) return rc;
    moe_in = u;
    res = add_residual ? (need_h ? h : attn_out) : nullptr;
  } else if (x) {  // no norm: the experts read h itself
    int rc = fr_add_rmsnorm(attn_out, H, x, H, nullptr, eps, dtype, M, H, h, H, nullptr, H, stream);
    if (rc) return rc;
    moe_in = h;
    res = add_residual ? h : nullptr;
  } else if (add_residual) {
    res = attn_out;
  }
  Carver c(workspace);
  void* aws;
  size_t aws_bytes;
  carve_align_ws(c, E, &aws, &aws_bytes);
  RouteWs rws = carve_route(c, M, H, E, topk);
  float* tw = c.take<float>(M * topk);
  int32_t* ti = c.take<int32_t>(M * topk);
  ExpertWs ews = carve_experts(c, M * topk, H, I, E);
  ews.align_ws = aws;
  ews.align_ws_bytes = aws_bytes;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = decode_prologue_dispatch(moe_in, dtype, M, H, H, gate, gate_stride_h, gate_stride_e, E, topk, renormalize,
                                    tw, ti, ews, st);
  if (rc == FR_OK) return experts_impl(moe_in, H, ti, tw, w1, w2, dtype, M, topk, H, I, E, out, H, ews, st, res, H, true);
  if (rc != FR_ERR_UNSUPPORTED) return rc;
  rc = route_fused_impl(moe_in, dtype, M, H, H, gate, gate_stride_h, gate_stride_e, E, topk, renormalize, tw, ti,
                        nullptr, rws, st);
  if (rc) return rc;
  return experts_impl(moe_in, H, ti, tw, w1, w2, dtype, M, topk, H, I, E, out, H, ews, st, res, H);
}

// ---- fp8 (E4M3) expert weights ---------------------------------------------------------------
struct Fp8Ws {
  uint8_t *a_q, *act_q;
  float *a_scale, *act_scale;
};
static size_t carve_fp8_layer(Carver& c, int64_t M, int H, int I, int E, int topk, void** aws, size_t* aws_bytes,
                              RouteWs* rws, float** tw, int32_t** ti, ExpertWs* ews, Fp8Ws* f8) {
  carve_align_ws(c, E, aws, aws_bytes);
  *rws = carve_route(c, M, H, E, topk);
  *tw = c.take<float>(M * topk);
  *ti = c.take<int32_t>(M * topk);
  *ews = carve_experts(c, M * topk, H, I, E);
  f8->a_q = c.take<uint8_t>(static_cast<size_t>(ews->rows) * H);
  f8->act_q = c.take<uint8_t>(static_cast<size_t>(ews->rows) * I);
  f8->a_scale = c.take<float>(ews->rows);
  f8->act_scale = c.take<float>(ews->rows);
  return c.total();
}

size_t fr_moe_fp8_workspace_bytes(int64_t M, int H, int I, int E, int topk) {
  if (M <= 0 || H <= 0 || I <= 0 || E <= 0 || topk <= 0) return 0;
  Carver c(nullptr);
  void* aws;
  size_t ab;
  RouteWs rws;
  float* tw;
  int32_t* ti;
  ExpertWs ews;
  Fp8Ws f8;
  return carve_fp8_layer(c, M, H, I, E, topk, &aws, &ab, &rws, &tw, &ti, &ews, &f8);
}

int fr_moe_layer_fp8(const void* x, const void* gate, int64_t gate_stride_h, int64_t gate_stride_e, const void* w1_q,
                     const float* w1_scale, const void* w2_q, const float* w2_scale, int dtype, int64_t M, int H, int I,
                     int E, int topk, int renormalize, void* out, float* topk_weights_out, int32_t* topk_ids_out,
                     void* workspace, size_t workspace_bytes, void* stream) {
  if (!x || !gate || !w1_q || !w1_scale || !w2_q || !w2_scale || !out || M < 0 || H <= 0 || I <= 0 || E <= 0 ||
      topk <= 0 || topk > E)
    return FR_ERR_ARG;
  if (dtype != FR_F16 && dtype != FR_BF16) return FR_ERR_UNSUPPORTED;
  if ((H % 16) || (I % 16)) return FR_ERR_ALIGN;
  if (H > 16384 || I > 16384) return FR_ERR_UNSUPPORTED;  // a row is quantised by one CTA holding it in registers
  if (M == 0) return FR_OK;
  if (!workspace || workspace_bytes < fr_moe_fp8_workspace_bytes(M, H, I, E, topk)) return FR_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 1023) return FR_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Carver c(workspace);
  void* aws;
  size_t ab;
  RouteWs rws;
  float* tw;
  int32_t* ti;
  ExpertWs w;
  Fp8Ws f8;
  carve_fp8_layer(c, M, H, I, E, topk, &aws, &ab, &rws, &tw, &ti, &w, &f8);
  w.align_ws = aws;
  w.align_ws_bytes = ab;
  if (topk_weights_out) tw = topk_weights_out;
  if (topk_ids_out) ti = topk_ids_out;
  int rc = route_fused_impl(x, dtype, M, H, H, gate, gate_stride_h, gate_stride_e, E, topk, renormalize, tw, ti,
                            nullptr, rws, st);
  if (rc) return rc;
  const int64_t n = M * topk;
  const bool tokenn = use_tokenn(n, E);
  rc = align_dispatch(ti, n, E, tokenn ? 16 : kBlockM, w.sorted, w.sorted_len, w.expert_ids, w.expert_ids_len,
                      w.num_post, w.counts, w.inv_pos, w.align_ws, w.align_ws_bytes, st);
  if (rc) return rc;
  const bool bf = dtype == FR_BF16;
  const unsigned rows = static_cast<unsigned>(w.rows);
  if (bf)
    permute_quant_rows_kernel<true><<<rows, 256, 0, st>>>(static_cast<const uint4*>(x), H / 8, w.sorted, w.num_post, n,
                                                          topk, reinterpret_cast<uint2*>(f8.a_q), H / 8, f8.a_scale,
                                                          H / 8);
  else
    permute_quant_rows_kernel<false><<<rows, 256, 0, st>>>(static_cast<const uint4*>(x), H / 8, w.sorted, w.num_post,
                                                           n, topk, reinterpret_cast<uint2*>(f8.a_q), H / 8,
                                                           f8.a_scale, H / 8);
  FR_CUDA_OK(cudaGetLastError());
  QuantArgs q1{f8.a_scale, w1_scale};
  QuantArgs q2{f8.act_scale, w2_scale};
  auto quant_act = [&]() -> int {
    if (bf)
      quant_rows_kernel<true><<<rows, 256, 0, st>>>(reinterpret_cast<const uint4*>(w.act), I / 8, w.num_post,
                                                    reinterpret_cast<uint2*>(f8.act_q), I / 8, f8.act_scale, I / 8);
    else
      quant_rows_kernel<false><<<rows, 256, 0, st>>>(reinterpret_cast<const uint4*>(w.act), I / 8, w.num_post,
                                                     reinterpret_cast<uint2*>(f8.act_q), I / 8, f8.act_scale, I / 8);
    return static_cast<int>(cudaGetLastError());
  };
  int deferred = 0;
  int64_t partial_cols = 0;
  if (tokenn) {
    rc = gemm_tokenn_dispatch(0, f8.a_q, H, w1_q, dtype, w.rows, H, I, E, 2 * I, w.counts, w.num_post, w.sorted, nullptr,
                              n, w.act, I, w.sp.s1, w.split, w.sp.bytes, st, nullptr, &q1);
    if (rc) return rc;
    if ((rc = quant_act())) return rc;
    rc = gemm_tokenn_dispatch(1, f8.act_q, I, w2_q, dtype, w.rows, I, H, E, H, w.counts, w.num_post, w.sorted, tw, n,
                              w.y_sorted, H, w.sp.s2, w.split, w.sp.bytes, st, &deferred, &q2);
    if (rc) return rc;
    partial_cols = static_cast<int64_t>((H + 127) / 128) * 128;
  } else {
    rc = gemm_grouped_dispatch(0, f8.a_q, H, w1_q, dtype, w.rows, H, I, E, 2 * I, w.expert_ids, w.num_post, w.sorted,
                               nullptr, n, w.act, I, w.sp.s1, w.split, w.sp.bytes, st, nullptr, &q1);
    if (rc) return rc;
    if ((rc = quant_act())) return rc;
    rc = gemm_grouped_dispatch(1, f8.act_q, I, w2_q, dtype, w.rows, I, H, E, H, w.expert_ids, w.num_post, w.sorted, tw,
                               n, w.y_sorted, H, w.sp.s2, w.split, w.sp.bytes, st, &deferred, &q2);
    if (rc) return rc;
    partial_cols = static_cast<int64_t>((H + kTileN - 1) / kTileN) * kTileN;
  }
  if (deferred > 1)
    return combine_partial_dispatch(w.split, deferred, n, H, partial_cols, tw, w.inv_pos, M, topk, dtype, nullptr, 0, out,
                                    H, st);
  if (bf)
    combine_kernel<true><<<static_cast<unsigned>(M), 256, 0, st>>>(reinterpret_cast<const uint4*>(w.y_sorted), H / 8,
                                                                   w.inv_pos, topk, H / 8, w.rows, nullptr, 0,
                                                                   static_cast<uint4*>(out), H / 8);
  else
    combine_kernel<false><<<static_cast<unsigned>(M), 256, 0, st>>>(reinterpret_cast<const uint4*>(w.y_sorted), H / 8,
                                                                    w.inv_pos, topk, H / 8, w.rows, nullptr, 0,
                                                                    static_cast<uint4*>(out), H / 8);
  return static_cast<int>(cudaGetLastError());
}

int fr_moe_layer_routed(const void* x, const int32_t* topk_ids, const float* topk_weights, const void* w1,
                        const void* w2, int dtype, int64_t M, int H, int I, int E, int topk, void* out,
                        void* workspace, size_t workspace_bytes, void* stream) {
  if (!x || !topk_ids || !w1 || !w2 || !out || M < 0 || H <= 0 || I <= 0 || E <= 0 || topk <= 0) return FR_ERR_ARG;
  if (dtype != FR_F16 && dtype != FR_BF16) return FR_ERR_UNSUPPORTED;
  if ((H % 8) || (I % 8)) return FR_ERR_ALIGN;
  if (M == 0) return FR_OK;
  if (!workspace || workspace_bytes < fr_moe_workspace_bytes(M, H, I, E, topk)) return FR_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 1023) return FR_ERR_ALIGN;
  Carver c(workspace);
  void* aws;
  size_t aws_bytes;
  carve_align_ws(c, E, &aws, &aws_bytes);
  carve_route(c, M, H, E, topk);
  c.take<float>(M * topk);
  c.take<int32_t>(M * topk);
  ExpertWs ews = carve_experts(c, M * topk, H, I, E);
  ews.align_ws = aws;
  ews.align_ws_bytes = aws_bytes;
  return experts_impl(x, H, topk_ids, topk_weights, w1, w2, dtype, M, topk, H, I, E, out, H, ews,
                      static_cast<cudaStream_t>(stream));
}

size_t fr_moe_experts_workspace_bytes(int64_t R, int H, int I, int E_local) {
  if (R <= 0 || H <= 0 || I <= 0 || E_local <= 0) return 0;
  Carver c(nullptr);
  void* aws;
  size_t aws_bytes;
  carve_align_ws(c, E_local, &aws, &aws_bytes);
  carve_experts(c, R, H, I, E_local);
  return c.total();
}

int fr_moe_experts(const void* rows, const int32_t* row_expert, const float* row_weight, const void* w1,
                   const void* w2, int dtype, int64_t R, int H, int I, int E_local, void* y, void* workspace,
                   size_t workspace_bytes, void* stream) {
  if (!rows || !row_expert || !w1 || !w2 || !y || R < 0 || H <= 0 || I <= 0 || E_local <= 0) return FR_ERR_ARG;
  if (dtype != FR_F16 && dtype != FR_BF16) return FR_ERR_UNSUPPORTED;
  if ((H % 8) || (I % 8)) return FR_ERR_ALIGN;
  if (R == 0) return FR_OK;
  if (!workspace || workspace_bytes < fr_moe_experts_workspace_bytes(R, H, I, E_local)) return FR_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 1023) return FR_ERR_ALIGN;
  Carver c(workspace);
  void* aws;
  size_t aws_bytes;
  carve_align_ws(c, E_local, &aws, &aws_bytes);
  ExpertWs ews = carve_experts(c, R, H, I, E_local);
  ews.align_ws = aws;
  ews.align_ws_bytes = aws_bytes;
  return experts_impl(rows, H, row_expert, row_weight, w1, w2, dtype, R, 1, H, I, E_local, y, H, ews,
                      static_cast<cudaStream_t>(stream));
}

}  // extern "C"
