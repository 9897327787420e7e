// Tensor-core kernels (tcgen05 + TMEM accumulators, TMA-fed, warp-specialised):
//   * grouped expert GEMM over expert-sorted row blocks, persistent tile loop, with three
//     epilogues: SiLU(gate)*up, routed-weight scaling, split-K fp32 partials;
//   * fused router: gate GEMM whose epilogue does the stable top-k and softmax in registers.
//
// What they stand in for in the reference: fused_moe_kernel
// (fast_route/fast_route/ops/fused_moe.py:10-130), ops.silu_and_mul
// (fast_route/fast_route/layers/stable_route.py:90) and route_kernel
// (fast_route/fast_route/ops/stable_route.py:32-121).
//
// Thread roles in both kernels (192 threads): warp 0 = TMA producer (one lane),
// warp 1 = TMEM owner + MMA issuer (one lane), warps 2..5 = epilogue (warp w reads the
// TMEM lane quarter w % 4).  Every CTA loads its own operands.
#include "fr_common.cuh"

namespace fr {

constexpr int BM = 128;                 // rows per tile = alignment block of the align stage
constexpr int BK = 64;                  // K elements per pipeline stage (128 bytes per row)
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int UMMA_K = 16;

enum { MODE_SILU = 0, MODE_WEIGHTED = 1, MODE_PARTIAL = 2 };

struct GemmParams {
  const int32_t* expert_ids;
  const int32_t* num_post;
  const int32_t* sorted_ids;
  const float* topk_w;
  int64_t n_valid;        // number of real assignments (sorted id >= n_valid marks padding)
  void* out;              // MODE_SILU / MODE_WEIGHTED output, two-byte elements
  int64_t ldo;
  float* partial;         // MODE_PARTIAL: [split][n_valid][partial_cols]
  int64_t partial_cols;
  int64_t max_rows;
  int K;
  int n_out;              // valid output columns (I for GEMM1, H for GEMM2)
  int b_rows_per_expert;  // rows of B per expert (2I or H)
  int b_half_offset;      // row offset of the second half box (I) when two_box
  int two_box;            // B tile = [gate half | up half]
  int num_nb;
  int split_k;
  int kb_per_split;
  int group_m;
  const float* row_scale;  // fp8 inputs only: activation scale per sorted row
  const float* col_scale;  // fp8 inputs only: weight scale per weight row (E * b_rows_per_expert)
};

struct PipeState {
  uint32_t stage = 0, phase = 0;
  template <int STAGES>
  __device__ __forceinline__ void advance() {
    if (++stage == STAGES) {
      stage = 0;
      phase ^= 1;
    }
  }
  __device__ __forceinline__ void advance_rt(uint32_t stages) {
    if (++stage == stages) {
      stage = 0;
      phase ^= 1;
    }
  }
};

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                              unsigned int where) {
  for (uint32_t it = 0; it < kWaitBudget; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  report(ST_WAIT_TIMEOUT, where);
  return false;
}

__device__ __forceinline__ float silu_f(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + BAR_BYTES + 1024;  // + alignment slack
};

// FP8: A and B are E4M3 bytes (128 elements per 128-byte smem row, MMA K = 32) and the epilogue applies
// row_scale[row] * col_scale[weight row]; the output / partial format is unchanged.
template <int BN, int STAGES, int MODE, bool BF16, bool FP8 = false>
__global__ void __launch_bounds__(192, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmParams p) {
  using SM = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(sB + STAGES * SM::B_STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulator buffers
  static_assert(TMEM_COLS == 512 || TMEM_COLS == 256 || TMEM_COLS == 128 || TMEM_COLS == 64, "TMEM cols");

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  int num_mb = __ldg(p.num_post) / BM;
  const int mb_cap = static_cast<int>(p.max_rows / BM);
  if (num_mb > mb_cap) num_mb = mb_cap;
  const int per_split = num_mb * p.num_nb;
  const int tiles = per_split * p.split_k;
  constexpr int BKE = FP8 ? 2 * BK : BK;  // elements per 128-byte row of a stage
  const int KB = (p.K + BKE - 1) / BKE;

  auto decode = [&](int tile, int& mb, int& nb, int& kb0, int& kb1) {
    const int ks = tile / per_split;
    const int t = tile - ks * per_split;
    const int gsz = p.group_m * p.num_nb;
    const int gid = t / gsz;
    const int first = gid * p.group_m;
    const int rows = min(num_mb - first, p.group_m);
    const int r = t - gid * gsz;
    mb = first + r % rows;
    nb = r / rows;
    kb0 = ks * p.kb_per_split;
    kb1 = min(KB, kb0 + p.kb_per_split);
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      PipeState ps;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        int mb, nb, kb0, kb1;
        decode(tile, mb, nb, kb0, kb1);
        const int e = __ldg(p.expert_ids + mb);
        const int brow = e * p.b_rows_per_expert + (p.two_box ? nb * (BN / 2) : nb * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_or_abort(&empty[ps.stage], ps.phase ^ 1, abort_flag, 0x100)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[ps.stage], A_STAGE_BYTES + SM::B_STAGE_BYTES);
          tma_load_2d(sA + ps.stage * A_STAGE_BYTES, &tmA, &full[ps.stage], kb * BKE, mb * BM);
          uint8_t* bdst = sB + ps.stage * SM::B_STAGE_BYTES;
          if (p.two_box) {
            tma_load_2d(bdst, &tmB, &full[ps.stage], kb * BKE, brow);
            tma_load_2d(bdst + (BN / 2) * BK * 2, &tmB, &full[ps.stage], kb * BKE, brow + p.b_half_offset);
          } else {
            tma_load_2d(bdst, &tmB, &full[ps.stage], kb * BKE, brow);
          }
          ps.advance<STAGES>();
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = FP8 ? umma_idesc_e4m3(BM, BN) : umma_idesc_f16(BF16, BM, BN);
      PipeState ps;
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++it) {
        int mb, nb, kb0, kb1;
        decode(tile, mb, nb, kb0, kb1);
        const uint32_t buf = it & 1u, aphase = (it >> 1) & 1u;
        if (!wait_or_abort(&tempty[buf], aphase ^ 1, abort_flag, 0x200)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_or_abort(&full[ps.stage], ps.phase, abort_flag, 0x201)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t adesc = umma_desc_sw128(smem_u32(sA + ps.stage * A_STAGE_BYTES));
          const uint64_t bdesc = umma_desc_sw128(smem_u32(sB + ps.stage * SM::B_STAGE_BYTES));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {  // 4 MMAs per stage, 32 bytes of K each
            if constexpr (FP8) tc_mma_f8(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            else tc_mma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty[ps.stage]);  // frees the smem stage once these MMAs have read it
          ps.advance<STAGES>();
        }
        if (ok) tc_commit(&tfull[buf]);
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
      int mb, nb, kb0, kb1;
      decode(tile, mb, nb, kb0, kb1);
      const uint32_t buf = it & 1u, aphase = (it >> 1) & 1u;
      if (!wait_or_abort(&tfull[buf], aphase, abort_flag, 0x300)) break;
      tc_fence_after();
      const int64_t row = static_cast<int64_t>(mb) * BM + q * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      float rs = 1.0f;
      const float* cs = nullptr;  // weight scales of this tile's expert
      if constexpr (FP8) {
        rs = __ldg(p.row_scale + row);
        cs = p.col_scale + static_cast<int64_t>(__ldg(p.expert_ids + mb)) * p.b_rows_per_expert;
      }

      if constexpr (MODE == MODE_SILU) {
        constexpr int HALF = BN / 2;
        uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + row * p.ldo + static_cast<int64_t>(nb) * HALF;
#pragma unroll 1
        for (int c0 = 0; c0 < HALF; c0 += 32) {
          uint32_t g[32], u[32];
          tmem_ld32(taddr + c0, g);
          tmem_ld32(taddr + HALF + c0, u);
          tc_wait_ld();
          uint32_t pk[16];
          const int col = nb * HALF + c0;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float g0 = __uint_as_float(g[2 * i]), g1 = __uint_as_float(g[2 * i + 1]);
            float u0 = __uint_as_float(u[2 * i]), u1 = __uint_as_float(u[2 * i + 1]);
            if constexpr (FP8) {
              const int c = min(col + 2 * i, p.n_out - 2);
              g0 *= rs * __ldg(cs + c);
              g1 *= rs * __ldg(cs + c + 1);
              u0 *= rs * __ldg(cs + p.b_half_offset + c);
              u1 *= rs * __ldg(cs + p.b_half_offset + c + 1);
            }
            pk[i] = pack2<BF16>(silu_f(g0) * u0, silu_f(g1) * u1);
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col + v * 8 + 8 <= p.n_out)
              *reinterpret_cast<uint4*>(orow + c0 + v * 8) =
                  make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
          }
        }
      } else if constexpr (MODE == MODE_WEIGHTED) {
        const int32_t sid = __ldg(p.sorted_ids + row);
        float w = 0.0f;
        if (sid >= 0 && sid < p.n_valid) w = p.topk_w ? __ldg(p.topk_w + sid) : 1.0f;
        uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + row * p.ldo + static_cast<int64_t>(nb) * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t a[32];
          tmem_ld32(taddr + c0, a);
          tc_wait_ld();
          uint32_t pk[16];
          const int col = nb * BN + c0;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float a0 = w * __uint_as_float(a[2 * i]), a1 = w * __uint_as_float(a[2 * i + 1]);
            if constexpr (FP8) {
              const int c = min(col + 2 * i, p.n_out - 2);
              a0 *= rs * __ldg(cs + c);
              a1 *= rs * __ldg(cs + c + 1);
            }
            pk[i] = pack2<BF16>(a0, a1);
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col + v * 8 + 8 <= p.n_out)
              *reinterpret_cast<uint4*>(orow + c0 + v * 8) =
                  make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
          }
        }
      } else {
        const int ks = tile / per_split;
        const int32_t sid = __ldg(p.sorted_ids + row);
        const bool valid = sid >= 0 && sid < p.n_valid;
        float* prow = p.partial + (static_cast<int64_t>(ks) * p.n_valid + (valid ? sid : 0)) * p.partial_cols +
                      static_cast<int64_t>(nb) * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t a[32];
          tmem_ld32(taddr + c0, a);
          tc_wait_ld();
          if (valid) {
            if constexpr (FP8) {  // partial sums leave the kernel already dequantised
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                int c = c0 + i;  // column inside the tile -> weight row of the expert
                int wr = p.two_box ? (c < BN / 2 ? nb * (BN / 2) + c : p.b_half_offset + nb * (BN / 2) + c - BN / 2)
                                   : nb * BN + c;
                wr = min(wr, p.b_rows_per_expert - 1);
                a[i] = __float_as_uint(__uint_as_float(a[i]) * rs * __ldg(cs + wr));
              }
            }
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              if (static_cast<int64_t>(nb) * BN + c0 + v * 4 + 4 <= p.partial_cols)
                *reinterpret_cast<uint4*>(prow + c0 + v * 4) =
                    make_uint4(a[4 * v], a[4 * v + 1], a[4 * v + 2], a[4 * v + 3]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ----------------------------------------------------------------------------------
// split-K reductions (small M): sum the fp32 partials in split order, apply the epilogue.
// ----------------------------------------------------------------------------------
// grid = (column chunks of 1024, sorted rows); padding rows are left untouched (nothing reads them)
template <bool BF16>
__global__ void __launch_bounds__(256)
splitk_reduce_silu_kernel(const float* __restrict__ partial, int64_t partial_cols, int split_k, int64_t n_valid,
                          const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ num_post, int I,
                          int half_tile, uint16_t* __restrict__ act, int64_t ld_act) {
  const int64_t row = blockIdx.y;
  if (row >= __ldg(num_post)) return;
  const int32_t sid = __ldg(sorted_ids + row);
  if (sid < 0 || sid >= n_valid) return;
  const int j = (blockIdx.x * 256 + threadIdx.x) * 4;  // half_tile is a multiple of 4: no straddling
  if (j >= I) return;
  const int nb = j / half_tile, c = j % half_tile;
  const int64_t gcol = static_cast<int64_t>(nb) * 2 * half_tile + c;
  float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
  for (int s = 0; s < split_k; ++s) {
    const float* pr = partial + (static_cast<int64_t>(s) * n_valid + sid) * partial_cols + gcol;
    const float4 gs = *reinterpret_cast<const float4*>(pr);
    const float4 us = *reinterpret_cast<const float4*>(pr + half_tile);
    g.x += gs.x; g.y += gs.y; g.z += gs.z; g.w += gs.w;
    u.x += us.x; u.y += us.y; u.z += us.z; u.w += us.w;
  }
  *reinterpret_cast<uint2*>(act + row * ld_act + j) =
      make_uint2(pack2<BF16>(silu_f(g.x) * u.x, silu_f(g.y) * u.y), pack2<BF16>(silu_f(g.z) * u.z, silu_f(g.w) * u.w));
}

template <bool BF16>
__global__ void __launch_bounds__(256)
splitk_reduce_weighted_kernel(const float* __restrict__ partial, int64_t partial_cols, int split_k, int64_t n_valid,
                              const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ num_post,
                              const float* __restrict__ topk_w, int H, uint16_t* __restrict__ y, int64_t ld_y) {
  const int64_t row = blockIdx.y;
  if (row >= __ldg(num_post)) return;
  const int32_t sid = __ldg(sorted_ids + row);
  if (sid < 0 || sid >= n_valid) return;
  const int j = (blockIdx.x * 256 + threadIdx.x) * 4;
  if (j >= H) return;
  const float w = topk_w ? __ldg(topk_w + sid) : 1.0f;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < split_k; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(
        partial + (static_cast<int64_t>(s) * n_valid + sid) * partial_cols + j);
    a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
  }
  *reinterpret_cast<uint2*>(y + row * ld_y + j) =
      make_uint2(pack2<BF16>(w * a.x, w * a.y), pack2<BF16>(w * a.z, w * a.w));
}

// Split-K GEMM2 with the reduction folded into the combine:
// out[t,h] = sum_j w[t*k+j] * sum_s partial[s][t*k+j][h]   (slot order, slice order, fp32)
template <bool BF16>
__global__ void __launch_bounds__(256)
combine_partial_kernel(const float* __restrict__ partial, int64_t partial_cols, int split_k, int64_t n_valid,
                       const float* __restrict__ topk_w, const int32_t* __restrict__ inv_pos, int topk, int H,
                       const uint16_t* __restrict__ residual, int64_t ld_res, uint16_t* __restrict__ out,
                       int64_t ld_out) {
  const int64_t t = blockIdx.y;
  const int j = (blockIdx.x * 256 + threadIdx.x) * 4;
  if (j >= H) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (residual) {  // read before the store below: out may alias residual
    const uint2 r = *reinterpret_cast<const uint2*>(residual + t * ld_res + j);
    const float2 r0 = unpack2<BF16>(r.x), r1 = unpack2<BF16>(r.y);
    acc = make_float4(r0.x, r0.y, r1.x, r1.y);
  }
  for (int q = 0; q < topk; ++q) {
    const int64_t sid = t * topk + q;
    if (inv_pos && __ldg(inv_pos + sid) < 0) continue;   // assignment rejected by the align stage: no partial rows
    const float w = topk_w ? __ldg(topk_w + sid) : 1.0f;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < split_k; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(
          partial + (static_cast<int64_t>(s) * n_valid + sid) * partial_cols + j);
      a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
    }
    acc.x += w * a.x; acc.y += w * a.y; acc.z += w * a.z; acc.w += w * a.w;
  }
  *reinterpret_cast<uint2*>(out + t * ld_out + j) =
      make_uint2(pack2<BF16>(acc.x, acc.y), pack2<BF16>(acc.z, acc.w));
}

// ----------------------------------------------------------------------------------
// host side: tensor maps, launchers
// ----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

int make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                 uint32_t box_rows, uint32_t box_cols, bool swizzle128, int elt_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return FR_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld_elems * elt_bytes) & 15)) return FR_ERR_ALIGN;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld_elems * elt_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, elt_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FR_OK : FR_ERR_DRIVER;
}

const DeviceInfo& device_info() {
  static thread_local DeviceInfo info;
  int dev = 0;
  cudaGetDevice(&dev);
  if (info.device != dev) {
    info.device = dev;
    cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  }
  return info;
}

constexpr int GEMM_BN = 256;
constexpr int GEMM_STAGES = 4;

template <int MODE, bool BF16, bool FP8 = false>
static int launch_grouped(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int grid,
                          cudaStream_t st) {
  auto kern = grouped_gemm_kernel<GEMM_BN, GEMM_STAGES, MODE, BF16, FP8>;
  constexpr int smem = GemmSmem<GEMM_BN, GEMM_STAGES>::TOTAL;
  FR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  kern<<<grid, 192, smem, st>>>(tmA, tmB, p);
  return static_cast<int>(cudaGetLastError());
}

// Picks how many K slices to use when there are too few tiles to fill the machine.
int choose_split_k(int64_t est_tiles, int KB, int sm_count, bool few_rows) {
  // Below two waves any gain in wave efficiency pays.  From two to eight waves only a handful of rows (pure
  // weight streaming, partial tiles of a few KB) make a split worth its reduction, and only if it recovers at
  // least 8 % of the machine: a partial last wave of such tiles costs a whole tile time (1 token on 2 experts:
  // 448 tiles = 3.03 waves).  Measured on one B200, Mixtral-8x7B shape: 1 token 165.5 -> 155.0 us, 2 tokens
  // 274 -> 262 us; from 64 tokens on the same rule loses 2-5 %, hence the row limit.
  if (est_tiles <= 0 || est_tiles >= (few_rows ? 8 : 2) * sm_count) return 1;
  const bool small = est_tiles < 2 * sm_count;
  int best = 1;
  double best_eff = 0.0, base_eff = 0.0;
  for (int s = 1; s <= 16; ++s) {
    if (KB / s < 4) break;
    if (!small && s > 4) break;
    const int64_t t = est_tiles * s;
    const int64_t waves = (t + sm_count - 1) / sm_count;
    const double eff = static_cast<double>(t) / static_cast<double>(waves * sm_count);
    if (s == 1) base_eff = eff;
    if (eff > best_eff + 0.03) {
      best_eff = eff;
      best = s;
    }
  }
  if (!small && best_eff < base_eff + 0.08) return 1;
  return best;
}

int gemm_grouped_dispatch(int which, const void* a, int64_t lda, const void* w, int dtype, int64_t max_rows,
                          int K, int n_out, int E, int b_rows_per_expert, const int32_t* expert_ids,
                          const int32_t* num_post, const int32_t* sorted_ids, const float* topk_w, int64_t n_valid,
                          void* out, int64_t ldo, int split_k, void* workspace, size_t workspace_bytes,
                          cudaStream_t st, int* deferred_split, const QuantArgs* quant, int64_t rows_hint = -1) {
  // quant != nullptr: a and w hold E4M3 bytes (lda and K count elements = bytes), dtype is the output type.
  // which: 0 = GEMM1 (two-box B, SiLU epilogue), 1 = GEMM2 (weighted epilogue).
  // deferred_split (GEMM2 only, may be null): when split-K is used, skip the reduction and
  // report the slice count; the caller then finishes with combine_partial_dispatch.
  if (deferred_split) *deferred_split = 0;
  if (!a || !w || !expert_ids || !num_post || !out || max_rows <= 0 || K <= 0 || n_out <= 0 || E <= 0)
    return FR_ERR_ARG;
  if (dtype != FR_F16 && dtype != FR_BF16) return FR_ERR_UNSUPPORTED;
  if (max_rows % BM) return FR_ERR_ARG;
  const bool fp8 = quant != nullptr;
  if (fp8 && (!quant->row_scale || !quant->col_scale)) return FR_ERR_ARG;
  if ((K % (fp8 ? 16 : 8)) || (n_out % 8) || (ldo % 8) || (lda % (fp8 ? 16 : 8))) return FR_ERR_ALIGN;
  if (reinterpret_cast<uintptr_t>(out) & 15) return FR_ERR_ALIGN;
  if (split_k < 1) split_k = 1;
  const int BKE = fp8 ? 2 * BK : BK;
  const int KB = (K + BKE - 1) / BKE;
  if (split_k > KB) split_k = KB;
  if ((which == 1 || split_k > 1) && !sorted_ids) return FR_ERR_ARG;
  const DeviceInfo& di = device_info();

  GemmParams p = {};
  p.expert_ids = expert_ids;
  p.num_post = num_post;
  p.sorted_ids = sorted_ids;
  p.topk_w = topk_w;
  p.n_valid = n_valid;
  p.out = out;
  p.ldo = ldo;
  p.max_rows = max_rows;
  p.K = K;
  p.n_out = n_out;
  p.b_rows_per_expert = b_rows_per_expert;
  p.row_scale = fp8 ? quant->row_scale : nullptr;
  p.col_scale = fp8 ? quant->col_scale : nullptr;
  p.two_box = (which == 0);
  p.b_half_offset = n_out;  // GEMM1: the linear ("up") branch starts I rows after the SiLU branch
  p.num_nb = p.two_box ? (n_out + GEMM_BN / 2 - 1) / (GEMM_BN / 2) : (n_out + GEMM_BN - 1) / GEMM_BN;
  p.split_k = split_k;
  p.kb_per_split = (KB + split_k - 1) / split_k;
  p.split_k = (KB + p.kb_per_split - 1) / p.kb_per_split;  // drop empty slices
  split_k = p.split_k;
  // Row blocks per tile group (all column tiles of a group are walked before the next group).
  // A group's A rows stay in L2 while its B tiles stream through; with ~32 row blocks per
  // expert a group of 32 lets each expert's weights be fetched from HBM once instead of twice,
  // with few blocks per expert a wider group only spreads the in-flight tiles over more experts.
  // rows_hint: the expected number of real rows when n_valid is only a capacity (expert-parallel callers)
  const int64_t blocks_per_expert = (rows_hint >= 0 ? rows_hint : n_valid) / (static_cast<int64_t>(BM) * E);
  p.group_m = blocks_per_expert >= 24 ? (which == 0 ? 32 : 24) : 16;
  p.partial_cols = static_cast<int64_t>(p.num_nb) * GEMM_BN;
  if (split_k > 1) {
    const size_t need = static_cast<size_t>(split_k) * static_cast<size_t>(n_valid) * p.partial_cols * sizeof(float);
    if (!workspace || workspace_bytes < need) return FR_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 15) return FR_ERR_ALIGN;
    p.partial = static_cast<float*>(workspace);
  }

  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, a, static_cast<uint64_t>(max_rows), static_cast<uint64_t>(K),
                        static_cast<uint64_t>(lda), BM, BKE, true, fp8 ? 1 : 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, w, static_cast<uint64_t>(E) * b_rows_per_expert, static_cast<uint64_t>(K),
                    static_cast<uint64_t>(K), p.two_box ? GEMM_BN / 2 : GEMM_BN, BKE, true, fp8 ? 1 : 2);
  if (rc) return rc;

  const int64_t max_tiles = (max_rows / BM) * p.num_nb * split_k;
  const int grid = static_cast<int>(max_tiles < di.sm_count ? max_tiles : di.sm_count);
  const bool bf = dtype == FR_BF16;
  if (split_k > 1) {
    if (fp8)
      rc = bf ? launch_grouped<MODE_PARTIAL, true, true>(tmA, tmB, p, grid, st)
              : launch_grouped<MODE_PARTIAL, false, true>(tmA, tmB, p, grid, st);
    else
      rc = bf ? launch_grouped<MODE_PARTIAL, true>(tmA, tmB, p, grid, st)
              : launch_grouped<MODE_PARTIAL, false>(tmA, tmB, p, grid, st);
    if (rc) return rc;
    if (which == 1 && deferred_split) {
      *deferred_split = split_k;
      return FR_OK;
    }
    const dim3 rgrid(static_cast<unsigned>((n_out + 1023) / 1024), static_cast<unsigned>(max_rows));
    if (which == 0) {
      if (bf)
        splitk_reduce_silu_kernel<true><<<rgrid, 256, 0, st>>>(p.partial, p.partial_cols, split_k, n_valid,
                                                               sorted_ids, num_post, n_out, GEMM_BN / 2,
                                                               static_cast<uint16_t*>(out), ldo);
      else
        splitk_reduce_silu_kernel<false><<<rgrid, 256, 0, st>>>(p.partial, p.partial_cols, split_k, n_valid,
                                                                sorted_ids, num_post, n_out, GEMM_BN / 2,
                                                                static_cast<uint16_t*>(out), ldo);
    } else {
      if (bf)
        splitk_reduce_weighted_kernel<true><<<rgrid, 256, 0, st>>>(p.partial, p.partial_cols, split_k, n_valid,
                                                                   sorted_ids, num_post, topk_w, n_out,
                                                                   static_cast<uint16_t*>(out), ldo);
      else
        splitk_reduce_weighted_kernel<false><<<rgrid, 256, 0, st>>>(p.partial, p.partial_cols, split_k, n_valid,
                                                                    sorted_ids, num_post, topk_w, n_out,
                                                                    static_cast<uint16_t*>(out), ldo);
    }
    return static_cast<int>(cudaGetLastError());
  }
  if (fp8) {
    if (which == 0)
      return bf ? launch_grouped<MODE_SILU, true, true>(tmA, tmB, p, grid, st)
                : launch_grouped<MODE_SILU, false, true>(tmA, tmB, p, grid, st);
    return bf ? launch_grouped<MODE_WEIGHTED, true, true>(tmA, tmB, p, grid, st)
              : launch_grouped<MODE_WEIGHTED, false, true>(tmA, tmB, p, grid, st);
  }
  if (which == 0)
    return bf ? launch_grouped<MODE_SILU, true>(tmA, tmB, p, grid, st)
              : launch_grouped<MODE_SILU, false>(tmA, tmB, p, grid, st);
  return bf ? launch_grouped<MODE_WEIGHTED, true>(tmA, tmB, p, grid, st)
            : launch_grouped<MODE_WEIGHTED, false>(tmA, tmB, p, grid, st);
}

int combine_partial_dispatch(const void* workspace, int split_k, int64_t n_valid, int n_out, int64_t partial_cols,
                             const float* topk_w, const int32_t* inv_pos, int64_t M, int topk, int dtype,
                             const void* residual, int64_t ld_res, void* out, int64_t ld_out, cudaStream_t st) {
  const dim3 grid(static_cast<unsigned>((n_out + 1023) / 1024), static_cast<unsigned>(M));
  if (dtype == FR_BF16)
    combine_partial_kernel<true><<<grid, 256, 0, st>>>(static_cast<const float*>(workspace), partial_cols, split_k,
                                                       n_valid, topk_w, inv_pos, topk, n_out,
                                                       static_cast<const uint16_t*>(residual), ld_res,
                                                       static_cast<uint16_t*>(out), ld_out);
  else
    combine_partial_kernel<false><<<grid, 256, 0, st>>>(static_cast<const float*>(workspace), partial_cols, split_k,
                                                        n_valid, topk_w, inv_pos, topk, n_out,
                                                        static_cast<const uint16_t*>(residual), ld_res,
                                                        static_cast<uint16_t*>(out), ld_out);
  return static_cast<int>(cudaGetLastError());
}

// ==================================================================================
// Fused router: one 128-row tile per CTA, N = padded expert count, whole K loop, then
// each epilogue thread owns one row of logits in TMEM and selects its top-k in registers.
// A thread can issue a tcgen05.mma only every hundred cycles or so, whatever its N, and
// with so few columns that — not the tensor pipe — is what the K loop costs.  So up to
// 128 experts the K stages are dealt round-robin to four (two) issuing threads on
// different warps, each with its own accumulator; the epilogue adds the accumulators in
// a fixed order.
// ==================================================================================
constexpr int RKMAX = 8;

struct RouterParams {
  int64_t M;
  int K;
  int E;
  int topk;
  int renormalize;
  int do_topk;
  float* weights;   // [M, topk]
  int32_t* ids;     // [M, topk]
  float* logits;    // [M, E] or null
};

template <int NPAD>
struct RouterSmem {
  // Several issuers pay while the K loop is the larger part and the stages stay deep enough: four up to 64 experts
  // (2048 tokens, 8 experts: 20.5 against 26.6 us), two at 128 (34.8 against 36.9 us; four, with one 32 KB stage each,
  // 41 us), one at 256 (two: 53-55 against 51 us: the epilogue has every extra accumulator to read).
  static constexpr int ISSUERS = NPAD > 128 ? 1 : (NPAD > 64 ? 2 : 4);
  static constexpr int THREADS = 32 * (1 + ISSUERS + 4);  // producer, issuers, four epilogue warps
  // A multiple of the issuer count, so that a stage is always consumed by the same issuer: a waiter then never
  // lags its barrier by more than one phase (a parity wait cannot tell phase n from phase n + 2).
  static constexpr int STAGES = NPAD > 128 ? 4 : (NPAD > 64 ? 6 : 8);   // 4 x 48 KB, 6 x 32 KB or 8 x <= 24 KB
  static_assert(STAGES % ISSUERS == 0, "a stage belongs to one issuer");
  static constexpr int B_STAGE_BYTES = NPAD * BK * 2;
  static constexpr int TOTAL = STAGES * (A_STAGE_BYTES + (B_STAGE_BYTES < 1024 ? 1024 : B_STAGE_BYTES)) + 256 + 1024;
};

template <int NPAD, bool BF16>
__global__ void __launch_bounds__(RouterSmem<NPAD>::THREADS, 1)
router_gemm_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmG,
                   const RouterParams p) {
  using SM = RouterSmem<NPAD>;
  constexpr int ROUTER_STAGES = SM::STAGES;
  constexpr int NI = SM::ISSUERS;
  constexpr int B_STRIDE = SM::B_STAGE_BYTES < 1024 ? 1024 : SM::B_STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + ROUTER_STAGES * A_STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(sB + ROUTER_STAGES * B_STRIDE);
  uint64_t* empty = full + ROUTER_STAGES;
  uint64_t* tfull = empty + ROUTER_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = NI * NPAD < 32 ? 32 : NI * NPAD;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ROUTER_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tfull, NI);            // one arrival per issuer, after its last MMA
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmG);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int KB = (p.K + BK - 1) / BK;
  const int m0 = blockIdx.x * BM;

  if (warp == 0) {
    if (lane == 0) {
      PipeState ps;
      for (int kb = 0; kb < KB; ++kb) {
        if (!wait_or_abort(&empty[ps.stage], ps.phase ^ 1, abort_flag, 0x400)) break;
        mbar_expect_tx(&full[ps.stage], A_STAGE_BYTES + SM::B_STAGE_BYTES);
        tma_load_2d(sA + ps.stage * A_STAGE_BYTES, &tmX, &full[ps.stage], kb * BK, m0);
        tma_load_2d(sB + ps.stage * B_STRIDE, &tmG, &full[ps.stage], kb * BK, 0);
        ps.advance<ROUTER_STAGES>();
      }
    }
  } else if (warp <= NI) {
    if (lane == 0) {
      // issuer i takes the K stages kb = i, i + NI, ... (always the same shared-memory stages) into accumulator i
      const int issuer = warp - 1;
      constexpr uint32_t idesc = umma_idesc_f16(BF16, BM, NPAD);
      const uint32_t d_tmem = tmem_base + issuer * NPAD;
      bool ok = true;
      for (int kb = issuer; kb < KB; kb += NI) {
        const int stage = kb % ROUTER_STAGES;
        if (!wait_or_abort(&full[stage], static_cast<uint32_t>(kb / ROUTER_STAGES) & 1u, abort_flag, 0x401)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t adesc = umma_desc_sw128(smem_u32(sA + stage * A_STAGE_BYTES));
        const uint64_t bdesc = umma_desc_sw128(smem_u32(sB + stage * B_STRIDE));
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          tc_mma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb >= NI || k > 0) ? 1u : 0u);
        tc_commit(&empty[stage]);
      }
      // all of this issuer's MMAs (none, if it had no stage) are complete when this arrives
      if (ok && issuer < KB) tc_commit(tfull);
      else mbar_arrive(tfull);
    }
  } else {
    const int q = warp & 3;
    if (wait_or_abort(tfull, 0, abort_flag, 0x402)) {
      tc_fence_after();
      const int64_t row = static_cast<int64_t>(m0) + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      // The sorted top list holds order-preserving integer images of the logits (fp32 bits with the sign folded,
      // -0 taken as +0), so "stays ahead of the newcomer" is one unsigned compare; 0 is below every image, -inf
      // included, and marks an empty slot.
      uint32_t tv[RKMAX];
      int tc[RKMAX];
#pragma unroll
      for (int j = 0; j < RKMAX; ++j) {
        tv[j] = 0u;
        tc[j] = 0x7fffffff;
      }
      float run_max = -INFINITY, run_sum = 0.0f;
      const int used = KB < NI ? KB : NI;       // accumulators that were written
#pragma unroll 1
      for (int c0 = 0; c0 < NPAD; c0 += 16) {
        uint32_t a[16];
        tmem_ld16(taddr + c0, a);
        tc_wait_ld();
        for (int acc = 1; acc < used; ++acc) {   // the issuers' partial sums, in issuer order
          uint32_t b[16];
          tmem_ld16(taddr + acc * NPAD + c0, b);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) a[i] = __float_as_uint(__fadd_rn(__uint_as_float(a[i]), __uint_as_float(b[i])));
        }
        if (c0 < p.E) {
          if (p.logits && row_ok) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (c0 + i < p.E) p.logits[row * p.E + c0 + i] = __uint_as_float(a[i]);
          }
          if (p.do_topk) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int c = c0 + i;
              float x = __uint_as_float(a[i]);
              if (x != x) x = -INFINITY;
              if (c < p.E) {
                if (!p.renormalize) {
                  const float nm = fmaxf(run_max, x);
                  run_sum = run_sum * __expf(run_max - nm) + __expf(x - nm);
                  run_max = nm;
                }
                // Insert into the sorted top list.  An entry stays ahead of the newcomer if it is larger, or equal:
                // columns arrive in ascending order, so an equal entry has the lower expert id.  keep[j] is monotone
                // in j; slot j keeps its entry, takes the newcomer (first slot that does not keep), or takes slot
                // j-1's entry.  All eight decisions are independent: no carry chain through the list.
                const uint32_t xb = __float_as_uint(x + 0.0f);                    // -0 -> +0
                const uint32_t xk = xb ^ ((xb & 0x80000000u) ? 0xFFFFFFFFu : 0x80000000u);
                bool keep[RKMAX];
#pragma unroll
                for (int j = 0; j < RKMAX; ++j) keep[j] = tv[j] >= xk;
#pragma unroll
                for (int j = RKMAX - 1; j >= 1; --j) {
                  tv[j] = keep[j] ? tv[j] : (keep[j - 1] ? xk : tv[j - 1]);
                  tc[j] = keep[j] ? tc[j] : (keep[j - 1] ? c : tc[j - 1]);
                }
                tv[0] = keep[0] ? tv[0] : xk;
                tc[0] = keep[0] ? tc[0] : c;
              }
            }
          }
        }
      }
      if (p.do_topk && row_ok) {
        float e[RKMAX];
        float s = 0.0f;
        auto value_of = [](uint32_t key) {        // back from the integer image
          return __uint_as_float(key ^ ((key & 0x80000000u) ? 0x80000000u : 0xFFFFFFFFu));
        };
        const float top = value_of(tv[0]);
#pragma unroll
        for (int j = 0; j < RKMAX; ++j) {
          e[j] = 0.0f;
          if (j < p.topk) {
            e[j] = exp_recipe(__fsub_rn(value_of(tv[j]), top));
            s = (j == 0) ? e[0] : __fadd_rn(s, e[j]);
          }
        }
        if (!p.renormalize) s = run_sum * __expf(run_max - top);
#pragma unroll
        for (int j = 0; j < RKMAX; ++j) {
          if (j < p.topk) {
            p.weights[row * p.topk + j] = __fdiv_rn(e[j], s);
            p.ids[row * p.topk + j] = tc[j];
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int NPAD>
static int launch_router(const CUtensorMap& tmX, const CUtensorMap& tmG, const RouterParams& p, bool bf,
                         cudaStream_t st) {
  constexpr int smem = RouterSmem<NPAD>::TOTAL;
  const unsigned grid = static_cast<unsigned>((p.M + BM - 1) / BM);
  if (bf) {
    auto kern = router_gemm_kernel<NPAD, true>;
    FR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<grid, RouterSmem<NPAD>::THREADS, smem, st>>>(tmX, tmG, p);
  } else {
    auto kern = router_gemm_kernel<NPAD, false>;
    FR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<grid, RouterSmem<NPAD>::THREADS, smem, st>>>(tmX, tmG, p);
  }
  return static_cast<int>(cudaGetLastError());
}

// gate_km: [E, H] with unit stride along H (K-major).
int router_gemm_dispatch(const void* x, int dtype, int64_t M, int H, int64_t ldx, const void* gate_km,
                         int64_t ld_gate, int E, int topk, int renormalize, int do_topk, float* weights,
                         int32_t* ids, float* logits_out, cudaStream_t st) {
  if (!x || !gate_km || M <= 0 || H <= 0 || E <= 0 || E > 256) return FR_ERR_ARG;
  if (dtype != FR_F16 && dtype != FR_BF16) return FR_ERR_UNSUPPORTED;
  if (do_topk && (topk > RKMAX || topk > E || !weights || !ids)) return FR_ERR_ARG;
  if (!do_topk && !logits_out) return FR_ERR_ARG;
  if ((H % 8) || (ldx % 8) || (ld_gate % 8)) return FR_ERR_ALIGN;
  int npad = 16;
  while (npad < E) npad <<= 1;
  CUtensorMap tmX, tmG;
  int rc = make_tmap_2d(&tmX, x, static_cast<uint64_t>(M), static_cast<uint64_t>(H), static_cast<uint64_t>(ldx),
                        BM, BK, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmG, gate_km, static_cast<uint64_t>(E), static_cast<uint64_t>(H),
                    static_cast<uint64_t>(ld_gate), static_cast<uint32_t>(npad), BK, true);
  if (rc) return rc;
  RouterParams p{M, H, E, topk, renormalize, do_topk, weights, ids, logits_out};
  const bool bf = dtype == FR_BF16;
  switch (npad) {
    case 16: return launch_router<16>(tmX, tmG, p, bf, st);
    case 32: return launch_router<32>(tmX, tmG, p, bf, st);
    case 64: return launch_router<64>(tmX, tmG, p, bf, st);
    case 128: return launch_router<128>(tmX, tmG, p, bf, st);
    default: return launch_router<256>(tmX, tmG, p, bf, st);
  }
}

}  // namespace fr
