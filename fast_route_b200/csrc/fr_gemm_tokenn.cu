// Grouped expert GEMM with the TOKENS on the MMA N axis ("token-N"): every tile is
//   D[128 weight rows, TN tokens] = W_tile[128, K] . X_tile[TN, K]^T,   TN = 16, 32, ... 256,
// so an expert's token count is padded to 16 instead of 128.  With few hundred tokens per expert the
// 128-row tiles of grouped_gemm_kernel (fr_gemm.cu) multiply up to half padding; here the tensor
// core always sees 128 full weight rows and only the token extent varies.  Same roles and pipeline
// as grouped_gemm_kernel (TMA producer lane, tcgen05.mma issuer lane, 4 epilogue warps, 4 smem
// stages of 16 KB weights + 32 KB tokens, two 256-column TMEM accumulators).  The accumulator comes
// out transposed (TMEM lane = output feature, column = token), so the epilogue goes through a
// 128 x 32 fp32 staging tile in shared memory and writes token-major rows.
//
// Reference counterpart: fused_moe_kernel + silu_and_mul (fast_route/fast_route/ops/fused_moe.py:10-130,
// layers/stable_route.py:85-95); the reference picks smaller Triton tiles for small batches
// (layers/stable_route.py:40-54), this is the tcgen05 equivalent of that choice.
#include "fr_common.cuh"

namespace fr {

constexpr int TN_MAX = 256;      // most tokens per tile (MMA N); the launch picks tn_box <= TN_MAX
constexpr int TW = 128;          // weight rows per tile (MMA M)
constexpr int TMAX_STAGES = 10;
constexpr int TW_STAGE_BYTES = TW * BK * 2;       // 16 KB, two boxes of 64 rows
constexpr int TPIPE_BYTES = 192 * 1024;           // shared memory given to the TMA pipeline
constexpr int TSTAGE_STRIDE = 33;                 // floats per staging row (32 tokens + 1: conflict-free)
constexpr int TMAX_EXPERTS = 256;

struct TokenNParams {
  const int32_t* counts;      // [E] tokens per expert
  const int32_t* sorted_ids;  // expert-sorted assignment ids, experts padded to 16
  const float* topk_w;
  int64_t n_valid;
  void* out;
  int64_t ldo;
  float* partial;             // MODE_PARTIAL: [split][n_valid][partial_cols]
  int64_t partial_cols;
  int E;
  int K;
  int n_out;                  // I (GEMM1) or H (GEMM2)
  int w_rows_per_expert;      // 2I or H
  int second_box_offset;      // row offset of the second 64-row box: I (gate/up pairing) or 64
  int features_per_tile;      // 64 (GEMM1: 64 gate + 64 up rows give 64 outputs) or 128
  int num_wt;                 // weight tiles per expert
  int split_k;
  int kb_per_split;
  const float* row_scale;     // fp8 inputs only: activation scale per sorted row
  const float* col_scale;     // fp8 inputs only: weight scale per weight row (E * w_rows_per_expert)
  int tn_box;                 // tokens per tile = TMA box height of the token operand: 16 ... 256
  int stages;                 // pipeline depth: TPIPE_BYTES / (16 KB + tn_box * 128 B), at most TMAX_STAGES
  int max_rows;               // rows of the token operand / output buffers
};

struct TileInfo {
  int e, wt, tt, ks;
  int row0;      // first sorted row of the token tile
  int tokens;    // real tokens in the tile
  int tn;        // MMA N: tokens rounded up to 16
};

template <int MODE, bool BF16, bool FP8 = false>
__global__ void __launch_bounds__(192, 1)
tokenn_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   const TokenNParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int STAGES = p.stages;
  const int TX_STAGE_BYTES = p.tn_box * BK * 2;   // a multiple of 2 KB: stage bases stay 1024-byte aligned
  uint8_t* sW = smem;
  uint8_t* sX = smem + STAGES * TW_STAGE_BYTES;
  float* stage_tile = reinterpret_cast<float*>(smem + TPIPE_BYTES);                   // [128][33]
  int* ex_start = reinterpret_cast<int*>(stage_tile + TW * TSTAGE_STRIDE);           // [E] first sorted row
  int* ex_count = ex_start + TMAX_EXPERTS;                                            // [E]
  int* ex_tile0 = ex_count + TMAX_EXPERTS;                                            // [E+1] first tile id
  uint64_t* full = reinterpret_cast<uint64_t*>(ex_tile0 + TMAX_EXPERTS + 2);
  uint64_t* empty = full + TMAX_STAGES;
  uint64_t* tfull = empty + TMAX_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * TN_MAX;

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
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
    // per-expert table: first sorted row (experts padded to 16 rows) and first tile id
    int row = 0, tile = 0;
    for (int e = 0; e < p.E; ++e) {
      int c = __ldg(p.counts + e);
      if (c < 0) c = 0;
      // counts that do not fit the buffers (an align stage that never ran) must not turn into stores past them
      if (c > p.max_rows - row) c = p.max_rows - row > 0 ? p.max_rows - row : 0;
      ex_start[e] = row;
      ex_count[e] = c;
      ex_tile0[e] = tile;
      row += (c + 15) & ~15;
      tile += ((c + p.tn_box - 1) / p.tn_box) * p.num_wt * p.split_k;
    }
    ex_tile0[p.E] = tile;
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int tiles = ex_tile0[p.E];
  constexpr int BKE = FP8 ? 2 * BK : BK;  // elements per 128-byte row of a stage
  const int KB = (p.K + BKE - 1) / BKE;

  // tiles are visited in increasing order by every role: the expert pointer only moves forward
  auto decode = [&](int tile, int& e_ptr, TileInfo& t) {
    while (tile >= ex_tile0[e_ptr + 1]) ++e_ptr;
    const int cnt = ex_count[e_ptr];
    const int tts = (cnt + p.tn_box - 1) / p.tn_box;
    const int rem = tile - ex_tile0[e_ptr];
    const int per_wt = tts * p.split_k;
    t.e = e_ptr;
    t.wt = rem / per_wt;
    const int r2 = rem - t.wt * per_wt;
    t.ks = r2 / tts;
    t.tt = r2 - t.ks * tts;
    t.row0 = ex_start[e_ptr] + t.tt * p.tn_box;
    t.tokens = min(p.tn_box, cnt - t.tt * p.tn_box);
    t.tn = (t.tokens + 15) & ~15;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      PipeState ps;
      int e_ptr = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        TileInfo t;
        decode(tile, e_ptr, t);
        const int wrow = t.e * p.w_rows_per_expert + t.wt * p.features_per_tile;
        const int kb0 = t.ks * p.kb_per_split, kb1 = min(KB, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_or_abort(&empty[ps.stage], ps.phase ^ 1, abort_flag, 0x600)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[ps.stage], static_cast<uint32_t>(TW_STAGE_BYTES + TX_STAGE_BYTES));
          uint8_t* wdst = sW + ps.stage * TW_STAGE_BYTES;
          tma_load_2d(wdst, &tmW, &full[ps.stage], kb * BKE, wrow);
          tma_load_2d(wdst + TW_STAGE_BYTES / 2, &tmW, &full[ps.stage], kb * BKE, wrow + p.second_box_offset);
          tma_load_2d(sX + ps.stage * TX_STAGE_BYTES, &tmX, &full[ps.stage], kb * BKE, t.row0);
          ps.advance_rt(STAGES);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      PipeState ps;
      uint32_t it = 0;
      int e_ptr = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++it) {
        TileInfo t;
        decode(tile, e_ptr, t);
        const uint32_t idesc = FP8 ? umma_idesc_e4m3(TW, t.tn) : umma_idesc_f16(BF16, TW, t.tn);
        const int kb0 = t.ks * p.kb_per_split, kb1 = min(KB, kb0 + p.kb_per_split);
        const uint32_t buf = it & 1u, aphase = (it >> 1) & 1u;
        if (!wait_or_abort(&tempty[buf], aphase ^ 1, abort_flag, 0x601)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * TN_MAX;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_or_abort(&full[ps.stage], ps.phase, abort_flag, 0x602)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t adesc = umma_desc_sw128(smem_u32(sW + ps.stage * TW_STAGE_BYTES));
          const uint64_t bdesc = umma_desc_sw128(smem_u32(sX + ps.stage * TX_STAGE_BYTES));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            if constexpr (FP8) tc_mma_f8(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            else tc_mma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty[ps.stage]);
          ps.advance_rt(STAGES);
        }
        if (ok) tc_commit(&tfull[buf]);
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    // warp q owns TMEM lanes (= output features of the tile) 32q..32q+31
    const int q = warp & 3;
    uint32_t it = 0;
    int e_ptr = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
      TileInfo t;
      decode(tile, e_ptr, t);
      const uint32_t buf = it & 1u, aphase = (it >> 1) & 1u;
      // The four epilogue warps share the staging tile and meet at a named barrier in every chunk, so they must
      // all take the same decision here: a vote over the 128 threads (every warp reaches it, its wait is bounded).
      const uint32_t got = wait_or_abort(&tfull[buf], aphase, abort_flag, 0x603) ? 1u : 0u;
      __syncwarp();
      uint32_t all_got;
      asm volatile(
          "{\n"
          ".reg .pred p, q;\n"
          "setp.ne.u32 p, %1, 0;\n"
          "bar.red.and.pred q, 1, 128, p;\n"
          "selp.u32 %0, 1, 0, q;\n"
          "}\n"
          : "=r"(all_got)
          : "r"(got)
          : "memory");
      if (!all_got) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * TN_MAX;
      const int nchunks = (t.tn + 31) / 32;
      for (int c = 0; c < nchunks; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tc_wait_ld();
        if (c == nchunks - 1) {  // accumulator fully read: hand the TMEM buffer back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty[buf]);
        }
        float* srow = stage_tile + (q * 32 + lane) * TSTAGE_STRIDE;
#pragma unroll
        for (int i = 0; i < 32; ++i) srow[i] = __uint_as_float(r[i]);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // second half: lane = token of the chunk, warp q = a slice of the tile's output features
        const int tok = c * 32 + lane;
        const bool tok_ok = tok < t.tokens;
        const int64_t row = static_cast<int64_t>(t.row0) + tok;
        float rs = 1.0f;
        const float* cs = nullptr;  // weight scales of this tile's expert
        if constexpr (FP8) {
          rs = tok_ok ? __ldg(p.row_scale + row) : 0.0f;
          cs = p.col_scale + static_cast<int64_t>(t.e) * p.w_rows_per_expert;
        }
        if constexpr (MODE == MODE_SILU) {
          // features: lanes 0..63 of the tile are the SiLU rows, 64..127 the linear rows of the same outputs
          const int f0 = q * 16;
          uint32_t pk[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float g0 = stage_tile[(f0 + 2 * i) * TSTAGE_STRIDE + lane];
            float g1 = stage_tile[(f0 + 2 * i + 1) * TSTAGE_STRIDE + lane];
            float u0 = stage_tile[(64 + f0 + 2 * i) * TSTAGE_STRIDE + lane];
            float u1 = stage_tile[(64 + f0 + 2 * i + 1) * TSTAGE_STRIDE + lane];
            if constexpr (FP8) {
              const int c = min(t.wt * 64 + f0 + 2 * i, p.n_out - 2);  // weight row of the SiLU branch
              g0 *= rs * __ldg(cs + c);
              g1 *= rs * __ldg(cs + c + 1);
              u0 *= rs * __ldg(cs + p.second_box_offset + c);
              u1 *= rs * __ldg(cs + p.second_box_offset + c + 1);
            }
            pk[i] = pack2<BF16>(silu_f(g0) * u0, silu_f(g1) * u1);
          }
          const int col = t.wt * 64 + f0;
          if (tok_ok) {
            uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + row * p.ldo + col;
            if (col + 8 <= p.n_out) *reinterpret_cast<uint4*>(o) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            if (col + 16 <= p.n_out) *reinterpret_cast<uint4*>(o + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
          }
        } else if constexpr (MODE == MODE_WEIGHTED) {
          const int f0 = q * 32;
          float w = 0.0f;
          if (tok_ok) {
            const int32_t sid = __ldg(p.sorted_ids + row);
            if (sid >= 0 && sid < p.n_valid) w = p.topk_w ? __ldg(p.topk_w + sid) : 1.0f;
          }
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float a0 = w * stage_tile[(f0 + 2 * i) * TSTAGE_STRIDE + lane];
            float a1 = w * stage_tile[(f0 + 2 * i + 1) * TSTAGE_STRIDE + lane];
            if constexpr (FP8) {
              const int c = min(t.wt * 128 + f0 + 2 * i, p.n_out - 2);
              a0 *= rs * __ldg(cs + c);
              a1 *= rs * __ldg(cs + c + 1);
            }
            pk[i] = pack2<BF16>(a0, a1);
          }
          const int col = t.wt * 128 + f0;
          if (tok_ok) {
            uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + row * p.ldo + col;
#pragma unroll
            for (int v = 0; v < 4; ++v)
              if (col + v * 8 + 8 <= p.n_out)
                *reinterpret_cast<uint4*>(o + v * 8) = make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
          }
        } else {
          const int f0 = q * 32;
          int32_t sid = -1;
          if (tok_ok) sid = __ldg(p.sorted_ids + row);
          if (sid >= 0 && sid < p.n_valid) {
            float* o = p.partial + (static_cast<int64_t>(t.ks) * p.n_valid + sid) * p.partial_cols +
                       static_cast<int64_t>(t.wt) * 128 + f0;
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              float4 val;
              val.x = stage_tile[(f0 + 4 * v) * TSTAGE_STRIDE + lane];
              val.y = stage_tile[(f0 + 4 * v + 1) * TSTAGE_STRIDE + lane];
              val.z = stage_tile[(f0 + 4 * v + 2) * TSTAGE_STRIDE + lane];
              val.w = stage_tile[(f0 + 4 * v + 3) * TSTAGE_STRIDE + lane];
              if constexpr (FP8) {  // partial sums leave the kernel already dequantised
                float* pv = &val.x;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  const int f = f0 + 4 * v + u;  // feature inside the tile -> weight row of the expert
                  int wr = (p.features_per_tile == 64)
                               ? (f < 64 ? t.wt * 64 + f : p.second_box_offset + t.wt * 64 + f - 64)
                               : t.wt * 128 + f;
                  wr = min(wr, p.w_rows_per_expert - 1);
                  pv[u] *= rs * __ldg(cs + wr);
                }
              }
              *reinterpret_cast<float4*>(o + 4 * v) = val;
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // staging tile free for the next chunk
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

constexpr int TOKENN_SMEM = TPIPE_BYTES + TW * TSTAGE_STRIDE * 4 + (3 * TMAX_EXPERTS + 2) * 4 + 512 + 1024;

template <int MODE, bool BF16, bool FP8 = false>
static int launch_tokenn(const CUtensorMap& tmW, const CUtensorMap& tmX, const TokenNParams& p, int grid,
                         cudaStream_t st) {
  auto kern = tokenn_gemm_kernel<MODE, BF16, FP8>;
  FR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TOKENN_SMEM));
  kern<<<grid, 192, TOKENN_SMEM, st>>>(tmW, tmX, p);
  return static_cast<int>(cudaGetLastError());
}

// which: 0 = GEMM1 (gate/up rows paired in one tile, SiLU epilogue), 1 = GEMM2 (routed-weight epilogue).
// a: expert-sorted rows, experts padded to 16 rows (align with block size 16); counts[E] on the device.
int gemm_tokenn_dispatch(int which, const void* a, int64_t lda, const void* w, int dtype, int64_t max_rows, int K,
                         int n_out, int E, int w_rows_per_expert, const int32_t* counts, const int32_t* num_post,
                         const int32_t* sorted_ids, const float* topk_w, int64_t n_valid, void* out, int64_t ldo,
                         int split_k, void* workspace, size_t workspace_bytes, cudaStream_t st, int* deferred_split,
                         const QuantArgs* quant) {
  if (deferred_split) *deferred_split = 0;
  const bool fp8 = quant != nullptr;  // a and w hold E4M3 bytes; dtype is the output type
  if (fp8 && (!quant->row_scale || !quant->col_scale)) return FR_ERR_ARG;
  if (!a || !w || !counts || !sorted_ids || !out || max_rows <= 0 || K <= 0 || n_out <= 0 || E <= 0) return FR_ERR_ARG;
  if (dtype != FR_F16 && dtype != FR_BF16) return FR_ERR_UNSUPPORTED;
  if (E > TMAX_EXPERTS) return FR_ERR_UNSUPPORTED;
  if ((K % (fp8 ? 16 : 8)) || (n_out % 8) || (ldo % 8) || (lda % (fp8 ? 16 : 8))) return FR_ERR_ALIGN;
  if (reinterpret_cast<uintptr_t>(out) & 15) return FR_ERR_ALIGN;
  const int BKE = fp8 ? 2 * BK : BK;
  const int KB = (K + BKE - 1) / BKE;
  if (split_k < 1) split_k = 1;
  if (split_k > KB) split_k = KB;
  const DeviceInfo& di = device_info();

  TokenNParams p = {};
  p.counts = counts;
  p.max_rows = static_cast<int>(max_rows < 0x7fffffff ? max_rows : 0x7fffffff);
  p.sorted_ids = sorted_ids;
  p.topk_w = topk_w;
  p.n_valid = n_valid;
  p.out = out;
  p.ldo = ldo;
  p.E = E;
  p.K = K;
  p.n_out = n_out;
  p.row_scale = fp8 ? quant->row_scale : nullptr;
  p.col_scale = fp8 ? quant->col_scale : nullptr;
  p.w_rows_per_expert = w_rows_per_expert;
  p.features_per_tile = (which == 0) ? 64 : 128;
  p.second_box_offset = (which == 0) ? n_out : 64;
  p.num_wt = (n_out + p.features_per_tile - 1) / p.features_per_tile;
  p.kb_per_split = (KB + split_k - 1) / split_k;
  p.split_k = (KB + p.kb_per_split - 1) / p.kb_per_split;
  split_k = p.split_k;
  p.partial_cols = static_cast<int64_t>(p.num_wt) * 128;
  // token tile: about twice the average tokens per expert, a power of two between 16 and 256; the
  // smaller the token operand, the more pipeline stages (= weight bytes in flight) fit
  {
    const int64_t avg = (n_valid + E - 1) / E;
    int box = 16;
    while (box < TN_MAX && box < 2 * avg) box <<= 1;
    p.tn_box = box;
    const int stage_bytes = TW_STAGE_BYTES + box * BK * 2;
    p.stages = TPIPE_BYTES / stage_bytes;
    if (p.stages > TMAX_STAGES) p.stages = TMAX_STAGES;
  }
  if (split_k > 1) {
    const size_t need = static_cast<size_t>(split_k) * static_cast<size_t>(n_valid) * p.partial_cols * sizeof(float);
    if (!workspace || workspace_bytes < need) return FR_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 15) return FR_ERR_ALIGN;
    p.partial = static_cast<float*>(workspace);
  }
  CUtensorMap tmW, tmX;
  int rc = make_tmap_2d(&tmW, w, static_cast<uint64_t>(E) * w_rows_per_expert, static_cast<uint64_t>(K),
                        static_cast<uint64_t>(K), 64, BKE, true, fp8 ? 1 : 2);
  if (rc) return rc;
  rc = make_tmap_2d(&tmX, a, static_cast<uint64_t>(max_rows), static_cast<uint64_t>(K), static_cast<uint64_t>(lda),
                    static_cast<uint32_t>(p.tn_box), BKE, true, fp8 ? 1 : 2);
  if (rc) return rc;
  const int64_t active = n_valid < E ? n_valid : E;
  const int64_t max_tiles = (n_valid / p.tn_box + active) * p.num_wt * split_k;
  const int grid = static_cast<int>(max_tiles < di.sm_count ? (max_tiles > 0 ? max_tiles : 1) : di.sm_count);
  const bool bf = dtype == FR_BF16;
  if (split_k > 1) {
    if (fp8)
      rc = bf ? launch_tokenn<MODE_PARTIAL, true, true>(tmW, tmX, p, grid, st)
              : launch_tokenn<MODE_PARTIAL, false, true>(tmW, tmX, p, grid, st);
    else
      rc = bf ? launch_tokenn<MODE_PARTIAL, true>(tmW, tmX, p, grid, st)
              : launch_tokenn<MODE_PARTIAL, false>(tmW, tmX, p, grid, st);
    if (rc) return rc;
    if (which == 1 && deferred_split) {
      *deferred_split = split_k;
      return FR_OK;
    }
    if (!num_post) return FR_ERR_ARG;
    const dim3 rgrid(static_cast<unsigned>((n_out + 1023) / 1024), static_cast<unsigned>(max_rows));
    if (which == 0) {
      if (bf)
        splitk_reduce_silu_kernel<true><<<rgrid, 256, 0, st>>>(p.partial, p.partial_cols, split_k, n_valid, sorted_ids,
                                                               num_post, n_out, 64, static_cast<uint16_t*>(out), ldo);
      else
        splitk_reduce_silu_kernel<false><<<rgrid, 256, 0, st>>>(p.partial, p.partial_cols, split_k, n_valid, sorted_ids,
                                                                num_post, n_out, 64, static_cast<uint16_t*>(out), ldo);
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
      return bf ? launch_tokenn<MODE_SILU, true, true>(tmW, tmX, p, grid, st)
                : launch_tokenn<MODE_SILU, false, true>(tmW, tmX, p, grid, st);
    return bf ? launch_tokenn<MODE_WEIGHTED, true, true>(tmW, tmX, p, grid, st)
              : launch_tokenn<MODE_WEIGHTED, false, true>(tmW, tmX, p, grid, st);
  }
  if (which == 0)
    return bf ? launch_tokenn<MODE_SILU, true>(tmW, tmX, p, grid, st) : launch_tokenn<MODE_SILU, false>(tmW, tmX, p, grid, st);
  return bf ? launch_tokenn<MODE_WEIGHTED, true>(tmW, tmX, p, grid, st)
            : launch_tokenn<MODE_WEIGHTED, false>(tmW, tmX, p, grid, st);
}

}  // namespace fr
