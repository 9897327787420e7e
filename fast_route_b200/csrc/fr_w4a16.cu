// W4A16 split-K GEMM for small batches:  c[m,n] = a[m,k] . dequant(qweight)[k,n],  fp16 activations, 4-bit
// GPTQ-packed weights with per-group fp16 scales and packed 4-bit zero points, fp32 accumulation, fp16 output.
// Stands in for matmul_split_k / hint_kernel of the reference (benchmarks/splitk_gemm/splitk.py:26-103, 178-216):
//   qweight[k/8, n] int32, nibble j of word [kk, n] is row k = 8*kk + j;   scales[k/g, n] fp16;
//   qzeros[k/g, n/8] int32, nibble j of word [gi, nn] belongs to column n = 8*nn + j;
//   w[k,n] = fp16(q) * s  -  fp16(z + 1) * s,  every operation rounded to fp16 (:83-87).
//
// B200 mapping.  The layer is bound by streaming the packed weights once, so weights sit on the MMA M axis
// (128 output columns per CTA) and the few activation rows on the MMA N axis (16..256):
//   warp 0    TMA producer: per 64-wide K step the packed tile (8 words x 128 columns, 4 KB) and the activation
//             tile (m_pad rows x 64, 128-byte swizzle) into a ring of input stages
//   warps 4-7 dequantise: thread t owns output column n0+t, expands 8 packed words into eight 16-byte rows of the
//             K-major, 128-byte-swizzled operand tile in shared memory, then drain the accumulator at the end
//   warp 1    one thread issues tcgen05.mma (M=128, N=m_pad, fp32 accumulator in TMEM)
// Split-K runs as a thread-block cluster along K (1, 2, 4 or 8 CTAs): every CTA parks its fp32 partial tile in its
// own shared memory, and after a cluster barrier CTA r sums rows r, r+S, ... over the ranks in rank order through
// distributed shared memory.  No workspace, no atomics: the result does not depend on timing (the reference
// accumulates the slices with fp16 atomics, :103).
#include <cooperative_groups.h>

#include "fr_common.cuh"

namespace fr {

namespace cgx = cooperative_groups;

constexpr int W4_BN = 128;                 // output columns (weight rows of the MMA) per CTA
constexpr int W4_BK = 64;                  // K step: one 128-byte operand row
constexpr int W4_WSTAGES = 3;              // dequantised operand ring
constexpr int W4_W_BYTES = W4_BN * W4_BK * 2;   // 16 KB
constexpr int W4_RAW_BYTES = 8 * W4_BN * 4;     // 4 KB of packed words
constexpr int W4_MAX_IN = 8;               // input ring depth (packed tile + activation tile)
constexpr int W4_SMEM_BUDGET = 200 * 1024;

struct W4Params {
  const __half* scales;    // [k/g, n]
  const int32_t* qzeros;   // [k/g, n/8]
  __half* c;
  int64_t ldc;
  int m;                   // valid activation rows of this launch (<= m_pad)
  int m_pad;               // MMA N: multiple of 16, <= 256
  int n, k;
  int groupsize;           // multiple of 64
  int in_stages;
  int x_bytes;             // m_pad * 128
  uint32_t tmem_cols;
};

// eight fp16 weights of one packed word: w_j = q_j * s - zs, each operation rounded to fp16 (no fused multiply-add)
__device__ __forceinline__ uint4 w4_dequant8(uint32_t v, __half2 s2, __half2 zs2) {
  const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
  uint32_t out[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // nibbles 2i (low half) and 2i+1 (high half) as 1024 + q in fp16, which is exact
    const uint32_t lo = (v >> (8 * i)) & 0xFu, hi = (v >> (8 * i + 4)) & 0xFu;
    const uint32_t bits = 0x64006400u | lo | (hi << 16);
    __half2 q = __hsub2_rn(*reinterpret_cast<const __half2*>(&bits), k1024);
    q = __hsub2_rn(__hmul2_rn(q, s2), zs2);
    out[i] = *reinterpret_cast<uint32_t*>(&q);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

__global__ void __launch_bounds__(256, 1)
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmX, const W4Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // layout: [W ring][X ring][packed ring][barriers]; the W ring doubles as the fp32 partial tile at the end
  uint8_t* sW = smem;
  uint8_t* sX = sW + W4_WSTAGES * W4_W_BYTES;
  uint8_t* sQ = sX + p.in_stages * p.x_bytes;
  uint64_t* in_full = reinterpret_cast<uint64_t*>(sQ + p.in_stages * W4_RAW_BYTES);
  uint64_t* in_empty = in_full + W4_MAX_IN;
  uint64_t* w_full = in_empty + W4_MAX_IN;
  uint64_t* w_empty = w_full + W4_WSTAGES;
  uint64_t* tfull = w_empty + W4_WSTAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  cgx::cluster_group cluster = cgx::this_cluster();
  const int S = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * W4_BN;

  // this CTA's K steps
  const int KB = p.k / W4_BK;
  const int per = (KB + S - 1) / S;
  const int kb_begin = min(KB, rank * per);
  const int kb_end = min(KB, kb_begin + per);
  const int nkb = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < W4_MAX_IN; ++s) {
      mbar_init(&in_full[s], 1);
      mbar_init(&in_empty[s], 1);
    }
    for (int s = 0; s < W4_WSTAGES; ++s) {
      mbar_init(&w_full[s], 4);
      mbar_init(&w_empty[s], 1);
    }
    mbar_init(tfull, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmX);
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc(tmem_slot, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t in_stages = static_cast<uint32_t>(p.in_stages);

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      PipeState ps;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        // a stage is free once the MMAs that read its activation tile are complete; they were issued after the
        // dequantisers had consumed its packed tile
        if (!wait_or_abort(&in_empty[ps.stage], ps.phase ^ 1, abort_flag, 0x800)) break;
        mbar_expect_tx(&in_full[ps.stage], W4_RAW_BYTES + p.x_bytes);
        // the packed matrix is addressed as 16-bit elements: column 2*n, row k/8
        tma_load_2d(sQ + ps.stage * W4_RAW_BYTES, &tmQ, &in_full[ps.stage], 2 * n0, kb * (W4_BK / 8));
        tma_load_2d(sX + ps.stage * p.x_bytes, &tmX, &in_full[ps.stage], kb * W4_BK, 0);
        ps.advance_rt(in_stages);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(false, W4_BN, p.m_pad);
      PipeState pin, pw;
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!wait_or_abort(&in_full[pin.stage], pin.phase, abort_flag, 0x810) ||
            !wait_or_abort(&w_full[pw.stage], pw.phase, abort_flag, 0x811)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t adesc = umma_desc_sw128(smem_u32(sW + pw.stage * W4_W_BYTES));
        const uint64_t bdesc = umma_desc_sw128(smem_u32(sX + pin.stage * p.x_bytes));
#pragma unroll
        for (int kk = 0; kk < W4_BK / 16; ++kk)
          tc_mma_f16(tmem_base, adesc + 2 * kk, bdesc + 2 * kk, idesc, (kb > kb_begin || kk > 0) ? 1u : 0u);
        tc_commit(&w_empty[pw.stage]);
        tc_commit(&in_empty[pin.stage]);
        pin.advance_rt(in_stages);
        pw.advance<W4_WSTAGES>();
      }
      if (ok) tc_commit(tfull);
    }
  } else if (warp >= 4) {
    // ---------------- dequantise, then drain ----------------
    const int t = threadIdx.x - 128;            // 0..127: output column n0 + t, TMEM lane t
    const int n = n0 + t;
    const bool n_ok = n < p.n;
    const int steps_per_group = p.groupsize / W4_BK;
    // byte offset of row t in a swizzled operand tile; the 16-byte chunk index is XORed with (t & 7)
    const uint32_t row_off = static_cast<uint32_t>(t >> 3) * 1024u + static_cast<uint32_t>(t & 7) * 128u;
    PipeState pin, pw;
    __half2 s2 = __half2half2(__ushort_as_half(0)), zs2 = s2;
    int cur_group = -1;
    bool ok = true;
    for (int kb = kb_begin; kb < kb_end && ok; ++kb) {
      const int g = kb / steps_per_group;
      if (g != cur_group) {
        cur_group = g;
        __half s = __ushort_as_half(0);
        uint32_t z = 0;
        if (n_ok) {
          s = __ldg(p.scales + static_cast<int64_t>(g) * p.n + n);
          z = (static_cast<uint32_t>(__ldg(p.qzeros + static_cast<int64_t>(g) * (p.n >> 3) + (n >> 3))) >> ((n & 7) * 4)) & 0xFu;
        }
        const __half zp1 = __ushort2half_rn(static_cast<unsigned short>(z + 1));
        s2 = __half2half2(s);
        zs2 = __half2half2(__hmul_rn(zp1, s));
      }
      if (!wait_or_abort(&in_full[pin.stage], pin.phase, abort_flag, 0x820) ||
          !wait_or_abort(&w_empty[pw.stage], pw.phase ^ 1, abort_flag, 0x821)) {
        ok = false;
        break;
      }
      const uint32_t* q = reinterpret_cast<const uint32_t*>(sQ + pin.stage * W4_RAW_BYTES) + t;
      uint8_t* wrow = sW + pw.stage * W4_W_BYTES + row_off;
      uint32_t words[8];
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) words[kk] = q[kk * W4_BN];
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        *reinterpret_cast<uint4*>(wrow + ((kk ^ (t & 7)) << 4)) = w4_dequant8(words[kk], s2, zs2);
      // make the generic-proxy writes visible to the tensor core (async proxy) before signalling
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&w_full[pw.stage]);
      pin.advance_rt(in_stages);
      pw.advance<W4_WSTAGES>();
    }

    // partial tile -> this CTA's shared memory as fp32 [m_pad][128] (column t contiguous across lanes)
    float* part = reinterpret_cast<float*>(sW);
    if (nkb > 0 && ok) ok = wait_or_abort(tfull, 0, abort_flag, 0x830);
    tc_fence_after();
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    for (int c0 = 0; c0 < p.m_pad; c0 += 16) {
      uint32_t acc[16];
      if (nkb > 0 && ok) {
        tmem_ld16(taddr + c0, acc);
        tc_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0u;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) part[(c0 + i) * W4_BN + t] = __uint_as_float(acc[i]);
    }
  }

  // every CTA of the cluster has parked its partial tile
  tc_fence_before();
  __syncthreads();
  cluster.sync();

  if (warp >= 4) {
    const int t = threadIdx.x - 128;
    const int n = n0 + t;
    if (n < p.n) {
      for (int row = rank; row < p.m; row += S) {
        float acc = 0.0f;
        for (int r = 0; r < S; ++r) {
          const float* remote = cluster.map_shared_rank(reinterpret_cast<float*>(sW), r);
          const float v = remote[row * W4_BN + t];
          acc = (r == 0) ? v : __fadd_rn(acc, v);
        }
        p.c[static_cast<int64_t>(row) * p.ldc + n] = __float2half_rn(acc);
      }
    }
  }
  // nobody leaves while another CTA may still read its shared memory
  cluster.sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

// Elementwise dequantisation to w[k,n] fp16 with the same arithmetic (for checking and for callers that want the
// dense matrix).
__global__ void w4a16_dequant_kernel(const int32_t* __restrict__ qweight, const __half* __restrict__ scales,
                                     const int32_t* __restrict__ qzeros, int n, int k, int groupsize,
                                     __half* __restrict__ w, int64_t ldw) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(k / 8) * n;
  if (idx >= total) return;
  const int kk = static_cast<int>(idx / n), col = static_cast<int>(idx % n);
  const int g = (kk * 8) / groupsize;
  const __half s = scales[static_cast<int64_t>(g) * n + col];
  const uint32_t z = (static_cast<uint32_t>(qzeros[static_cast<int64_t>(g) * (n >> 3) + (col >> 3)]) >> ((col & 7) * 4)) & 0xFu;
  const __half zs = __hmul_rn(__ushort2half_rn(static_cast<unsigned short>(z + 1)), s);
  const uint4 v = w4_dequant8(static_cast<uint32_t>(qweight[idx]), __half2half2(s), __half2half2(zs));
  const __half* h = reinterpret_cast<const __half*>(&v);
#pragma unroll
  for (int j = 0; j < 8; ++j) w[static_cast<int64_t>(kk * 8 + j) * ldw + col] = h[j];
}

int w4a16_dequant_dispatch(const int32_t* qweight, const void* scales, const int32_t* qzeros, int n, int k,
                           int groupsize, void* w, int64_t ldw, cudaStream_t st) {
  if (!qweight || !scales || !qzeros || !w || n <= 0 || k <= 0 || groupsize <= 0) return FR_ERR_ARG;
  if ((n % 8) || (k % 8) || (groupsize % 8) || (k % groupsize) || ldw < n) return FR_ERR_ALIGN;
  const int64_t total = static_cast<int64_t>(k / 8) * n;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  w4a16_dequant_kernel<<<blocks, 256, 0, st>>>(qweight, static_cast<const __half*>(scales), qzeros, n, k, groupsize,
                                               static_cast<__half*>(w), ldw);
  return static_cast<int>(cudaGetLastError());
}

// split_k: 0 = choose (largest of 1,2,4,8 that keeps the grid within the SM count and every slice non-empty).
int w4a16_gemm_dispatch(const void* a, int64_t lda, const int32_t* qweight, const void* scales, const int32_t* qzeros,
                        int64_t m, int n, int k, int groupsize, void* c, int64_t ldc, int split_k, cudaStream_t st) {
  if (!a || !qweight || !scales || !qzeros || !c || m < 0 || n <= 0 || k <= 0 || groupsize <= 0) return FR_ERR_ARG;
  if (m == 0) return FR_OK;
  if ((n % 8) || (k % W4_BK) || (groupsize % W4_BK) || (k % groupsize) || (lda % 8) || ldc < n) return FR_ERR_ALIGN;
  if (split_k != 0 && split_k != 1 && split_k != 2 && split_k != 4 && split_k != 8) return FR_ERR_ARG;
  const DeviceInfo& di = device_info();
  const int n_tiles = (n + W4_BN - 1) / W4_BN;
  const int KB = k / W4_BK;
  int S = split_k;
  if (S == 0) {
    S = 1;
    while (S < 8 && n_tiles * (S * 2) <= di.sm_count && KB >= S * 2 * 4) S *= 2;
  }
  while (S > 1 && KB < S) S /= 2;

  CUtensorMap tmQ;
  int rc = make_tmap_2d(&tmQ, qweight, static_cast<uint64_t>(k / 8), static_cast<uint64_t>(n) * 2,
                        static_cast<uint64_t>(n) * 2, 8, 2 * W4_BN, false);
  if (rc) return rc;

  auto kern = w4a16_gemm_kernel;
  for (int64_t m0 = 0; m0 < m; m0 += 256) {
    const int mc = static_cast<int>(m - m0 < 256 ? m - m0 : 256);
    W4Params p = {};
    p.scales = static_cast<const __half*>(scales);
    p.qzeros = qzeros;
    p.c = static_cast<__half*>(c) + m0 * ldc;
    p.ldc = ldc;
    p.m = mc;
    p.m_pad = (mc + 15) & ~15;
    p.n = n;
    p.k = k;
    p.groupsize = groupsize;
    p.x_bytes = p.m_pad * 128;
    int stages = (W4_SMEM_BUDGET - W4_WSTAGES * W4_W_BYTES) / (W4_RAW_BYTES + p.x_bytes);
    p.in_stages = stages > W4_MAX_IN ? W4_MAX_IN : stages;
    if (p.in_stages < 2) return FR_ERR_UNSUPPORTED;
    uint32_t cols = 32;
    while (cols < static_cast<uint32_t>(p.m_pad)) cols *= 2;
    p.tmem_cols = cols;
    // the partial tile (m_pad x 128 fp32) reuses the operand ring and the start of the activation ring
    if (p.m_pad * W4_BN * 4 > W4_WSTAGES * W4_W_BYTES + p.in_stages * p.x_bytes) return FR_ERR_UNSUPPORTED;
    CUtensorMap tmX;
    rc = make_tmap_2d(&tmX, static_cast<const __half*>(a) + m0 * lda, static_cast<uint64_t>(mc),
                      static_cast<uint64_t>(k), static_cast<uint64_t>(lda), p.m_pad, W4_BK, true);
    if (rc) return rc;
    const int smem = W4_WSTAGES * W4_W_BYTES + p.in_stages * (p.x_bytes + W4_RAW_BYTES) + 512 + 1024;
    FR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles, S, 1);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = S;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    FR_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tmQ, tmX, p));
  }
  return FR_OK;
}

}  // namespace fr
