// Low-latency routing: (1) top-k on packed sortable keys for 16-bit logits, (2) a
// cooperative align kernel that spreads the counting sort over every SM with a single
// bounded grid barrier.  Same outputs, bit for bit, as the kernels in fr_route.cu; these exist because the
// routing stage moves well under 10 MB and is bound by instruction issue and launch latency,
// not by HBM (reference stage: route_kernel epilogue, ops/stable_route.py:91-121, followed by
// moe_align_block_size, ops/fused_moe.py:133-175).
#include <cooperative_groups.h>

#include <atomic>
#include <cstdlib>

#include "fr_common.cuh"

namespace fr {

// ----------------------------------------------------------------------------------
// packed keys: (order-preserving 16-bit image of the value) << 16 | (0xFFFF - column).
// A larger key is a larger value, or the same value in a lower column: one unsigned max
// implements the tie rule.  0 marks an empty slot.
// ----------------------------------------------------------------------------------
template <typename T>
struct Bits16;
template <>
struct Bits16<__half> {
  static __device__ __forceinline__ bool is_nan(uint32_t u) { return (u & 0x7FFFu) > 0x7C00u; }
  static constexpr uint32_t kNegInf = 0xFC00u;
  static __device__ __forceinline__ float to_float(uint32_t u) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(u)));
  }
};
template <>
struct Bits16<__nv_bfloat16> {
  static __device__ __forceinline__ bool is_nan(uint32_t u) { return (u & 0x7FFFu) > 0x7F80u; }
  static constexpr uint32_t kNegInf = 0xFF80u;
  static __device__ __forceinline__ float to_float(uint32_t u) { return __uint_as_float(u << 16); }
};

template <typename T>
__device__ __forceinline__ uint32_t make_key(uint32_t u, int col) {
  if (Bits16<T>::is_nan(u)) u = Bits16<T>::kNegInf;  // NaN is outside the contract: ranked last
  if (u == 0x8000u) u = 0;                           // -0 and +0 are the same value
  const uint32_t mono = (u & 0x8000u) ? (~u & 0xFFFFu) : (u | 0x8000u);
  return (mono << 16) | (0xFFFFu - static_cast<uint32_t>(col));
}
template <typename T>
__device__ __forceinline__ float key_value(uint32_t key) {
  const uint32_t mono = key >> 16;
  const uint32_t u = (mono & 0x8000u) ? (mono & 0x7FFFu) : (~mono & 0xFFFFu);
  return Bits16<T>::to_float(u);
}
__device__ __forceinline__ int key_col(uint32_t key) { return static_cast<int>(0xFFFFu - (key & 0xFFFFu)); }

#define FR_CE(a, b)                      \
  do {                                   \
    const uint32_t hi_ = max(a, b);      \
    const uint32_t lo_ = min(a, b);      \
    a = hi_;                             \
    b = lo_;                             \
  } while (0)

// Descending sort of 8 keys (Batcher odd-even merge network, 19 compare-exchanges).
__device__ __forceinline__ void sort8_desc(uint32_t (&k)[8]) {
  FR_CE(k[0], k[1]); FR_CE(k[2], k[3]); FR_CE(k[4], k[5]); FR_CE(k[6], k[7]);
  FR_CE(k[0], k[2]); FR_CE(k[1], k[3]); FR_CE(k[4], k[6]); FR_CE(k[5], k[7]);
  FR_CE(k[1], k[2]); FR_CE(k[5], k[6]);
  FR_CE(k[0], k[4]); FR_CE(k[1], k[5]); FR_CE(k[2], k[6]); FR_CE(k[3], k[7]);
  FR_CE(k[2], k[4]); FR_CE(k[3], k[5]);
  FR_CE(k[1], k[2]); FR_CE(k[3], k[4]); FR_CE(k[5], k[6]);
}

constexpr int PK = 8;  // most experts per token on this path

// L lanes hold one row, 8 sorted keys each.  Round j: the maximum of the lane heads is the
// j-th winner (one redux over the group); its owner pops it.  Returns the winners in win[].
template <int L>
__device__ __forceinline__ void select_topk(uint32_t (&keys)[8], int k, unsigned group_mask, uint32_t (&win)[PK]) {
#pragma unroll
  for (int j = 0; j < PK; ++j) {
    win[j] = 0;
    if (j < k) {
      uint32_t m = keys[0];
      if (L > 1) m = __reduce_max_sync(group_mask, m);
      win[j] = m;
      const bool mine = (keys[0] == m);
#pragma unroll
      for (int i = 0; i < 7; ++i) keys[i] = mine ? keys[i + 1] : keys[i];
      keys[7] = mine ? 0u : keys[7];
    }
  }
}

// Softmax over the k winners with the fixed fp32 recipe.  Lane `sub` of the group owns the
// slots sub, sub+L, ...: it evaluates their exponentials, all lanes form the same sequential
// sum from the exchanged values, and the owner divides and stores its slots (one IEEE division
// per owned slot; consecutive lanes write consecutive addresses).
template <typename T, int L>
__device__ __forceinline__ void write_topk(const uint32_t (&win)[PK], int k, int sub, int lane, unsigned group_mask,
                                           bool row_ok, float* wrow, int32_t* irow, int32_t* sm_ids) {
  const float v0 = key_value<T>(win[0]);
  constexpr int PER = (PK + L - 1) / L;
  float e[PK], mine[PER];
  uint32_t mykey[PER];
#pragma unroll
  for (int j = 0; j < PK; ++j) e[j] = 0.0f;
#pragma unroll
  for (int r = 0; r < PER; ++r) {
    mine[r] = 0.0f;
    mykey[r] = 0;
    if (r * L < k) {  // uniform over the warp
      const int myj = sub + r * L;
      uint32_t kk = win[0];
#pragma unroll
      for (int j = 1; j < PK; ++j) kk = (myj == j) ? win[j] : kk;
      mykey[r] = kk;
      mine[r] = exp_recipe(__fsub_rn(key_value<T>(kk), v0));
#pragma unroll
      for (int j = r * L; j < PK && j < (r + 1) * L; ++j) {
        if (L > 1) e[j] = __shfl_sync(group_mask, mine[r], (lane & ~(L - 1)) + (j - r * L));
        else e[j] = mine[r];
      }
    }
  }
  float s = e[0];
#pragma unroll
  for (int j = 1; j < PK; ++j)
    if (j < k) s = __fadd_rn(s, e[j]);
#pragma unroll
  for (int r = 0; r < PER; ++r) {
    const int myj = sub + r * L;
    if (r * L < k && myj < k && row_ok) {
      wrow[myj] = __fdiv_rn(mine[r], s);
      const int c = key_col(mykey[r]);
      irow[myj] = c;
      if (sm_ids) sm_ids[myj] = c;
    }
  }
}

template <typename T, int L>
__device__ __forceinline__ void load_keys(const T* row, int64_t stride_e, int E, int sub, bool vec_ok,
                                          uint32_t (&keys)[8]) {
  const int c0 = sub * 8;
  if (vec_ok) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(row + c0));
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      keys[2 * i] = make_key<T>(w[i] & 0xFFFFu, c0 + 2 * i);
      keys[2 * i + 1] = make_key<T>(w[i] >> 16, c0 + 2 * i + 1);
    }
  } else {
    const unsigned short* r16 = reinterpret_cast<const unsigned short*>(row);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = c0 + i;
      keys[i] = (c < E) ? make_key<T>(r16[static_cast<int64_t>(c) * stride_e], c) : 0u;
    }
  }
}

template <typename T, int L>
__global__ void __launch_bounds__(256) topk16_kernel(const T* __restrict__ logits, int64_t M, int E, int64_t stride_m,
                                                     int64_t stride_e, int k, float* __restrict__ weights,
                                                     int64_t w_stride, int32_t* __restrict__ ids, int64_t id_stride,
                                                     int vec_ok) {
  const int64_t gthread = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t row = gthread / L;
  const int sub = static_cast<int>(gthread % L);
  const int lane = threadIdx.x & 31;
  const bool row_ok = row < M;
  const int64_t r = row_ok ? row : (M - 1);
  const unsigned group_mask = (L == 32) ? 0xffffffffu : (((1u << L) - 1u) << (lane & ~(L - 1)));
  uint32_t keys[8], win[PK];
  load_keys<T, L>(logits + r * stride_m, stride_e, E, sub, vec_ok != 0, keys);
  sort8_desc(keys);
  select_topk<L>(keys, k, group_mask, win);
  write_topk<T, L>(win, k, sub, lane, group_mask, row_ok, weights + r * w_stride, ids + r * id_stride, nullptr);
}

template <typename T>
int launch_topk16(const void* logits, int64_t M, int E, int64_t stride_m, int64_t stride_e, int k, float* weights,
                  int64_t w_stride, int32_t* ids, int64_t id_stride, cudaStream_t st) {
  const T* lp = static_cast<const T*>(logits);
  const int threads = 256;
#define FR_LAUNCH_TOPK16(L_)                                                                                   \
  do {                                                                                                         \
    const int vec_ok = (stride_e == 1) && (E == (L_) * 8) && ((stride_m * 2) % 16 == 0) &&                     \
                       ((reinterpret_cast<uintptr_t>(lp) & 15) == 0);                                          \
    const int64_t total = M * (L_);                                                                            \
    const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);                            \
    topk16_kernel<T, L_><<<blocks, threads, 0, st>>>(lp, M, E, stride_m, stride_e, k, weights, w_stride, ids,  \
                                                     id_stride, vec_ok);                                       \
  } while (0)
  if (E <= 8) FR_LAUNCH_TOPK16(1);
  else if (E <= 16) FR_LAUNCH_TOPK16(2);
  else if (E <= 32) FR_LAUNCH_TOPK16(4);
  else if (E <= 64) FR_LAUNCH_TOPK16(8);
  else if (E <= 128) FR_LAUNCH_TOPK16(16);
  else FR_LAUNCH_TOPK16(32);
#undef FR_LAUNCH_TOPK16
  return static_cast<int>(cudaGetLastError());
}
template int launch_topk16<__half>(const void*, int64_t, int, int64_t, int64_t, int, float*, int64_t, int32_t*,
                                   int64_t, cudaStream_t);
template int launch_topk16<__nv_bfloat16>(const void*, int64_t, int, int64_t, int64_t, int, float*, int64_t,
                                          int32_t*, int64_t, cudaStream_t);

// ----------------------------------------------------------------------------------
// cooperative route + align
// ----------------------------------------------------------------------------------
// Bounded, self-resetting grid barrier for a cooperative launch (all blocks co-resident).
// bar[0] = arrival count, bar[1] = generation; both start at zero and the count is zero
// again after every completed barrier.  If the wait runs out the status block records it
// and every block leaves the kernel; the two words must then be cleared before reuse.
// bar[3] = how many polls a block may spend waiting (0 = the default, about a second); a
// caller that wants a shorter limit writes it there, next to the barrier words it owns.
__device__ __forceinline__ bool grid_barrier(unsigned int* bar, unsigned int nblocks) {
  __shared__ int ok_flag;
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = 1;
    volatile unsigned int* vgen = bar + 1;
    const unsigned int gen = *vgen;
    __threadfence();
    const unsigned int prev = atomicAdd(bar, 1u);
    if (prev == nblocks - 1) {
      bar[0] = 0;
      __threadfence();
      atomicAdd(bar + 1, 1u);
    } else {
      const unsigned int asked = __ldcg(bar + 3);
      const uint32_t budget = asked ? asked : (1u << 22);
      uint32_t it = 0;
      while (*vgen == gen) {
        if (++it > budget) {
          ok = 0;
          report(ST_WAIT_TIMEOUT, 0x500);
          break;
        }
      }
    }
    __threadfence();
    ok_flag = ok;
  }
  __syncthreads();
  return ok_flag != 0;
}

struct CoopParams {
  const int32_t* ids_in;
  int64_t n;
  int E, bs, nbits;
  int32_t* sorted;
  int64_t sorted_len;
  int32_t* expert_ids;
  int64_t expert_ids_len;
  int32_t* num_post;
  int32_t* counts;
  int32_t* inv_pos;
  // scratch
  int32_t* hist;          // [gridDim][E]
  unsigned int* barrier;  // [2]
  int64_t per_block;      // assignments per block
  int64_t seg;            // assignments per warp, multiple of 32
};

// The kernel body; load_ids(sids, lo_blk, slice) fills this block's slice of the flat expert ids in shared memory.
// (Ranking the block's own rows of logits in that phase, to make routing + align one launch, was measured and is
// not faster than the two kernels: the ranking runs slower inside a one-block-per-SM cooperative kernel than as
// its own full-occupancy launch, and the cost of a cooperative launch is paid either way.)
template <typename LoadIds>
__device__ __forceinline__ void align_coop_body(const CoopParams& p, LoadIds&& load_ids) {
  extern __shared__ int csm[];
  const int nwarps = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int E = p.E;
  const int ES = E | 1;            // odd row stride: column reads across warps hit distinct banks
  const int B = gridDim.x;
  int* cnt = csm;                  // [nwarps][ES] per-warp counts, then exclusive prefixes over the warps
  int* total = cnt + nwarps * ES;  // [E]   totals over the grid
  int* before = total + E;         // [E]   counts of lower-numbered blocks, later + padded start
  int* start = before + E;         // [E+1] padded starts
  int* padded = start + E + 1;     // [E]
  int32_t* sids = padded + E;      // [per_block] this block's slice of the flat ids

  const int64_t lo_blk = static_cast<int64_t>(blockIdx.x) * p.per_block;
  const int64_t hi_blk = min(p.n, lo_blk + p.per_block);
  const int slice = hi_blk > lo_blk ? static_cast<int>(hi_blk - lo_blk) : 0;
  for (int i = threadIdx.x; i < nwarps * ES + 2 * E; i += blockDim.x) cnt[i] = 0;  // cnt, total, before
  load_ids(sids, lo_blk, slice);
  __syncthreads();

  // pass 1: per-warp counts over the warp's contiguous sub-slice (order of the atomics is irrelevant)
  const int wlo = static_cast<int>(min(static_cast<int64_t>(slice), static_cast<int64_t>(warp) * p.seg));
  const int whi = static_cast<int>(min(static_cast<int64_t>(slice), static_cast<int64_t>(warp + 1) * p.seg));
  int* my = cnt + warp * ES;
  for (int i = wlo + lane; i < whi; i += 32) {
    const int e = sids[i];
    if (e >= 0) atomicAdd(&my[e], 1);
  }
  __syncthreads();
  // exclusive prefix over the warps, one expert per warp pass: lane l holds warp l's count
  for (int e = warp; e < E; e += nwarps) {
    const int c = (lane < nwarps) ? cnt[lane * ES + e] : 0;
    int incl = c;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += o;
    }
    if (lane < nwarps) cnt[lane * ES + e] = incl - c;
    if (lane == 31) __stcg(p.hist + static_cast<int64_t>(blockIdx.x) * E + e, incl);
  }
  if (!grid_barrier(p.barrier, B)) return;

  // totals and the counts of lower-numbered blocks: thread (g, e) sums the blocks g, g+G, ...
  // Every block starts its walk at a different histogram row so that the SMs do not all ask
  // the L2 for the same line at the same time.
  {
    const int G = max(1, static_cast<int>(blockDim.x) / E);
    const int g = threadIdx.x / E, e = threadIdx.x - g * E;
    const int me = static_cast<int>(blockIdx.x);
    if (g < G) {
      for (int ee = e; ee < E; ee += blockDim.x) {  // one trip unless E > blockDim
        int t = 0, bfr = 0;
        const int trips = (B - g + G - 1) / G;      // blocks g, g+G, ... handled by this thread
        int j = (me * 7) % (trips > 0 ? trips : 1);
        constexpr int BATCH = 8;                    // independent loads issued back to back
        for (int it = 0; it < trips; it += BATCH) {
          int v[BATCH], bb[BATCH];
#pragma unroll
          for (int u = 0; u < BATCH; ++u) {
            bb[u] = g + j * G;
            v[u] = (it + u < trips) ? __ldcg(p.hist + static_cast<int64_t>(bb[u]) * E + ee) : 0;
            if (++j >= trips) j = 0;
          }
#pragma unroll
          for (int u = 0; u < BATCH; ++u) {
            t += v[u];
            if (bb[u] < me) bfr += v[u];
          }
        }
        atomicAdd(&total[ee], t);
        atomicAdd(&before[ee], bfr);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) padded[e] = (total[e] + p.bs - 1) / p.bs * p.bs;
  __syncthreads();
  if (warp == 0) {
    const int chunk = (E + 31) / 32;
    const int e0 = lane * chunk;
    int sum = 0;
    for (int e = e0; e < e0 + chunk && e < E; ++e) sum += padded[e];
    int incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += o;
    }
    int run = incl - sum;
    for (int e = e0; e < e0 + chunk && e < E; ++e) {
      start[e] = run;
      before[e] += run;   // write base of this block for expert e = padded start + lower blocks
      run += padded[e];
    }
    if (lane == 31) start[E] = incl;
  }
  __syncthreads();
  // pass 2: stable scatter; position = block base + prefix over lower warps + rank in the row
  for (int b0 = wlo; b0 < whi; b0 += 32) {
    const int i = b0 + lane;
    const int e = (i < whi) ? sids[i] : -1;
    const unsigned grp = same_expert_lanes(e, p.nbits);
    int pos = 0;
    if (e >= 0) pos = before[e] + my[e] + __popc(grp & ((1u << lane) - 1u));
    __syncwarp();
    if (e >= 0) {
      if (lane == (__ffs(grp) - 1)) my[e] += __popc(grp);
      const int64_t flat = lo_blk + i;
      if (pos < p.sorted_len) p.sorted[pos] = static_cast<int32_t>(flat);
      if (p.inv_pos) p.inv_pos[flat] = pos;
    } else if (i < whi && p.inv_pos) {
      p.inv_pos[lo_blk + i] = -1;   // rejected id: the combine must not pick up a stale position
    }
    __syncwarp();
  }
  // padding entries, block -> expert table, tails: spread over the grid
  const int num_post = start[E];
  const int gwarp = blockIdx.x * nwarps + warp;
  const int gwarps = B * nwarps;
  for (int e = gwarp; e < E; e += gwarps) {
    const int s = start[e], t = total[e], pe = start[e + 1];
    for (int q = s + t + lane; q < pe; q += 32)
      if (q < p.sorted_len) p.sorted[q] = static_cast<int32_t>(p.n);
    for (int blk = s / p.bs + lane; blk < pe / p.bs; blk += 32)
      if (blk < p.expert_ids_len) p.expert_ids[blk] = e;
    if (p.counts && lane == 0) p.counts[e] = t;
  }
  const int64_t gthread = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t gthreads = static_cast<int64_t>(B) * blockDim.x;
  for (int64_t q = num_post + gthread; q < p.sorted_len; q += gthreads) p.sorted[q] = static_cast<int32_t>(p.n);
  for (int64_t blk = num_post / p.bs + gthread; blk < p.expert_ids_len; blk += gthreads) p.expert_ids[blk] = -1;
  if (blockIdx.x == 0 && threadIdx.x == 0) *p.num_post = num_post;
}

__global__ void __launch_bounds__(1024) align_coop_kernel(const CoopParams p) {
  align_coop_body(p, [&](int32_t* sids, int64_t lo_blk, int slice) {
    for (int i = threadIdx.x; i < slice; i += blockDim.x) {
      int e = __ldg(p.ids_in + lo_blk + i);
      if (e < 0 || e >= p.E) {
        report(ST_BAD_EXPERT_ID, static_cast<unsigned int>(e));
        e = -1;
      }
      sids[i] = e;
    }
  });
}

constexpr int kCoopMaxPerBlock = 8192;

size_t coop_workspace_bytes(int E) {
  // histogram for up to 256 blocks + the two barrier words (kept 256 bytes apart from the histogram)
  return 256 + static_cast<size_t>(256) * E * sizeof(int32_t);
}

// Returns FR_ERR_UNSUPPORTED when the case does not fit this kernel; the caller then uses the
// cluster kernel.
int align_coop_dispatch(const int32_t* ids_in, int64_t n, int E, int bs, int32_t* sorted_ids, int64_t sorted_len,
                        int32_t* expert_ids, int64_t expert_ids_len, int32_t* num_post, int32_t* counts,
                        int32_t* inv_pos, void* workspace, size_t workspace_bytes, cudaStream_t st, int64_t min_n) {
  if (!workspace || workspace_bytes < coop_workspace_bytes(E) || (reinterpret_cast<uintptr_t>(workspace) & 15))
    return FR_ERR_UNSUPPORTED;
  if (n < min_n || n < 1 || E > 1024) return FR_ERR_UNSUPPORTED;
  const DeviceInfo& di = device_info();
  int grid = di.sm_count < 256 ? di.sm_count : 256;
  if (grid <= 0) return FR_ERR_UNSUPPORTED;
  int64_t per_block = (n + grid - 1) / grid;
  if (per_block < 1024) {  // do not spread thinner than one assignment per thread
    per_block = 1024;
    grid = static_cast<int>((n + per_block - 1) / per_block);
  }
  if (per_block > kCoopMaxPerBlock) return FR_ERR_UNSUPPORTED;
  const int threads = 1024, nwarps = 32;
  int64_t seg = (per_block + nwarps - 1) / nwarps;
  seg = (seg + 31) / 32 * 32;

  CoopParams p = {};
  p.ids_in = ids_in;
  p.n = n;
  p.E = E;
  p.bs = bs;
  while ((1 << p.nbits) < E) ++p.nbits;
  p.sorted = sorted_ids;
  p.sorted_len = sorted_len;
  p.expert_ids = expert_ids;
  p.expert_ids_len = expert_ids_len;
  p.num_post = num_post;
  p.counts = counts;
  p.inv_pos = inv_pos;
  p.barrier = static_cast<unsigned int*>(workspace);
  p.hist = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(workspace) + 256);
  p.per_block = per_block;
  p.seg = seg;

  const size_t smem = (static_cast<size_t>(nwarps) * (E | 1) + 4 * static_cast<size_t>(E) + 1 + per_block) * sizeof(int);
  if (smem > 200 * 1024) return FR_ERR_UNSUPPORTED;
  if (smem > 48 * 1024)
    FR_CUDA_OK(cudaFuncSetAttribute(align_coop_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(smem)));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FR_CUDA_OK(cudaLaunchKernelEx(&cfg, align_coop_kernel, p));
  return FR_OK;
}

// ----------------------------------------------------------------------------------
// fr_align_noalloc: the cooperative align kernel with its scratch in library-owned device
// memory instead of a caller workspace.
// ----------------------------------------------------------------------------------
constexpr int kNoAllocMaxExperts = FR_ALIGN_NOALLOC_MAX_EXPERTS;
constexpr size_t kNoAllocScratchBytes = 256 + static_cast<size_t>(256) * kNoAllocMaxExperts * sizeof(int32_t);

// Barrier words + per-block histograms for up to kNoAllocMaxExperts experts.  Every GPU that
// loads the library holds these 262,400 bytes (256.25 KB) until the process exits.
static __device__ __align__(256) unsigned char g_align_noalloc_scratch[kNoAllocScratchBytes];

// In host code the array's name is only a handle; the device address comes from
// cudaGetSymbolAddress, looked up once per device with that device current.  The table is
// read and filled from any host thread (two threads that race on the first call both store
// the same address).  The look-up is refused while the stream is being captured: the first
// call on a device belongs before any capture.
static int noalloc_scratch_ptr(void** out, cudaStream_t st) {
  constexpr int kMaxDevices = 64;
  static std::atomic<void*> cached[kMaxDevices];
  int dev = 0;
  FR_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return FR_ERR_UNSUPPORTED;
  void* ptr = cached[dev].load(std::memory_order_acquire);
  if (!ptr) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    FR_CUDA_OK(cudaStreamIsCapturing(st, &cap));
    if (cap != cudaStreamCaptureStatusNone) return FR_ERR_UNSUPPORTED;
    FR_CUDA_OK(cudaGetSymbolAddress(&ptr, g_align_noalloc_scratch));
    if (!ptr) return FR_ERR_DRIVER;
    cached[dev].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return FR_OK;
}

int align_noalloc_dispatch(const int32_t* topk_ids, int64_t n, int E, int bs, int32_t* sorted_ids,
                           int64_t sorted_len, int32_t* expert_ids, int64_t expert_ids_len, int32_t* num_post,
                           int32_t* counts, int32_t* inv_pos, cudaStream_t st) {
  if (!topk_ids || !sorted_ids || !expert_ids || !num_post || n < 1 || E <= 0 || bs <= 0) return FR_ERR_ARG;
  if (E > kNoAllocMaxExperts) return FR_ERR_UNSUPPORTED;                      // beyond the built-in scratch
  const DeviceInfo& di = device_info();
  if (n > static_cast<int64_t>(di.sm_count < 256 ? di.sm_count : 256) * kCoopMaxPerBlock) return FR_ERR_UNSUPPORTED;
  if (sorted_len < n + static_cast<int64_t>(E) * (bs - 1)) return FR_ERR_ARG;
  if (expert_ids_len < (n + static_cast<int64_t>(E) * (bs - 1)) / bs) return FR_ERR_ARG;
  void* scratch = nullptr;
  const int rc = noalloc_scratch_ptr(&scratch, st);
  if (rc) return rc;
  // The array keeps whatever the previous call left.  Only its first 16 bytes must start at
  // zero: the two barrier words (a call that ended in a reported timeout could have left a
  // count behind) and the wait-budget word; the histogram rows are fully rewritten before
  // they are read.
  FR_CUDA_OK(cudaMemsetAsync(scratch, 0, 16, st));
  return align_coop_dispatch(topk_ids, n, E, bs, sorted_ids, sorted_len, expert_ids, expert_ids_len, num_post,
                             counts, inv_pos, scratch, kNoAllocScratchBytes, st, /*min_n=*/1);
}

}  // namespace fr
