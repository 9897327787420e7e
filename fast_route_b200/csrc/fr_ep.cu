// Expert parallelism over peer memory with no host in the loop.
//
// The reference layer (fast_route/fast_route/layers/stable_route.py:10-102) is single-GPU; this is its
// sharded form: rank r of W owns experts [r*E/W, (r+1)*E/W) and brings its own tokens.  Every rank keeps, in
// a region all GPUs of the node can read (same layout on every rank):
//     x[rows, H]          its tokens
//     sorted[n]           its assignments ordered by expert (align with block size 1: no padding)
//     tw[n]               its routing weights, by flat assignment id
//     y[y_rows, H]        the results of ITS experts, in expert-sorted order
// plus, after one all-gather of E integers per rank, the table counts[W][E] (tokens of rank s for expert e).
// From that table alone every rank derives, with the same arithmetic,
//   * as expert owner: where each (local expert j, source rank s) segment starts in its expert-sorted
//     operand (experts padded to 128 rows, sources in rank order inside an expert) and where the segment
//     starts in the source's sorted list;
//   * as token owner: in which row of the owner's y each of its assignments ends up.
// So no sizes travel to the host, no send / receive buffers exist and no position list comes back: the gather
// kernel pulls token rows straight from their owners (16-byte peer loads over NVLink) while it builds the GEMM
// operand, and the combine kernel pulls the k result rows of a token straight from the experts' owners.
// Peer memory is only touched by plain loads in these two kernels (no TMA, no multicast, no multimem).
#include "fr_common.cuh"

namespace fr {

constexpr int kEpMaxExperts = 1024;
constexpr int kEpBlock = FR_GEMM_BLOCK_M;

enum : unsigned int { ST_EP_CAPACITY = 4 };   // more rows arrived than the receive capacity holds

struct EpPlanParams {
  const int32_t* counts;  // [W][E]
  int W, E, El, rank;
  int64_t cap_rows;       // capacity of the expert-sorted buffers, multiple of 128
  int32_t* seg_start;     // [El*W + 1] first operand row of segment (j, s); the last entry is num_post
  int32_t* seg_count;     // [El*W]
  int32_t* seg_src_off;   // [El*W] first entry of the segment in source s's sorted list
  int32_t* comb_base;     // [E] row in the owner's y of this rank's first assignment to expert e, minus the
                          //     position of that assignment in this rank's sorted list
  int32_t* num_post;      // [1]
  int32_t* expert_ids;    // [cap_rows / 128] local expert of every 128-row block
};

// One block.  E <= 1024, so every table fits in shared memory and the serial scans are a few hundred adds.
__global__ void __launch_bounds__(256) ep_plan_kernel(const EpPlanParams p) {
  __shared__ int tot[kEpMaxExperts];      // tokens per expert over all ranks
  __shared__ int start[kEpMaxExperts];    // padded start of expert e in its owner's operand
  __shared__ int below[kEpMaxExperts];    // tokens for expert e from ranks below this one
  __shared__ int selfpre[kEpMaxExperts];  // position of expert e's first entry in this rank's sorted list
  __shared__ int s_num_post;
  const int W = p.W, E = p.E, El = p.El;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0, b = 0;
    for (int s = 0; s < W; ++s) {
      int c = __ldg(p.counts + s * E + e);
      if (c < 0) c = 0;
      t += c;
      if (s < p.rank) b += c;
    }
    tot[e] = t;
    below[e] = b;
  }
  __syncthreads();
  for (int o = threadIdx.x; o < W; o += blockDim.x) {   // one owner per thread: padded starts of its experts
    int run = 0;
    for (int j = 0; j < El; ++j) {
      start[o * El + j] = run;
      run += (tot[o * El + j] + kEpBlock - 1) / kEpBlock * kEpBlock;
    }
    if (o == p.rank) s_num_post = run;
  }
  if (threadIdx.x == blockDim.x - 1) {                  // this rank's own sorted list
    int run = 0;
    for (int e = 0; e < E; ++e) {
      selfpre[e] = run;
      int c = __ldg(p.counts + p.rank * E + e);
      run += c < 0 ? 0 : c;
    }
  }
  __syncthreads();
  int num_post = s_num_post;
  if (num_post > p.cap_rows) {
    if (threadIdx.x == 0) report(ST_EP_CAPACITY, static_cast<unsigned int>(num_post));
    num_post = static_cast<int>(p.cap_rows);
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) p.comb_base[e] = start[e] + below[e] - selfpre[e];
  const int lo = p.rank * El;
  for (int i = threadIdx.x; i < El * W; i += blockDim.x) {
    const int j = i / W, s = i - j * W;
    int st = start[lo + j], off = 0;
    for (int s2 = 0; s2 < s; ++s2) {
      const int c = __ldg(p.counts + s2 * E + lo + j);
      st += c < 0 ? 0 : c;
    }
    for (int e = 0; e < lo + j; ++e) {
      const int c = __ldg(p.counts + s * E + e);
      off += c < 0 ? 0 : c;
    }
    int c = __ldg(p.counts + s * E + lo + j);
    if (c < 0) c = 0;
    if (st > num_post) st = num_post;            // beyond the capacity: the segment is dropped (and reported)
    if (st + c > num_post) c = num_post - st;
    p.seg_start[i] = st;
    p.seg_count[i] = c;
    p.seg_src_off[i] = off;
  }
  if (threadIdx.x == 0) {
    p.seg_start[El * W] = num_post;
    *p.num_post = num_post;
  }
  for (int j = 0; j < El; ++j) {
    const int b0 = start[lo + j] / kEpBlock;
    const int b1 = min(num_post, start[lo + j] + (tot[lo + j] + kEpBlock - 1) / kEpBlock * kEpBlock) / kEpBlock;
    for (int b = b0 + threadIdx.x; b < b1; b += blockDim.x) p.expert_ids[b] = j;
  }
}

struct EpGatherParams {
  const uint8_t* const* peer_base;   // [W] base of every rank's region
  int64_t x_off, sorted_off, tw_off; // byte offsets inside a region
  int64_t ld_x_v;                    // row pitch of x in 16-byte vectors
  int64_t peer_rows, n_per_rank;
  int W, El, topk, row_v;
  const int32_t* seg_start;
  const int32_t* seg_count;
  const int32_t* seg_src_off;
  const int32_t* num_post;
  uint4* a_sorted;                   // [cap_rows, H]
  int64_t ld_a_v;
  float* w_sorted;                   // [cap_rows] routing weight of the row (0 for padding)
  int32_t* sorted_local;             // [cap_rows] row index for real rows, cap_rows for padding
  int64_t cap_rows;
};

// a_sorted[p,:] = x of the rank that owns the token of operand row p, read over NVLink.  Blocks stride over
// the rows in use (the row count is only known on the device).
__global__ void __launch_bounds__(256) ep_gather_kernel(const EpGatherParams p) {
  extern __shared__ int seg_sm[];    // seg_start[nseg + 1]
  const int nseg = p.El * p.W;
  for (int i = threadIdx.x; i <= nseg; i += blockDim.x) seg_sm[i] = __ldg(p.seg_start + i);
  __syncthreads();
  const int num_post = seg_sm[nseg];
  // Which source rank a row comes from and which of its assignments it is: a search in the segment table and one
  // load from the source's sorted list.  Returns false for a padding row.
  auto lookup = [&](int64_t row, int& s, int32_t& sid) -> bool {
    int lo = 0, hi = nseg - 1;   // last segment whose start is <= row (empty segments share their start with the next)
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (seg_sm[mid] <= row) lo = mid; else hi = mid - 1;
    }
    const int off = static_cast<int>(row) - seg_sm[lo];
    if (off >= __ldg(p.seg_count + lo)) return false;
    s = lo % p.W;
    const int64_t q = static_cast<int64_t>(__ldg(p.seg_src_off + lo)) + off;
    if (q < 0 || q >= p.n_per_rank) {
      sid = -1;
      return true;
    }
    sid = reinterpret_cast<const int32_t*>(p.peer_base[s] + p.sorted_off)[q];
    return true;
  };
  int64_t row = blockIdx.x;
  int s_cur = 0, s_nxt = 0;
  int32_t sid_cur = -1, sid_nxt = -1;
  bool real_cur = row < num_post && lookup(row, s_cur, sid_cur);
  for (; row < num_post; row += gridDim.x) {
    // the next row's look-up (a trip over NVLink) is issued now and consumed in the next iteration
    const int64_t nrow = row + gridDim.x;
    const bool real_nxt = nrow < num_post && lookup(nrow, s_nxt, sid_nxt);
    bool ok = real_cur && sid_cur >= 0 && sid_cur < p.n_per_rank;
    const int token = ok ? sid_cur / p.topk : 0;
    ok = ok && token < p.peer_rows;
    if (real_cur && !ok && threadIdx.x == 0) report(ST_BAD_SORTED_ID, static_cast<unsigned int>(row));
    uint4* d = p.a_sorted + row * p.ld_a_v;
    if (ok) {
      const uint8_t* base = p.peer_base[s_cur];
      const uint4* src = reinterpret_cast<const uint4*>(base + p.x_off) + static_cast<int64_t>(token) * p.ld_x_v;
      float w = 0.0f;
      if (threadIdx.x == 0) w = reinterpret_cast<const float*>(base + p.tw_off)[sid_cur];   // in flight with the row
      // a row crosses NVLink with a latency of microseconds: keep four 16-byte loads per thread in flight
      for (int v0 = threadIdx.x; v0 < p.row_v; v0 += 4 * blockDim.x) {
        uint4 t[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = v0 + u * static_cast<int>(blockDim.x);
          if (v < p.row_v) t[u] = src[v];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = v0 + u * static_cast<int>(blockDim.x);
          if (v < p.row_v) d[v] = t[u];
        }
      }
      if (threadIdx.x == 0) {
        p.w_sorted[row] = w;
        p.sorted_local[row] = static_cast<int32_t>(row);
      }
    } else {
      for (int v = threadIdx.x; v < p.row_v; v += blockDim.x) d[v] = make_uint4(0, 0, 0, 0);
      if (threadIdx.x == 0) {
        p.w_sorted[row] = 0.0f;
        p.sorted_local[row] = static_cast<int32_t>(p.cap_rows);
      }
    }
    real_cur = real_nxt;
    s_cur = s_nxt;
    sid_cur = sid_nxt;
  }
}

// out[t,:] = sum_j y of the owner of expert ids[t,j], row comb_base[e] + inv_pos[t*k+j]; fp32, slot order.
template <bool BF16>
__global__ void __launch_bounds__(256) ep_combine_kernel(const uint8_t* const* __restrict__ peer_base, int64_t y_off,
                                                         int64_t ld_y_v, int64_t y_rows, int W, int El, int E,
                                                         const int32_t* __restrict__ ids,
                                                         const int32_t* __restrict__ inv_pos,
                                                         const int32_t* __restrict__ comb_base, int topk, int row_v,
                                                         uint4* __restrict__ out, int64_t ld_out_v) {
  const int64_t t = blockIdx.x;
  for (int v = threadIdx.x; v < row_v; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    for (int j = 0; j < topk; ++j) {
      const int e = __ldg(ids + t * topk + j);
      const int q = __ldg(inv_pos + t * topk + j);
      if (e < 0 || e >= E || q < 0) continue;
      const int64_t pos = static_cast<int64_t>(__ldg(comb_base + e)) + q;
      if (pos < 0 || pos >= y_rows) continue;
      const uint4* y = reinterpret_cast<const uint4*>(peer_base[e / El] + y_off);
      const uint4 raw = y[pos * ld_y_v + v];
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

}  // namespace fr
