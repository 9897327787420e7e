// W4A16 split-K GEMM for small batches:  c[m,n] = a[m,k] . dequant(qweight)[k,n],  fp16 activations, 4-bit
// GPTQ-packed weights with per-group fp16 scales and packed 4-bit zero points, fp32 accumulation, fp16 output.
// Stands in for matmul_split_k / hint_kernel of the reference (benchmarks/splitk_gemm/splitk.py:26-103, 178-216):
//   qweight[k/8, n] int32, nibble j of word [kk, n] is row k = 8*kk + j;   scales[k/g, n] fp16;
//   qzeros[k/g, n/8] int32, nibble j of word [gi, nn] belongs to column n = 8*nn + j;
//   w[k,n] = fp16(q) * s  -  fp16(z + 1) * s,  every operation rounded to fp16 (:83-87).
//
// B200 mapping.  The packed weights are streamed once, so weights sit on the MMA M axis (128 output columns per
// CTA) and the few activation rows on the MMA N axis (16..128 per launch); a K step is 64 wide.
// The K steps of a CTA are dealt round-robin to four independent pipelines ("groups"), each with its own input
// stages, operand buffers, an fp32 accumulator in TMEM and its own barriers:
//   warp p (p = 0..3), one thread: TMA producer and MMA issuer of group p.  Loads the packed tile (8 words x 128
//              columns per step, 4 KB) and the activation tile (m_pad rows x 64, 128-byte swizzle) of the group's
//              steps, and issues tcgen05.mma (M=128, N=m_pad) on every operand the dequantisers hand over.
//   warps 4+4p .. 7+4p: the 128 dequantisers of group p.  Thread t owns output column n0+t and expands the 8 packed
//              words of a step into 64 fp16 weights.
// Two kernels share this frame:
//   w4a16_gemm_pair_kernel (up to 64 activation rows): the weights go from registers straight into lane t of a
//              tensor-memory buffer (tcgen05.st) and the MMA reads its A operand there; a group works on pairs of
//              consecutive K steps; the eight weights of a packed word come out with k interleaved (0, 4, 1, 5, 2, 6,
//              3, 7: one shift and four mask-or operations per word instead of four byte permutes) and a helper warp
//              per group (warps 20..23) gives the activation tile the same order in shared memory before the MMA
//              reads it (a sum over k does not care about the order).
//   w4a16_gemm_smem_kernel (65 to 128 rows, where the accumulators need the tensor-memory columns): the weights go
//              into row t of a K-major, 128-byte-swizzled shared-memory tile, natural k order, one K step at a time.
// A thread can issue a tcgen05.mma only every hundred cycles or so, whatever its shape, so one issuing thread per
// CTA was the bottleneck; four pipelines that never wait for one another hide it.  The dequantising warps drain the
// four accumulators at the end; warp 1 also allocates and frees TMEM.
// At these sizes the kernels are bound by instruction issue, most of it the bookkeeping of a pipeline turn (scale and zero
// point, addresses, barrier polls, fences, the arrive) rather than the expansion itself, not by HBM or the tensor pipe.
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
constexpr int W4_GROUPS = 4;               // dequantising groups of 128 threads, each with its own accumulator
constexpr int W4_WBUFS = 2;                // dequantised operand tiles per group
constexpr int W4_WSTAGES = W4_GROUPS * W4_WBUFS;
constexpr int W4_W_BYTES = W4_BN * W4_BK * 2;   // 16 KB
constexpr int W4_RAW_BYTES = 8 * W4_BN * 4;     // 4 KB of packed words
constexpr int W4_MAX_IN = 16;              // input ring depth (packed tile + activation tile)
constexpr int W4_SMEM_BUDGET = 224 * 1024;
constexpr int W4_MAX_M = 128;              // activation rows per launch (MMA N); larger batches run in chunks
constexpr int W4_HELPER_WARP0 = 4 + W4_GROUPS * 4;   // first of the four warps that reorder the activation tiles
constexpr int W4_THREADS = 128 + W4_GROUPS * 128 + W4_GROUPS * 32;
constexpr int W4_THREADS_SMEM = 128 + W4_GROUPS * 128;          // the shared-memory-operand kernel has no helper warps
constexpr int W4_ATMEM_MAX_M = 64;         // up to this many rows the dequantised operand lives in tensor memory


struct W4Params {
  const __half* scales;    // [k/g, n]
  const int32_t* qzeros;   // [k/g, n/8]
  __half* c;
  int64_t ldc;
  int m;                   // valid activation rows of this launch (<= m_pad)
  int m_pad;               // MMA N: multiple of 16, <= 128
  int n, k;
  int groupsize;           // multiple of 64 (a K step never straddles two groups)
  int in_stages;
  int x_bytes;             // m_pad * 128
  uint32_t tmem_cols;
};

// Scale-dependent constants of one (column, group) and the expansion of one packed word into eight fp16 weights
// w_j = q_j * s - zs, both operations rounded to fp16 and not fused with each other.
//
// Fast path (2^-9 <= |s| < 32).  Byte i of the word holds nibbles 2i and 2i+1.  Replicating the byte into both
// halves and masking with 0x00F0000F | 0x64006400 gives the fp16 pair (1024 + q_2i, 1024 + 16 * q_2i+1), exactly.
// One fused multiply-add per pair, fma(1024 + q, s, -1024 s) and fma(1024 + 16 q, s / 16, -64 s), evaluates
// q * s exactly and rounds it once, which is what fp16(q) * s does: s / 16, 1024 s and 64 s are exact in this
// range.  The pair comes out in memory order.
// Slow path (any other scale, zero and subnormal-prone ones included): integer nibbles -> fp16 -> multiply.
struct W4Group {
  __half2 s2, zs2, mul2, add2;
  __half2 s16_2, add1024_2, add64_2;
  bool fast;
  __device__ __forceinline__ void set(__half s, uint32_t z) {
    s2 = __half2half2(s);
    zs2 = __half2half2(__hmul_rn(__ushort2half_rn(static_cast<unsigned short>(z + 1)), s));
    const unsigned short mag = __half_as_ushort(s) & 0x7FFFu;
    fast = mag >= 0x1800u && mag < 0x5000u;
    const __half s16 = __hmul_rn(s, __ushort_as_half(0x2C00));          // s / 16
    const __half m1024 = __hneg(__hmul_rn(s, __ushort_as_half(0x6400)));     // -1024 s
    const __half m64 = __hneg(__hmul_rn(s, __ushort_as_half(0x5400)));       // -64 s
    mul2 = __halves2half2(s, s16);
    add2 = __halves2half2(m1024, m64);
    s16_2 = __half2half2(s16);
    add1024_2 = __half2half2(m1024);
    add64_2 = __half2half2(m64);
  }
  // eight weights in memory order k = 0 .. 7
  template <bool FAST>
  __device__ __forceinline__ uint4 expand(uint32_t v) const {
    uint32_t out[4];
    if constexpr (FAST) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t bits = (__byte_perm(v, 0u, 0x4040u | (i << 8) | i) & 0x00F0000Fu) | 0x64006400u;
        __half2 q = __hfma2(*reinterpret_cast<const __half2*>(&bits), mul2, add2);
        q = __hsub2_rn(q, zs2);
        out[i] = *reinterpret_cast<uint32_t*>(&q);
      }
    } else {
      const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t bits = 0x64006400u | ((v >> (8 * i)) & 0xFu) | (((v >> (8 * i + 4)) & 0xFu) << 16);
        __half2 q = __hmul2_rn(__hsub2_rn(*reinterpret_cast<const __half2*>(&bits), k1024), s2);
        q = __hsub2_rn(q, zs2);
        out[i] = *reinterpret_cast<uint32_t*>(&q);
      }
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
  }
  // The same eight weights in the order k = 0, 4, 1, 5, 2, 6, 3, 7: nibbles j and j + 4 sit 16 bits apart in the
  // word, so a mask alone puts them into the two mantissas (nibbles 1, 3, 5, 7 land four bits up: 1024 + 16 q).
  // One shift and four mask-or operations per word instead of four byte permutes and four mask-ors; the GEMM
  // permutes the activation tile the same way, and a sum over k does not care about the order.
  template <bool FAST>
  __device__ __forceinline__ uint4 expand_interleaved(uint32_t v) const {
    uint32_t out[4];
    if constexpr (FAST) {
      const uint32_t v8 = v >> 8;
      const uint32_t b0 = (v & 0x000F000Fu) | 0x64006400u;      // 1024 + (q0, q4)
      const uint32_t b1 = (v & 0x00F000F0u) | 0x64006400u;      // 1024 + 16 (q1, q5)
      const uint32_t b2 = (v8 & 0x000F000Fu) | 0x64006400u;     // 1024 + (q2, q6)
      const uint32_t b3 = (v8 & 0x00F000F0u) | 0x64006400u;     // 1024 + 16 (q3, q7)
      __half2 q0 = __hsub2_rn(__hfma2(*reinterpret_cast<const __half2*>(&b0), s2, add1024_2), zs2);
      __half2 q1 = __hsub2_rn(__hfma2(*reinterpret_cast<const __half2*>(&b1), s16_2, add64_2), zs2);
      __half2 q2 = __hsub2_rn(__hfma2(*reinterpret_cast<const __half2*>(&b2), s2, add1024_2), zs2);
      __half2 q3 = __hsub2_rn(__hfma2(*reinterpret_cast<const __half2*>(&b3), s16_2, add64_2), zs2);
      out[0] = *reinterpret_cast<uint32_t*>(&q0);
      out[1] = *reinterpret_cast<uint32_t*>(&q1);
      out[2] = *reinterpret_cast<uint32_t*>(&q2);
      out[3] = *reinterpret_cast<uint32_t*>(&q3);
    } else {
      const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t bits = 0x64006400u | ((v >> (4 * i)) & 0xFu) | (((v >> (4 * i + 16)) & 0xFu) << 16);
        __half2 q = __hmul2_rn(__hsub2_rn(*reinterpret_cast<const __half2*>(&bits), k1024), s2);
        q = __hsub2_rn(q, zs2);
        out[i] = *reinterpret_cast<uint32_t*>(&q);
      }
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
  }
  __device__ __forceinline__ uint4 expand_any(uint32_t v) const { return fast ? expand<true>(v) : expand<false>(v); }
};

// Batches of more than 64 rows (the accumulators then need the tensor-memory columns): the dequantised operand goes
// through shared memory, one K step at a time, weights in natural k order.
__global__ void __launch_bounds__(W4_THREADS_SMEM, 1)
w4a16_gemm_smem_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmX, const W4Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // layout: [W ring][X ring][packed ring][barriers]; the front of it doubles as the fp32 partial tile at the end
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
  const int in_stages = p.in_stages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < W4_MAX_IN; ++s) {
      mbar_init(&in_full[s], 1);
      mbar_init(&in_empty[s], 1);
    }
    for (int s = 0; s < W4_WSTAGES; ++s) {
      mbar_init(&w_full[s], 4);      // the four warps of the owning group
      mbar_init(&w_empty[s], 1);
    }
    mbar_init(tfull, W4_GROUPS);     // one arrival per group, after its last MMA
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

  // Step i of the CTA belongs to group i % 4; its input stage is i % in_stages.  in_stages is a multiple of four, so
  // a group always meets the same stages: own step j (i = grp + 4 j) uses stage grp + 4 * (j % spg).
  const int spg = in_stages / W4_GROUPS;           // input stages per group

  if (warp < W4_GROUPS) {
    // ---------------- per group: TMA producer + MMA issuer (one thread) ----------------
    if (lane == 0) {
      const int grp_id = warp;
      const int own = nkb > grp_id ? (nkb - grp_id + W4_GROUPS - 1) / W4_GROUPS : 0;   // steps of this group
      uint64_t* my_w_full = w_full + grp_id * W4_WBUFS;
      uint64_t* my_w_empty = w_empty + grp_id * W4_WBUFS;
      const uint32_t idesc = umma_idesc_f16(false, W4_BN, p.m_pad);
      const uint32_t d_tmem = tmem_base + grp_id * p.m_pad;       // the group's own accumulator
      auto load = [&](int j) {           // own step j -> its stage (the caller has made sure the stage is free)
        const int st = grp_id + W4_GROUPS * (j % spg);
        const int kb = kb_begin + grp_id + W4_GROUPS * j;
        mbar_expect_tx(&in_full[st], W4_RAW_BYTES + p.x_bytes);
        // the packed matrix is addressed as 16-bit elements: column 2*n, row k/8
        tma_load_2d(sQ + st * W4_RAW_BYTES, &tmQ, &in_full[st], 2 * n0, kb * (W4_BK / 8));
        tma_load_2d(sX + st * p.x_bytes, &tmX, &in_full[st], kb * W4_BK, 0);
      };
      const int pre = own < spg ? own : spg;
      for (int j = 0; j < pre; ++j) load(j);
      bool ok = true;
      for (int j = 0; j < own && ok; ++j) {
        // refill the stage of the previous own step first (its MMAs were issued a whole step ago)
        if (j >= 1 && j - 1 + spg < own) {
          const int pst = grp_id + W4_GROUPS * ((j - 1) % spg);
          if (!wait_or_abort(&in_empty[pst], static_cast<uint32_t>((j - 1) / spg) & 1u, abort_flag, 0x800)) {
            ok = false;
            break;
          }
          load(j - 1 + spg);
        }
        const int buf = j % W4_WBUFS;
        const int st = grp_id + W4_GROUPS * (j % spg);
        // the dequantisers waited for this step's input stage before they wrote the operand tile
        if (!wait_or_abort(&my_w_full[buf], static_cast<uint32_t>(j / W4_WBUFS) & 1u, abort_flag, 0x811)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t bdesc = umma_desc_sw128(smem_u32(sX + st * p.x_bytes));
        const uint64_t adesc = umma_desc_sw128(smem_u32(sW + (grp_id * W4_WBUFS + buf) * W4_W_BYTES));
#pragma unroll
        for (int kk = 0; kk < W4_BK / 16; ++kk)
          tc_mma_f16(d_tmem, adesc + 2 * kk, bdesc + 2 * kk, idesc, (j > 0 || kk > 0) ? 1u : 0u);
        tc_commit(&my_w_empty[buf]);
        tc_commit(&in_empty[st]);
      }
      // all of the group's MMAs (none, for a group without steps) are complete when this arrives
      if (ok && own > 0) tc_commit(tfull);
      else mbar_arrive(tfull);
    }
  } else {
    // ---------------- dequantise, then drain ----------------
    const int t = (threadIdx.x - 128) & 127;        // output column n0 + t, TMEM lane t
    const int grp_id = (threadIdx.x - 128) >> 7;    // owns steps grp_id, grp_id + 4, ...
    const int n = n0 + t;
    const bool n_ok = n < p.n;
    // byte offset of row t in a swizzled operand tile; the 16-byte chunk index is XORed with (t & 7)
    const uint32_t row_off = static_cast<uint32_t>(t >> 3) * 1024u + static_cast<uint32_t>(t & 7) * 128u;
    uint8_t* w_base = sW + grp_id * (W4_WBUFS * W4_W_BYTES);
    uint64_t* my_w_full = w_full + grp_id * W4_WBUFS;
    uint64_t* my_w_empty = w_empty + grp_id * W4_WBUFS;
    const __half* sp = p.scales + n;
    const int32_t* zp = p.qzeros + (n >> 3);
    const int zshift = (n & 7) * 4;
    // scale and zero point of the group's next step are loaded while it works on the current one
    // (the quantisation group of a step advances by 4 / kpg, plus a carry, per own step: no division in the loop)
    __half s_next = __ushort_as_half(0);
    uint32_t z_next = 0;
    const int kpg = p.groupsize / W4_BK;              // K steps per quantisation group
    const int g_adv = W4_GROUPS / kpg, g_rem_adv = W4_GROUPS % kpg;
    int g_rem = 0;
    if (grp_id < nkb) {
      const int g0 = (kb_begin + grp_id) / kpg;
      g_rem = (kb_begin + grp_id) % kpg;
      sp += static_cast<int64_t>(g0) * p.n;
      zp += static_cast<int64_t>(g0) * (p.n >> 3);
      if (n_ok) {
        s_next = __ldg(sp);
        z_next = static_cast<uint32_t>(__ldg(zp));
      }
    }
    bool ok = true;
    int st = grp_id;
    uint32_t in_ph = 0, buf = 0, w_ph = 0;
    for (int i = grp_id; i < nkb; i += W4_GROUPS) {
      W4Group grp;
      grp.set(s_next, (z_next >> zshift) & 0xFu);
      if (i + W4_GROUPS < nkb) {
        g_rem += g_rem_adv;
        const int carry = g_rem >= kpg ? 1 : 0;
        g_rem -= carry ? kpg : 0;
        sp += (g_adv + carry) * p.n;
        zp += (g_adv + carry) * (p.n >> 3);
        if (n_ok) {
          s_next = __ldg(sp);
          z_next = static_cast<uint32_t>(__ldg(zp));
        }
      }
      // The operand buffer is free once the group's MMAs of two steps ago are complete, and the packed tile has
      // usually landed: ask both barriers at once and only fall back to the bounded waits if one is not there yet.
      {
        const bool r1 = mbar_try_wait(&my_w_empty[buf], w_ph ^ 1), r2 = mbar_try_wait(&in_full[st], in_ph);
        if (!(r1 && r2)) {
          if (!wait_or_abort(&my_w_empty[buf], w_ph ^ 1, abort_flag, 0x821) ||
              !wait_or_abort(&in_full[st], in_ph, abort_flag, 0x820)) {
            ok = false;
            break;
          }
        }
      }
      const uint32_t* q = reinterpret_cast<const uint32_t*>(sQ + st * W4_RAW_BYTES) + t;
      uint32_t words[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) words[j] = q[j * W4_BN];
      // row t of the operand tile; chunk j goes to position j ^ (t & 7): one XOR on the shared-memory address
      const uint32_t wrow = smem_u32(w_base + buf * W4_W_BYTES + row_off) ^ (static_cast<uint32_t>(t & 7) << 4);
      if (grp.fast) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 w8 = grp.expand<true>(words[j]);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(wrow ^ (j << 4)), "r"(w8.x), "r"(w8.y),
                       "r"(w8.z), "r"(w8.w) : "memory");
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 w8 = grp.expand<false>(words[j]);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(wrow ^ (j << 4)), "r"(w8.x), "r"(w8.y),
                       "r"(w8.z), "r"(w8.w) : "memory");
        }
      }
      // make the generic-proxy writes visible to the tensor core (async proxy) before signalling
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&my_w_full[buf]);
      st += W4_GROUPS;
      if (st >= in_stages) {
        st -= in_stages;
        in_ph ^= 1;
      }
      if (++buf == W4_WBUFS) {
        buf = 0;
        w_ph ^= 1;
      }
    }

    // partial tile -> this CTA's shared memory as fp32 [m_pad][128] (column t contiguous across lanes);
    // the four groups take 16-row chunks in turn and add the groups' accumulators in a fixed order
    float* partial = reinterpret_cast<float*>(sW);
    ok = wait_or_abort(tfull, 0, abort_flag, 0x830) && (*abort_flag == 0);
    tc_fence_after();
    // (every group's MMAs are complete once tfull completes, so the operand tiles may be overwritten)
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const int used = nkb < W4_GROUPS ? nkb : W4_GROUPS;
    for (int c0 = grp_id * 16; c0 < p.m_pad; c0 += W4_GROUPS * 16) {
      float acc[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
      if (ok) {
        for (int a = 0; a < used; ++a) {
          uint32_t raw[16];
          tmem_ld16(taddr + a * p.m_pad + c0, raw);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = (a == 0) ? __uint_as_float(raw[i]) : __fadd_rn(acc[i], __uint_as_float(raw[i]));
        }
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) partial[(c0 + i) * W4_BN + t] = acc[i];
    }
  }

  // every CTA of the cluster has parked its partial tile
  tc_fence_before();
  __syncthreads();
  cluster.sync();

  if (warp >= 4) {
    const int t = (threadIdx.x - 128) & 127;
    const int grp_id = (threadIdx.x - 128) >> 7;
    const int n = n0 + t;
    if (n < p.n) {
      for (int row = rank + grp_id * S; row < p.m; row += W4_GROUPS * S) {
        // all remote loads in flight together (one trip through the cluster network instead of S), then the
        // sum in rank order
        float v[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          v[r] = 0.0f;
          if (r < S) v[r] = cluster.map_shared_rank(reinterpret_cast<float*>(sW), r)[row * W4_BN + t];
        }
        float acc = v[0];
#pragma unroll
        for (int r = 1; r < 8; ++r)
          if (r < S) acc = __fadd_rn(acc, v[r]);
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

// ----------------------------------------------------------------------------------------------------------------
// Batches of up to 64 rows: the same four pipelines, but a pipeline takes its K steps in PAIRS (128 of K at a time).
// A dequantising warp issues about 350 instructions per 64-wide step of which only about 110 expand weights; the rest
// is the step's bookkeeping (scale and zero point, addresses, barrier polls, fences, the arrive).  With two steps per
// turn that bookkeeping is paid once per 16 packed words: one scale / zero point when the quantisation group covers
// both steps, one pair of barrier polls, one tcgen05.wait::st, one arrive, and the issuing thread wakes once for eight
// MMAs.  The two operand buffers of a group (32 columns each, adjacent) then hold the two halves of one pair, so a
// group's dequantisers expand the first half of the next pair in registers while the MMAs of the current one run and
// store it once those are complete.
// K steps of the CTA: pair q covers steps 2q and 2q + 1; pair q belongs to group q % 4; its input stage is
// q % in_stages (in_stages is a multiple of four, counted in pairs).
// ----------------------------------------------------------------------------------------------------------------
constexpr int W4P_STAGE_RAW = 2 * W4_RAW_BYTES;       // packed words of a pair: 16 rows x 128 columns, 8 KB

// Eight consecutive k of one activation row (a 16-byte chunk, wherever the swizzle put it) into the order the
// weights are expanded in: k = 0, 4, 1, 5, 2, 6, 3, 7.
__device__ __forceinline__ void permute_chunk(uint4* px) {
  const uint4 x = *px;
  *px = make_uint4(__byte_perm(x.x, x.z, 0x5410), __byte_perm(x.x, x.z, 0x7632), __byte_perm(x.y, x.w, 0x5410),
                   __byte_perm(x.y, x.w, 0x7632));
}

__global__ void __launch_bounds__(W4_THREADS, 1)
w4a16_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmX,
                       const W4Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // layout: [X ring: two 64-wide tiles per stage][packed ring][barriers]; the front doubles as the fp32 partial tile
  const int xs_bytes = 2 * p.x_bytes;
  uint8_t* sX = smem;
  uint8_t* sQ = sX + p.in_stages * xs_bytes;
  uint64_t* in_full = reinterpret_cast<uint64_t*>(sQ + p.in_stages * W4P_STAGE_RAW);
  uint64_t* in_empty = in_full + W4_MAX_IN;
  uint64_t* w_full = in_empty + W4_MAX_IN;         // [group]
  uint64_t* w_empty = w_full + W4_GROUPS;          // [group]
  uint64_t* tfull = w_empty + W4_GROUPS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  cgx::cluster_group cluster = cgx::this_cluster();
  const int S = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * W4_BN;

  // this CTA's K steps; a slice starts on an even step, so that pairs never straddle two CTAs
  const int KB = p.k / W4_BK;
  const int per = ((KB + S - 1) / S + 1) & ~1;
  const int kb_begin = min(KB, rank * per);
  const int kb_end = min(KB, kb_begin + per);
  const int nkb = kb_end - kb_begin;
  const int npairs = (nkb + 1) / 2;
  const int in_stages = p.in_stages;
  const int spg = in_stages / W4_GROUPS;           // input stages per group

  if (threadIdx.x == 0) {
    for (int s = 0; s < W4_MAX_IN; ++s) {
      mbar_init(&in_full[s], 1);
      mbar_init(&in_empty[s], 1);
    }
    for (int g = 0; g < W4_GROUPS; ++g) {
      mbar_init(&w_full[g], 5);      // the four warps of the group and its helper warp
      mbar_init(&w_empty[g], 1);
    }
    mbar_init(tfull, W4_GROUPS);     // one arrival per group, after its last MMA
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmX);
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // columns [0, 4 m_pad): the groups' accumulators; [256, 512): the groups' operand buffers, 64 columns each

  if (warp < W4_GROUPS) {
    // ---------------- per group: TMA producer + MMA issuer (one thread) ----------------
    if (lane == 0) {
      const int grp_id = warp;
      const int own = npairs > grp_id ? (npairs - grp_id + W4_GROUPS - 1) / W4_GROUPS : 0;   // pairs of this group
      const uint32_t idesc = umma_idesc_f16(false, W4_BN, p.m_pad);
      const uint32_t d_tmem = tmem_base + grp_id * p.m_pad;
      const uint32_t a_tmem = tmem_base + 256 + grp_id * 64;
      auto load = [&](int j) {           // own pair j -> its stage (the caller has made sure the stage is free)
        const int st = grp_id + W4_GROUPS * (j % spg);
        const int kb = kb_begin + 2 * (grp_id + W4_GROUPS * j);
        mbar_expect_tx(&in_full[st], W4P_STAGE_RAW + xs_bytes);
        // the packed matrix is addressed as 16-bit elements: column 2*n, row k/8; steps past the end of K read zeros
        tma_load_2d(sQ + st * W4P_STAGE_RAW, &tmQ, &in_full[st], 2 * n0, kb * (W4_BK / 8));
        tma_load_2d(sQ + st * W4P_STAGE_RAW + W4_RAW_BYTES, &tmQ, &in_full[st], 2 * n0, (kb + 1) * (W4_BK / 8));
        tma_load_2d(sX + st * xs_bytes, &tmX, &in_full[st], kb * W4_BK, 0);
        tma_load_2d(sX + st * xs_bytes + p.x_bytes, &tmX, &in_full[st], (kb + 1) * W4_BK, 0);
      };
      const int pre = own < spg ? own : spg;
      for (int j = 0; j < pre; ++j) load(j);
      bool ok = true;
      for (int j = 0; j < own && ok; ++j) {
        // refill the stage of the previous own pair first (its MMAs were issued a whole pair ago)
        if (j >= 1 && j - 1 + spg < own) {
          const int pst = grp_id + W4_GROUPS * ((j - 1) % spg);
          if (!wait_or_abort(&in_empty[pst], static_cast<uint32_t>((j - 1) / spg) & 1u, abort_flag, 0x900)) {
            ok = false;
            break;
          }
          load(j - 1 + spg);
        }
        const int st = grp_id + W4_GROUPS * (j % spg);
        const int kb = kb_begin + 2 * (grp_id + W4_GROUPS * j);
        const int halves = kb + 1 < kb_end ? 2 : 1;
        if (!wait_or_abort(&w_full[grp_id], static_cast<uint32_t>(j) & 1u, abort_flag, 0x911)) {
          ok = false;
          break;
        }
        tc_fence_after();
        for (int h = 0; h < halves; ++h) {
          const uint64_t bdesc = umma_desc_sw128(smem_u32(sX + st * xs_bytes + h * p.x_bytes));
#pragma unroll
          for (int kk = 0; kk < W4_BK / 16; ++kk)
            tc_mma_f16_a_tmem(d_tmem, a_tmem + 32 * h + 8 * kk, bdesc + 2 * kk, idesc, (j > 0 || h > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&w_empty[grp_id]);
        tc_commit(&in_empty[st]);
      }
      // all of the group's MMAs (none, for a group without pairs) are complete when this arrives
      if (ok && own > 0) tc_commit(tfull);
      else mbar_arrive(tfull);
    }
  } else if (warp < W4_HELPER_WARP0) {
    // ---------------- dequantise, then drain ----------------
    const int t = (threadIdx.x - 128) & 127;        // output column n0 + t, TMEM lane t
    const int grp_id = (threadIdx.x - 128) >> 7;    // owns pairs grp_id, grp_id + 4, ...
    const int own = npairs > grp_id ? (npairs - grp_id + W4_GROUPS - 1) / W4_GROUPS : 0;
    const int n = n0 + t;
    const bool n_ok = n < p.n;
    const __half* sp = p.scales + n;
    const int32_t* zp = p.qzeros + (n >> 3);
    const int zshift = (n & 7) * 4;
    const int kpg = p.groupsize / W4_BK;            // K steps per quantisation group
    const bool one_group = (kpg & 1) == 0;          // a pair (an even step and its successor) lies in one group
    const int last_group = p.k / p.groupsize - 1;
    // scale and zero point of the pair's two steps; those of the next own pair are loaded while this one is expanded
    auto fetch = [&](int j, __half (&sv)[2], uint32_t (&zv)[2]) {
      const int kb = kb_begin + 2 * (grp_id + W4_GROUPS * j);
      const int g0 = kb / kpg;
      int g1 = (kb + 1) / kpg;
      g1 = g1 > last_group ? last_group : g1;       // a second step past the end of K multiplies zeros
      sv[0] = sv[1] = __ushort_as_half(0);
      zv[0] = zv[1] = 0;
      if (n_ok) {
        sv[0] = __ldg(sp + static_cast<int64_t>(g0) * p.n);
        zv[0] = static_cast<uint32_t>(__ldg(zp + static_cast<int64_t>(g0) * (p.n >> 3)));
        if (!one_group) {
          sv[1] = __ldg(sp + static_cast<int64_t>(g1) * p.n);
          zv[1] = static_cast<uint32_t>(__ldg(zp + static_cast<int64_t>(g1) * (p.n >> 3)));
        }
      }
    };
    const uint32_t a_tmem = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + 256 + grp_id * 64;
    auto expand_step = [&](const W4Group& grp, const uint32_t (&words)[8], uint32_t (&regs)[32]) {
      if (grp.fast) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint4 w8 = grp.expand_interleaved<true>(words[i]);
          regs[4 * i] = w8.x, regs[4 * i + 1] = w8.y, regs[4 * i + 2] = w8.z, regs[4 * i + 3] = w8.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint4 w8 = grp.expand_interleaved<false>(words[i]);
          regs[4 * i] = w8.x, regs[4 * i + 1] = w8.y, regs[4 * i + 2] = w8.z, regs[4 * i + 3] = w8.w;
        }
      }
    };
    bool ok = true;
    __half s_next[2];
    uint32_t z_next[2];
    s_next[0] = s_next[1] = __ushort_as_half(0);
    z_next[0] = z_next[1] = 0;
    if (own > 0) fetch(0, s_next, z_next);
    int st = grp_id;
    uint32_t in_ph = 0;
    for (int j = 0; j < own; ++j) {
      const int kb = kb_begin + 2 * (grp_id + W4_GROUPS * j);
      const bool two = kb + 1 < kb_end;
      W4Group grp_a, grp_b;
      grp_a.set(s_next[0], (z_next[0] >> zshift) & 0xFu);
      if (one_group) grp_b = grp_a;
      else grp_b.set(s_next[1], (z_next[1] >> zshift) & 0xFu);
      if (j + 1 < own) fetch(j + 1, s_next, z_next);
      if (!wait_or_abort(&in_full[st], in_ph, abort_flag, 0x920)) {
        ok = false;
        break;
      }
      const uint32_t* q = reinterpret_cast<const uint32_t*>(sQ + st * W4P_STAGE_RAW) + t;
      uint32_t words[8], regs[32];
#pragma unroll
      for (int i = 0; i < 8; ++i) words[i] = q[i * W4_BN];
      expand_step(grp_a, words, regs);            // in registers while the previous pair's MMAs still run
      if (two) {
#pragma unroll
        for (int i = 0; i < 8; ++i) words[i] = q[(8 + i) * W4_BN];
      }
      // the group's operand buffers are free once the MMAs of its previous pair are complete
      if (!wait_or_abort(&w_empty[grp_id], (static_cast<uint32_t>(j) & 1u) ^ 1u, abort_flag, 0x921)) {
        ok = false;
        break;
      }
      tc_fence_after();
      tmem_st32(a_tmem, regs);
      if (two) {
        expand_step(grp_b, words, regs);
        tmem_st32(a_tmem + 32, regs);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&w_full[grp_id]);
      st += W4_GROUPS;
      if (st >= in_stages) {
        st -= in_stages;
        in_ph ^= 1;
      }
    }

    // partial tile -> this CTA's shared memory as fp32 [m_pad][128] (column t contiguous across lanes);
    // the four groups take 16-row chunks in turn and add the groups' accumulators in a fixed order
    float* partial = reinterpret_cast<float*>(smem);
    ok = wait_or_abort(tfull, 0, abort_flag, 0x930) && (*abort_flag == 0);
    tc_fence_after();
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const int used = npairs < W4_GROUPS ? npairs : W4_GROUPS;
    for (int c0 = grp_id * 16; c0 < p.m_pad; c0 += W4_GROUPS * 16) {
      float acc[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
      if (ok) {
        for (int a = 0; a < used; ++a) {
          uint32_t raw[16];
          tmem_ld16(taddr + a * p.m_pad + c0, raw);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = (a == 0) ? __uint_as_float(raw[i]) : __fadd_rn(acc[i], __uint_as_float(raw[i]));
        }
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) partial[(c0 + i) * W4_BN + t] = acc[i];
    }
  } else {
    // ---------------- helper warp of a group: activation tiles into the weights' k order ----------------
    const int grp_id = warp - W4_HELPER_WARP0;
    int st = grp_id;
    uint32_t in_ph = 0;
    for (int q = grp_id, j = 0; q < npairs; q += W4_GROUPS, ++j) {
      // not ahead of the dequantisers: its arrival belongs to the same phase of w_full as theirs
      if (!wait_or_abort(&w_empty[grp_id], (static_cast<uint32_t>(j) & 1u) ^ 1u, abort_flag, 0x941)) break;
      if (!wait_or_abort(&in_full[st], in_ph, abort_flag, 0x940)) break;
      for (int ch = lane; ch < 2 * p.m_pad * 8; ch += 32) permute_chunk(reinterpret_cast<uint4*>(sX + st * xs_bytes) + ch);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&w_full[grp_id]);
      st += W4_GROUPS;
      if (st >= in_stages) {
        st -= in_stages;
        in_ph ^= 1;
      }
    }
  }

  // every CTA of the cluster has parked its partial tile
  tc_fence_before();
  __syncthreads();
  cluster.sync();

  if (warp >= 4 && warp < W4_HELPER_WARP0) {
    const int t = (threadIdx.x - 128) & 127;
    const int grp_id = (threadIdx.x - 128) >> 7;
    const int n = n0 + t;
    if (n < p.n) {
      for (int row = rank + grp_id * S; row < p.m; row += W4_GROUPS * S) {
        // all remote loads in flight together, then the sum in rank order
        float v[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          v[r] = 0.0f;
          if (r < S) v[r] = cluster.map_shared_rank(reinterpret_cast<float*>(smem), r)[row * W4_BN + t];
        }
        float acc = v[0];
#pragma unroll
        for (int r = 1; r < 8; ++r)
          if (r < S) acc = __fadd_rn(acc, v[r]);
        p.c[static_cast<int64_t>(row) * p.ldc + n] = __float2half_rn(acc);
      }
    }
  }
  // nobody leaves while another CTA may still read its shared memory
  cluster.sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
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
  W4Group grp;
  grp.set(s, z);
  const uint4 v = grp.expand_any(static_cast<uint32_t>(qweight[idx]));
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
  if ((n % 8) || (k % W4_BK) || (groupsize % 64) || (k % groupsize) || (lda % 8) || ldc < n) return FR_ERR_ALIGN;
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

  for (int64_t m0 = 0; m0 < m; m0 += W4_MAX_M) {
    const int mc = static_cast<int>(m - m0 < W4_MAX_M ? m - m0 : W4_MAX_M);
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
    const bool a_tmem = p.m_pad <= W4_ATMEM_MAX_M;
    auto kern = a_tmem ? w4a16_gemm_pair_kernel : w4a16_gemm_smem_kernel;
    // a pipeline stage: one K step (shared-memory operand) or a pair of them (tensor-memory operand)
    const int w_ring = a_tmem ? 0 : W4_WSTAGES * W4_W_BYTES;
    const int stage_bytes = (a_tmem ? 2 : 1) * (W4_RAW_BYTES + p.x_bytes);
    int stages = (W4_SMEM_BUDGET - w_ring) / stage_bytes;
    const int steps = (KB + S - 1) / S;
    const int units = a_tmem ? (steps + 2) / 2 : steps;
    if (stages > units) stages = units;
    if (stages > W4_MAX_IN) stages = W4_MAX_IN;
    // A multiple of the group count: the previous use of a stage then belongs to the same dequantising group,
    // which keeps every waiter within one phase of its barrier.
    p.in_stages = (stages + W4_GROUPS - 1) / W4_GROUPS * W4_GROUPS;
    if (stage_bytes * p.in_stages + w_ring > W4_SMEM_BUDGET) p.in_stages -= W4_GROUPS;
    if (p.in_stages < W4_GROUPS) return FR_ERR_UNSUPPORTED;
    uint32_t cols = 32;
    while (cols < static_cast<uint32_t>(p.m_pad * W4_GROUPS)) cols *= 2;
    p.tmem_cols = a_tmem ? 512u : cols;
    // the partial tile (m_pad x 128 fp32) reuses the front of the rings
    if (p.m_pad * W4_BN * 4 > w_ring + p.in_stages * stage_bytes) return FR_ERR_UNSUPPORTED;
    CUtensorMap tmX;
    rc = make_tmap_2d(&tmX, static_cast<const __half*>(a) + m0 * lda, static_cast<uint64_t>(mc),
                      static_cast<uint64_t>(k), static_cast<uint64_t>(lda), p.m_pad, 64, true);
    if (rc) return rc;
    const int smem = w_ring + p.in_stages * stage_bytes + 512 + 1024;
    FR_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles, S, 1);
    cfg.blockDim = dim3(a_tmem ? W4_THREADS : W4_THREADS_SMEM);
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
