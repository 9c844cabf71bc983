// out[m, N] = x[m, K] . W[N, K]^T for 1..16 tokens per CTA against a BF16 (or, for the router, FP32)
// weight, as a persistent streaming walk over the weight with register-level tensor-core MMAs
// (mma.sync m16n8k16): the latency-bound
// regime between the one-token GEMV and the TMEM kernel, where allocating tensor memory, building a
// shared-memory pipeline and reducing split-K partials across a cluster cost more than they save.
// Extends the reference's m = 1 GEMV (bf16_proj/gemv1.cu:27-125) to the smallest of the m <= 32 calls
// that its swap-AB kernel serves (_swab_kernel, best_submissions/muse_bf16_proj.py:236-257).
//
// A persistent grid of CTAs of NW warps. x (m rows, padded by 64 bytes so that the 8 tokens of a fragment
// fall in different banks) is brought into shared memory once by bulk copies. The CTA then takes
// groups of 8 weight rows (one contiguous 8 x K block of W) round robin; the NW warps split K, each
// lane streaming 16-byte pieces of W straight from global memory into the B fragments of two MMAs:
// lane (g, q) loads W[row0 + g][kb + 8q .. kb + 8q + 7]. The MMA's k slots are a permutation of those
// eight elements, and the same permutation is applied to x (the A fragment is the 16 bytes of
// x[token g] at the same offset), so the dot products are unchanged. Tokens are the MMA's M (16),
// weight rows its N (8). Warps reduce through shared memory in a fixed order (deterministic).
//
// When one batch of the CTA's loads covers a whole row (K <= 32 * NW * U), every warp meets the same
// pieces of K in every group, so its A fragments never change: fewtok_xreg_kernel loads them once from
// global memory into registers and runs with no shared-memory copy of x at all. Tokens 8..15 double
// those registers, which a 32-warp CTA only has for U <= 2; 16 warps x 8 loads serve K = 4096 there.
// That kernel also runs column-parallel (self-validating lines into the peers' staging) and as several
// interleaved walks over disjoint token blocks; fewtok_xreg_f32_kernel is its FP32-weight form.
#include "boundary.cuh"
#include "common.cuh"

namespace muse {

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

MUSE_TRACE_SETTER(fewtok_trace_set)

constexpr int FEWTOK_X_PAD = 64;   // bytes added to each x row in shared memory
static inline bool peer_active_host(const PeerSync& ps) { return ps.world > 1; }

// HI = tokens 8..15 exist (second half of the A fragment); otherwise those MMA rows are fed zeros.
template <int NW, int U, bool HI>
__global__ void __launch_bounds__(NW * 32) fewtok_mma_kernel(const __nv_bfloat16* __restrict__ W,
                                                             const __nv_bfloat16* __restrict__ x,
                                                             __nv_bfloat16* __restrict__ out, int m, int N, int K, int ld_x,
                                                             int ld_out, int* __restrict__ status) {
  unsigned long long* const trace = MUSE_TRACE_BASE();
  // Diagnostic builds: thread 0 of every CTA stamps clock64() into its 16 slots (0 entry, 1 first loads issued,
  // 2 x arrived, 3/4/5 first group multiplied / reduced in shared memory / stored, 6 last group multiplied,
  // 7 end, 8 groups walked; 15 and 11 = entry and exit on the global nanosecond timer).
  unsigned long long* const tr = trace && threadIdx.x == 0 ? trace + 16ull * blockIdx.x : nullptr;
#define FEWTOK_STAMP(slot) do { if (tr) tr[slot] = static_cast<unsigned long long>(clock64()); } while (0)
  if (tr) { FEWTOK_STAMP(0); tr[15] = global_ns(); }
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t xbar;
  constexpr int TOK = HI ? 16 : 8;
  constexpr int OUTS = TOK * 8;                  // outputs of one row group
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const uint32_t x_stride = static_cast<uint32_t>(K) * 2u + FEWTOK_X_PAD;
  float* red = reinterpret_cast<float*>(smem + static_cast<size_t>(m) * x_stride);   // [2][NW][OUTS]
  const int kblocks = K >> 5;                    // 32-element (64-byte) pieces of a row
  const int nb = (kblocks + NW * U - 1) / (NW * U);
  const int groups = (N + 7) >> 3;
  const int my_groups = blockIdx.x < groups ? (groups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int steps = my_groups * nb;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&xbar), 1);
    fence_mbar_init();
    mbar_expect_tx(smem_u32(&xbar), static_cast<uint32_t>(K) * 2u * static_cast<uint32_t>(m));
    for (int t = 0; t < m; ++t)
      bulk_load_1d(smem_u32(smem) + static_cast<uint32_t>(t) * x_stride, x + static_cast<size_t>(t) * ld_x,
                   static_cast<uint32_t>(K) * 2u, smem_u32(&xbar));
  }
  // Lane's piece of batch b of row group i: W[min(8 * group + g, N - 1)][32 * (b * NW * U + warp * U + u) + 8q ..].
  auto load = [&](uint4 (&w)[U], int i, int b) {
    int row = (blockIdx.x + i * static_cast<int>(gridDim.x)) * 8 + g;
    row = row < N ? row : N - 1;
    const uint4* p = reinterpret_cast<const uint4*>(W + static_cast<size_t>(row) * K) + q;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int kb = b * NW * U + warp * U + u;
      w[u] = kb < kblocks ? ldg_stream16(p + kb * 4) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  uint4 w[U], wn[U];
  if (steps > 0) load(w, 0, 0);
  FEWTOK_STAMP(1);
  __syncthreads();
  if (!mbar_wait(smem_u32(&xbar), 0)) {
    if (threadIdx.x == 0) atomicOr(status, ST_X_TIMEOUT);
    return;
  }
  FEWTOK_STAMP(2);
  // MMA rows of tokens that do not exist read the last real token (fewer distinct shared-memory
  // addresses per load than zero rows would cost); their results are never stored.
  const uint8_t* xg = smem + static_cast<size_t>(min(g, m - 1)) * x_stride + q * 16;        // token g
  const uint8_t* xh = smem + static_cast<size_t>(min(g + 8, m - 1)) * x_stride + q * 16;    // token g + 8
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  int i = 0, b = 0;
  for (int s = 0; s < steps; ++s) {
    int in = i, bn = b + 1;
    if (bn == nb) { bn = 0; ++in; }
    if (s + 1 < steps) load(wn, in, bn);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int kb = b * NW * U + warp * U + u;
      if (kb < kblocks) {
        const uint4 xa = *reinterpret_cast<const uint4*>(xg + kb * 64);
        uint4 xb = make_uint4(0u, 0u, 0u, 0u);
        if constexpr (HI) xb = *reinterpret_cast<const uint4*>(xh + kb * 64);
        mma_bf16_16816(acc, xa.x, xb.x, xa.y, xb.y, w[u].x, w[u].y);
        mma_bf16_16816(acc, xa.z, xb.z, xa.w, xb.w, w[u].z, w[u].w);
      }
    }
    if (b == nb - 1) {
      if (i == 0) FEWTOK_STAMP(3);
      if (i == my_groups - 1) FEWTOK_STAMP(6);
      // acc[0..1]: token g, rows 2q, 2q+1 of the group; acc[2..3]: token g + 8.
      float* mine = red + (static_cast<size_t>(i & 1) * NW + warp) * OUTS;
      *reinterpret_cast<float2*>(mine + g * 8 + 2 * q) = make_float2(acc[0], acc[1]);
      if constexpr (HI) *reinterpret_cast<float2*>(mine + (g + 8) * 8 + 2 * q) = make_float2(acc[2], acc[3]);
      acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
      __syncthreads();   // the buffer written two groups ago is free again once every warp passed this
      if (i == 0) FEWTOK_STAMP(4);
      if (threadIdx.x < OUTS) {
        const float* col = red + static_cast<size_t>(i & 1) * NW * OUTS + threadIdx.x;
        float sum = 0.f;
#pragma unroll 8
        for (int wv = 0; wv < NW; ++wv) sum += col[wv * OUTS];
        const int t = threadIdx.x >> 3;
        const int row = (blockIdx.x + i * static_cast<int>(gridDim.x)) * 8 + (threadIdx.x & 7);
        if (t < m && row < N) out[static_cast<size_t>(t) * ld_out + row] = __float2bfloat16_rn(sum);
      }
      if (i == 0) FEWTOK_STAMP(5);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) w[u] = wn[u];
    i = in;
    b = bn;
  }
  if (tr) { FEWTOK_STAMP(7); tr[8] = static_cast<unsigned long long>(my_groups); tr[11] = global_ns(); }
#undef FEWTOK_STAMP
}

constexpr int RP_TOKENS = 8;   // most tokens of a row-parallel call
// Byte offset, inside a rank's staging, of the lines `src` sends for token t of call e: 8 bytes per output row.
__device__ __forceinline__ size_t rp_row_offset(int e, int world, int src, int t, int n) {
  return ((static_cast<size_t>(e & 1) * world + src) * RP_TOKENS + t) * static_cast<size_t>(n) * 8;
}

// K <= 32 * NW * U: one batch per group, A fragments resident in registers (no shared-memory x).
// HI = tokens 8..15 exist. With tok_split > 1 the grid is tok_split interleaved copies of the walk, copy j
// multiplying tokens [j * TOKS, (j + 1) * TOKS): CTAs c and c + 1 stream the same groups at the same time,
// so W still leaves HBM once (the second reader finds it in L2) while each SM keeps only its own tokens.
// PEERS = column-parallel: every CTA stores its rows at columns [col0, col0 + N) of this rank's gathered
// output and sends them to every peer's staging as self-validating lines; when its groups are done it
// unpacks its share of the lines the peers sent here. No fence, no flag, no wait on another CTA.
// VEC (one GPU) = 16-byte output stores: the caller guarantees N % 8 == 0 and 16-byte aligned rows of out.
// BND = x is not read but rebuilt by the post-attention boundary prologue (boundary.cuh) from `bd`: up to 8
// tokens, one walk, one GPU; `x` and `ld_x` are ignored.
// RP = row-parallel: W and x are this rank's K slice, so every output is a partial sum that has to meet the other
// ranks' (the reference's tensor-parallel `o` projection, bf16_proj/reference.py:17; its all-reduce is the
// identity on one GPU, decode_layer/reference.py:451). One-shot all-reduce inside the kernel: every CTA sends
// its FP32 partial sums to EVERY rank's staging (its own included) as self-validating 16-byte lines
// {sum, call number, sum, call number}, and when its groups are done it adds up, for the same groups, the lines
// of all ranks in rank order (so every rank computes the same bits) and stores BF16 into its own `out`.
// Up to 8 tokens, N % 8 == 0; staging per rank: 2 x world x 8 tokens x N x 8 bytes.
template <int NW, int U, bool HI, bool PEERS, bool VEC, bool BND = false, bool RP = false>
__global__ void __launch_bounds__(NW * 32) fewtok_xreg_kernel(const __nv_bfloat16* __restrict__ W,
                                                              const __nv_bfloat16* __restrict__ x,
                                                              __nv_bfloat16* __restrict__ out, int m, int N, int K, int ld_x,
                                                              int ld_out, int tok_split, int* __restrict__ status,
                                                              const __grid_constant__ PeerSync ps,
                                                              const __grid_constant__ BoundaryArgs bd) {
  static_assert(!BND || (!HI && !PEERS && NW * 32 >= 256), "the boundary prologue serves one 8-token walk on one GPU");
  static_assert(!RP || (!HI && !PEERS && !BND && !VEC), "the row-parallel exchange serves one 8-token walk");
  unsigned long long* const trace = MUSE_TRACE_BASE();
  // Diagnostic builds, the exchange (PEERS only): per CTA 16 slots of the global nanosecond timer, 0 entry,
  // 1 first group stored, 2 groups done, 3 peers' lines unpacked; first group: 5 multiplied, 6 synchronised, 7 stored locally.
  unsigned long long* const tr = PEERS && trace ? trace + 16ull * blockIdx.x : nullptr;
  if (tr && threadIdx.x == 0) tr[0] = global_ns();
  constexpr int OUTS = HI ? 128 : 64;            // 8 or 16 tokens x 8 rows
  constexpr int TOKS = HI ? 16 : 8;
  __shared__ __align__(16) float red[2][NW][OUTS];
  __shared__ int s_epoch;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int C = static_cast<int>(gridDim.x) / tok_split, c = static_cast<int>(blockIdx.x) / tok_split;
  if constexpr (PEERS) {
    out = reinterpret_cast<__nv_bfloat16*>(ps.out[ps.rank]) + ps.col0;
  }
  const int m_all = m;
  int t0 = 0;
  {
    t0 = (static_cast<int>(blockIdx.x) % tok_split) * TOKS;
    x += static_cast<size_t>(t0) * ld_x;
    out += static_cast<size_t>(t0) * ld_out;
    m = m - t0 < TOKS ? m - t0 : TOKS;
    if (!PEERS && m <= 0) return;
  }
  const int kblocks = K >> 5;
  const int groups = (N + 7) >> 3;
  const int my_groups = (c < groups && m > 0) ? (groups - c + C - 1) / C : 0;
  const int first = warp * U;                    // this warp's 64-byte pieces of every row: first .. first + U - 1
  auto load = [&](uint4 (&w)[U], int i) {
    int row = (c + i * C) * 8 + g;
    row = row < N ? row : N - 1;
    const uint4* p = reinterpret_cast<const uint4*>(W + static_cast<size_t>(row) * K) + q;
#pragma unroll
    for (int u = 0; u < U; ++u) w[u] = first + u < kblocks ? ldg_stream16(p + (first + u) * 4) : make_uint4(0u, 0u, 0u, 0u);
  };
  // One register buffer: a group's loads are re-issued into it as soon as its MMAs have read it, and stay
  // in flight across the reduction below. (A second buffer costs 16 registers the 32-warp CTA does not have.)
  uint4 w[U], xr[U], xh[HI ? U : 1];
  if (my_groups > 0) load(w, 0);
  // Only the weights have been touched so far: everything below waits for the kernels ahead in the stream (no-ops
  // unless this launch was allowed to start under the previous kernel's tail).
  griddep_launch_dependents();
  griddep_wait();
  if constexpr (BND) {
    // The first weight loads are in flight; every CTA now rebuilds h for all tokens and takes its fragments from it.
    extern __shared__ __align__(16) float bnd_s1[];
    __shared__ float bnd_red[NW][BND_TOKENS];
    __shared__ float bnd_inv1[BND_TOKENS], bnd_inv2[BND_TOKENS];
    boundary_prologue<NW * 32>(bd, m, K, bnd_s1, bnd_red, bnd_inv1, bnd_inv2);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      xr[u] = make_uint4(0u, 0u, 0u, 0u);
      if (g < m && first + u < kblocks) {
        float h[8];
        boundary_h8(bd, bnd_s1, bnd_inv2, K, g, (first + u) * 32 + q * 8, h);
        xr[u] = make_uint4(pack_bf16x2(h[0], h[1]), pack_bf16x2(h[2], h[3]), pack_bf16x2(h[4], h[5]), pack_bf16x2(h[6], h[7]));
      }
    }
    xh[0] = make_uint4(0u, 0u, 0u, 0u);
  } else {
    const uint4* px = reinterpret_cast<const uint4*>(x + static_cast<size_t>(g < m ? g : 0) * ld_x) + q;
#pragma unroll
    for (int u = 0; u < U; ++u)
      xr[u] = (g < m && first + u < kblocks) ? __ldcg(px + (first + u) * 4) : make_uint4(0u, 0u, 0u, 0u);
    if constexpr (HI) {
      const uint4* ph = reinterpret_cast<const uint4*>(x + static_cast<size_t>(g + 8 < m ? g + 8 : 0) * ld_x) + q;
#pragma unroll
      for (int u = 0; u < U; ++u)
        xh[u] = (g + 8 < m && first + u < kblocks) ? __ldcg(ph + (first + u) * 4) : make_uint4(0u, 0u, 0u, 0u);
    } else {
      xh[0] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  if constexpr (PEERS || RP) {   // after the first loads are in flight: none of this delays them
    if (threadIdx.x == 0) {
      // The call number, and the book-keeping that advances it: the last CTA to get HERE closes the number,
      // because by then every CTA of the grid has read it. Done first so that nothing waits on it at the end.
      int* mine = ps.flags[ps.rank];
      const int e = ld_acquire_sys(mine + 16) + 1;   // acquire: the count below may not overtake this read
      s_epoch = e;
      if (atomicAdd(mine + 17, 1) == static_cast<int>(gridDim.x) - 1) {
        mine[17] = 0;
        mine[16] = e;
      }
    } else if (threadIdx.x >= NW * 32 - ps.world && static_cast<int>(threadIdx.x) - (NW * 32 - ps.world) != ps.rank) {
      // One lane per peer touches that peer's staging now, so that the address translation of the first
      // real store (several microseconds later) is already cached. The value is never used.
      uint32_t unused;
      asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(unused) : "l"(ps.ll[threadIdx.x - (NW * 32 - ps.world)]) : "memory");
    }
  }
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int i = 0; i < my_groups; ++i) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint4 hi = xh[HI ? u : 0];
      mma_bf16_16816(acc, xr[u].x, hi.x, xr[u].y, hi.y, w[u].x, w[u].y);
      mma_bf16_16816(acc, xr[u].z, hi.z, xr[u].w, hi.w, w[u].z, w[u].w);
    }
    if (tr && i == 0 && threadIdx.x == 0) tr[5] = global_ns();
    if (i + 1 < my_groups) load(w, i + 1);
    *reinterpret_cast<float2*>(&red[i & 1][warp][g * 8 + 2 * q]) = make_float2(acc[0], acc[1]);
    if constexpr (HI) *reinterpret_cast<float2*>(&red[i & 1][warp][(g + 8) * 8 + 2 * q]) = make_float2(acc[2], acc[3]);
    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
    __syncthreads();   // the buffer written two groups ago is free again once every warp passed this
    if (tr && i == 0 && threadIdx.x == 0) tr[6] = global_ns();
    if (threadIdx.x < OUTS) {
      float sum = 0.f;
#pragma unroll 8
      for (int wv = 0; wv < NW; ++wv) sum += red[i & 1][wv][threadIdx.x];
      const int t = threadIdx.x >> 3, r = threadIdx.x & 7;
      const int grp = c + i * C, row0 = grp * 8;
      if constexpr (!PEERS && VEC) {
        // 8 rows of a token = 8 neighbouring lanes: one 16-byte store per token and group instead of eight
        // 2-byte ones (what makes an output in page-locked host memory affordable: one PCIe write each).
        const uint32_t v = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(sum)));
        const uint32_t p01 = v | (__shfl_down_sync(0xffffffffu, v, 1) << 16);
        const uint32_t p23 = __shfl_down_sync(0xffffffffu, p01, 2);
        const uint32_t p45 = __shfl_down_sync(0xffffffffu, p01, 4), p67 = __shfl_down_sync(0xffffffffu, p23, 4);
        if (r == 0 && t < m) *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * ld_out + row0) = make_uint4(p01, p23, p45, p67);
      } else if constexpr (RP) {
        // Rows r, r + 1 of a token sit in neighbouring lanes: one line carries both partial sums.
        const float other = __shfl_down_sync(0xffffffffu, sum, 1);
        if ((r & 1) == 0 && t < m) {
          const int e = s_epoch;
          const size_t off = rp_row_offset(e, ps.world, ps.rank, t, N) + static_cast<size_t>(row0 + r) * 8;
          for (int p = 0; p < ps.world; ++p)
            st_volatile_v4(static_cast<char*>(ps.ll[p]) + off, __float_as_uint(sum), static_cast<uint32_t>(e), __float_as_uint(other),
                           static_cast<uint32_t>(e));
        }
      } else if constexpr (!PEERS) {
        if (t < m && row0 + r < N) out[static_cast<size_t>(t) * ld_out + row0 + r] = __float2bfloat16_rn(sum);
      } else {
        // The 8 rows of a token sit in 8 neighbouring lanes: gather them into one 16-byte vector (N % 8 == 0 here).
        const uint32_t v = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(sum)));
        const uint32_t p01 = v | (__shfl_down_sync(0xffffffffu, v, 1) << 16);
        const uint32_t p23 = __shfl_down_sync(0xffffffffu, p01, 2);
        const uint32_t p45 = __shfl_down_sync(0xffffffffu, p01, 4), p67 = __shfl_down_sync(0xffffffffu, p23, 4);
        if (r == 0 && t < m) {
          const uint4 val = make_uint4(p01, p23, p45, p67);
          *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * ld_out + row0) = val;
          if (tr && i == 0 && threadIdx.x == 0) tr[7] = global_ns();
          const int e = s_epoch;
          const size_t off = ll_row_offset(e, ps.world, ps.rank, t0 + t, N) + static_cast<size_t>(grp) * 32;
          for (int p = 0; p < ps.world; ++p)
            if (p != ps.rank) ll_send16(static_cast<char*>(ps.ll[p]) + off, val, e);
        }
      }
    }
    if (tr && i == 0 && threadIdx.x == 0) tr[1] = global_ns();
  }
  if constexpr (RP) {
    // Add up, for this CTA's own groups, the partial sums of every rank (this rank's own came the same way).
    // Units of (group, token, row pair): one thread polls `world` lines and stores two BF16 outputs.
    __syncthreads();
    const int e = s_epoch;
    const uint32_t want = static_cast<uint32_t>(e);
    bool ok = true;
    for (int u = threadIdx.x; u < my_groups * 32; u += NW * 32) {
      const int i = u >> 5, t = (u >> 2) & 7, j = u & 3;
      if (t >= m) continue;
      const int row = (c + i * C) * 8 + 2 * j;
      float a0 = 0.f, a1 = 0.f;
      for (int src = 0; src < ps.world && ok; ++src) {
        const char* line = static_cast<const char*>(ps.ll[ps.rank]) + rp_row_offset(e, ps.world, src, t, N) + static_cast<size_t>(row) * 8;
        uint4 v = ld_volatile_v4(line);
        if (v.y != want || v.w != want) {
          const unsigned long long t_start = global_ns();
          for (;;) {
            v = ld_volatile_v4(line);
            if (v.y == want && v.w == want) break;
            if (global_ns() - t_start > WAIT_LIMIT_NS) { ok = false; break; }
          }
        }
        a0 += __uint_as_float(v.x);
        a1 += __uint_as_float(v.z);
      }
      if (ok) *reinterpret_cast<uint32_t*>(out + static_cast<size_t>(t) * ld_out + row) = pack_bf16x2(a0, a1);
    }
    if (!ok) atomicOr(status, ST_PEER_DONE_TIMEOUT);
  }
  if constexpr (PEERS) {
    // Unpack this CTA's share of what the peers sent: (sending rank, token, group) units, 16 bytes of output each.
    __syncthreads();
    if (tr && threadIdx.x == 0) tr[2] = global_ns();
    const int e = s_epoch, gpr = N >> 3;
    const int units = (ps.world - 1) * m_all * gpr;
    bool ok = true;
    for (int u = static_cast<int>(blockIdx.x) * NW * 32 + threadIdx.x; u < units; u += static_cast<int>(gridDim.x) * NW * 32) {
      const int si = u / (m_all * gpr), rem = u - si * (m_all * gpr);
      const int t = rem / gpr, grp = rem - t * gpr;
      const int src = si < ps.rank ? si : si + 1;
      uint4 val;
      if (ll_recv16(static_cast<const char*>(ps.ll[ps.rank]) + ll_row_offset(e, ps.world, src, t, N) + static_cast<size_t>(grp) * 32, e, val))
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(ps.out[ps.rank]) + static_cast<size_t>(t) * ld_out +
                                  static_cast<size_t>(src) * N + grp * 8) = val;
      else
        ok = false;
    }
    if (!ok) atomicOr(status, ST_PEER_DONE_TIMEOUT);
    if (tr && threadIdx.x == 0) tr[3] = global_ns();
  }
}

// The same walk over FP32 weights (the MoE router): each lane loads 32 bytes (8 FP32) per piece, splits
// them in registers into BF16 hi = bf16(w) and lo = bf16(w - hi) -- the split the reference's prepare()
// stores (best_submissions/muse_bf16_proj.py:346-349) -- and feeds both to MMAs on one FP32
// accumulator (its _router_kernel, :260-287), so W is read once, as FP32, with no pre-split copy.
// Up to 8 tokens per CTA (tok_split copies for more); output FP32.
// XF32 = the router's FP32-input mode of the reference's decode layer (X_F32,
// best_submissions/muse_decode_layer.py:165-200): x is FP32, split the same way once into registers, and
// out = x_hi (hi + lo) + x_lo hi, three MMAs per step. Its x fragments take twice the registers, so a
// group's weights then pass through in two halves (one half in flight at a time).
// BND (with XF32) = the FP32 x is rebuilt by the post-attention boundary prologue from `bd` (up to 8 tokens).
template <int NW, int U, bool XF32, bool BND = false>
__global__ void __launch_bounds__(NW * 32) fewtok_xreg_f32_kernel(const float* __restrict__ W, const void* __restrict__ xv,
                                                                  float* __restrict__ out, int m, int N, int K, int ld_x,
                                                                  int ld_out, int tok_split,
                                                                  const __grid_constant__ BoundaryArgs bd) {
  static_assert(!BND || XF32, "the boundary hands the router FP32 activations");
  constexpr int OUTS = 64, TOKS = 8;
  constexpr int SUBS = XF32 && U > 1 ? 2 : 1, PS = U / SUBS;   // weight sub-batches of a group, pieces in each
  __shared__ __align__(16) float red[2][NW][OUTS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int C = static_cast<int>(gridDim.x) / tok_split, c = static_cast<int>(blockIdx.x) / tok_split;
  const int t0 = (static_cast<int>(blockIdx.x) % tok_split) * TOKS;
  out += static_cast<size_t>(t0) * ld_out;
  m = m - t0 < TOKS ? m - t0 : TOKS;
  if (m <= 0) return;
  const int kblocks = K >> 5;
  const int groups = (N + 7) >> 3;
  const int my_groups = c < groups ? (groups - c + C - 1) / C : 0;
  const int first = warp * U;
  uint4 w[2 * PS], xr[U], xl[XF32 ? U : 1];
  auto load = [&](int i, int h) {
    int row = (c + i * C) * 8 + g;
    row = row < N ? row : N - 1;
    const uint4* p = reinterpret_cast<const uint4*>(W + static_cast<size_t>(row) * K) + 2 * q;   // 8 FP32 = two vectors
#pragma unroll
    for (int u = 0; u < PS; ++u) {
      const int piece = first + h * PS + u;
      const bool ok = piece < kblocks;
      w[2 * u] = ok ? ldg_stream16(p + piece * 8) : make_uint4(0u, 0u, 0u, 0u);
      w[2 * u + 1] = ok ? ldg_stream16(p + piece * 8 + 1) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  if (my_groups > 0) load(0, 0);
  griddep_launch_dependents();   // only the weights have been touched so far; the rest waits for the kernels ahead
  griddep_wait();
  // (a, b) -> BF16 pair of the hi halves (a in the low 16 bits) and of the lo halves.
  auto split = [](uint32_t a_bits, uint32_t b_bits, uint32_t& hi, uint32_t& lo) {
    const float a = __uint_as_float(a_bits), b = __uint_as_float(b_bits);
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    const float ra = a - __uint_as_float(hi << 16), rb = b - __uint_as_float(hi & 0xffff0000u);
    const __nv_bfloat162 l = __floats2bfloat162_rn(ra, rb);
    lo = *reinterpret_cast<const uint32_t*>(&l);
  };
  if constexpr (BND) {
    extern __shared__ __align__(16) float bnd_s1[];
    __shared__ float bnd_red[NW][BND_TOKENS];
    __shared__ float bnd_inv1[BND_TOKENS], bnd_inv2[BND_TOKENS];
    boundary_prologue<NW * 32>(bd, m, K, bnd_s1, bnd_red, bnd_inv1, bnd_inv2);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      xr[u] = xl[XF32 ? u : 0] = make_uint4(0u, 0u, 0u, 0u);
      if (g < m && first + u < kblocks) {
        float h[8];
        boundary_h8(bd, bnd_s1, bnd_inv2, K, g, (first + u) * 32 + q * 8, h);
        split(__float_as_uint(h[0]), __float_as_uint(h[1]), xr[u].x, xl[XF32 ? u : 0].x);
        split(__float_as_uint(h[2]), __float_as_uint(h[3]), xr[u].y, xl[XF32 ? u : 0].y);
        split(__float_as_uint(h[4]), __float_as_uint(h[5]), xr[u].z, xl[XF32 ? u : 0].z);
        split(__float_as_uint(h[6]), __float_as_uint(h[7]), xr[u].w, xl[XF32 ? u : 0].w);
      }
    }
  } else if constexpr (XF32) {
    const float* xf = reinterpret_cast<const float*>(xv) + static_cast<size_t>(t0 + (g < m ? g : 0)) * ld_x;
    const uint4* px = reinterpret_cast<const uint4*>(xf) + 2 * q;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool ok = g < m && first + u < kblocks;
      const uint4 a = ok ? __ldcg(px + (first + u) * 8) : make_uint4(0u, 0u, 0u, 0u);
      const uint4 b = ok ? __ldcg(px + (first + u) * 8 + 1) : make_uint4(0u, 0u, 0u, 0u);
      split(a.x, a.y, xr[u].x, xl[u].x);
      split(a.z, a.w, xr[u].y, xl[u].y);
      split(b.x, b.y, xr[u].z, xl[u].z);
      split(b.z, b.w, xr[u].w, xl[u].w);
    }
  } else {
    const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(xv) + static_cast<size_t>(t0 + (g < m ? g : 0)) * ld_x;
    const uint4* px = reinterpret_cast<const uint4*>(xb) + q;
#pragma unroll
    for (int u = 0; u < U; ++u)
      xr[u] = (g < m && first + u < kblocks) ? __ldcg(px + (first + u) * 4) : make_uint4(0u, 0u, 0u, 0u);
    xl[0] = make_uint4(0u, 0u, 0u, 0u);
  }
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int i = 0; i < my_groups; ++i) {
#pragma unroll
    for (int h = 0; h < SUBS; ++h) {
#pragma unroll
      for (int u = 0; u < PS; ++u) {
        uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
        split(w[2 * u].x, w[2 * u].y, h0, l0);
        split(w[2 * u].z, w[2 * u].w, h1, l1);
        split(w[2 * u + 1].x, w[2 * u + 1].y, h2, l2);
        split(w[2 * u + 1].z, w[2 * u + 1].w, h3, l3);
        const uint4 xa = xr[h * PS + u];
        mma_bf16_16816(acc, xa.x, 0u, xa.y, 0u, h0, h1);
        mma_bf16_16816(acc, xa.z, 0u, xa.w, 0u, h2, h3);
        mma_bf16_16816(acc, xa.x, 0u, xa.y, 0u, l0, l1);
        mma_bf16_16816(acc, xa.z, 0u, xa.w, 0u, l2, l3);
        if constexpr (XF32) {
          const uint4 xb = xl[h * PS + u];
          mma_bf16_16816(acc, xb.x, 0u, xb.y, 0u, h0, h1);
          mma_bf16_16816(acc, xb.z, 0u, xb.w, 0u, h2, h3);
        }
      }
      if (h + 1 < SUBS) load(i, h + 1);
      else if (i + 1 < my_groups) load(i + 1, 0);
    }
    *reinterpret_cast<float2*>(&red[i & 1][warp][g * 8 + 2 * q]) = make_float2(acc[0], acc[1]);
    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
    __syncthreads();
    if (threadIdx.x < OUTS) {
      float sum = 0.f;
#pragma unroll 8
      for (int wv = 0; wv < NW; ++wv) sum += red[i & 1][wv][threadIdx.x];
      const int t = threadIdx.x >> 3;
      const int row = (c + i * C) * 8 + (threadIdx.x & 7);
      if (t < m && row < N) out[static_cast<size_t>(t) * ld_out + row] = sum;
    }
  }
}


static size_t fewtok_smem(int K, int m, int nw) {
  const int tok = m > 8 ? 16 : 8;
  return static_cast<size_t>(m) * (static_cast<size_t>(K) * 2 + FEWTOK_X_PAD) + 2ull * nw * tok * 8 * sizeof(float);
}

template <int NW, int U, bool HI>
static cudaError_t launch_fewtok(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out,
                                 int* status, cudaStream_t s) {
  auto kern = fewtok_mma_kernel<NW, U, HI>;
  static int configured[64] = {0}, sms[64] = {0}, optin[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    if ((e = cudaDeviceGetAttribute(&optin[dev], cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) return e;
    cudaFuncAttributes fa;
    if ((e = cudaFuncGetAttributes(&fa, kern)) != cudaSuccess) return e;
    optin[dev] -= static_cast<int>(fa.sharedSizeBytes);
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, optin[dev])) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    configured[dev] = 1;
  }
  const size_t smem = fewtok_smem(K, m, NW);
  if (smem > static_cast<size_t>(optin[dev])) return cudaErrorInvalidConfiguration;
  int resident = 0;
  if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, NW * 32, smem)) != cudaSuccess) return e;
  if (resident < 1) return cudaErrorInvalidConfiguration;
  int grid = sms[dev] * resident;
  const int groups = (N + 7) / 8;
  if (grid > groups) grid = groups;
  kern<<<grid, NW * 32, smem, s>>>(reinterpret_cast<const __nv_bfloat16*>(W), reinterpret_cast<const __nv_bfloat16*>(x),
                                   reinterpret_cast<__nv_bfloat16*>(out), m, N, K, ld_x, ld_out, status);
  return cudaGetLastError();
}

template <int NW, int U, bool HI, bool PEERS, bool VEC>
static cudaError_t launch_xreg_with(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out,
                                    int tok_split, int* status, const PeerSync& ps, cudaStream_t s) {
  auto kern = fewtok_xreg_kernel<NW, U, HI, PEERS, VEC>;
  static int per_sm[64] = {0}, sms[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!per_sm[dev]) {
    if ((e = cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    int resident = 0;
    if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, NW * 32, 0)) != cudaSuccess) return e;
    if (resident < 1) return cudaErrorInvalidConfiguration;
    per_sm[dev] = resident;
  }
  int walkers = sms[dev] * per_sm[dev] / tok_split;   // CTAs per copy of the walk
  const int groups = (N + 7) / 8;
  if (walkers > groups) walkers = groups;
  if (walkers < 1) return cudaErrorInvalidConfiguration;
  return launch_dependent(kern, dim3(walkers * tok_split), dim3(NW * 32), 0, s, reinterpret_cast<const __nv_bfloat16*>(W),
                          reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(out), m, N, K, ld_x, ld_out,
                          tok_split, status, ps, BoundaryArgs{});
}

// Row-parallel launch: the same persistent walk, the all-reduce inside (see RP above).
template <int NW, int U>
static cudaError_t launch_xreg_rowpar(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out,
                                      int* status, const PeerSync& ps, cudaStream_t s) {
  auto kern = fewtok_xreg_kernel<NW, U, false, false, false, false, true>;
  static int per_sm[64] = {0}, sms[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!per_sm[dev]) {
    if ((e = cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    int resident = 0;
    if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, NW * 32, 0)) != cudaSuccess) return e;
    if (resident < 1) return cudaErrorInvalidConfiguration;
    per_sm[dev] = resident;
  }
  int walkers = sms[dev] * per_sm[dev];
  if (walkers > N / 8) walkers = N / 8;
  return launch_dependent(kern, dim3(walkers), dim3(NW * 32), 0, s, reinterpret_cast<const __nv_bfloat16*>(W),
                          reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(out), m, N, K, ld_x, ld_out, 1, status, ps,
                          BoundaryArgs{});
}

// out[m, N] = sum over ranks of x_r[m, K_r] . W_r[N, K_r]^T, 1..8 tokens; K_r (this rank's slice) <= 4096 in whole
// 32-element pieces. `peers`: world, rank, flags[] and ll[] (the staging of every rank) are used; out[] is not.
int fewtok_rowpar_dispatch(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out, int* status,
                           const PeerSync* peers, cudaStream_t stream) {
  if (!W || !x || !out || !status || !peers || N <= 0 || K <= 0) return -1;
  const PeerSync ps = *peers;
  if (ps.world < 2 || ps.world > MAX_WORLD || ps.rank < 0 || ps.rank >= ps.world) return -8;
  for (int p = 0; p < ps.world; ++p)
    if (!ps.ll[p] || !ps.flags[p] || (reinterpret_cast<uintptr_t>(ps.ll[p]) & 15)) return -8;
  if (m < 1 || m > RP_TOKENS) return -9;
  if (K % 32 != 0 || K / 32 > 128 || N % 8 != 0 || ld_x % 8 != 0 || ld_x < K || ld_out < N || ld_out % 2 != 0) return -2;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(out) & 3)) return -2;
  const int kb = K / 32;
  cudaError_t e;
  if (kb <= 16) e = launch_xreg_rowpar<16, 1>(W, x, out, m, N, K, ld_x, ld_out, status, ps, stream);
  else if (kb <= 32) e = launch_xreg_rowpar<16, 2>(W, x, out, m, N, K, ld_x, ld_out, status, ps, stream);
  else if (kb <= 64) e = launch_xreg_rowpar<16, 4>(W, x, out, m, N, K, ld_x, ld_out, status, ps, stream);
  else e = launch_xreg_rowpar<32, 4>(W, x, out, m, N, K, ld_x, ld_out, status, ps, stream);
  return static_cast<int>(e);
}

// The single-GPU instantiation carries no exchange code.
template <int NW, int U, bool HI>
static cudaError_t launch_xreg(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out,
                               int tok_split, int* status, const PeerSync& ps, cudaStream_t s) {
  if (peer_active_host(ps)) return launch_xreg_with<NW, U, HI, true, false>(W, x, out, m, N, K, ld_x, ld_out, tok_split, status, ps, s);
  const bool vec = N % 8 == 0 && ((reinterpret_cast<uintptr_t>(out) | (static_cast<uintptr_t>(ld_out) * 2)) & 15) == 0;
  return vec ? launch_xreg_with<NW, U, HI, false, true>(W, x, out, m, N, K, ld_x, ld_out, tok_split, status, ps, s)
             : launch_xreg_with<NW, U, HI, false, false>(W, x, out, m, N, K, ld_x, ld_out, tok_split, status, ps, s);
}

template <int NW, int U, bool XF32>
static cudaError_t launch_xreg_f32(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out,
                                   int tok_split, cudaStream_t s) {
  auto kern = fewtok_xreg_f32_kernel<NW, U, XF32>;
  static int per_sm[64] = {0}, sms[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!per_sm[dev]) {
    if ((e = cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    int resident = 0;
    if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, NW * 32, 0)) != cudaSuccess) return e;
    if (resident < 1) return cudaErrorInvalidConfiguration;
    per_sm[dev] = resident;
  }
  int walkers = sms[dev] * per_sm[dev] / tok_split;
  const int groups = (N + 7) / 8;
  if (walkers > groups) walkers = groups;
  if (walkers < 1) return cudaErrorInvalidConfiguration;
  return launch_dependent(kern, dim3(walkers * tok_split), dim3(NW * 32), 0, s, reinterpret_cast<const float*>(W), x,
                          reinterpret_cast<float*>(out), m, N, K, ld_x, ld_out, tok_split, BoundaryArgs{});
}

// FP32 weight and output, 1..8 * tok_split tokens, 16 warps, unroll in {2, 4, 8} with K <= 512 * unroll;
// x BF16, or FP32 when x_is_f32 (ld_x counts elements of x's type).
int fewtok_f32_dispatch(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out, int unroll,
                        int tok_split, int x_is_f32, cudaStream_t stream) {
  if (!W || !x || !out || N <= 0 || K <= 0) return -1;
  if (tok_split < 1 || tok_split > 4 || m < 1 || m > 8 * tok_split) return -9;
  if (K % 32 != 0 || ld_x % 8 != 0 || ld_x < K || ld_out < N || K / 32 > 16 * unroll) return -2;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return -2;
  cudaError_t e = cudaErrorInvalidValue;
#define MUSE_F32(U_)                                                                                         \
  if (unroll == U_)                                                                                          \
    e = x_is_f32 ? launch_xreg_f32<16, U_, true>(W, x, out, m, N, K, ld_x, ld_out, tok_split, stream)        \
                 : launch_xreg_f32<16, U_, false>(W, x, out, m, N, K, ld_x, ld_out, tok_split, stream);
  MUSE_F32(8) MUSE_F32(4) MUSE_F32(2)
#undef MUSE_F32
  return static_cast<int>(e);
}

size_t fewtok_smem_bytes(int m, int K, int warps) { return fewtok_smem(K, m, warps); }

// ---------------------------------------------------------------- the post-attention boundary

// Stand-alone form, one CTA of 256 threads per token; D % 8 == 0 and D <= 8192 (four 8-element chunks per thread,
// held in registers between the two reductions).
__global__ void __launch_bounds__(256) attn_boundary_kernel(const __grid_constant__ BoundaryArgs bd, int D) {
  constexpr int NT = 256, CH = 4;
  __shared__ float red[NT / 32];
  __shared__ float s_inv;
  griddep_launch_dependents();   // everything here depends on the kernels ahead: only the launch itself overlaps them
  griddep_wait();
  const int t = blockIdx.x, cpt = D >> 3, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  auto block_inv = [&](float v, float eps) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
      float r = lane < NT / 32 ? red[lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
      if (lane == 0) s_inv = rsqrtf(r / static_cast<float>(D) + eps);
    }
    __syncthreads();
    return s_inv;
  };
  float v[CH][8], a[CH][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + j * NT;
    if (c < cpt) {
      bf16x8_to_f32(__ldcg(reinterpret_cast<const uint4*>(bd.attn + static_cast<size_t>(t) * D) + c), a[j]);
      const float4 s0 = __ldcg(reinterpret_cast<const float4*>(bd.stream + static_cast<size_t>(t) * D) + 2 * c);
      const float4 s1 = __ldcg(reinterpret_cast<const float4*>(bd.stream + static_cast<size_t>(t) * D) + 2 * c + 1);
      const float4 a0 = __ldg(reinterpret_cast<const float4*>(bd.alpha) + 2 * c), a1 = __ldg(reinterpret_cast<const float4*>(bd.alpha) + 2 * c + 1);
      const float4 b0 = __ldg(reinterpret_cast<const float4*>(bd.beta) + 2 * c), b1 = __ldg(reinterpret_cast<const float4*>(bd.beta) + 2 * c + 1);
      const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      const float al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float be[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        ss = fmaf(a[j][i], a[j][i], ss);
        v[j][i] = al[i] * sv[i];
        a[j][i] *= be[i];
      }
    }
  }
  const float r1 = block_inv(ss, BND_POST_EPS);
  ss = 0.f;
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + j * NT;
    if (c < cpt) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[j][i] = fmaf(a[j][i], r1, v[j][i]);
        ss = fmaf(v[j][i], v[j][i], ss);
      }
      if (bd.stream1) {
        float4* gp = reinterpret_cast<float4*>(bd.stream1 + static_cast<size_t>(t) * D) + 2 * c;
        gp[0] = make_float4(v[j][0], v[j][1], v[j][2], v[j][3]);
        gp[1] = make_float4(v[j][4], v[j][5], v[j][6], v[j][7]);
      }
    }
  }
  const float r2 = block_inv(ss, BND_RMS_EPS);
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + j * NT;
    if (c < cpt) {
      float w[8], h[8];
      bf16x8_to_f32(__ldg(reinterpret_cast<const uint4*>(bd.norm_w) + c), w);
#pragma unroll
      for (int i = 0; i < 8; ++i) h[i] = v[j][i] * r2 * (1.f + w[i]);
      if (bd.h)
        reinterpret_cast<uint4*>(bd.h + static_cast<size_t>(t) * D)[c] =
            make_uint4(pack_bf16x2(h[0], h[1]), pack_bf16x2(h[2], h[3]), pack_bf16x2(h[4], h[5]), pack_bf16x2(h[6], h[7]));
      if (bd.h_f32) {
        float4* gp = reinterpret_cast<float4*>(bd.h_f32 + static_cast<size_t>(t) * D) + 2 * c;
        gp[0] = make_float4(h[0], h[1], h[2], h[3]);
        gp[1] = make_float4(h[4], h[5], h[6], h[7]);
      }
    }
  }
}

// ---------------------------------------------------------------- boundary + pooler + router in one launch
//
// The three kernels the decode layer runs between the `o` projection and the experts (boundary, pooler, and the
// router on a side stream: best_submissions/muse_decode_layer.py:855-869) as ONE launch for up to 8 tokens.
// Every CTA first issues the weight loads of its first row group. One CTA per token then computes its boundary
// (one 8-element chunk per thread, values in registers between the two CTA-wide reductions), writes stream1, h as
// BF16 hi (the layer's BF16 h) + BF16 lo (the remainder of the FP32 value) and, where asked, the FP32 h to global
// memory and releases flag t. Every CTA waits (bounded) for the m flags and takes its x from those rows: the first
// `pooler_ctas` CTAs walk the pooler's BF16 rows with the hi fragments held in registers (as fewtok_xreg_kernel),
// the others the router's rows, given as the BF16 hi + lo halves of the FP32 weight, with the hi and lo rows of h
// copied to shared memory: x_hi W_hi + x_hi W_lo + x_lo W_hi, the three MMAs of the FP32-input mode with both
// splits made once instead of per use, which leaves the registers for a whole 8-row group (hi and lo) in flight. Rebuilding h in every CTA instead costs about a
// microsecond per token of shared-memory traffic on every SM; here it is computed once and read from L2.
// The producers wait for nobody, so nothing can wait in a circle; the grid is at most one CTA per SM. The last
// CTA to have read its fragments (a counter) puts the flags and the counter back to zero for the next call.
__device__ __forceinline__ void split_hi_lo_pair(uint32_t a_bits, uint32_t b_bits, uint32_t& hi, uint32_t& lo) {
  const float a = __uint_as_float(a_bits), b = __uint_as_float(b_bits);
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  const float ra = a - __uint_as_float(hi << 16), rb = b - __uint_as_float(hi & 0xffff0000u);
  const __nv_bfloat162 l = __floats2bfloat162_rn(ra, rb);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}
__device__ __forceinline__ uint4 ld_cg16(const void* p) {   // L2 load of data another CTA of this launch wrote
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

constexpr int FB_NW = 16, FB_U = 8, FB_NT = FB_NW * 32;   // 512 threads: 16 warps x 8 pieces of 32 elements = K up to 4096
constexpr int FB_DONE = BND_TOKENS;                        // cnt[0..7]: token ready flags; cnt[8]: CTAs that have read them
// Every CTA but the producers sleeps this long before its first weight loads, so that the producers' 40 KB of
// input is ahead of 12 MB of weight in the memory system's queues: measured on cold weights 8.0 / 8.7 / 10.0 us
// per call at 1 / 4 / 8 tokens against 8.7 / 9.3 / 10.5 without (600 and 1000 ns: no better).
constexpr int FB_STAGGER_NS = 300;

// Sum over the CTA; every thread gets the total. red: [FB_NW] floats.
__device__ __forceinline__ float fb_block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();   // red is free again
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x & 31) < FB_NW ? red[threadIdx.x & 31] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// Every thread of the CTA: wait (bounded) until the m tokens are published, thread t on flag t. CTA-uniform result.
__device__ __forceinline__ bool fb_wait_tokens(const int* cnt, int m) {
  bool ready = true;
  if (threadIdx.x < m) {
    const unsigned long long t0 = global_ns();
    while (ld_acquire_gpu(cnt + threadIdx.x) == 0) {
      if (global_ns() - t0 > WAIT_LIMIT_NS) {
        ready = false;
        break;
      }
    }
  }
  return __syncthreads_and(ready ? 1 : 0) != 0;
}

// One row group's 64 partial sums per warp -> out[t][8 rows]: every warp has written red[warp][64] and the CTA has
// synchronised; threads 0..63 add the warps up.
template <typename OutT>
__device__ __forceinline__ void fb_store_group(const float (*red)[64], OutT* out, int ld_out, int m, int N, int row0) {
  if (threadIdx.x < 64) {
    float sum = 0.f;
#pragma unroll 8
    for (int wv = 0; wv < FB_NW; ++wv) sum += red[wv][threadIdx.x];
    const int t = threadIdx.x >> 3, r = row0 + (threadIdx.x & 7);
    if (t < m && r < N) {
      if constexpr (sizeof(OutT) == 4) out[static_cast<size_t>(t) * ld_out + r] = sum;
      else out[static_cast<size_t>(t) * ld_out + r] = __float2bfloat16_rn(sum);
    }
  }
}

__global__ void __launch_bounds__(FB_NT, 1)
fused_boundary_kernel(const __nv_bfloat16* __restrict__ Wp, const __nv_bfloat16* __restrict__ Wr_hi,
                      const __nv_bfloat16* __restrict__ Wr_lo, const __grid_constant__ BoundaryArgs bd,
                      __nv_bfloat16* __restrict__ h_lo, __nv_bfloat16* __restrict__ outp, float* __restrict__ outr, int m, int Np,
                      int Nr, int K, int ld_outp, int ld_outr, int pooler_ctas, int stagger_ns, int* __restrict__ cnt,
                      int* __restrict__ status) {
  extern __shared__ __align__(16) uint8_t fb_x[];        // router CTAs: h hi rows then h lo rows, [2][m][2 K + pad]
  __shared__ __align__(16) float red[2][FB_NW][64];
  __shared__ float bsum[FB_NW];
  __shared__ __align__(8) uint64_t xbar;
  // Diagnostic builds: thread 0 of every CTA stamps the global nanosecond timer into its 16 slots (0 entry, 1 first
  // loads issued, 7 / 8 / 2 producers: input arrived / rows stored / token published, 3 all tokens seen,
  // 4 fragments ready, 5 first group multiplied, 6 exit).
  unsigned long long* const trace = MUSE_TRACE_BASE();
  unsigned long long* const tr = trace && threadIdx.x == 0 ? trace + 16ull * blockIdx.x : nullptr;
#define FB_STAMP(slot) do { if (tr) tr[slot] = global_ns(); } while (0)
  FB_STAMP(0);
  griddep_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  const int kblocks = K >> 5, first = warp * FB_U;
  bool ok;
  int arrived = 0;   // thread 0: this CTA's number among those that have seen the tokens

  if (static_cast<int>(blockIdx.x) >= pooler_ctas) {
    // ================================================================ router CTAs
    const int C = static_cast<int>(gridDim.x) - pooler_ctas, c = static_cast<int>(blockIdx.x) - pooler_ctas;
    const int groups = (Nr + 7) >> 3, my_groups = c < groups ? (groups - c + C - 1) / C : 0;
    const uint32_t xrow = static_cast<uint32_t>(K) * 2u + FEWTOK_X_PAD;
    if (threadIdx.x == 0) {
      mbar_init(smem_u32(&xbar), 1);
      fence_mbar_init();
    }
    if (stagger_ns > 0) __nanosleep(stagger_ns);   // the producers' input goes to the memory system first
    // A WHOLE group in flight, hi and lo halves: 8 pieces of 16 bytes each (x stays in shared memory, which leaves
    // the registers for it).
    uint4 wh[FB_U], wl[FB_U];
    auto load = [&](int i) {
      int r = (c + i * C) * 8 + g;
      r = r < Nr ? r : Nr - 1;
      const uint4* ph = reinterpret_cast<const uint4*>(Wr_hi + static_cast<size_t>(r) * K) + q;
      const uint4* pl = reinterpret_cast<const uint4*>(Wr_lo + static_cast<size_t>(r) * K) + q;
#pragma unroll
      for (int u = 0; u < FB_U; ++u) {
        const bool in = first + u < kblocks;
        wh[u] = in ? ldg_stream16(ph + (first + u) * 4) : make_uint4(0u, 0u, 0u, 0u);
        wl[u] = in ? ldg_stream16(pl + (first + u) * 4) : make_uint4(0u, 0u, 0u, 0u);
      }
    };
    if (my_groups > 0) load(0);
    griddep_wait();   // only weights so far (they may have left under the previous kernel's tail); flags and h come after
    FB_STAMP(1);
    ok = fb_wait_tokens(cnt, m);
    if (threadIdx.x == 0) arrived = atomicAdd(cnt + FB_DONE, 1);   // consumed at the end: the round trip overlaps the walk
    FB_STAMP(3);
    // The rows into shared memory by one thread's bulk copies (they were written through the generic proxy, hence
    // the proxy fence).
    if (ok && threadIdx.x == 0) {
      asm volatile("fence.proxy.async;" ::: "memory");
      mbar_expect_tx(smem_u32(&xbar), static_cast<uint32_t>(m) * static_cast<uint32_t>(K) * 4u);
      for (int t = 0; t < m; ++t) {
        bulk_load_1d(smem_u32(fb_x) + static_cast<uint32_t>(t) * xrow, bd.h + static_cast<size_t>(t) * K, static_cast<uint32_t>(K) * 2u,
                     smem_u32(&xbar));
        bulk_load_1d(smem_u32(fb_x) + static_cast<uint32_t>(m + t) * xrow, h_lo + static_cast<size_t>(t) * K,
                     static_cast<uint32_t>(K) * 2u, smem_u32(&xbar));
      }
    }
    if (ok) ok = __syncthreads_and(mbar_wait(smem_u32(&xbar), 0) ? 1 : 0) != 0;
    FB_STAMP(4);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const uint8_t* const xh = fb_x + static_cast<uint32_t>(g < m ? g : 0) * xrow + q * 16;
    const uint8_t* const xl = xh + static_cast<uint32_t>(m) * xrow;
    for (int i = 0; i < (ok ? my_groups : 0); ++i) {
#pragma unroll
      for (int u = 0; u < FB_U; ++u) {
        uint4 xa = make_uint4(0u, 0u, 0u, 0u), xb = xa;
        if (g < m && first + u < kblocks) {
          xa = *reinterpret_cast<const uint4*>(xh + (first + u) * 64);
          xb = *reinterpret_cast<const uint4*>(xl + (first + u) * 64);
        }
        mma_bf16_16816(acc, xa.x, 0u, xa.y, 0u, wh[u].x, wh[u].y);   // x_hi W_hi, x_hi W_lo, x_lo W_hi
        mma_bf16_16816(acc, xa.z, 0u, xa.w, 0u, wh[u].z, wh[u].w);
        mma_bf16_16816(acc, xa.x, 0u, xa.y, 0u, wl[u].x, wl[u].y);
        mma_bf16_16816(acc, xa.z, 0u, xa.w, 0u, wl[u].z, wl[u].w);
        mma_bf16_16816(acc, xb.x, 0u, xb.y, 0u, wh[u].x, wh[u].y);
        mma_bf16_16816(acc, xb.z, 0u, xb.w, 0u, wh[u].z, wh[u].w);
      }
      if (i + 1 < my_groups) load(i + 1);
      *reinterpret_cast<float2*>(&red[i & 1][warp][g * 8 + 2 * q]) = make_float2(acc[0], acc[1]);
      acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
      __syncthreads();   // the buffer written two groups ago is free again once every warp passed this
      if (i == 0) FB_STAMP(5);
      fb_store_group(red[i & 1], outr, ld_outr, m, Nr, (c + i * C) * 8);
    }
  } else {
    // ================================================================ pooler CTAs (the last m of them produce h)
    const int C = pooler_ctas, c = static_cast<int>(blockIdx.x);
    const int groups = (Np + 7) >> 3, my_groups = c < groups ? (groups - c + C - 1) / C : 0;
    // The producer of token t is pooler CTA pooler_ctas - 1 - t (the last CTAs walk the fewest groups). Its own
    // input loads go out ahead of its weight loads: everybody waits for it.
    const int tok = pooler_ctas - 1 - c;
    const bool producer = tok < m;
    const int ch = threadIdx.x;
    const bool live = producer && ch < (K >> 3);
    uint4 av = make_uint4(0u, 0u, 0u, 0u), nw = av;
    float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s4 = s0, a0 = s0, a1 = s0, b0 = s0, b1 = s0;
    if (producer) griddep_wait();   // its input is the output of the kernels ahead in the stream
    if (live) {
      av = __ldcg(reinterpret_cast<const uint4*>(bd.attn + static_cast<size_t>(tok) * K) + ch);
      s0 = __ldcg(reinterpret_cast<const float4*>(bd.stream + static_cast<size_t>(tok) * K) + 2 * ch);
      s4 = __ldcg(reinterpret_cast<const float4*>(bd.stream + static_cast<size_t>(tok) * K) + 2 * ch + 1);
      a0 = __ldg(reinterpret_cast<const float4*>(bd.alpha) + 2 * ch);
      a1 = __ldg(reinterpret_cast<const float4*>(bd.alpha) + 2 * ch + 1);
      b0 = __ldg(reinterpret_cast<const float4*>(bd.beta) + 2 * ch);
      b1 = __ldg(reinterpret_cast<const float4*>(bd.beta) + 2 * ch + 1);
      nw = __ldg(reinterpret_cast<const uint4*>(bd.norm_w) + ch);
    }
    uint4 w[FB_U];
    auto load = [&](int i) {
      int r = (c + i * C) * 8 + g;
      r = r < Np ? r : Np - 1;
      const uint4* p = reinterpret_cast<const uint4*>(Wp + static_cast<size_t>(r) * K) + q;
#pragma unroll
      for (int u = 0; u < FB_U; ++u) w[u] = first + u < kblocks ? ldg_stream16(p + (first + u) * 4) : make_uint4(0u, 0u, 0u, 0u);
    };
    // A producer loads its first weights only after it has published (its release would wait for them).
    if (!producer) {
      if (stagger_ns > 0) __nanosleep(stagger_ns);   // the producers' input goes to the memory system first
      if (my_groups > 0) load(0);
      griddep_wait();   // only weights so far; flags and h come after
    }
    FB_STAMP(1);
    if (producer) {   // token `tok`'s boundary, one chunk of 8 elements per thread (K / 8 <= 512)
      float a[8], s1[8], ow[8];
      const float be[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      bf16x8_to_f32(av, a);
      bf16x8_to_f32(nw, ow);
      s1[0] = a0.x * s0.x; s1[1] = a0.y * s0.y; s1[2] = a0.z * s0.z; s1[3] = a0.w * s0.w;
      s1[4] = a1.x * s4.x; s1[5] = a1.y * s4.y; s1[6] = a1.z * s4.z; s1[7] = a1.w * s4.w;
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(a[i], a[i], ss);
      const float r1 = rsqrtf(fb_block_sum(ss, bsum) / static_cast<float>(K) + BND_POST_EPS);
      FB_STAMP(7);
      ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        s1[i] = fmaf(be[i] * a[i], r1, s1[i]);
        ss = fmaf(s1[i], s1[i], ss);
      }
      const float r2 = rsqrtf(fb_block_sum(ss, bsum) / static_cast<float>(K) + BND_RMS_EPS);
      if (live) {
        float h[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = s1[i] * r2 * (1.f + ow[i]);
        if (bd.h_f32) {
          float4* hf = reinterpret_cast<float4*>(bd.h_f32 + static_cast<size_t>(tok) * K) + 2 * ch;
          hf[0] = make_float4(h[0], h[1], h[2], h[3]);
          hf[1] = make_float4(h[4], h[5], h[6], h[7]);
        }
        uint4 hi, lo;   // h = hi + lo in BF16: hi is the layer's BF16 h, lo the remainder the router adds back
        split_hi_lo_pair(__float_as_uint(h[0]), __float_as_uint(h[1]), hi.x, lo.x);
        split_hi_lo_pair(__float_as_uint(h[2]), __float_as_uint(h[3]), hi.y, lo.y);
        split_hi_lo_pair(__float_as_uint(h[4]), __float_as_uint(h[5]), hi.z, lo.z);
        split_hi_lo_pair(__float_as_uint(h[6]), __float_as_uint(h[7]), hi.w, lo.w);
        reinterpret_cast<uint4*>(bd.h + static_cast<size_t>(tok) * K)[ch] = hi;
        reinterpret_cast<uint4*>(h_lo + static_cast<size_t>(tok) * K)[ch] = lo;
        if (bd.stream1) {
          float4* gp = reinterpret_cast<float4*>(bd.stream1 + static_cast<size_t>(tok) * K) + 2 * ch;
          gp[0] = make_float4(s1[0], s1[1], s1[2], s1[3]);
          gp[1] = make_float4(s1[4], s1[5], s1[6], s1[7]);
        }
      }
      __syncthreads();   // every thread's stores precede thread 0's release (cumulative at GPU scope)
      FB_STAMP(8);
      if (threadIdx.x == 0) st_release_gpu(cnt + tok, 1);
      FB_STAMP(2);
      if (my_groups > 0) load(0);
    }
    ok = fb_wait_tokens(cnt, m);
    if (threadIdx.x == 0) arrived = atomicAdd(cnt + FB_DONE, 1);   // consumed at the end: the round trip overlaps the walk
    FB_STAMP(3);
    uint4 xr[FB_U];   // the BF16 fragments, straight from L2
#pragma unroll
    for (int u = 0; u < FB_U; ++u)
      xr[u] = (ok && g < m && first + u < kblocks) ? ld_cg16(bd.h + static_cast<size_t>(g) * K + (first + u) * 32 + q * 8)
                                                   : make_uint4(0u, 0u, 0u, 0u);
    FB_STAMP(4);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < (ok ? my_groups : 0); ++i) {
#pragma unroll
      for (int u = 0; u < FB_U; ++u) {
        mma_bf16_16816(acc, xr[u].x, 0u, xr[u].y, 0u, w[u].x, w[u].y);
        mma_bf16_16816(acc, xr[u].z, 0u, xr[u].w, 0u, w[u].z, w[u].w);
      }
      if (i + 1 < my_groups) load(i + 1);
      *reinterpret_cast<float2*>(&red[i & 1][warp][g * 8 + 2 * q]) = make_float2(acc[0], acc[1]);
      acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
      __syncthreads();
      if (i == 0) FB_STAMP(5);
      fb_store_group(red[i & 1], outp, ld_outp, m, Np, (c + i * C) * 8);
    }
  }
  if (!ok && threadIdx.x == 0) atomicOr(status, ST_X_TIMEOUT);
  // Every CTA counted itself once it had seen the flags; the last one to do so re-arms them for the next call.
  if (threadIdx.x == 0 && arrived == static_cast<int>(gridDim.x) - 1) {
    for (int t = 0; t < BND_TOKENS; ++t) cnt[t] = 0;
    cnt[FB_DONE] = 0;
  }
  FB_STAMP(6);
#undef FB_STAMP
}

static int boundary_args_ok(const BoundaryArgs& bd, int m, int D) {
  if (!bd.stream || !bd.attn || !bd.alpha || !bd.beta || !bd.norm_w || m < 1 || D < 8 || D % 8) return -1;
  const uintptr_t all = reinterpret_cast<uintptr_t>(bd.stream) | reinterpret_cast<uintptr_t>(bd.attn) |
                        reinterpret_cast<uintptr_t>(bd.alpha) | reinterpret_cast<uintptr_t>(bd.beta) |
                        reinterpret_cast<uintptr_t>(bd.norm_w) | reinterpret_cast<uintptr_t>(bd.stream1) |
                        reinterpret_cast<uintptr_t>(bd.h) | reinterpret_cast<uintptr_t>(bd.h_f32);
  return (all & 15) ? -2 : 0;   // contiguous rows of 16-byte vectors
}

int attn_boundary_dispatch(const BoundaryArgs& bd, int m, int D, cudaStream_t stream) {
  const int bad = boundary_args_ok(bd, m, D);
  if (bad) return bad;
  if (D > 8192) return -2;
  if (!bd.stream1 && !bd.h && !bd.h_f32) return -1;
  return static_cast<int>(launch_dependent(attn_boundary_kernel, dim3(m), dim3(256), 0, stream, bd, D));
}

// The projection with the boundary as its prologue: 16 warps x 8 loads (K <= 4096), up to 8 tokens, and at least
// as many 8-row groups as tokens (CTA t publishes token t). f32w = the router's FP32 weight and output.
template <bool F32W>
static cudaError_t launch_boundary(const void* W, void* out, int m, int N, int K, int ld_out, int* status, const BoundaryArgs& bd,
                                   cudaStream_t s) {
  static int sms[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  const size_t smem = boundary_smem_bytes(K);
  if (!sms[dev]) {
    int v = 0;
    if ((e = cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    if constexpr (F32W) {
      if ((e = cudaFuncSetAttribute(fewtok_xreg_f32_kernel<16, 8, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(boundary_smem_bytes(4096)))) != cudaSuccess) return e;
    } else {
      if ((e = cudaFuncSetAttribute(fewtok_xreg_kernel<16, 8, false, false, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(boundary_smem_bytes(4096)))) != cudaSuccess) return e;
      if ((e = cudaFuncSetAttribute(fewtok_xreg_kernel<16, 8, false, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(boundary_smem_bytes(4096)))) != cudaSuccess) return e;
    }
    sms[dev] = v;
  }
  int walkers = sms[dev];   // 512 threads with up to 128 registers and 128 KB of shared memory: one CTA per SM
  const int groups = (N + 7) / 8;
  if (walkers > groups) walkers = groups;
  if constexpr (F32W) {
    return launch_dependent(fewtok_xreg_f32_kernel<16, 8, true, true>, dim3(walkers), dim3(512), smem, s, reinterpret_cast<const float*>(W),
                            nullptr, reinterpret_cast<float*>(out), m, N, K, K, ld_out, 1, bd);
  } else {
    const bool vec = N % 8 == 0 && ((reinterpret_cast<uintptr_t>(out) | (static_cast<uintptr_t>(ld_out) * 2)) & 15) == 0;
    if (vec)
      return launch_dependent(fewtok_xreg_kernel<16, 8, false, false, true, true>, dim3(walkers), dim3(512), smem, s,
                              reinterpret_cast<const __nv_bfloat16*>(W), nullptr, reinterpret_cast<__nv_bfloat16*>(out), m, N, K, K, ld_out,
                              1, status, PeerSync{}, bd);
    return launch_dependent(fewtok_xreg_kernel<16, 8, false, false, false, true>, dim3(walkers), dim3(512), smem, s,
                            reinterpret_cast<const __nv_bfloat16*>(W), nullptr, reinterpret_cast<__nv_bfloat16*>(out), m, N, K, K, ld_out, 1,
                            status, PeerSync{}, bd);
  }
}

int fewtok_boundary_dispatch(const void* W, int w_is_f32, const BoundaryArgs& bd, void* out, int m, int N, int K, int ld_out,
                             int* status, cudaStream_t stream) {
  if (!W || !out || N <= 0 || (!w_is_f32 && !status)) return -1;
  const int bad = boundary_args_ok(bd, m, K);
  if (bad) return bad;
  if (m > BND_TOKENS || (N + 7) / 8 < m) return -9;
  if (K % 32 != 0 || K / 32 > 128 || ld_out < N || (reinterpret_cast<uintptr_t>(W) & 15)) return -2;
  const cudaError_t e = w_is_f32 ? launch_boundary<true>(W, out, m, N, K, ld_out, status, bd, stream)
                                 : launch_boundary<false>(W, out, m, N, K, ld_out, status, bd, stream);
  return static_cast<int>(e);
}

// Whether (warps, unroll) has a register-resident instantiation for CTAs of `toks` (8 or 16) tokens.
static bool xreg_serves(int toks, int K, int warps, int unroll) {
  if (K / 32 > warps * unroll) return false;
  if (warps == 16) return unroll == 1 || unroll == 2 || unroll == 4 || unroll == 8;
  if (warps == 32) return unroll == 1 || unroll == 2 || (unroll == 4 && toks <= 8);
  return false;
}

// 1..16 tokens, BF16 weight and output; warps in {16, 32}, unroll in {1, 2, 4}, and 8 with 16 warps when
// that covers a whole row (K <= 4096). Negative = argument error.
int fewtok_mma_dispatch(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out, int warps,
                        int unroll, int tok_split, int* status, const PeerSync* peers, cudaStream_t stream) {
  PeerSync ps = {};
  if (peers && peers->world > 1) {
    ps = *peers;
    if (ps.world > MAX_WORLD || ps.rank < 0 || ps.rank >= ps.world || ps.col0 < 0) return -8;
    for (int p = 0; p < ps.world; ++p)
      if (!ps.out[p] || !ps.flags[p]) return -8;
    out = ps.out[ps.rank];
    // the exchange: equal slices side by side, whole 16-byte vectors, staging for LL_TOKENS tokens
    if (ld_out < ps.world * N || ps.col0 != ps.rank * N || N % 8 != 0 || ld_out % 8 != 0 || m > LL_TOKENS) return -8;
    for (int p = 0; p < ps.world; ++p)
      if (!ps.ll[p] || (reinterpret_cast<uintptr_t>(ps.ll[p]) & 15) || (reinterpret_cast<uintptr_t>(ps.out[p]) & 15)) return -8;
  }
  if (!W || !x || !out || !status || N <= 0 || K <= 0) return -1;
  if (tok_split < 1 || tok_split > 4 || m < 1 || m > 16 * tok_split) return -9;
  const int toks = m <= 8 * tok_split ? 8 : 16;   // tokens per CTA
  if (K % 32 != 0 || ld_x % 8 != 0 || ld_x < K || ld_out < N) return -2;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return -2;
  cudaError_t e = cudaErrorInvalidValue;
  if (xreg_serves(toks, K, warps, unroll)) {   // a whole row per batch: the A fragments stay in registers
#define MUSE_XREG(NW_, U_, HI_)                                 \
    if (warps == NW_ && unroll == U_ && (toks > 8) == HI_)      \
      e = launch_xreg<NW_, U_, HI_>(W, x, out, m, N, K, ld_x, ld_out, tok_split, status, ps, stream);
    MUSE_XREG(32, 1, false) MUSE_XREG(32, 2, false) MUSE_XREG(32, 4, false) MUSE_XREG(32, 1, true) MUSE_XREG(32, 2, true)
    MUSE_XREG(16, 1, false) MUSE_XREG(16, 2, false) MUSE_XREG(16, 4, false) MUSE_XREG(16, 8, false)
    MUSE_XREG(16, 1, true) MUSE_XREG(16, 2, true) MUSE_XREG(16, 4, true) MUSE_XREG(16, 8, true)
#undef MUSE_XREG
    return static_cast<int>(e);
  }
  if (tok_split != 1) return -9;   // the shared-memory path holds all of a call's tokens in one CTA
  if (peer_active_host(ps)) return -8;   // and has no exchange epilogue
  if (fewtok_smem(K, m, warps) > 227 * 1024) return -5;
#define MUSE_FEWTOK(NW_, U_)                                                                                    \
  if (warps == NW_ && unroll == U_)                                                                             \
    e = m > 8 ? launch_fewtok<NW_, U_, true>(W, x, out, m, N, K, ld_x, ld_out, status, stream)                  \
              : launch_fewtok<NW_, U_, false>(W, x, out, m, N, K, ld_x, ld_out, status, stream);
  MUSE_FEWTOK(32, 1) MUSE_FEWTOK(32, 2) MUSE_FEWTOK(32, 4) MUSE_FEWTOK(16, 1) MUSE_FEWTOK(16, 2) MUSE_FEWTOK(16, 4)
#undef MUSE_FEWTOK
  if (e == cudaErrorInvalidConfiguration) return -5;
  return static_cast<int>(e);
}

// One launch for boundary -> pooler + router (up to 8 tokens, K <= 4096 in whole 32-element pieces, at least 8 m
// pooler rows so that CTA t exists for every token t). At most one CTA per SM: the consumers of a token's h
// spin while its producer runs. cnt: 9 ints, zero before the first call and again after every call. h_lo: [m, K]
// BF16 scratch the CTAs hand the low half of h to one another through.
int fused_boundary_dispatch(const void* Wp, const void* Wr_hi, const void* Wr_lo, const BoundaryArgs& bd, void* h_lo, void* outp,
                            void* outr, int m, int Np, int Nr, int K, int ld_outp, int ld_outr, int* cnt, int* status,
                            cudaStream_t stream) {
  if (!Wp || !Wr_hi || !Wr_lo || !h_lo || !outp || !outr || !cnt || !status || Np <= 0 || Nr <= 0 || !bd.h) return -1;
  const int bad = boundary_args_ok(bd, m, K);
  if (bad) return bad;
  if (m > BND_TOKENS) return -9;
  if (K % 32 != 0 || K / 32 > FB_NW * FB_U || ld_outp < Np || ld_outr < Nr) return -2;
  if ((reinterpret_cast<uintptr_t>(Wp) | reinterpret_cast<uintptr_t>(Wr_hi) | reinterpret_cast<uintptr_t>(Wr_lo) |
       reinterpret_cast<uintptr_t>(h_lo)) & 15)
    return -2;
  static int sms[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return static_cast<int>(cudaErrorInvalidDevice);
  const auto x_bytes = [](int tokens, int k) { return static_cast<size_t>(2 * tokens) * (static_cast<size_t>(k) * 2 + FEWTOK_X_PAD); };
  if (!sms[dev]) {
    int v = 0;
    if ((e = cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return static_cast<int>(e);
    if ((e = cudaFuncSetAttribute(fused_boundary_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(x_bytes(BND_TOKENS, FB_NW * FB_U * 32)))) != cudaSuccess)
      return static_cast<int>(e);
    sms[dev] = v;
  }
  // The router's groups are twice the bytes of the pooler's: give each router group a CTA of its own (up to a
  // quarter of the SMs), the pooler the rest.
  const int gp = (Np + 7) / 8, gr = (Nr + 7) / 8;
  const int rc = gr < sms[dev] / 4 ? gr : sms[dev] / 4;
  const int pc = sms[dev] - rc < gp ? sms[dev] - rc : gp;
  if (pc < m) return -9;   // one pooler CTA per token publishes it
  return static_cast<int>(launch_dependent(
      fused_boundary_kernel, dim3(pc + rc), dim3(FB_NT), x_bytes(m, K), stream, reinterpret_cast<const __nv_bfloat16*>(Wp),
      reinterpret_cast<const __nv_bfloat16*>(Wr_hi), reinterpret_cast<const __nv_bfloat16*>(Wr_lo), bd, reinterpret_cast<__nv_bfloat16*>(h_lo),
      reinterpret_cast<__nv_bfloat16*>(outp), reinterpret_cast<float*>(outr), m, Np, Nr, K, ld_outp, ld_outr, pc, FB_STAGGER_NS, cnt, status));
}

}  // namespace muse
