// out[m, n] = x[m, K] . W[n, K]^T for small m, computed as out^T = W . x^T ("swap AB") so that a
// 128-row weight tile is the wide tensor-core operand and all tokens of a token tile ride along as
// the narrow one. Replaces the reference's Triton kernels: _swab_kernel
// (best_submissions/muse_bf16_proj.py:236-257), _router_kernel (:260-287), the split-K hand-off
// _finish (:215-233) and, with NTOK up to 256, the cuBLAS call for m > 32 (:390).
//
// One CTA = one (weight-row tile, K slice, token tile) unit:
//   warp 0 / lane 0   TMA producer: per 64-wide K chunk, one W box [128 x 64] (plus the "lo" box for the
//                     router's BF16 hi+lo pair) and one x box [NTOK x 64], 128-byte swizzled, into a
//                     ring of `stages` shared-memory stages, completion counted on an mbarrier. The
//                     first `stages` chunks are requested before anything else in the CTA is set up;
//   warp 1 / lane 0   MMA issuer: four tcgen05.mma (M=128, N=NTOK, K=16) per chunk -- eight for hi+lo,
//                     both halves into the same FP32 accumulator in TMEM -- then tcgen05.commit frees
//                     the stage; a last commit signals the epilogue;
//   all four warps    epilogue: thread = weight row (TMEM lane), registers = tokens.
//
// Split-K reduction. The `split` K slices of a tile are `groups` clusters of `cluster` CTAs
// (cluster dims (1, cluster, 1), consecutive blockIdx.y). Inside a cluster the partial tiles never
// leave the chip: the tile's tokens are dealt out to the cluster's CTAs in blocks of T, and every CTA
// PUSHES, straight from its accumulator registers, each block to its owner's shared memory with
// st.async (slot = sender's rank), counted in bytes on the owner's mbarrier. The owner waits for its
// barrier only, sums the slots in rank order (bit-reproducible) and writes the output. The only
// cluster-wide barrier is armed at start-up and has long completed when it is waited on.
// Only when groups > 1 do the cluster sums go through an FP32 workspace with vector red.global.add;
// the last CTA to arrive on the tile's counter reads the totals back, writes the output and restores
// workspace and counter to zero. No CTA waits on a CTA outside its (co-scheduled) cluster, the launch
// is a single kernel and leaves every scratch byte as it found it, so it can be captured in a CUDA
// graph and replayed.
#include "common.cuh"

namespace muse {

constexpr int TILE_ROWS = 128;  // weight rows per CTA = MMA M
constexpr int BK = 64;          // K elements per stage = one 128-byte swizzle span of BF16
constexpr int MAX_STAGES = 12;
constexpr int MAX_CLUSTER = 16;

template <int NTOK, bool HILO>
struct SkinnyCfg {
  static constexpr int A_BYTES = TILE_ROWS * BK * 2;
  static constexpr int B_BYTES = NTOK * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES * (HILO ? 2 : 1) + B_BYTES;
  static constexpr int TMEM_COLS = NTOK < 32 ? 32 : NTOK;
};

// Tokens per owner CTA when `mvalid` tokens are dealt to `cluster` CTAs: whole groups of four
// (one 16-byte st.async each). Shared by the kernel and the host-side shared-memory sizing.
__host__ __device__ constexpr int owner_block(int mvalid, int cluster) {
  return (((mvalid + cluster - 1) / cluster) + 3) & ~3;
}

// ---- thread-block cluster helpers (a launch without a cluster attribute is a cluster of one)
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
// Arrival without its own release: the caller has already fenced what the peers need to see.
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_smem, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem), "r"(rank));
  return r;
}
// 16 bytes from registers into a peer's (or our own) shared memory; the peer's mbarrier counts them.
__device__ __forceinline__ void st_async_f32x4(uint32_t remote_addr, float a, float b, float c, float d,
                                               uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1,%2,%3,%4}, [%5];" ::"r"(
                   remote_addr),
               "f"(a), "f"(b), "f"(c), "f"(d), "r"(remote_bar)
               : "memory");
}
__device__ __forceinline__ void red_add_f32x4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ float4 ldg_cg_f32x4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void stg_cg_f32x4(float* p, float4 v) {
  asm volatile("st.global.cg.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// Eight consecutive output features of one token, starting at feature n0 (a multiple of 8).
// `col0` shifts the destination column (this rank's slice inside a gathered output); bounds use n0 < n.
__device__ __forceinline__ void store_out8(void* out, int out_f32, bool vec_ok, size_t token, int ld_out, int n0, int n,
                                           int col0, const float4& lo, const float4& hi) {
  if (n0 >= n) return;
  const float a[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  if (out_f32) {
    float* o = reinterpret_cast<float*>(out) + token * ld_out + col0 + n0;
    if (vec_ok && n0 + 8 <= n) {
      *reinterpret_cast<float4*>(o) = lo;
      *reinterpret_cast<float4*>(o + 4) = hi;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (n0 + i < n) o[i] = a[i];
    }
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + token * ld_out + col0 + n0;
    if (vec_ok && n0 + 8 <= n) {
      __nv_bfloat162 p0 = __floats2bfloat162_rn(a[0], a[1]), p1 = __floats2bfloat162_rn(a[2], a[3]);
      __nv_bfloat162 p2 = __floats2bfloat162_rn(a[4], a[5]), p3 = __floats2bfloat162_rn(a[6], a[7]);
      uint4 v;
      v.x = *reinterpret_cast<uint32_t*>(&p0);
      v.y = *reinterpret_cast<uint32_t*>(&p1);
      v.z = *reinterpret_cast<uint32_t*>(&p2);
      v.w = *reinterpret_cast<uint32_t*>(&p3);
      *reinterpret_cast<uint4*>(o) = v;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (n0 + i < n) o[i] = __float2bfloat16_rn(a[i]);
    }
  }
}

// More tokens per thread than this go out through a shared-memory transpose as 16-byte vectors.
constexpr int DIRECT_STORE_TOKENS = 16;

template <int NTOK, bool HILO, bool PEERS>
__global__ void __launch_bounds__(128)
skinny_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_wlo,
                 const __grid_constant__ CUtensorMap tm_x, void* __restrict__ out, float* __restrict__ ws,
                 int* __restrict__ cnt, int* __restrict__ status, int m, int n, int chunks, int split, int stages,
                 int out_f32, int ld_out, const __grid_constant__ PeerSync ps) {
  using Cfg = SkinnyCfg<NTOK, HILO>;
  // Per-CTA phase stamps of diagnostic builds (SM cycle counter; slot 15 / 11 = global nanosecond timer at entry / exit).
  unsigned long long* const trace = MUSE_TRACE_BASE();
  unsigned long long* const tr =
      trace ? trace + 16ull * (blockIdx.x + gridDim.x * (blockIdx.y + static_cast<size_t>(gridDim.y) * blockIdx.z)) : nullptr;
#define MUSE_STAMP(slot) do { if (tr) tr[slot] = static_cast<unsigned long long>(clock64()); } while (0)
  if (tr && threadIdx.x == 0) { MUSE_STAMP(0); tr[15] = global_ns(); }
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_empty[MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_acc;
  __shared__ __align__(8) uint64_t bar_rx;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_abort;
  __shared__ int s_last;
  __shared__ int s_issued;
  __shared__ int s_epoch;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile_n = blockIdx.x, tile_m = blockIdx.z;
  const int tile_id = tile_m * gridDim.x + tile_n;
  // Balanced K slices (the host keeps chunks and split below 65536, so 32-bit products are exact).
  const int c0 = static_cast<int>(blockIdx.y * static_cast<uint32_t>(chunks) / static_cast<uint32_t>(split));
  const int c1 = static_cast<int>((blockIdx.y + 1u) * static_cast<uint32_t>(chunks) / static_cast<uint32_t>(split));
  const int nchunks = c1 - c0;
  // 1024-byte alignment: the 128-byte swizzle pattern repeats every 8 rows x 128 bytes.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  // ---- producer state lives in thread 0 across the set-up barrier
  uint64_t pol_w = 0, pol_x = 0;
  int issued = 0;
  auto issue_w = [&](int i, int s) {   // arms the stage's barrier for all of its bytes, then the weight tiles
    const uint32_t full = smem_u32(&bar_full[s]);
    const uint32_t a = smem_base + static_cast<uint32_t>(s) * Cfg::STAGE_BYTES;
    mbar_expect_tx(full, Cfg::STAGE_BYTES);
    tma_load_2d(a, &tm_w, (c0 + i) * BK, tile_n * TILE_ROWS, full, pol_w);
    if (HILO) tma_load_2d(a + Cfg::A_BYTES, &tm_wlo, (c0 + i) * BK, tile_n * TILE_ROWS, full, pol_w);
  };
  auto issue_x = [&](int i, int s) {
    const uint32_t full = smem_u32(&bar_full[s]);
    const uint32_t a = smem_base + static_cast<uint32_t>(s) * Cfg::STAGE_BYTES;
    tma_load_2d(a + Cfg::A_BYTES * (HILO ? 2 : 1), &tm_x, (c0 + i) * BK, tile_m * NTOK, full, pol_x);
    ++issued;
  };
  auto issue = [&](int i, int s) {
    issue_w(i, s);
    issue_x(i, s);
  };

  // The first thing a CTA does is get weight bytes moving: every stage starts empty, so thread 0
  // requests the first `stages` chunks before TMEM, the other warps or the cluster are ready.
  if (tid == 0) {
    MUSE_STAMP(13);
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_acc), 1);
    mbar_init(smem_u32(&bar_rx), 1);
    fence_mbar_init();
    MUSE_STAMP(14);
    pol_w = l2_policy_evict_first();  // weights are read once
    pol_x = l2_policy_evict_last();   // every CTA of the same K slice re-reads x
    // The weight tiles of the first stages leave now, the x tiles once the kernels ahead in the stream have completed
    // (a launch allowed to start under the previous kernel's tail touches only weights until then).
    const int pre = min(stages, nchunks);
    for (int i = 0; i < pre; ++i) issue_w(i, i);
    griddep_launch_dependents();
    griddep_wait();
    for (int i = 0; i < pre; ++i) issue_x(i, i);
    s_abort = 0;
    s_issued = 0;
    if constexpr (PEERS) {
      s_epoch = peer_epoch(ps);
      if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) peer_announce_enter(ps, s_epoch);
    }
    MUSE_STAMP(1);
  }

  const int csize = static_cast<int>(cluster_size()), crank = static_cast<int>(cluster_rank());
  const int groups = split / csize;
  const int tok0 = tile_m * NTOK;
  const int mvalid = min(NTOK, m - tok0);
  const int mpad = (mvalid + 3) & ~3;               // whole groups of four tokens (the padding tokens are zero)
  const int T = owner_block(mvalid, csize);         // tokens per owner CTA
  const int my_cnt = max(0, min(T, mpad - crank * T));  // tokens this CTA owns
  // Receive slots [sender rank][row][T tokens] sit behind the ring: peers may push while our ring is busy.
  // (The vector-store staging area overlays the ring and may be the larger of the two.)
  const uint32_t ring_bytes = static_cast<uint32_t>(stages) * Cfg::STAGE_BYTES;
  const int staged_tokens = csize == 1 ? mpad : T;  // what one CTA ever stages: all tokens, or the block it owns
  const uint32_t stage_bytes = staged_tokens > DIRECT_STORE_TOKENS ? static_cast<uint32_t>(staged_tokens) * TILE_ROWS * 4u : 0u;
  const uint32_t rx_base = smem_base + (ring_bytes > stage_bytes ? ring_bytes : stage_bytes);
  const float* const rx = reinterpret_cast<const float*>(smem_raw + (rx_base - smem_u32(smem_raw)));
  // Arm the receive barrier: every sender (ourselves included) pushes 128 rows x my_cnt tokens. This
  // precedes our arrival on the cluster barrier below, and no peer pushes before that barrier completes.
  if (tid == 0 && csize > 1 && my_cnt > 0)
    mbar_expect_tx(smem_u32(&bar_rx), static_cast<uint32_t>(csize) * TILE_ROWS * my_cnt * 4u);

  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
    if (lane == 0) MUSE_STAMP(12);
  }
  griddep_wait();   // every thread, before the first barrier: what follows reads and writes more than weights
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_acc = tmem_slot;
  // Tell the cluster that this CTA's barriers exist. Nobody waits for this until its own main loop
  // is over, by which time every peer arrived long ago.
  // (thread 0 released its barrier initialisation to the cluster with fence.mbarrier_init above.)
  if (csize > 1) cluster_arrive_relaxed();
  if (tid == 0) MUSE_STAMP(2);

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer, chunks beyond the first ring fill: wait for the stage's previous use to drain
      int s = 0;
      uint32_t phase = 0;
      for (int i = stages; i < nchunks; ++i) {
        if (!mbar_wait(smem_u32(&bar_empty[s]), phase)) {
          atomicOr(status, ST_PRODUCER_TIMEOUT);
          s_abort = 1;
          break;
        }
        issue(i, s);
        if (++s == stages) {
          s = 0;
          phase ^= 1u;
        }
      }
      s_issued = issued;
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer
      constexpr uint32_t idesc = umma_idesc_bf16(TILE_ROWS, NTOK);
      int s = 0;
      uint32_t phase = 0;
      for (int i = 0; i < nchunks; ++i) {
        if (!mbar_wait(smem_u32(&bar_full[s]), phase)) {
          atomicOr(status, ST_MMA_TIMEOUT);
          s_abort = 1;
          break;
        }
        tc_fence_after_sync();
        if (i == 0) MUSE_STAMP(3);
        const uint32_t a = smem_base + static_cast<uint32_t>(s) * Cfg::STAGE_BYTES;
        const uint64_t a_desc = umma_desc_k_sw128(a);
        const uint64_t b_desc = umma_desc_k_sw128(a + Cfg::A_BYTES * (HILO ? 2 : 1));
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          // 16 BF16 = 32 bytes further along K inside the swizzle span: +2 in 16-byte units.
          umma_bf16(tmem_acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
          if (HILO) {
            const uint64_t alo_desc = umma_desc_k_sw128(a + Cfg::A_BYTES);
            umma_bf16(tmem_acc, alo_desc + 2 * k, b_desc + 2 * k, idesc, 1u);
          }
        }
        umma_commit(smem_u32(&bar_empty[s]));
        if (++s == stages) {
          s = 0;
          phase ^= 1u;
        }
      }
      umma_commit(smem_u32(&bar_acc));  // also on the abort path, so that the epilogue is released
      MUSE_STAMP(4);
    }
    __syncwarp();
  }

  // ---- epilogue, all four warps: thread = weight row; warp w may only touch TMEM lanes [32w, 32w + 32)
  bool ok = mbar_wait(smem_u32(&bar_acc), 0);
  if (!ok && lane == 0) atomicOr(status, ST_EPILOGUE_TIMEOUT);
  ok = __syncthreads_and(ok && !s_abort);
  tc_fence_after_sync();
  if (tid == 0) MUSE_STAMP(5);

  const int r = warp * 32 + lane;
  const int n_idx = tile_n * TILE_ROWS + r;
  const bool row_ok = n_idx < n;
  const uint32_t taddr = tmem_acc + (static_cast<uint32_t>(warp * 32) << 16);
  // Workspace of a tile: [row][NTOK tokens], so that four tokens of a row are one 16-byte vector.
  float* const ws_row = ws + static_cast<size_t>(tile_id) * (TILE_ROWS * NTOK) + static_cast<size_t>(r) * NTOK;
  // Destinations: the caller's `out`, or every rank's gathered output (this rank's columns start at col0).
  const int ndst = PEERS ? ps.world : 1;
  const int col0 = PEERS ? ps.col0 : 0;
  int pe = 0;
  if constexpr (PEERS) {
    // No store may reach a peer that has not entered this call: its previous output may still be in use.
    pe = s_epoch;
    peer_wait_all_entered(ps, pe, status);
  }
  auto dst = [&](int d) -> void* { return PEERS ? ps.out[d] : out; };
  auto store_tok = [&](int j, float f) {
    if (row_ok && j < mvalid) {
      const size_t o = static_cast<size_t>(tok0 + j) * ld_out + col0 + n_idx;
      for (int d = 0; d < ndst; ++d) {
        if (out_f32) reinterpret_cast<float*>(dst(d))[o] = f;
        else reinterpret_cast<__nv_bfloat16*>(dst(d))[o] = __float2bfloat16_rn(f);
      }
    }
  };

  // Staging area for vector stores: [token][128 rows] FP32 over the ring, which is idle once bar_acc fired.
  float* const stage = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)));
  const bool vec_ok = (reinterpret_cast<uintptr_t>(dst(0)) & 15) == 0 && ld_out % (out_f32 ? 4 : 8) == 0 &&
                      col0 % (out_f32 ? 4 : 8) == 0;
  // All threads: tokens [first, first + cnt) of the tile wait in `stage`; write them as 8-feature vectors.
  auto staged_store = [&](int first, int cnt) {
    __syncthreads();
    const int items = cnt * 16;
#pragma unroll 4
    for (int it = tid; it < items; it += 128) {
      const int t = it >> 4, g8 = it & 15;
      const float4 lo = *reinterpret_cast<const float4*>(stage + t * TILE_ROWS + g8 * 8);
      const float4 hi = *reinterpret_cast<const float4*>(stage + t * TILE_ROWS + g8 * 8 + 4);
      if (first + t < mvalid)
        for (int d = 0; d < ndst; ++d)
          store_out8(dst(d), out_f32, vec_ok, static_cast<size_t>(tok0 + first + t), ld_out, tile_n * TILE_ROWS + g8 * 8, n,
                     col0, lo, hi);
    }
  };

  if (csize == 1) {
    // One K slice per cluster: straight from the accumulator to the output (or the workspace).
    if (groups == 1 && mpad > DIRECT_STORE_TOKENS) {
      if (ok) {
#pragma unroll 1
        for (int c = 0; c < mpad; c += 32) {
          uint32_t v[16], w[16];
          tmem_ld16(taddr + c, v);
          if (c + 16 < mpad) tmem_ld16(taddr + c + 16, w);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) stage[(c + j) * TILE_ROWS + r] = __uint_as_float(v[j]);
          if (c + 16 < mpad) {
#pragma unroll
            for (int j = 0; j < 16; ++j) stage[(c + 16 + j) * TILE_ROWS + r] = __uint_as_float(w[j]);
          }
        }
      }
      staged_store(0, ok ? mvalid : 0);
    } else if (ok) {
#pragma unroll 1
      for (int c = 0; c < mpad; c += 16) {
        uint32_t v[16];
        tmem_ld16(taddr + c, v);
        tmem_ld_wait();
        if (groups == 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j) store_tok(c + j, __uint_as_float(v[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 16; j += 4)
            if (c + j < mpad)
              red_add_f32x4(ws_row + c + j, __uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                            __uint_as_float(v[j + 3]));
        }
      }
    }
    if (tid == 0) { MUSE_STAMP(6); MUSE_STAMP(7); }
  } else {
    cluster_wait();  // pairs with the arrive after set-up: every peer's receive barrier is initialised
    if (tid == 0) MUSE_STAMP(6);
    if (ok) {
      // Push: tokens [q T, (q + 1) T) go to CTA q, into the slot of our rank. The walk over the
      // tokens is in order, so the owner and the offset inside its block advance by counting (T is
      // a multiple of four), and a peer's addresses are translated once per owner, not per store.
      const uint32_t my_slot = rx_base + static_cast<uint32_t>((crank * TILE_ROWS + r) * T) * 4u;
      const uint32_t bar_local = smem_u32(&bar_rx);
      int owner = 0, t = 0;
      uint32_t slot_remote = dsmem_addr(my_slot, 0), bar_remote = dsmem_addr(bar_local, 0);
      auto push16 = [&](const uint32_t (&val)[16], int base) {
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          if (base + j < mpad) {
            st_async_f32x4(slot_remote + static_cast<uint32_t>(t) * 4u, __uint_as_float(val[j]), __uint_as_float(val[j + 1]),
                           __uint_as_float(val[j + 2]), __uint_as_float(val[j + 3]), bar_remote);
            t += 4;
            if (t == T) {
              t = 0;
              if (++owner < csize) {
                slot_remote = dsmem_addr(my_slot, owner);
                bar_remote = dsmem_addr(bar_local, owner);
              }
            }
          }
        }
      };
#pragma unroll 1
      for (int c = 0; c < mpad; c += 32) {
        uint32_t v[16], w[16];
        const bool two = c + 16 < mpad;
        tmem_ld16(taddr + c, v);
        if (two) tmem_ld16(taddr + c + 16, w);   // both loads in flight before the one wait
        tmem_ld_wait();
        push16(v, c);
        if (two) push16(w, c + 16);
      }
    }
    if (tid == 0) MUSE_STAMP(7);
    if (my_cnt > 0) {
      bool got = mbar_wait(smem_u32(&bar_rx), 0);
      if (!got && lane == 0) atomicOr(status, ST_EPILOGUE_TIMEOUT);
      if (got) {
        const bool staged = groups == 1 && my_cnt > DIRECT_STORE_TOKENS;
        for (int t = 0; t < my_cnt; t += 4) {
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int p = 0; p < csize; ++p) {  // fixed order: the sum does not depend on arrival order
            const float4 u = *reinterpret_cast<const float4*>(rx + (p * TILE_ROWS + r) * T + t);
            acc.x += u.x; acc.y += u.y; acc.z += u.z; acc.w += u.w;
          }
          const int j = crank * T + t;
          if (staged) {
            stage[t * TILE_ROWS + r] = acc.x;
            stage[(t + 1) * TILE_ROWS + r] = acc.y;
            stage[(t + 2) * TILE_ROWS + r] = acc.z;
            stage[(t + 3) * TILE_ROWS + r] = acc.w;
          } else if (groups == 1) {
            store_tok(j, acc.x); store_tok(j + 1, acc.y); store_tok(j + 2, acc.z); store_tok(j + 3, acc.w);
          } else {
            red_add_f32x4(ws_row + j, acc.x, acc.y, acc.z, acc.w);
          }
        }
      }
      if (groups == 1 && my_cnt > DIRECT_STORE_TOKENS) staged_store(crank * T, got ? my_cnt : 0);  // CTA-uniform condition
    }
  }
  if (tid == 0) MUSE_STAMP(8);

  if (groups > 1) {
    // Every add of this CTA is ordered before its arrival; the last of the tile's `split` CTAs sees all.
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int prev = atomicAdd(&cnt[tile_id], 1);
      const int last = prev == split - 1;
      if (last) __threadfence();
      s_last = last;
    }
    __syncthreads();
    if (s_last) {
      // Each thread reads back and clears its own row's words: no other thread touches them.
      for (int j = 0; j < mpad; j += 4) {
        const float4 u = ldg_cg_f32x4(ws_row + j);
        store_tok(j, u.x); store_tok(j + 1, u.y); store_tok(j + 2, u.z); store_tok(j + 3, u.w);
        stg_cg_f32x4(ws_row + j, make_float4(0.f, 0.f, 0.f, 0.f));
      }
      if (tid == 0) cnt[tile_id] = 0;
    }
  }

  // Column-parallel: publish "this rank's slice is everywhere" and wait for the same from every peer.
  if constexpr (PEERS) peer_finish(ps, pe, static_cast<int>(gridDim.x * gridDim.y * gridDim.z), status, &s_last);

  // ---- teardown
  if (tid == 0) MUSE_STAMP(9);
  tc_fence_before_sync();
  __syncthreads();
  if (s_abort && tid == 0) {
    // Let every copy this CTA issued land (or give up) before its shared memory is released.
    const int n_issued = s_issued;
    for (int j = max(0, n_issued - stages); j < n_issued; ++j)
      if (!mbar_wait(smem_u32(&bar_full[j % stages]), static_cast<uint32_t>(j / stages) & 1u))
        atomicOr(status, ST_DRAIN_TIMEOUT);
  }
  if (warp == 2) tmem_dealloc(tmem_acc, Cfg::TMEM_COLS);
  if (tid == 0) { MUSE_STAMP(10); if (tr) tr[11] = global_ns(); }
#undef MUSE_STAMP
}

// ---------------------------------------------------------------- host side

MUSE_TRACE_SETTER(skinny_trace_set)

int skinny_stage_bytes(int ntok, int hilo) { return TILE_ROWS * BK * 2 * (hilo ? 2 : 1) + ntok * BK * 2; }

// Dynamic shared memory of a launch: the ring, the receive slots of a clustered launch, alignment slack.
int skinny_smem_bytes(int ntok, int hilo, int stages, int cluster, int m) {
  const int mvalid = m < ntok ? m : ntok;
  const int rx = cluster > 1 ? cluster * TILE_ROWS * owner_block(mvalid, cluster) * 4 : 0;
  const int ring = stages * skinny_stage_bytes(ntok, hilo);
  const int staged_tokens = cluster > 1 ? owner_block(mvalid, cluster) : ((mvalid + 3) & ~3);
  const int staged = staged_tokens > 16 ? staged_tokens * TILE_ROWS * 4 : 0;  // the vector-store staging area overlays the ring
  return (ring > staged ? ring : staged) + rx + 1024;
}

template <int NTOK, bool HILO, bool PEERS>
static cudaError_t configure(int dev, int* room_out) {
  static int dyn_max[64] = {0};  // per device: opt-in ceiling for dynamic shared memory, once raised
  auto kern = skinny_tc_kernel<NTOK, HILO, PEERS>;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!dyn_max[dev]) {
    cudaFuncAttributes fa;
    int optin = 0;
    cudaError_t e;
    if ((e = cudaFuncGetAttributes(&fa, kern)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) return e;
    const int room = optin - static_cast<int>(fa.sharedSizeBytes);  // static shared memory counts against the limit
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, room)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1)) != cudaSuccess) return e;
    // Ask for the largest shared-memory carveout, or two CTAs of ~80 KB each do not share an SM.
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared)) !=
        cudaSuccess)
      return e;
    dyn_max[dev] = room;
  }
  *room_out = dyn_max[dev];
  return cudaSuccess;
}

template <int NTOK, bool HILO>
static void fill_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int m, int n, int cluster, int groups,
                        size_t smem, cudaStream_t stream, bool pdl) {
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3((n + TILE_ROWS - 1) / TILE_ROWS, cluster * groups, (m + NTOK - 1) / NTOK);
  cfg->blockDim = dim3(128, 1, 1);
  cfg->dynamicSmemBytes = smem;
  cfg->stream = stream;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = static_cast<unsigned>(cluster);
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // may start under the previous kernel's tail
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg->attrs = attr;
  cfg->numAttrs = pdl && g_programmatic_launch ? 2 : 1;
}

template <int NTOK, bool HILO, bool PEERS>
static cudaError_t launch_with(const CUtensorMap* tw, const CUtensorMap* twlo, const CUtensorMap* tx, void* out, float* ws,
                               int* cnt, int* status, int m, int n, int chunks, int cluster, int groups, int stages,
                               int out_f32, int ld_out, const PeerSync& ps, cudaStream_t stream);

// The single-GPU instantiation carries no trace of the peer exchange (PEERS = false).
template <int NTOK, bool HILO>
static cudaError_t launch(const CUtensorMap* tw, const CUtensorMap* twlo, const CUtensorMap* tx, void* out, float* ws,
                          int* cnt, int* status, int m, int n, int chunks, int cluster, int groups, int stages,
                          int out_f32, int ld_out, const PeerSync& ps, cudaStream_t stream) {
  if (ps.world > 1) return launch_with<NTOK, HILO, true>(tw, twlo, tx, out, ws, cnt, status, m, n, chunks, cluster, groups,
                                                         stages, out_f32, ld_out, ps, stream);
  return launch_with<NTOK, HILO, false>(tw, twlo, tx, out, ws, cnt, status, m, n, chunks, cluster, groups, stages, out_f32,
                                        ld_out, ps, stream);
}

template <int NTOK, bool HILO, bool PEERS>
static cudaError_t launch_with(const CUtensorMap* tw, const CUtensorMap* twlo, const CUtensorMap* tx, void* out, float* ws,
                               int* cnt, int* status, int m, int n, int chunks, int cluster, int groups, int stages,
                               int out_f32, int ld_out, const PeerSync& ps, cudaStream_t stream) {
  int dev = 0, room = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if ((e = configure<NTOK, HILO, PEERS>(dev, &room)) != cudaSuccess) return e;
  const size_t smem = static_cast<size_t>(skinny_smem_bytes(NTOK, HILO, stages, cluster, m));
  if (smem > static_cast<size_t>(room)) return cudaErrorInvalidValue;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  fill_config<NTOK, HILO>(&cfg, attr, m, n, cluster, groups, smem, stream, true);
  return cudaLaunchKernelEx(&cfg, skinny_tc_kernel<NTOK, HILO, PEERS>, *tw, HILO ? *twlo : *tw, *tx, out, ws, cnt, status, m, n,
                            chunks, cluster * groups, stages, out_f32, ld_out, ps);
}

// How many clusters of this shape the device can hold at once (0 = the shape cannot launch).
template <int NTOK, bool HILO>
static int max_clusters(int m, int stages, int cluster) {
  int dev = 0, room = 0, num = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (configure<NTOK, HILO, false>(dev, &room) != cudaSuccess) return -1;
  const size_t smem = static_cast<size_t>(skinny_smem_bytes(NTOK, HILO, stages, cluster, m));
  if (smem > static_cast<size_t>(room)) return 0;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  // the grid only has to be a legal multiple of the cluster for the query
  fill_config<NTOK, HILO>(&cfg, attr, m, TILE_ROWS, cluster, 1, smem, nullptr, false);
  if (cudaOccupancyMaxActiveClusters(&num, skinny_tc_kernel<NTOK, HILO, false>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return num;
}

#define MUSE_FOR_NTOK(NT_VAR, HILO_VAR, EXPR_T, EXPR_F) \
  switch (NT_VAR) {                                     \
    case 16: return (HILO_VAR) ? EXPR_T(16) : EXPR_F(16);     \
    case 32: return (HILO_VAR) ? EXPR_T(32) : EXPR_F(32);     \
    case 64: return (HILO_VAR) ? EXPR_T(64) : EXPR_F(64);     \
    case 128: return (HILO_VAR) ? EXPR_T(128) : EXPR_F(128);  \
    case 256: return (HILO_VAR) ? EXPR_T(256) : EXPR_F(256);  \
    default: break;                                     \
  }

int skinny_max_clusters(int ntok, int hilo, int m, int stages, int cluster) {
  if (cluster < 1 || cluster > MAX_CLUSTER || stages < 1 || stages > MAX_STAGES || m < 1) return -1;
#define MC_T(NT) max_clusters<NT, true>(m, stages, cluster)
#define MC_F(NT) max_clusters<NT, false>(m, stages, cluster)
  MUSE_FOR_NTOK(ntok, hilo, MC_T, MC_F)
#undef MC_T
#undef MC_F
  return -7;
}

// Everything skinny_tc_dispatch rejects that can be decided without touching the device: returns 0 or the
// negative code. `ps` = the peer descriptor already copied (world <= 1: single GPU).
static int skinny_check_args(const CUtensorMap* tw, const CUtensorMap* tx, const void* out, const float* ws, const int* cnt,
                             const int* status, int m, int n, int k, int ld_out, int ntok, int cluster, int groups,
                             int stages, const PeerSync& ps) {
  if (!tw || !tx || !out || !status || m <= 0 || n <= 0 || k <= 0) return -1;
  if (k % 8 != 0) return -2;
  const int chunks = (k + BK - 1) / BK;
  if (cluster < 1 || cluster > MAX_CLUSTER || groups < 1) return -3;
  const long long split = static_cast<long long>(cluster) * groups;
  if (split > chunks || split > 65535 || chunks > 65535) return -3;
  if (groups > 1 && (!ws || !cnt)) return -4;
  if (stages < 1 || stages > MAX_STAGES) return -5;
  if (ld_out < n + ps.col0) return -6;
  if (ntok != 16 && ntok != 32 && ntok != 64 && ntok != 128 && ntok != 256) return -7;
  return 0;
}

// Negative = argument error, positive = cudaError_t, 0 = launched.
int skinny_tc_dispatch(const CUtensorMap* tw, const CUtensorMap* twlo, const CUtensorMap* tx, void* out, float* ws,
                       int* cnt, int* status, int m, int n, int k, int ld_out, int ntok, int cluster, int groups,
                       int stages, int out_f32, const PeerSync* peers, cudaStream_t stream) {
  PeerSync ps = {};
  if (peers && peers->world > 1) {
    ps = *peers;
    if (ps.world > MAX_WORLD || ps.rank < 0 || ps.rank >= ps.world || ps.col0 < 0) return -8;
    for (int p = 0; p < ps.world; ++p)
      if (!ps.out[p] || !ps.flags[p]) return -8;
    out = ps.out[ps.rank];
  }
  const int bad = skinny_check_args(tw, tx, out, ws, cnt, status, m, n, k, ld_out, ntok, cluster, groups, stages, ps);
  if (bad) return bad;
  const int chunks = (k + BK - 1) / BK;
  const bool hilo = twlo != nullptr;
#define L_T(NT) static_cast<int>(launch<NT, true>(tw, twlo, tx, out, ws, cnt, status, m, n, chunks, cluster, groups, stages, out_f32, ld_out, ps, stream))
#define L_F(NT) static_cast<int>(launch<NT, false>(tw, twlo, tx, out, ws, cnt, status, m, n, chunks, cluster, groups, stages, out_f32, ld_out, ps, stream))
  MUSE_FOR_NTOK(ntok, hilo, L_T, L_F)
#undef L_T
#undef L_F
  return -7;
}

// ---------------------------------------------------------------- launch without any allocation
//
// Split-K scratch that lives in the library image instead of in memory the caller allocates:
// STATIC_WS_FLOATS floats of partial sums followed by STATIC_CNT_INTS tile counters. Every GPU that
// loads the library carries these 4 MiB + 16 KiB until the process exits.
constexpr long long STATIC_WS_FLOATS = 1ll << 20;
constexpr int STATIC_CNT_INTS = 4096;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_WS_FLOATS * 4 + STATIC_CNT_INTS * 4];

long long skinny_static_ws_floats() { return STATIC_WS_FLOATS; }
int skinny_static_cnt_ints() { return STATIC_CNT_INTS; }

// In host code `g_static_scratch` is only a handle for the symbol, not an address a kernel can use.
// The device address is looked up once per device, with that device current, and cached. Two threads
// making the first call on a device at the same time both look it up and store the same value.
static cudaError_t static_scratch_address(unsigned char** out) {
  static unsigned char* volatile addr[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  unsigned char* a = addr[dev];
  if (!a) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return e;
    addr[dev] = a = static_cast<unsigned char*>(p);
  }
  *out = a;
  return cudaSuccess;
}

// Same launch as skinny_tc_dispatch with the workspace and counters taken from g_static_scratch.
// -20: the shape needs more scratch than the library carries (only launches with groups > 1 use any).
// Every argument is validated before anything is put on the stream. Calls nothing that allocates.
int skinny_tc_static_dispatch(const CUtensorMap* tw, const CUtensorMap* twlo, const CUtensorMap* tx, void* out,
                              int* status, int m, int n, int k, int ld_out, int ntok, int cluster, int groups,
                              int stages, int out_f32, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || ntok <= 0) return -1;
  const long long tiles = static_cast<long long>((n + TILE_ROWS - 1) / TILE_ROWS) * ((m + ntok - 1) / ntok);
  const long long floats = tiles * TILE_ROWS * ntok;
  if (groups > 1 && (floats > STATIC_WS_FLOATS || tiles > STATIC_CNT_INTS)) return -20;
  unsigned char* base = nullptr;
  cudaError_t e = static_scratch_address(&base);
  if (e != cudaSuccess) return static_cast<int>(e);
  float* ws = reinterpret_cast<float*>(base);
  int* cnt = reinterpret_cast<int*>(base + STATIC_WS_FLOATS * 4);
  const int bad = skinny_check_args(tw, tx, out, ws, cnt, status, m, n, k, ld_out, ntok, cluster, groups, stages, PeerSync{});
  if (bad) return bad;
  if (groups > 1) {
    // The shared-memory fit is the one check left to the launch itself; decide it before the clears too.
    int dev = 0, room = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return static_cast<int>(e);
    if ((e = cudaDeviceGetAttribute(&room, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) return static_cast<int>(e);
    if (skinny_smem_bytes(ntok, twlo != nullptr, stages, cluster, m) + 512 > room) return static_cast<int>(cudaErrorInvalidValue);
    // The array keeps whatever the previous call (of anyone in this process) left. A completed call
    // leaves zeros, an aborted one may not: clear exactly what this launch will accumulate into.
    if ((e = cudaMemsetAsync(ws, 0, static_cast<size_t>(floats) * 4, stream)) != cudaSuccess) return static_cast<int>(e);
    if ((e = cudaMemsetAsync(cnt, 0, static_cast<size_t>(tiles) * 4, stream)) != cudaSuccess) return static_cast<int>(e);
  }
  return skinny_tc_dispatch(tw, twlo, tx, out, ws, cnt, status, m, n, k, ld_out, ntok, cluster, groups, stages, out_f32,
                            nullptr, stream);
}

}  // namespace muse
