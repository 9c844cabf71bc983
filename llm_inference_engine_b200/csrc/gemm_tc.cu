// out[m, n] = x[m, K] . W[n, K]^T (BF16 in, FP32 accumulate, BF16 out) for many tokens: the m > 32 GEMM
// of the path, which the reference hands to cuBLAS (best_submissions/muse_bf16_proj.py:390). Swap-AB like
// muse_skinny_tc (the weight tile is the MMA's M = 128, the tokens its N), TMA -> shared-memory ring ->
// tcgen05.mma -> tensor memory, but shaped for what bounds these sizes:
//   * the token tile is as wide as the call (N = m rounded up to 16, a run-time value; one tile up to 256 tokens),
//     so W leaves HBM once and is never re-read through L2;
//   * traffic from L2 into shared memory, not HBM or the tensor pipe, limits a swap-AB kernel at 64..256
//     tokens (every 128-row weight tile wants the whole x tile beside it). With PAIR a CTA owns two 128-row
//     tiles and brings each x chunk in once for both: two MMAs per K step into two FP32 accumulators that share
//     the SM's tensor memory (2 x 256 columns at 256 tokens). Without PAIR it owns one tile (small weights want
//     more CTAs rather than less x traffic), which may be SHORT (tile_rows < 128: a weight of any height then
//     fills the SMs in one wave without any K split; used at few tokens, where the tensor pipe has time to spare);
//   * a pipeline stage holds k_atoms 64-wide pieces of K (each its own swizzled box), so that one step asks DRAM
//     for k_atoms x 128 contiguous bytes of every weight row;
//   * K slices fill the SMs in one wave, one CTA per SM, and meet in one of two ways, both with a fixed
//     summation order (bit-reproducible). Cluster: tokens are dealt to the cluster's CTAs in blocks of 16, every
//     CTA pushes the blocks it does not own from tensor memory into the owner's shared memory (16-byte
//     st.shared::cluster, a warp writing 512 contiguous bytes); the receive area overlays the idle ring: one
//     cluster barrier after the main loop says the rings are idle, a second one that the pushes have landed.
//     Workspace: no cluster; every slice writes the blocks it does not own to its slot of a global workspace
//     (plain 16-byte stores that stay in L2), counts itself in on the tile's counter, waits (bounded) for the
//     others, reads its own block's slots back, and the last slice to finish reading zeroes the counters;
//   * 128 .. 512 threads: thread 0 = TMA producer (cp.async.bulk.tensor.2d, weights with an evict-first L2
//     policy, x evict-last; no cluster multicast), warp 1 lane 0 = MMA issuer, everybody else parked on a CTA
//     barrier during the main loop; then every warpgroup reads accumulators out (warp w touches TMEM lanes
//     32 (w % 4) ..), 16 tokens per warpgroup and step: TMEM (+ received slots) -> shared-memory transpose ->
//     16-byte global stores.
// Every wait is bounded and reports through the status word. Column-parallel (PEERS) the output goes to every
// rank's gathered buffer with the flag exchange of common.cuh.
#include "common.cuh"

namespace muse {

constexpr int GT_ROWS = 128;       // rows of one weight tile = MMA M
constexpr int GT_BK = 64;          // K elements per stage
constexpr int GT_MAX_STAGES = 12;
constexpr int GT_MAX_KATOMS = 8;     // 64-wide K atoms per pipeline stage
constexpr int GT_MAX_CLUSTER = 16;
constexpr int GT_SUB = 16;         // tokens summed, staged and stored at a time; owner blocks are multiples of it
constexpr int GT_MIN_SMEM = 116 * 1024;   // more than half of the 228 KB of an SM: one CTA per SM
constexpr int GT_MAX_THREADS = 512;       // 1 .. 4 warpgroups; all of them work in the epilogue

// Tokens per owner CTA when the (padded) tokens of a tile are dealt to `cluster` CTAs.
__host__ __device__ constexpr int gt_owner_block(int mpad16, int cluster) {
  return (((mpad16 + cluster - 1) / cluster) + GT_SUB - 1) / GT_SUB * GT_SUB;
}

__device__ __forceinline__ uint32_t gt_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t gt_cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void gt_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void gt_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t gt_dsmem_addr(uint32_t local_smem, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem), "r"(rank));
  return r;
}
// 16 bytes into a peer's shared memory. Plain stores: an st.async per 16 bytes would also update the owner's
// mbarrier once per store, and thousands of updates of one barrier word serialise (measured: 25 GB/s per CTA).
__device__ __forceinline__ void gt_st_cluster_v4(uint32_t remote_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(remote_addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// One barrier per epilogue warpgroup (ids 1 .. 4; id 0 is __syncthreads).
__device__ __forceinline__ void gt_group_sync(int wg) { asm volatile("bar.sync %0, 128;" ::"r"(wg + 1) : "memory"); }

template <bool PAIR, bool PEERS>
__global__ void __launch_bounds__(GT_MAX_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
               __nv_bfloat16* __restrict__ out, float* __restrict__ ws, int* __restrict__ cnt, int* __restrict__ status, int m,
               int n, int chunks, int ntok, int stages, int tmem_cols, int ld_out, int tile_rows, int katoms,
               const __grid_constant__ PeerSync ps) {
  constexpr int H = PAIR ? 2 : 1;          // weight tiles (accumulators) per CTA
  constexpr int ROWS = GT_ROWS * H;        // accumulator rows per CTA (row stride of the staging and the slots)
  // Weight rows this CTA owns: 256 for a pair; else `tile_rows` (a multiple of 8 up to 128 = the box of tm_w). A
  // short tile lets a weight of any height fill the SMs in one wave without splitting K: the MMA is still M = 128
  // and reads 128 rows of shared memory, but the rows past the tile are whatever lies there, they only reach
  // accumulator lanes nobody reads, and the tensor pipe has the time at the few tokens this is used for.
  const int own_rows = PAIR ? ROWS : tile_rows;
  const uint32_t A_BYTES = static_cast<uint32_t>(PAIR ? GT_ROWS : tile_rows) * (GT_BK * 2);
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[GT_MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_empty[GT_MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_acc;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_abort;
  __shared__ int s_last;
  __shared__ int s_issued;
  __shared__ int s_epoch;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile_n = blockIdx.x, tile_m = blockIdx.z;
  // Phase stamps of diagnostic builds: 16 slots per CTA, SM clock; slots 15 / 14 = global nanosecond timer at entry / exit.
  unsigned long long* const trace = MUSE_TRACE_BASE();
  unsigned long long* const tr =
      trace ? trace + 16ull * (blockIdx.x + gridDim.x * (blockIdx.y + static_cast<size_t>(gridDim.y) * blockIdx.z)) : nullptr;
#define GT_STAMP(slot) do { if (tr) tr[slot] = static_cast<unsigned long long>(clock64()); } while (0)
  if (tr && tid == 0) { GT_STAMP(0); tr[15] = global_ns(); }
  // K slices = gridDim.y. Either they are the CTAs of one thread-block cluster (cluster dims (1, slices, 1)) and
  // meet in distributed shared memory, or the launch has no cluster and they meet in the global workspace.
  const bool dsm = gt_cluster_size() > 1;
  const int csize = static_cast<int>(gridDim.y), crank = static_cast<int>(blockIdx.y);
  // A pipeline stage holds `katoms` 64-wide K atoms of every operand (each its own swizzled box), so that one step
  // asks DRAM for katoms x 128 contiguous bytes of every weight row instead of 128. K is dealt to the slices in
  // whole steps; atoms past the end of K read as zeros.
  const int steps = (chunks + katoms - 1) / katoms;
  const int c0 = static_cast<int>(static_cast<uint32_t>(crank) * static_cast<uint32_t>(steps) / static_cast<uint32_t>(csize));
  const int c1 = static_cast<int>((static_cast<uint32_t>(crank) + 1u) * static_cast<uint32_t>(steps) / static_cast<uint32_t>(csize));
  const int nchunks = c1 - c0;   // steps of this slice
  const uint32_t b_bytes = static_cast<uint32_t>(ntok) * (GT_BK * 2);
  const uint32_t a_all = A_BYTES * H * static_cast<uint32_t>(katoms);      // all A atoms of a stage, then all B atoms
  const uint32_t stage_bytes = a_all + b_bytes * static_cast<uint32_t>(katoms);
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // the 128-byte swizzle repeats every 1024 bytes

  uint64_t pol_w = 0, pol_x = 0;
  int issued = 0;
  auto issue_w = [&](int i, int s) {   // arms the stage's barrier for all of its bytes, then the weight atoms
    const uint32_t full = smem_u32(&bar_full[s]);
    const uint32_t a = smem_base + static_cast<uint32_t>(s) * stage_bytes;
    mbar_expect_tx(full, stage_bytes);
    for (int t = 0; t < katoms; ++t) {
      const int kcol = ((c0 + i) * katoms + t) * GT_BK;
      tma_load_2d(a + static_cast<uint32_t>(t) * A_BYTES * H, &tm_w, kcol, tile_n * own_rows, full, pol_w);
      if (PAIR) tma_load_2d(a + static_cast<uint32_t>(t) * A_BYTES * H + A_BYTES, &tm_w, kcol, tile_n * own_rows + GT_ROWS, full, pol_w);
    }
  };
  auto issue_x = [&](int i, int s) {
    const uint32_t full = smem_u32(&bar_full[s]);
    const uint32_t a = smem_base + static_cast<uint32_t>(s) * stage_bytes;
    for (int t = 0; t < katoms; ++t)
      tma_load_2d(a + a_all + static_cast<uint32_t>(t) * b_bytes, &tm_x, ((c0 + i) * katoms + t) * GT_BK, tile_m * ntok, full, pol_x);
    ++issued;
  };
  auto issue = [&](int i, int s) {
    issue_w(i, s);
    issue_x(i, s);
  };

  const int tok0 = tile_m * ntok;
  const int mvalid = min(ntok, m - tok0);
  const int mpad = (mvalid + GT_SUB - 1) / GT_SUB * GT_SUB;      // <= ntok; the padding tokens are zero rows of x
  const int T = csize > 1 ? gt_owner_block(mpad, csize) : mpad;  // tokens per owner CTA
  const int my_first = crank * T;
  const int my_cnt = max(0, min(T, mpad - my_first));            // tokens this CTA sums and stores

  // Weight bytes start moving before anything else in the CTA is set up.
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_acc), 1);
    fence_mbar_init();
    pol_w = l2_policy_evict_first();
    pol_x = l2_policy_evict_last();
    // The first stages: the weight tiles leave now, the x tiles once the kernels ahead in the stream have completed
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
    GT_STAMP(1);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_slot), static_cast<uint32_t>(tmem_cols));
    tmem_relinquish();
  }
  griddep_wait();   // every thread, before the first barrier: what follows reads and writes more than weights
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_acc = tmem_slot;
  const uint32_t acc_stride = static_cast<uint32_t>(tmem_cols / H);   // second accumulator: the upper half of the columns

  if (warp == 0) {
    if (lane == 0) {
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
      const uint32_t idesc = umma_idesc_bf16(GT_ROWS, ntok);
      int s = 0;
      uint32_t phase = 0;
      for (int i = 0; i < nchunks; ++i) {
        if (!mbar_wait(smem_u32(&bar_full[s]), phase)) {
          atomicOr(status, ST_MMA_TIMEOUT);
          s_abort = 1;
          break;
        }
        tc_fence_after_sync();
        if (i == 0) GT_STAMP(2);
        const uint32_t a = smem_base + static_cast<uint32_t>(s) * stage_bytes;
#pragma unroll 1
        for (int t = 0; t < katoms; ++t) {
          const uint64_t a0_desc = umma_desc_k_sw128(a + static_cast<uint32_t>(t) * A_BYTES * H);
          const uint64_t a1_desc = umma_desc_k_sw128(a + static_cast<uint32_t>(t) * A_BYTES * H + A_BYTES);
          const uint64_t b_desc = umma_desc_k_sw128(a + a_all + static_cast<uint32_t>(t) * b_bytes);
#pragma unroll
          for (int k = 0; k < GT_BK / 16; ++k) {
            // 16 BF16 = 32 bytes further along K inside the swizzle span: +2 in 16-byte units.
            const uint32_t accumulate = (i > 0 || t > 0 || k > 0) ? 1u : 0u;
            umma_bf16(tmem_acc, a0_desc + 2 * k, b_desc + 2 * k, idesc, accumulate);
            if (PAIR) umma_bf16(tmem_acc + acc_stride, a1_desc + 2 * k, b_desc + 2 * k, idesc, accumulate);
          }
        }
        umma_commit(smem_u32(&bar_empty[s]));
        if (++s == stages) {
          s = 0;
          phase ^= 1u;
        }
      }
      umma_commit(smem_u32(&bar_acc));   // also on the abort path, so that the epilogue is released
      GT_STAMP(3);
      // Only this thread watches the accumulators complete; everybody else is parked on the barrier below.
      if (!mbar_wait(smem_u32(&bar_acc), 0)) {
        atomicOr(status, ST_EPILOGUE_TIMEOUT);
        s_abort = 1;
      }
    }
    __syncwarp();
  }

  // ---- epilogue, all warps. Warp w may only touch TMEM lanes [32 (w % 4), 32 (w % 4) + 32): thread = weight row
  // of each tile; the warpgroups (4 warps each) take the 16-token groups of every step round robin.
  __syncthreads();
  tc_fence_after_sync();
  const bool ok = !s_abort;
  if (tid == 0) GT_STAMP(4);

  const int G = static_cast<int>(blockDim.x) >> 7, wg = tid >> 7;
  const int r = tid & 127;
  const uint32_t taddr = tmem_acc + (static_cast<uint32_t>((warp & 3) * 32) << 16);
  // After the main loop the ring is idle and becomes: receive slots, then one store staging area per warpgroup.
  // A slot holds one sender's partial sums of one tile for this CTA's T tokens as [T / 4 token quads][128 rows]
  // float4: the 32 lanes of a warp (32 neighbouring rows, the same token quad) write and read 512 contiguous bytes.
  const uint32_t rx_base = smem_base;
  const uint32_t slot_bytes = static_cast<uint32_t>(T) * GT_ROWS * 4u;
  const uint32_t rx_bytes = dsm ? static_cast<uint32_t>(csize - 1) * H * slot_bytes : 0u;
  const float4* const rx = reinterpret_cast<const float4*>(smem_raw + (rx_base - smem_u32(smem_raw)));
  float* const stage = reinterpret_cast<float*>(smem_raw + (rx_base + rx_bytes - smem_u32(smem_raw))) + wg * (GT_SUB * ROWS);

  // Global mode: the partial sums that slice `sender` holds for owner `q` of this tile live at
  // ws[((unit * csize + q) * (csize - 1) + slot) * H + h] as [T / 4 token quads][128 rows] float4, like a slot.
  const size_t unit = tile_n + static_cast<size_t>(gridDim.x) * tile_m;
  float4* const ws4 = reinterpret_cast<float4*>(ws);
  const size_t slot_vec = static_cast<size_t>(T >> 2) * GT_ROWS;   // float4 per (slot, tile)
  if (csize > 1 && !dsm) {
    if (ok) {
#pragma unroll 1
      for (int q = 0; q < csize; ++q) {
        if (q == crank) continue;
        const int first = q * T, cnt_q = min(T, mpad - first);
        if (cnt_q <= 0) break;
        const int slot = crank < q ? crank : crank - 1;
#pragma unroll
        for (int h = 0; h < H; ++h) {
          float4* dst = ws4 + (((unit * csize + q) * (csize - 1) + slot) * H + h) * slot_vec + r;
#pragma unroll 1
          for (int c = wg * GT_SUB; c < cnt_q; c += G * GT_SUB) {
            uint32_t v[16];
            tmem_ld16(taddr + h * acc_stride + first + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; j += 4)
              __stcg(dst + static_cast<size_t>((c + j) >> 2) * GT_ROWS,
                     make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])));
          }
        }
      }
    }
    if (tid == 0) GT_STAMP(5);
    // Arrive (every CTA, also an aborted one, so that nobody waits for it in vain), then wait for all slices of
    // this tile: a bounded spin of one thread. All CTAs of the grid are resident at once (one per SM, the host
    // keeps the grid within the SM count), so the slices being waited for are running.
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      atomicAdd(cnt + 2 * unit, 1);
      bool all = ld_acquire_gpu(cnt + 2 * unit) >= csize;
      const unsigned long long t0 = global_ns();
      while (!all) {
#pragma unroll 1
        for (int i = 0; i < 32 && !all; ++i) all = ld_acquire_gpu(cnt + 2 * unit) >= csize;
        if (!all && global_ns() - t0 > WAIT_LIMIT_NS) break;
      }
      if (!all) {
        atomicOr(status, ST_EPILOGUE_TIMEOUT);
        s_abort = 1;
      }
      GT_STAMP(6);
    }
    __syncthreads();
  }
  if (dsm) {
    // Every CTA of the cluster has finished reading its ring (its last MMA completed): the rings may be written.
    gt_cluster_arrive();
    gt_cluster_wait();
    if (tid == 0) GT_STAMP(5);
    if (ok) {
#pragma unroll 1
      for (int q = 0; q < csize; ++q) {
        if (q == crank) continue;
        const int first = q * T, cnt_q = min(T, mpad - first);
        if (cnt_q <= 0) break;
        const int slot = crank < q ? crank : crank - 1;   // the owner keeps no slot for itself
#pragma unroll
        for (int h = 0; h < H; ++h) {
          const uint32_t dst = gt_dsmem_addr(rx_base + static_cast<uint32_t>(slot * H + h) * slot_bytes + static_cast<uint32_t>(r) * 16u,
                                             static_cast<uint32_t>(q));
#pragma unroll 1
          for (int c = wg * GT_SUB; c < cnt_q; c += G * GT_SUB) {
            uint32_t v[16];
            tmem_ld16(taddr + h * acc_stride + first + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; j += 4)
              gt_st_cluster_v4(dst + static_cast<uint32_t>((c + j) >> 2) * (GT_ROWS * 16u), v[j], v[j + 1], v[j + 2], v[j + 3]);
          }
        }
      }
    }
    if (tid == 0) GT_STAMP(6);
    // Second cluster barrier: every push of every CTA has landed (release / acquire at cluster scope).
    gt_cluster_arrive();
    gt_cluster_wait();
  }

  // Destinations: the caller's `out`, or every rank's gathered output (this rank's columns start at col0).
  const int ndst = PEERS ? ps.world : 1;
  const int col0 = PEERS ? ps.col0 : 0;
  int pe = 0;
  if constexpr (PEERS) {
    pe = s_epoch;
    peer_wait_all_entered(ps, pe, status);   // no store may reach a peer that has not entered this call
  }
  auto dst_of = [&](int d) -> __nv_bfloat16* { return PEERS ? reinterpret_cast<__nv_bfloat16*>(ps.out[d]) : out; };
  const bool vec_ok = (reinterpret_cast<uintptr_t>(dst_of(0)) & 15) == 0 && ld_out % 8 == 0 && col0 % 8 == 0;

  const bool got = ok && !s_abort;
  if (tid == 0) GT_STAMP(7);

  // Own block, GT_SUB tokens per warpgroup and step: accumulator + received slots (fixed order) -> staging ->
  // 16-byte stores. Conditions on `sub` and `got` are uniform per warpgroup, which is what its barrier needs.
#pragma unroll 1
  for (int sub = wg * GT_SUB; sub < my_cnt; sub += G * GT_SUB) {
    if (got) {
#pragma unroll
      for (int h = 0; h < H; ++h) {
        uint32_t v[16];
        tmem_ld16(taddr + h * acc_stride + my_first + sub, v);
        tmem_ld_wait();
        float f[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(v[j]);
        if (dsm) {
          for (int p = 0; p < csize - 1; ++p) {
            const float4* src = rx + (static_cast<size_t>(p * H + h) * (T >> 2) + (sub >> 2)) * GT_ROWS + r;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float4 u = src[j * GT_ROWS];
              f[4 * j] += u.x; f[4 * j + 1] += u.y; f[4 * j + 2] += u.z; f[4 * j + 3] += u.w;
            }
          }
        } else {
          for (int p = 0; p < csize - 1; ++p) {
            const float4* src = ws4 + (((unit * csize + crank) * (csize - 1) + p) * H + h) * slot_vec +
                                static_cast<size_t>(sub >> 2) * GT_ROWS + r;
            float4 u[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) u[j] = __ldcg(src + j * GT_ROWS);   // all four in flight, straight from L2
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              f[4 * j] += u[j].x; f[4 * j + 1] += u[j].y; f[4 * j + 2] += u[j].z; f[4 * j + 3] += u[j].w;
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) stage[j * ROWS + h * GT_ROWS + r] = f[j];
      }
    }
    gt_group_sync(wg);
    if (got) {
      constexpr int VPT = ROWS / 8;   // 8-row vectors per token
      for (int it = r; it < GT_SUB * VPT; it += 128) {
        const int j = it / VPT, g8 = it % VPT;
        const int tok = my_first + sub + j;
        const int n0 = tile_n * own_rows + g8 * 8;
        if (tok >= mvalid || n0 >= n || g8 * 8 >= own_rows) continue;
        const float4 lo = *reinterpret_cast<const float4*>(stage + j * ROWS + g8 * 8);
        const float4 hi = *reinterpret_cast<const float4*>(stage + j * ROWS + g8 * 8 + 4);
        const size_t o = static_cast<size_t>(tok0 + tok) * ld_out + col0 + n0;
        if (vec_ok && n0 + 8 <= n) {
          const __nv_bfloat162 p0 = __floats2bfloat162_rn(lo.x, lo.y), p1 = __floats2bfloat162_rn(lo.z, lo.w);
          const __nv_bfloat162 p2 = __floats2bfloat162_rn(hi.x, hi.y), p3 = __floats2bfloat162_rn(hi.z, hi.w);
          uint4 pk;
          pk.x = *reinterpret_cast<const uint32_t*>(&p0);
          pk.y = *reinterpret_cast<const uint32_t*>(&p1);
          pk.z = *reinterpret_cast<const uint32_t*>(&p2);
          pk.w = *reinterpret_cast<const uint32_t*>(&p3);
          for (int d = 0; d < ndst; ++d) *reinterpret_cast<uint4*>(dst_of(d) + o) = pk;
        } else {
          const float a[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
          for (int d = 0; d < ndst; ++d)
            for (int i = 0; i < 8; ++i)
              if (n0 + i < n) dst_of(d)[o + i] = __float2bfloat16_rn(a[i]);
        }
      }
    }
    gt_group_sync(wg);
  }

  if (tid == 0) GT_STAMP(8);
  if (csize > 1 && !dsm) {
    // The last slice of the tile to finish reading puts both counters back to zero for the next launch.
    __syncthreads();
    if (tid == 0 && atomicAdd(cnt + 2 * unit + 1, 1) == csize - 1) {
      cnt[2 * unit] = 0;
      cnt[2 * unit + 1] = 0;
    }
  }
  if constexpr (PEERS) peer_finish(ps, pe, static_cast<int>(gridDim.x * gridDim.y * gridDim.z), status, &s_last);

  // ---- teardown
  if (tid == 0) GT_STAMP(9);
  tc_fence_before_sync();
  __syncthreads();
  if (s_abort && tid == 0) {
    // Let every copy this CTA issued land (or give up) before its shared memory is released.
    const int n_issued = s_issued;
    for (int j = max(0, n_issued - stages); j < n_issued; ++j)
      if (!mbar_wait(smem_u32(&bar_full[j % stages]), static_cast<uint32_t>(j / stages) & 1u))
        atomicOr(status, ST_DRAIN_TIMEOUT);
  }
  // No push is in flight towards this CTA any more: the second cluster barrier above came after all of them.
  if (warp == 2) tmem_dealloc(tmem_acc, static_cast<uint32_t>(tmem_cols));
  if (tr && tid == 0) { GT_STAMP(10); tr[14] = global_ns(); }
#undef GT_STAMP
}

MUSE_TRACE_SETTER(gemm_trace_set)

// ---------------------------------------------------------------- host side

static int gt_tmem_cols(int ntok, int pair) {
  int cols = 32;
  while (cols < ntok * (pair ? 2 : 1)) cols <<= 1;
  return cols;   // 32 .. 512, a power of two
}

int gemm_tc_stage_bytes(int ntok, int pair, int tile_rows, int katoms) {
  return katoms * ((pair ? 2 * GT_ROWS : tile_rows) * GT_BK * 2 + ntok * GT_BK * 2);
}

// Dynamic shared memory of a launch: the ring, or the receive slots plus the store staging (one area per warpgroup)
// that replace it after the main loop, whichever is larger, plus alignment slack.
// (`cluster` = K slices that meet in distributed shared memory; slices that meet in the global workspace need none.)
int gemm_tc_smem_bytes(int ntok, int pair, int stages, int cluster, int m, int warpgroups, int tile_rows, int katoms) {
  const int rows = GT_ROWS * (pair ? 2 : 1);
  const int mvalid = m < ntok ? m : ntok;
  const int mpad = (mvalid + GT_SUB - 1) / GT_SUB * GT_SUB;
  const int T = cluster > 1 ? gt_owner_block(mpad, cluster) : mpad;
  const int rx = cluster > 1 ? (cluster - 1) * rows * T * 4 : 0;
  const int after = rx + warpgroups * GT_SUB * rows * 4;
  // (a short tile's MMA reads 128 rows from where its tile starts: keep the last stage's over-read inside)
  const int ring = stages * gemm_tc_stage_bytes(ntok, pair, tile_rows, katoms) + (pair ? 0 : (GT_ROWS - tile_rows) * GT_BK * 2);
  const int need = (ring > after ? ring : after) + 1024;
  // Never less than half an SM's shared memory: two of these CTAs must not share an SM, because together
  // they could ask for more tensor memory than the SM has, and tcgen05.alloc waits without a limit.
  return need > GT_MIN_SMEM ? need : GT_MIN_SMEM;
}

template <bool PAIR, bool PEERS>
static cudaError_t gt_configure(int dev, int* room_out) {
  static int dyn_max[64] = {0};
  auto kern = gemm_tc_kernel<PAIR, PEERS>;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!dyn_max[dev]) {
    cudaFuncAttributes fa;
    int optin = 0;
    cudaError_t e;
    if ((e = cudaFuncGetAttributes(&fa, kern)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) return e;
    const int room = optin - static_cast<int>(fa.sharedSizeBytes);
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, room)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared)) !=
        cudaSuccess)
      return e;
    dyn_max[dev] = room;
  }
  *room_out = dyn_max[dev];
  return cudaSuccess;
}

static void gt_fill_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int m, int n, int ntok, int pair, int cluster,
                           int split, int warpgroups, int tile_rows, size_t smem, cudaStream_t stream, bool pdl) {
  const int rows = pair ? 2 * GT_ROWS : tile_rows;
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3((n + rows - 1) / rows, cluster * split, (m + ntok - 1) / ntok);
  cfg->blockDim = dim3(128 * warpgroups, 1, 1);
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

template <bool PAIR, bool PEERS>
static cudaError_t gt_launch(const CUtensorMap* tw, const CUtensorMap* tx, void* out, float* ws, int* cnt, int* status, int m,
                             int n, int chunks, int ntok, int cluster, int split, int stages, int warpgroups, int tile_rows,
                             int katoms, int ld_out, const PeerSync& ps, cudaStream_t stream) {
  int dev = 0, room = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if ((e = gt_configure<PAIR, PEERS>(dev, &room)) != cudaSuccess) return e;
  const size_t smem = static_cast<size_t>(gemm_tc_smem_bytes(ntok, PAIR, stages, cluster, m, warpgroups, tile_rows, katoms));
  if (smem > static_cast<size_t>(room)) return cudaErrorInvalidValue;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  gt_fill_config(&cfg, attr, m, n, ntok, PAIR, cluster, split, warpgroups, tile_rows, smem, stream, true);
  return cudaLaunchKernelEx(&cfg, gemm_tc_kernel<PAIR, PEERS>, *tw, *tx, reinterpret_cast<__nv_bfloat16*>(out), ws, cnt, status,
                            m, n, chunks, ntok, stages, gt_tmem_cols(ntok, PAIR), ld_out, tile_rows, katoms, ps);
}

// How many clusters of this launch shape the device holds at once (0: the shape cannot launch; negative: bad argument).
int gemm_tc_max_clusters(int ntok, int pair, int stages, int cluster, int m, int warpgroups, int tile_rows, int katoms) {
  if (cluster < 1 || cluster > GT_MAX_CLUSTER || stages < 1 || stages > GT_MAX_STAGES || m < 1 || ntok < 16 || ntok > 256 ||
      ntok % 16 || warpgroups < 1 || warpgroups > GT_MAX_THREADS / 128 || tile_rows < 8 || tile_rows > GT_ROWS || tile_rows % 8 || katoms < 1 || katoms > GT_MAX_KATOMS)
    return -1;
  int dev = 0, room = 0, num = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  const cudaError_t e = pair ? gt_configure<true, false>(dev, &room) : gt_configure<false, false>(dev, &room);
  if (e != cudaSuccess) return -1;
  const size_t smem = static_cast<size_t>(gemm_tc_smem_bytes(ntok, pair, stages, cluster, m, warpgroups, tile_rows, katoms));
  if (smem > static_cast<size_t>(room)) return 0;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  gt_fill_config(&cfg, attr, m < ntok ? m : ntok, pair ? 2 * GT_ROWS : tile_rows, ntok, pair, cluster, 1, warpgroups, tile_rows, smem,
                 nullptr, false);
  const cudaError_t q = pair ? cudaOccupancyMaxActiveClusters(&num, gemm_tc_kernel<true, false>, &cfg)
                             : cudaOccupancyMaxActiveClusters(&num, gemm_tc_kernel<false, false>, &cfg);
  if (q != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return num;
}

// Workspace floats and counters a launch with `split` K slices meeting in global memory needs (0 when split == 1).
long long gemm_tc_ws_floats(int m, int n, int ntok, int pair, int split, int tile_rows) {
  if (split <= 1) return 0;
  const int rows = GT_ROWS * (pair ? 2 : 1);   // slots are sized for whole 128-row tiles, whatever the tile height
  const int own = pair ? rows : tile_rows;
  const long long units = static_cast<long long>((n + own - 1) / own) * ((m + ntok - 1) / ntok);
  const int mvalid = m < ntok ? m : ntok;
  const int T = gt_owner_block((mvalid + GT_SUB - 1) / GT_SUB * GT_SUB, split);
  return units * split * (split - 1) * rows * T;
}
int gemm_tc_cnt_ints(int m, int n, int ntok, int pair, int split, int tile_rows) {
  if (split <= 1) return 0;
  const int own = pair ? 2 * GT_ROWS : tile_rows;
  return 2 * ((n + own - 1) / own) * ((m + ntok - 1) / ntok);
}

// Negative = argument error, positive = cudaError_t, 0 = launched.
int gemm_tc_dispatch(const CUtensorMap* tw, const CUtensorMap* tx, void* out, float* ws, int* cnt, int* status, int m, int n,
                     int k, int ld_out, int ntok, int pair, int cluster, int split, int stages, int warpgroups, int tile_rows,
                     int katoms, const PeerSync* peers, cudaStream_t stream) {
  PeerSync ps = {};
  if (peers && peers->world > 1) {
    ps = *peers;
    if (ps.world > MAX_WORLD || ps.rank < 0 || ps.rank >= ps.world || ps.col0 < 0) return -8;
    for (int p = 0; p < ps.world; ++p)
      if (!ps.out[p] || !ps.flags[p]) return -8;
    out = ps.out[ps.rank];
  }
  if (!tw || !tx || !out || !status || m <= 0 || n <= 0 || k <= 0) return -1;
  if (k % 8 != 0) return -2;
  const int chunks = (k + GT_BK - 1) / GT_BK;
  if (cluster < 1 || cluster > GT_MAX_CLUSTER || split < 1 || split > 64 || (cluster > 1 && split > 1)) return -3;
  if (katoms < 1 || katoms > GT_MAX_KATOMS) return -12;
  if (cluster * split > (chunks + katoms - 1) / katoms || chunks > 65535) return -3;
  if (split > 1) {
    if (!ws || !cnt || (reinterpret_cast<uintptr_t>(ws) & 15)) return -4;
    // Slices wait for one another: every CTA of the grid has to be resident at once, one per SM.
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return -1;
    const int rows = pair ? 2 * GT_ROWS : tile_rows;
    if (static_cast<long long>((n + rows - 1) / rows) * split * ((m + ntok - 1) / ntok) > sms) return -10;
  }
  if (tile_rows < 8 || tile_rows > GT_ROWS || tile_rows % 8 || (pair && tile_rows != GT_ROWS)) return -11;
  if (stages < 1 || stages > GT_MAX_STAGES) return -5;
  if (ld_out < n + ps.col0) return -6;
  if (ntok < 16 || ntok > 256 || ntok % 16) return -7;
  if (warpgroups < 1 || warpgroups > GT_MAX_THREADS / 128) return -9;
  cudaError_t e;
  if (ps.world > 1)
    e = pair ? gt_launch<true, true>(tw, tx, out, ws, cnt, status, m, n, chunks, ntok, cluster, split, stages, warpgroups, tile_rows, katoms, ld_out, ps, stream)
             : gt_launch<false, true>(tw, tx, out, ws, cnt, status, m, n, chunks, ntok, cluster, split, stages, warpgroups, tile_rows, katoms, ld_out, ps, stream);
  else
    e = pair ? gt_launch<true, false>(tw, tx, out, ws, cnt, status, m, n, chunks, ntok, cluster, split, stages, warpgroups, tile_rows, katoms, ld_out, ps, stream)
             : gt_launch<false, false>(tw, tx, out, ws, cnt, status, m, n, chunks, ntok, cluster, split, stages, warpgroups, tile_rows, katoms, ld_out, ps, stream);
  return static_cast<int>(e);
}

}  // namespace muse
