// Persistent "stream-K" variant of the swap-AB tensor-core projection for tall weights at up to
// 64 tokens: out[m, n] = x[m, K] . W[n, K]^T with the same operands, tiles and MMA shape as
// skinny_tc.cu (128 weight rows x NTOK tokens per tile, 64-wide K chunks through a TMA -> shared
// memory ring -> tcgen05.mma -> TMEM), but a different decomposition of the work.
//
// The (tile, K chunk) pairs of the whole problem form one line of L = tiles x chunks units,
// tile-major. The grid is one CTA per SM, resident for the whole call, and CTA b takes the
// contiguous run [b L / G, (b + 1) L / G): every SM streams the same number of weight bytes to
// within one chunk, set-up (barriers, TMEM, tensor-map fetch) is paid once per SM instead of once
// per unit, and the producer never stops at a tile boundary, so HBM stays busy from the first
// request to the last. A run crosses at most a few tile boundaries; each piece of a tile is a
// "segment". Warps are specialised:
//   warp 0 / lane 0    TMA producer over the whole run (ring of `stages` stages);
//   warp 1 / lane 0    MMA issuer; segments alternate between two TMEM accumulators, so the next
//                      segment's MMAs run while the previous one is being drained;
//   warps 2..5         epilogue: drain an accumulator (thread = weight row, registers = tokens),
//                      release it, and either store the output (the segment covers the tile's whole
//                      K) or park the partial tile in a workspace slot of its own and count itself
//                      in; the last contributor of a tile sums the slots in slot order (so the
//                      result does not depend on arrival order), stores, and resets the counter.
// Slots are overwritten, never accumulated into, so the workspace needs no zeroing: only the
// counters return to zero. No CTA waits for another CTA. Replaces, for these shapes, the same
// reference code as skinny_tc.cu (best_submissions/muse_bf16_proj.py:215-287).
#include "common.cuh"

namespace muse {

constexpr int SK_ROWS = 128;
constexpr int SK_BK = 64;
constexpr int SK_MAX_STAGES = 12;
constexpr int SK_THREADS = 192;   // producer warp, MMA warp, four epilogue warps

__device__ __forceinline__ void sk_epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ float4 sk_ldcg4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void sk_stcg4(float* p, float a, float b, float c, float d) {
  asm volatile("st.global.cg.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// First unit of CTA b's run; shared by the kernel and the host (workspace sizing).
__host__ __device__ inline long long sk_start(long long b, long long L, long long G) { return b * L / G; }
// The CTA whose run contains unit u.
__host__ __device__ inline int sk_owner(long long u, long long L, long long G) {
  long long b = u * G / L;
  while (b + 1 < G && sk_start(b + 1, L, G) <= u) ++b;
  while (b > 0 && sk_start(b, L, G) > u) --b;
  return static_cast<int>(b);
}

template <int NTOK, bool HILO, bool PEERS>
__global__ void __launch_bounds__(SK_THREADS, 1)
streamk_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_wlo,
                  const __grid_constant__ CUtensorMap tm_x, void* __restrict__ out, float* __restrict__ ws,
                  int* __restrict__ cnt, int* __restrict__ status, int m, int n, int chunks, int n_tiles, int m_tiles,
                  int stages, int max_contrib, int out_f32, int ld_out, const __grid_constant__ PeerSync ps,
                  unsigned long long* __restrict__ trace) {
  // Optional per-CTA phase stamps (SM cycle counter; slots 15 / 11: global nanosecond timer at entry / exit).
  unsigned long long* const tr = trace ? trace + 16ull * blockIdx.x : nullptr;
#define SK_STAMP(slot) do { if (tr) tr[slot] = static_cast<unsigned long long>(clock64()); } while (0)
  if (tr && threadIdx.x == 0) { SK_STAMP(0); tr[15] = global_ns(); }
  static_assert(NTOK <= 64, "the epilogue keeps a whole accumulator row in registers");
  constexpr int A_BYTES = SK_ROWS * SK_BK * 2;
  constexpr int STAGE_BYTES = A_BYTES * (HILO ? 2 : 1) + NTOK * SK_BK * 2;
  constexpr int TMEM_COLS = 2 * NTOK < 32 ? 32 : 2 * NTOK;   // two accumulators
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[SK_MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_empty[SK_MAX_STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_abort;
  __shared__ int s_flag;    // epilogue: "this CTA is the tile's last contributor"; later: peer finish
  __shared__ int s_epoch;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long G = gridDim.x;
  const long long L = static_cast<long long>(n_tiles) * m_tiles * chunks;
  const long long lo = sk_start(blockIdx.x, L, G), hi = sk_start(blockIdx.x + 1, L, G);
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  uint64_t pol_w = 0, pol_x = 0;
  // Producer cursor: (tile, chunk) of the next unit to request.
  int p_tile = static_cast<int>(lo / chunks), p_chunk = static_cast<int>(lo - static_cast<long long>(p_tile) * chunks);
  auto issue = [&](int s) {
    const int tile_n = p_tile % n_tiles, tile_m = p_tile / n_tiles;
    const uint32_t full = smem_u32(&bar_full[s]);
    const uint32_t a = smem_base + static_cast<uint32_t>(s) * STAGE_BYTES;
    mbar_expect_tx(full, STAGE_BYTES);
    tma_load_2d(a, &tm_w, p_chunk * SK_BK, tile_n * SK_ROWS, full, pol_w);
    if (HILO) tma_load_2d(a + A_BYTES, &tm_wlo, p_chunk * SK_BK, tile_n * SK_ROWS, full, pol_w);
    tma_load_2d(a + A_BYTES * (HILO ? 2 : 1), &tm_x, p_chunk * SK_BK, tile_m * NTOK, full, pol_x);
    if (++p_chunk == chunks) {
      p_chunk = 0;
      ++p_tile;
    }
  };

  const int total = static_cast<int>(hi - lo);
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&acc_full[0]), 1);
    mbar_init(smem_u32(&acc_full[1]), 1);
    mbar_init(smem_u32(&acc_empty[0]), 128);
    mbar_init(smem_u32(&acc_empty[1]), 128);
    fence_mbar_init();
    pol_w = l2_policy_evict_first();
    pol_x = l2_policy_evict_last();
    const int pre = min(stages, total);
    for (int i = 0; i < pre; ++i) issue(i);   // every stage starts empty: weight bytes move first
    SK_STAMP(1);
    s_abort = 0;
    if constexpr (PEERS) {
      s_epoch = peer_epoch(ps);
      if (blockIdx.x == 0) peer_announce_enter(ps, s_epoch);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  if (tid == 0) SK_STAMP(2);

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer: the rest of the run, each request waiting for its stage to drain
      int s = 0;
      uint32_t phase = 0;
      for (int i = stages; i < total; ++i) {
        if (!mbar_wait(smem_u32(&bar_empty[s]), phase)) {
          atomicOr(status, ST_PRODUCER_TIMEOUT);
          s_abort = 1;
          break;
        }
        issue(s);
        if (++s == stages) {
          s = 0;
          phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer: one accumulator per segment, alternating between the two
      constexpr uint32_t idesc = umma_idesc_bf16(SK_ROWS, NTOK);
      int s = 0, seg = 0;
      uint32_t phase = 0;
      long long idx = lo;
      bool dead = false;
      while (idx < hi && !dead) {
        const long long tile = idx / chunks;
        const long long seg_end = min(hi, (tile + 1) * chunks);
        const int a = seg & 1;
        if (seg >= 2) {   // the epilogue must have drained this accumulator's previous segment
          if (!mbar_wait(smem_u32(&acc_empty[a]), static_cast<uint32_t>((seg >> 1) - 1) & 1u)) {
            atomicOr(status, ST_MMA_TIMEOUT);
            s_abort = 1;
            dead = true;
            break;
          }
          tc_fence_after_sync();
        }
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(a * NTOK);
        bool first = true;
        for (; idx < seg_end; ++idx) {
          if (!mbar_wait(smem_u32(&bar_full[s]), phase)) {
            atomicOr(status, ST_MMA_TIMEOUT);
            s_abort = 1;
            dead = true;
            break;
          }
          tc_fence_after_sync();
          if (idx == lo) SK_STAMP(3);
          const uint32_t sa = smem_base + static_cast<uint32_t>(s) * STAGE_BYTES;
          const uint64_t a_desc = umma_desc_k_sw128(sa);
          const uint64_t b_desc = umma_desc_k_sw128(sa + A_BYTES * (HILO ? 2 : 1));
#pragma unroll
          for (int k = 0; k < SK_BK / 16; ++k) {
            umma_bf16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (!first || k > 0) ? 1u : 0u);
            if (HILO) {
              const uint64_t alo_desc = umma_desc_k_sw128(sa + A_BYTES);
              umma_bf16(d_tmem, alo_desc + 2 * k, b_desc + 2 * k, idesc, 1u);
            }
          }
          first = false;
          umma_commit(smem_u32(&bar_empty[s]));
          if (++s == stages) {
            s = 0;
            phase ^= 1u;
          }
        }
        umma_commit(smem_u32(&acc_full[a]));   // also when giving up, so that the epilogue is released
        ++seg;
      }
      SK_STAMP(4);
    }
    __syncwarp();
  } else {
    // ---- epilogue warps 2..5: warp w may only touch TMEM lanes [32 (w % 4), 32 (w % 4) + 32)
    const int et = tid - 64;                 // 0..127
    const int q = warp & 3, r = q * 32 + lane;
    const int ndst = PEERS ? ps.world : 1;
    const int col0 = PEERS ? ps.col0 : 0;
    bool entered = !PEERS;
    long long idx = lo;
    int seg = 0;
    while (idx < hi) {
      const long long tile = idx / chunks;
      const long long seg_begin = idx, seg_end = min(hi, (tile + 1) * chunks);
      const int a = seg & 1;
      bool ok = mbar_wait(smem_u32(&acc_full[a]), static_cast<uint32_t>(seg >> 1) & 1u);
      if (!ok && lane == 0) atomicOr(status, ST_EPILOGUE_TIMEOUT);
      if (!ok || s_abort) break;
      tc_fence_after_sync();
      if (et == 0) { if (seg == 0) SK_STAMP(5); if (seg_end == hi) SK_STAMP(6); }
      float v[NTOK];
      const uint32_t taddr = tmem_base + static_cast<uint32_t>(a * NTOK) + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
      for (int c = 0; c < NTOK; c += 16) {
        uint32_t t16[16];
        tmem_ld16(taddr + c, t16);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) v[c + j] = __uint_as_float(t16[j]);
      }
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&acc_empty[a]));   // the MMA warp may start the segment after next

      const int tile_n = static_cast<int>(tile % n_tiles), tile_m = static_cast<int>(tile / n_tiles);
      const int tok0 = tile_m * NTOK;
      const int mvalid = min(NTOK, m - tok0);
      const int n_idx = tile_n * SK_ROWS + r;
      const bool row_ok = n_idx < n;
      auto store_row = [&](const float (&val)[NTOK]) {
        if constexpr (PEERS) {
          if (!entered) {   // no store may reach a peer that has not entered this call
            if (et < ps.world && !peer_wait_flag(ps.flags[ps.rank] + et, s_epoch)) atomicOr(status, ST_PEER_ENTER_TIMEOUT);
            sk_epilogue_sync();
            entered = true;
          }
        }
        if (!row_ok) return;
        for (int d = 0; d < ndst; ++d) {
          void* dst = PEERS ? ps.out[d] : out;
#pragma unroll
          for (int j = 0; j < NTOK; ++j) {
            if (j < mvalid) {
              const size_t o = static_cast<size_t>(tok0 + j) * ld_out + col0 + n_idx;
              if (out_f32) reinterpret_cast<float*>(dst)[o] = val[j];
              else reinterpret_cast<__nv_bfloat16*>(dst)[o] = __float2bfloat16_rn(val[j]);
            }
          }
        }
      };

      const bool whole_k = seg_begin == tile * chunks && seg_end == (tile + 1) * chunks;
      if (whole_k) {
        store_row(v);
      } else {
        // Park this segment's partial tile in the slot of this CTA, then count in.
        const int bf = sk_owner(tile * chunks, L, G), bl = sk_owner((tile + 1) * chunks - 1, L, G);
        const int contrib = bl - bf + 1, slot = static_cast<int>(blockIdx.x) - bf;
        float* const tile_ws = ws + static_cast<size_t>(tile) * max_contrib * (SK_ROWS * NTOK);
        float* const mine = tile_ws + (static_cast<size_t>(slot) * SK_ROWS + r) * NTOK;
#pragma unroll
        for (int j = 0; j < NTOK; j += 4) sk_stcg4(mine + j, v[j], v[j + 1], v[j + 2], v[j + 3]);
        __threadfence();
        sk_epilogue_sync();
        if (et == 0 && seg_end == hi) SK_STAMP(7);
        if (et == 0) {
          const int last = atomicAdd(&cnt[tile], 1) == contrib - 1;
          if (last) {
            cnt[tile] = 0;   // everyone has arrived: the counter is ready for the next call
            __threadfence();
          }
          s_flag = last;
        }
        sk_epilogue_sync();
        if (et == 0 && seg_end == hi) SK_STAMP(8);
        if (s_flag) {
          float acc[NTOK];
#pragma unroll
          for (int j = 0; j < NTOK; ++j) acc[j] = 0.f;
          for (int sl = 0; sl < contrib; ++sl) {   // slot order = K order: independent of who arrived when
            const float* p = tile_ws + (static_cast<size_t>(sl) * SK_ROWS + r) * NTOK;
#pragma unroll
            for (int j = 0; j < NTOK; j += 4) {
              const float4 u = sk_ldcg4(p + j);
              acc[j] += u.x; acc[j + 1] += u.y; acc[j + 2] += u.z; acc[j + 3] += u.w;
            }
          }
          store_row(acc);
        }
        sk_epilogue_sync();   // s_flag is reused by the next segment
      }
      if (et == 0 && seg_end == hi) SK_STAMP(9);
      idx = seg_end;
      ++seg;
    }
  }

  // ---- teardown
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (PEERS) peer_finish(ps, s_epoch, static_cast<int>(gridDim.x), status, &s_flag);
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  if (tid == 0) { SK_STAMP(10); if (tr) tr[11] = global_ns(); }
#undef SK_STAMP
}

unsigned long long* skinny_get_trace();

// ---------------------------------------------------------------- host side

int streamk_stage_bytes(int ntok, int hilo) { return SK_ROWS * SK_BK * 2 * (hilo ? 2 : 1) + ntok * SK_BK * 2; }
int streamk_smem_bytes(int ntok, int hilo, int stages) { return stages * streamk_stage_bytes(ntok, hilo) + 1024; }

// Most CTAs that ever share one tile, for a grid of `grid` CTAs: the number of workspace slots per tile.
int streamk_max_contrib(int m, int n, int k, int ntok, int grid) {
  if (m <= 0 || n <= 0 || k <= 0 || ntok <= 0 || grid <= 0) return -1;
  const long long chunks = (k + SK_BK - 1) / SK_BK;
  const long long tiles = static_cast<long long>((n + SK_ROWS - 1) / SK_ROWS) * ((m + ntok - 1) / ntok);
  const long long L = tiles * chunks, G = grid;
  int worst = 1;
  for (long long t = 0; t < tiles; ++t) {
    const int c = sk_owner((t + 1) * chunks - 1, L, G) - sk_owner(t * chunks, L, G) + 1;
    if (c > worst) worst = c;
  }
  return worst;
}

long long streamk_ws_floats(int m, int n, int k, int ntok, int grid) {
  const int mc = streamk_max_contrib(m, n, k, ntok, grid);
  if (mc < 0) return -1;
  const long long tiles = static_cast<long long>((n + SK_ROWS - 1) / SK_ROWS) * ((m + ntok - 1) / ntok);
  return tiles * mc * SK_ROWS * ntok;
}

template <int NTOK, bool HILO, bool PEERS>
static cudaError_t sk_launch(const CUtensorMap* tw, const CUtensorMap* twlo, const CUtensorMap* tx, void* out, float* ws,
                             int* cnt, int* status, int m, int n, int k, int grid, int stages, int out_f32, int ld_out,
                             const PeerSync& ps, cudaStream_t stream) {
  auto kern = streamk_tc_kernel<NTOK, HILO, PEERS>;
  static int dyn_max[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!dyn_max[dev]) {
    cudaFuncAttributes fa;
    int optin = 0;
    if ((e = cudaFuncGetAttributes(&fa, kern)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) return e;
    const int room = optin - static_cast<int>(fa.sharedSizeBytes);
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, room)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared)) !=
        cudaSuccess)
      return e;
    dyn_max[dev] = room;
  }
  const int smem = streamk_smem_bytes(NTOK, HILO, stages);
  if (smem > dyn_max[dev]) return cudaErrorInvalidValue;
  const int chunks = (k + SK_BK - 1) / SK_BK;
  const int n_tiles = (n + SK_ROWS - 1) / SK_ROWS, m_tiles = (m + NTOK - 1) / NTOK;
  const int mc = streamk_max_contrib(m, n, k, NTOK, grid);
  kern<<<grid, SK_THREADS, smem, stream>>>(*tw, HILO ? *twlo : *tw, *tx, out, ws, cnt, status, m, n, chunks, n_tiles,
                                           m_tiles, stages, mc, out_f32, ld_out, ps, skinny_get_trace());
  return cudaGetLastError();
}

// Negative = argument error, positive = cudaError_t, 0 = launched.
int streamk_tc_dispatch(const CUtensorMap* tw, const CUtensorMap* twlo, const CUtensorMap* tx, void* out, float* ws,
                        int* cnt, int* status, int m, int n, int k, int ld_out, int ntok, int grid, int stages,
                        int out_f32, const PeerSync* peers, cudaStream_t stream) {
  PeerSync ps = {};
  if (peers && peers->world > 1) {
    ps = *peers;
    if (ps.world > MAX_WORLD || ps.rank < 0 || ps.rank >= ps.world || ps.col0 < 0) return -8;
    for (int p = 0; p < ps.world; ++p)
      if (!ps.out[p] || !ps.flags[p]) return -8;
    out = ps.out[ps.rank];
  }
  if (!tw || !tx || !out || !ws || !cnt || !status || m <= 0 || n <= 0 || k <= 0) return -1;
  if (k % 8 != 0) return -2;
  const long long chunks = (k + SK_BK - 1) / SK_BK;
  const long long tiles = static_cast<long long>((n + SK_ROWS - 1) / SK_ROWS) * ((m + ntok - 1) / (ntok > 0 ? ntok : 1));
  if (grid < 1 || grid > tiles * chunks || grid > 65535) return -3;
  if (stages < 1 || stages > SK_MAX_STAGES) return -5;
  if (ld_out < n + ps.col0) return -6;
  const bool hilo = twlo != nullptr, pe = ps.world > 1;
#define SK_CASE(NT)                                                                                                    \
  case NT:                                                                                                             \
    if (hilo)                                                                                                          \
      return static_cast<int>(pe ? sk_launch<NT, true, true>(tw, twlo, tx, out, ws, cnt, status, m, n, k, grid, stages, \
                                                             out_f32, ld_out, ps, stream)                              \
                                 : sk_launch<NT, true, false>(tw, twlo, tx, out, ws, cnt, status, m, n, k, grid, stages, \
                                                              out_f32, ld_out, ps, stream));                           \
    return static_cast<int>(pe ? sk_launch<NT, false, true>(tw, twlo, tx, out, ws, cnt, status, m, n, k, grid, stages,  \
                                                            out_f32, ld_out, ps, stream)                               \
                               : sk_launch<NT, false, false>(tw, twlo, tx, out, ws, cnt, status, m, n, k, grid, stages, \
                                                             out_f32, ld_out, ps, stream));
  switch (ntok) {
    SK_CASE(16)
    SK_CASE(32)
    SK_CASE(64)
    default:
      return -7;
  }
#undef SK_CASE
}

}  // namespace muse
