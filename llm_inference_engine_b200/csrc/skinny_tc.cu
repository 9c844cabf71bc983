// out[m, n] = x[m, K] . W[n, K]^T for small m, computed as out^T = W . x^T ("swap AB") so that a
// 128-row weight tile is the wide tensor-core operand and all tokens of a token tile ride along as
// the narrow one. Replaces the reference's Triton kernels: _swab_kernel
// (best_submissions/muse_bf16_proj.py:236-257), _router_kernel (:260-287), the split-K hand-off
// _finish (:215-233) and, with NTOK up to 256, the cuBLAS call for m > 32 (:390).
//
// One CTA = one (weight-row tile, K slice, token tile) unit:
//   warp 0 / lane 0   TMA producer: per 64-wide K chunk, one W box [128 x 64] (plus the "lo" box for the
//                     router's BF16 hi+lo pair) and one x box [NTOK x 64], 128-byte swizzled, into a
//                     ring of `stages` shared-memory stages, completion counted on an mbarrier;
//   warp 1 / lane 0   MMA issuer: four tcgen05.mma (M=128, N=NTOK, K=16) per chunk -- eight for hi+lo,
//                     both halves into the same FP32 accumulator in TMEM -- then tcgen05.commit frees
//                     the stage; a last commit signals the epilogue;
//   all four warps    epilogue: tcgen05.ld the accumulator (lane = weight row, column = token) and
//                     either store the output directly (split == 1) or add it into an FP32 workspace
//                     with red.global.add; the last CTA to arrive on the tile's counter reads the sums
//                     back, writes the output and restores workspace and counter to zero.
// No CTA waits on another, the launch is a single kernel and touches no memory it does not restore,
// so it can be captured in a CUDA graph and replayed.
#include "common.cuh"

namespace muse {

constexpr int TILE_ROWS = 128;  // weight rows per CTA = MMA M
constexpr int BK = 64;          // K elements per stage = one 128-byte swizzle span of BF16
constexpr int MAX_STAGES = 12;

template <int NTOK, bool HILO>
struct SkinnyCfg {
  static constexpr int A_BYTES = TILE_ROWS * BK * 2;
  static constexpr int B_BYTES = NTOK * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES * (HILO ? 2 : 1) + B_BYTES;
  static constexpr int TMEM_COLS = NTOK < 32 ? 32 : NTOK;
};

template <int NTOK, bool HILO>
__global__ void __launch_bounds__(128)
skinny_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_wlo,
                 const __grid_constant__ CUtensorMap tm_x, void* __restrict__ out, float* __restrict__ ws,
                 int* __restrict__ cnt, int* __restrict__ status, int m, int n, int chunks, int split, int stages,
                 int out_f32, int ld_out) {
  using Cfg = SkinnyCfg<NTOK, HILO>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_empty[MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_acc;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_abort;
  __shared__ int s_last;
  __shared__ int s_issued;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile_n = blockIdx.x, tile_m = blockIdx.z;
  const int tile_id = tile_m * gridDim.x + tile_n;
  const int c0 = static_cast<int>(static_cast<long long>(blockIdx.y) * chunks / split);
  const int c1 = static_cast<int>(static_cast<long long>(blockIdx.y + 1) * chunks / split);
  const int nchunks = c1 - c0;

  // 1024-byte alignment: the 128-byte swizzle pattern repeats every 8 rows x 128 bytes.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_acc), 1);
    fence_mbar_init();
    s_abort = 0;
    s_issued = 0;
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
    if (HILO) tma_prefetch_desc(&tm_wlo);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_acc = tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer
      const uint64_t pol_w = l2_policy_evict_first();  // weights are read once
      const uint64_t pol_x = l2_policy_evict_last();   // every CTA of the same K slice re-reads x
      int s = 0, issued = 0;
      uint32_t phase = 0;  // parity of the "empty" phase this stage's previous use will complete
      for (int i = 0; i < nchunks; ++i) {
        if (i >= stages && !mbar_wait(smem_u32(&bar_empty[s]), phase)) {
          atomicOr(status, ST_PRODUCER_TIMEOUT);
          s_abort = 1;
          break;
        }
        const uint32_t full = smem_u32(&bar_full[s]);
        const uint32_t a = smem_base + static_cast<uint32_t>(s) * Cfg::STAGE_BYTES;
        mbar_expect_tx(full, Cfg::STAGE_BYTES);
        tma_load_2d(a, &tm_w, (c0 + i) * BK, tile_n * TILE_ROWS, full, pol_w);
        if (HILO) tma_load_2d(a + Cfg::A_BYTES, &tm_wlo, (c0 + i) * BK, tile_n * TILE_ROWS, full, pol_w);
        tma_load_2d(a + Cfg::A_BYTES * (HILO ? 2 : 1), &tm_x, (c0 + i) * BK, tile_m * NTOK, full, pol_x);
        ++issued;
        if (++s == stages) {
          s = 0;
          if (i >= stages) phase ^= 1u;
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
    }
    __syncwarp();
  }

  // ---- epilogue, all four warps: warp w may only touch TMEM lanes [32w, 32w + 32)
  bool ok = mbar_wait(smem_u32(&bar_acc), 0);
  if (!ok && lane == 0) atomicOr(status, ST_EPILOGUE_TIMEOUT);
  ok = __syncthreads_and(ok && !s_abort);
  tc_fence_after_sync();

  if (ok) {
    const int r = warp * 32 + lane;
    const int n_idx = tile_n * TILE_ROWS + r;
    const bool row_ok = n_idx < n;
    const int tok0 = tile_m * NTOK;
    const int mvalid = min(NTOK, m - tok0);
    const uint32_t taddr = tmem_acc + (static_cast<uint32_t>(warp * 32) << 16);
    float* wsp = ws + static_cast<size_t>(tile_id) * (TILE_ROWS * NTOK) + r;
    __nv_bfloat16* out_bf = reinterpret_cast<__nv_bfloat16*>(out) + static_cast<size_t>(tok0) * ld_out + n_idx;
    float* out_f = reinterpret_cast<float*>(out) + static_cast<size_t>(tok0) * ld_out + n_idx;

#pragma unroll 1
    for (int c = 0; c < NTOK; c += 16) {
      if (c >= mvalid) break;  // CTA-uniform
      uint32_t v[16];
      tmem_ld16(taddr + c, v);
      tmem_ld_wait();
      if (split == 1) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c + j < mvalid && row_ok) {
            const float f = __uint_as_float(v[j]);
            if (out_f32) out_f[static_cast<size_t>(c + j) * ld_out] = f;
            else out_bf[static_cast<size_t>(c + j) * ld_out] = __float2bfloat16_rn(f);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (c + j < mvalid && row_ok) red_add_f32(wsp + (c + j) * TILE_ROWS, __uint_as_float(v[j]));
      }
    }

    if (split > 1) {
      // Every add of this CTA is ordered before its arrival; the last arriver sees all of them.
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
        // Each thread reads back and clears exactly the addresses it added to itself, so the
        // clearing store can never overtake another thread's read.
        if (row_ok) {
          for (int j = 0; j < mvalid; ++j) {
            float* p = wsp + j * TILE_ROWS;
            const float f = ldg_cg_f32(p);
            if (out_f32) out_f[static_cast<size_t>(j) * ld_out] = f;
            else out_bf[static_cast<size_t>(j) * ld_out] = __float2bfloat16_rn(f);
            stg_cg_f32(p, 0.f);
          }
        }
        if (tid == 0) cnt[tile_id] = 0;
      }
    }
  }

  // ---- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (s_abort && tid == 0) {
    // Let every copy this CTA issued land (or give up) before its shared memory is released.
    const int issued = s_issued;
    for (int j = max(0, issued - stages); j < issued; ++j)
      if (!mbar_wait(smem_u32(&bar_full[j % stages]), static_cast<uint32_t>(j / stages) & 1u))
        atomicOr(status, ST_DRAIN_TIMEOUT);
  }
  if (warp == 2) tmem_dealloc(tmem_acc, Cfg::TMEM_COLS);
}

// ---------------------------------------------------------------- host side

template <int NTOK, bool HILO>
static cudaError_t launch(const CUtensorMap* tw, const CUtensorMap* twlo, const CUtensorMap* tx, void* out, float* ws,
                          int* cnt, int* status, int m, int n, int chunks, int split, int stages, int out_f32,
                          int ld_out, cudaStream_t stream) {
  using Cfg = SkinnyCfg<NTOK, HILO>;
  auto kern = skinny_tc_kernel<NTOK, HILO>;
  static int dyn_max[64] = {0};  // per device: opt-in ceiling for dynamic shared memory, once raised
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!dyn_max[dev]) {
    cudaFuncAttributes fa;
    int optin = 0;
    if ((e = cudaFuncGetAttributes(&fa, kern)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) return e;
    const int room = optin - static_cast<int>(fa.sharedSizeBytes);  // static shared memory counts against the limit
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, room)) != cudaSuccess) return e;
    dyn_max[dev] = room;
  }
  const size_t smem = static_cast<size_t>(stages) * Cfg::STAGE_BYTES + 1024;
  if (smem > static_cast<size_t>(dyn_max[dev])) return cudaErrorInvalidValue;
  const dim3 grid((n + TILE_ROWS - 1) / TILE_ROWS, split, (m + NTOK - 1) / NTOK);
  kern<<<grid, 128, smem, stream>>>(*tw, HILO ? *twlo : *tw, *tx, out, ws, cnt, status, m, n, chunks, split, stages,
                                    out_f32, ld_out);
  return cudaGetLastError();
}

int skinny_stage_bytes(int ntok, int hilo) { return TILE_ROWS * BK * 2 * (hilo ? 2 : 1) + ntok * BK * 2; }

// Negative = argument error, positive = cudaError_t, 0 = launched.
int skinny_tc_dispatch(const CUtensorMap* tw, const CUtensorMap* twlo, const CUtensorMap* tx, void* out, float* ws,
                       int* cnt, int* status, int m, int n, int k, int ld_out, int ntok, int split, int stages,
                       int out_f32, cudaStream_t stream) {
  if (!tw || !tx || !out || !status || m <= 0 || n <= 0 || k <= 0) return -1;
  if (k % 8 != 0) return -2;
  const int chunks = (k + BK - 1) / BK;
  if (split < 1 || split > chunks || split > 65535) return -3;
  if (split > 1 && (!ws || !cnt)) return -4;
  if (stages < 1 || stages > MAX_STAGES) return -5;
  if (ld_out < n) return -6;
  const bool hilo = twlo != nullptr;
  cudaError_t e;
#define MUSE_CASE(NT)                                                                                              \
  case NT:                                                                                                         \
    e = hilo ? launch<NT, true>(tw, twlo, tx, out, ws, cnt, status, m, n, chunks, split, stages, out_f32, ld_out,  \
                                stream)                                                                            \
             : launch<NT, false>(tw, twlo, tx, out, ws, cnt, status, m, n, chunks, split, stages, out_f32, ld_out, \
                                 stream);                                                                          \
    break;
  switch (ntok) {
    MUSE_CASE(16)
    MUSE_CASE(32)
    MUSE_CASE(64)
    MUSE_CASE(128)
    MUSE_CASE(256)
    default:
      return -7;
  }
#undef MUSE_CASE
  return static_cast<int>(e);
}

}  // namespace muse
