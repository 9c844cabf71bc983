// One-token projection y[N] = W[N,K] . x[K] as a streaming GEMV (no tensor cores: at m = 1 the
// weight bytes are the whole cost). Replaces bf16_proj/gemv1.cu:27-125 of the reference.
//
// A CTA is 8 warps. WPR warps share one weight row (each owns a contiguous K segment), so a CTA
// covers 8 / WPR rows. Each lane streams its segment with 16-byte no-allocate loads, U loads per
// batch, the next batch in flight in registers while the current one is multiplied. x is brought
// into shared memory by one bulk (TMA 1-D) copy that overlaps the first weight batch. Lanes reduce
// by shuffle, the warps of a row through shared memory. One launch, no workspace.
//
// W is BF16 (output BF16, round-to-nearest) or FP32 (router: output FP32); x is BF16; the
// accumulation is FP32. Requires K % 8 == 0 (BF16 W) or K % 4 == 0 (FP32 W), K % WPR == 0 with
// each segment a whole number of 16-byte vectors, and x 16-byte aligned.
#include "common.cuh"

namespace muse {

template <int U>
__device__ __forceinline__ void load_batch(uint4 (&w)[U], const uint4* wp, int v0, int nvec) {
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int v = v0 + u * 32;
    w[u] = v < nvec ? ldg_stream16(wp + v) : make_uint4(0u, 0u, 0u, 0u);
  }
}

// One output feature goes to the caller's `out`, or, column-parallel, to column col0 + row of this
// rank's OWN gathered output; the grid's last CTA then ships the whole slice to the peers.
template <bool F32W>
__device__ __forceinline__ void store_row(const PeerSync& ps, void* out, int row, float acc) {
  void* dst = peer_active(ps) ? ps.out[ps.rank] : out;
  const int col = peer_active(ps) ? ps.col0 + row : row;
  if constexpr (F32W) reinterpret_cast<float*>(dst)[col] = acc;
  else reinterpret_cast<__nv_bfloat16*>(dst)[col] = __float2bfloat16_rn(acc);
}

// All threads of every CTA, after their rows are stored locally. The last CTA copies this rank's
// [col0, col0 + N) slice to every peer in 16-byte vectors (a few KB over NVLink instead of one tiny
// remote store per row) once all peers have entered the call, then publishes and waits.
template <bool F32W>
__device__ __forceinline__ void gemv_peer_finish(const PeerSync& ps, int e, int N, int* status, int* s_flag) {
  if (!peer_last_cta(ps, static_cast<int>(gridDim.x), s_flag)) return;
  peer_wait_all_entered(ps, e, status);
  constexpr int ES = F32W ? 4 : 2;
  const char* src = reinterpret_cast<const char*>(ps.out[ps.rank]) + static_cast<size_t>(ps.col0) * ES;
  const int bytes = N * ES;
  const bool vec = ((reinterpret_cast<uintptr_t>(src) | static_cast<unsigned>(bytes)) & 15) == 0;
  for (int p = 0; p < ps.world; ++p) {
    if (p == ps.rank) continue;
    char* dst = reinterpret_cast<char*>(ps.out[p]) + static_cast<size_t>(ps.col0) * ES;
    if (vec && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
      for (int i = threadIdx.x * 16; i < bytes; i += blockDim.x * 16)
        *reinterpret_cast<uint4*>(dst + i) = __ldcg(reinterpret_cast<const uint4*>(src + i));
    } else {
      for (int i = threadIdx.x * 2; i < bytes; i += blockDim.x * 2)
        *reinterpret_cast<unsigned short*>(dst + i) = __ldcg(reinterpret_cast<const unsigned short*>(src + i));
    }
  }
  peer_publish(ps, e, status);
}

template <int WPR, int U, bool F32W>
__global__ void __launch_bounds__(256) gemv1_kernel(const void* __restrict__ W, const __nv_bfloat16* __restrict__ x,
                                                    void* __restrict__ out, int N, int K, int* __restrict__ status,
                                                    const __grid_constant__ PeerSync ps) {
  constexpr int RPC = 8 / WPR;        // rows per CTA
  constexpr int EPV = F32W ? 4 : 8;   // weights per 16-byte vector
  constexpr int WB = F32W ? 4 : 2;    // bytes per weight
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t xbar;
  __shared__ float part[8];
  __shared__ int s_last;
  __shared__ int s_epoch;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * RPC + warp / WPR;
  const int seg = warp % WPR;
  const int ks = K / WPR;             // elements in one warp's segment
  const int nvec = ks / EPV;
  const bool live = row < N;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&xbar), 1);
    fence_mbar_init();
  }
  const uint4* wp = reinterpret_cast<const uint4*>(
      reinterpret_cast<const char*>(W) + (static_cast<size_t>(live ? row : 0) * K + static_cast<size_t>(seg) * ks) * WB);
  uint4 w[U], wn[U];
  const int nb = live ? (nvec + 32 * U - 1) / (32 * U) : 0;
  if (nb > 0) load_batch<U>(w, wp, lane, nvec);
  // Only the weights have been touched so far: x, the output and the exchange wait for the kernels ahead in the
  // stream (no-ops unless this launch was allowed to start under the previous kernel's tail).
  griddep_launch_dependents();
  griddep_wait();
  if (threadIdx.x == 0) {
    mbar_expect_tx(smem_u32(&xbar), static_cast<uint32_t>(K) * 2u);
    bulk_load_1d(smem_u32(smem), x, static_cast<uint32_t>(K) * 2u, smem_u32(&xbar));
    if (peer_active(ps)) {
      s_epoch = peer_epoch(ps);
      if (blockIdx.x == 0) peer_announce_enter(ps, s_epoch);
    }
  }

  __syncthreads();  // barrier initialised for everyone
  // A CTA-uniform verdict on the copy of x: on a time-out nobody multiplies (x is not there), but every
  // thread still reaches the barriers below and the column-parallel book-keeping, so that the arrival
  // count and the call number stay consistent for the next call.
  const bool x_ok = __syncthreads_and(mbar_wait(smem_u32(&xbar), 0)) != 0;
  if (!x_ok && threadIdx.x == 0) atomicOr(status, ST_X_TIMEOUT);
  const int nb_run = x_ok ? nb : 0;

  const uint8_t* xseg = smem + static_cast<size_t>(seg) * ks * 2;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  for (int b = 0; b < nb_run; ++b) {
    if (b + 1 < nb) load_batch<U>(wn, wp, (b + 1) * 32 * U + lane, nvec);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = b * 32 * U + u * 32 + lane;
      if (v < nvec) {
        if constexpr (F32W) {
          const uint2 xv = *reinterpret_cast<const uint2*>(xseg + static_cast<size_t>(v) * 8);
          a0 = fmaf(__uint_as_float(w[u].x), bf16lo_f32(xv.x), a0);
          a1 = fmaf(__uint_as_float(w[u].y), bf16hi_f32(xv.x), a1);
          a2 = fmaf(__uint_as_float(w[u].z), bf16lo_f32(xv.y), a2);
          a3 = fmaf(__uint_as_float(w[u].w), bf16hi_f32(xv.y), a3);
        } else {
          const uint4 xv = *reinterpret_cast<const uint4*>(xseg + static_cast<size_t>(v) * 16);
          a0 = fmaf(bf16lo_f32(w[u].x), bf16lo_f32(xv.x), a0);
          a1 = fmaf(bf16hi_f32(w[u].x), bf16hi_f32(xv.x), a1);
          a2 = fmaf(bf16lo_f32(w[u].y), bf16lo_f32(xv.y), a2);
          a3 = fmaf(bf16hi_f32(w[u].y), bf16hi_f32(xv.y), a3);
          a0 = fmaf(bf16lo_f32(w[u].z), bf16lo_f32(xv.z), a0);
          a1 = fmaf(bf16hi_f32(w[u].z), bf16hi_f32(xv.z), a1);
          a2 = fmaf(bf16lo_f32(w[u].w), bf16lo_f32(xv.w), a2);
          a3 = fmaf(bf16hi_f32(w[u].w), bf16hi_f32(xv.w), a3);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) w[u] = wn[u];
  }
  float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if constexpr (WPR > 1) {
    if (lane == 0) part[warp] = acc;
    __syncthreads();
    if (lane == 0 && seg == 0) {
#pragma unroll
      for (int s = 1; s < WPR; ++s) acc += part[warp + s];
    }
  }
  if (x_ok && live && lane == 0 && seg == 0) store_row<F32W>(ps, out, row, acc);
  if (peer_active(ps)) gemv_peer_finish<F32W>(ps, s_epoch, N, status, &s_last);
}

// Whole-row variant for tall weights: a persistent grid (every CTA resident at once), warp g of the
// grid takes rows g, g + G, g + 2G, ... . The (row, batch) steps of a warp form one stream that stays
// double-buffered across row boundaries, x is fetched once per CTA instead of once per 8 rows, and
// every SM ends up with the same number of rows to within one, so the grid drains together.
template <int U, bool F32W>
__global__ void __launch_bounds__(256) gemv1_rows_kernel(const void* __restrict__ W, const __nv_bfloat16* __restrict__ x,
                                                         void* __restrict__ out, int N, int K, int* __restrict__ status,
                                                         const __grid_constant__ PeerSync ps) {
  constexpr int EPV = F32W ? 4 : 8;
  constexpr int WB = F32W ? 4 : 2;
  __shared__ int s_last;
  __shared__ int s_epoch;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t xbar;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_warps = gridDim.x * 8;
  const int gw = blockIdx.x * 8 + warp;
  const int nvec = K / EPV;
  const int nb = (nvec + 32 * U - 1) / (32 * U);            // batches per row
  const int my_rows = gw < N ? (N - gw + total_warps - 1) / total_warps : 0;
  const int steps = my_rows * nb;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&xbar), 1);
    fence_mbar_init();
  }
  auto row_ptr = [&](int r) {
    return reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(W) +
                                          static_cast<size_t>(gw + r * total_warps) * K * WB);
  };
  uint4 w[U], wn[U];
  if (steps > 0) load_batch<U>(w, row_ptr(0), lane, nvec);
  griddep_launch_dependents();   // only the weights so far: see gemv1_kernel
  griddep_wait();
  if (threadIdx.x == 0) {
    mbar_expect_tx(smem_u32(&xbar), static_cast<uint32_t>(K) * 2u);
    bulk_load_1d(smem_u32(smem), x, static_cast<uint32_t>(K) * 2u, smem_u32(&xbar));
    if (peer_active(ps)) {
      s_epoch = peer_epoch(ps);
      if (blockIdx.x == 0) peer_announce_enter(ps, s_epoch);
    }
  }
  __syncthreads();
  // CTA-uniform, and without an early return: see gemv1_kernel.
  const bool x_ok = __syncthreads_and(mbar_wait(smem_u32(&xbar), 0)) != 0;
  if (!x_ok && threadIdx.x == 0) atomicOr(status, ST_X_TIMEOUT);
  const int steps_run = x_ok ? steps : 0;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  int r = 0, b = 0;
  for (int s = 0; s < steps_run; ++s) {
    int rn = r, bn = b + 1;
    if (bn == nb) { bn = 0; ++rn; }
    if (s + 1 < steps) load_batch<U>(wn, row_ptr(rn), bn * 32 * U + lane, nvec);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = b * 32 * U + u * 32 + lane;
      if (v < nvec) {
        if constexpr (F32W) {
          const uint2 xv = *reinterpret_cast<const uint2*>(smem + static_cast<size_t>(v) * 8);
          a0 = fmaf(__uint_as_float(w[u].x), bf16lo_f32(xv.x), a0);
          a1 = fmaf(__uint_as_float(w[u].y), bf16hi_f32(xv.x), a1);
          a2 = fmaf(__uint_as_float(w[u].z), bf16lo_f32(xv.y), a2);
          a3 = fmaf(__uint_as_float(w[u].w), bf16hi_f32(xv.y), a3);
        } else {
          const uint4 xv = *reinterpret_cast<const uint4*>(smem + static_cast<size_t>(v) * 16);
          a0 = fmaf(bf16lo_f32(w[u].x), bf16lo_f32(xv.x), a0);
          a1 = fmaf(bf16hi_f32(w[u].x), bf16hi_f32(xv.x), a1);
          a2 = fmaf(bf16lo_f32(w[u].y), bf16lo_f32(xv.y), a2);
          a3 = fmaf(bf16hi_f32(w[u].y), bf16hi_f32(xv.y), a3);
          a0 = fmaf(bf16lo_f32(w[u].z), bf16lo_f32(xv.z), a0);
          a1 = fmaf(bf16hi_f32(w[u].z), bf16hi_f32(xv.z), a1);
          a2 = fmaf(bf16lo_f32(w[u].w), bf16lo_f32(xv.w), a2);
          a3 = fmaf(bf16hi_f32(w[u].w), bf16hi_f32(xv.w), a3);
        }
      }
    }
    if (b == nb - 1) {  // row finished: reduce across the warp and store
      float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) store_row<F32W>(ps, out, gw + r * total_warps, acc);
      a0 = a1 = a2 = a3 = 0.f;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) w[u] = wn[u];
    r = rn;
    b = bn;
  }
  if (peer_active(ps)) gemv_peer_finish<F32W>(ps, s_epoch, N, status, &s_last);
}

template <int U, bool F32W>
static cudaError_t launch_rows(const void* W, const void* x, void* out, int N, int K, int* status, const PeerSync& ps,
                               cudaStream_t s) {
  auto kern = gemv1_rows_kernel<U, F32W>;
  static int per_sm[64] = {0}, sms[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  const int smem = K * 2;
  if (!per_sm[dev]) {
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    int nblk = 0;
    if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nblk, kern, 256, 16 * 1024)) != cudaSuccess) return e;
    per_sm[dev] = nblk > 0 ? nblk : 1;
  }
  int resident = per_sm[dev];
  if (smem > 16 * 1024) {  // long rows: recompute residency for this K
    if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, 256, smem)) != cudaSuccess) return e;
    if (resident < 1) resident = 1;
  }
  int grid = sms[dev] * resident;
  const int need = (N + 7) / 8;
  if (grid > need) grid = need;
  return launch_dependent(kern, dim3(grid), dim3(256), smem, s, W, reinterpret_cast<const __nv_bfloat16*>(x), out, N, K, status, ps);
}

template <bool F32W>
static cudaError_t pick_rows(const void* W, const void* x, void* out, int N, int K, int u, int* st, const PeerSync& ps, cudaStream_t s) {
  switch (u) {
    case 1: return launch_rows<1, F32W>(W, x, out, N, K, st, ps, s);
    case 2: return launch_rows<2, F32W>(W, x, out, N, K, st, ps, s);
    case 4: return launch_rows<4, F32W>(W, x, out, N, K, st, ps, s);
    case 8: return launch_rows<8, F32W>(W, x, out, N, K, st, ps, s);
  }
  return cudaErrorInvalidValue;
}

template <int WPR, int U, bool F32W>
static cudaError_t launch(const void* W, const void* x, void* out, int N, int K, int* status, const PeerSync& ps,
                          cudaStream_t s) {
  constexpr int RPC = 8 / WPR;
  const int smem = K * 2;
  auto kern = gemv1_kernel<WPR, U, F32W>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
  }
  return launch_dependent(kern, dim3((N + RPC - 1) / RPC), dim3(256), smem, s, W, reinterpret_cast<const __nv_bfloat16*>(x), out, N, K,
                          status, ps);
}

template <int WPR, bool F32W>
static cudaError_t pick_u(const void* W, const void* x, void* out, int N, int K, int u, int* st, const PeerSync& ps, cudaStream_t s) {
  switch (u) {
    case 1: return launch<WPR, 1, F32W>(W, x, out, N, K, st, ps, s);
    case 2: return launch<WPR, 2, F32W>(W, x, out, N, K, st, ps, s);
    case 4: return launch<WPR, 4, F32W>(W, x, out, N, K, st, ps, s);
    case 8: return launch<WPR, 8, F32W>(W, x, out, N, K, st, ps, s);
  }
  return cudaErrorInvalidValue;
}

template <bool F32W>
static cudaError_t pick_wpr(const void* W, const void* x, void* out, int N, int K, int wpr, int u, int* st,
                            const PeerSync& ps, cudaStream_t s) {
  switch (wpr) {
    case 1: return pick_u<1, F32W>(W, x, out, N, K, u, st, ps, s);
    case 2: return pick_u<2, F32W>(W, x, out, N, K, u, st, ps, s);
    case 4: return pick_u<4, F32W>(W, x, out, N, K, u, st, ps, s);
    case 8: return pick_u<8, F32W>(W, x, out, N, K, u, st, ps, s);
  }
  return cudaErrorInvalidValue;
}

// Argument checks live here so that the C-ABI wrapper stays a one-liner. Negative = argument error.
int gemv1_dispatch(const void* W, const void* x, void* out, int N, int K, int w_is_f32, int wpr, int unroll,
                   int persistent, int* status, const PeerSync* peers, cudaStream_t stream) {
  PeerSync ps = {};
  if (peers && peers->world > 1) {
    ps = *peers;
    if (ps.world > MAX_WORLD || ps.rank < 0 || ps.rank >= ps.world || ps.col0 < 0) return -8;
    for (int p = 0; p < ps.world; ++p)
      if (!ps.out[p] || !ps.flags[p]) return -8;
    out = ps.out[ps.rank];
  }
  if (!W || !x || !out || !status || N <= 0 || K <= 0) return -1;
  const int epv = w_is_f32 ? 4 : 8;
  if (K % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return -2;
  if (wpr != 1 && wpr != 2 && wpr != 4 && wpr != 8) return -3;
  if (K % wpr != 0 || (K / wpr) % epv != 0) return -4;
  if (K * 2 > 200 * 1024) return -5;
  if (persistent) {
    if (wpr != 1) return -6;  // whole rows per warp only
    return static_cast<int>(w_is_f32 ? pick_rows<true>(W, x, out, N, K, unroll, status, ps, stream)
                                     : pick_rows<false>(W, x, out, N, K, unroll, status, ps, stream));
  }
  const cudaError_t e = w_is_f32 ? pick_wpr<true>(W, x, out, N, K, wpr, unroll, status, ps, stream)
                                 : pick_wpr<false>(W, x, out, N, K, wpr, unroll, status, ps, stream);
  return static_cast<int>(e);
}

}  // namespace muse
