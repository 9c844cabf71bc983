// out[m, N] = x[m, K] . W[N, K]^T for 1..8 tokens with W read in a LOSSLESS 12-bit form: 25 % fewer bytes on a
// path that is bound by the weight stream.
//
// The format is the reference author's (bf16_proj/probe18.py:332-362 `_zip`, notes in bf16_proj/LOG.md "lossless
// 12-bit weight compression"): the low byte of every BF16 weight is kept raw; the high byte (sign + exponent bits
// 7..1) of trained or Gaussian weights falls into a window of 8 neighbouring values for all but ~1e-4 of them, so
// it is stored as a 4-bit code (sign, index into the window, window base `b2` per matrix). A weight whose high
// byte is outside the window is coded as the window's smallest magnitude with its own sign, and listed with its
// true value in a small per-row-group table; the kernel adds x * true - x * coded for it in FP32 (both products
// are exact), so every weight enters the sum with exactly its BF16 value.
//
// The reference decoded tiles in Triton in front of wgmma and lost to its plain kernel. Here the decode runs in
// the registers of the persistent register-MMA walk (fewtok_xreg_kernel): a lane's 16-byte load of 8 weights
// becomes 8 raw bytes + 4 code bytes, laid out by prepare so that every load is still a 16-byte vector:
//   low plane  [N, K]     bytes, per 64-byte span (two 32-weight pieces): lane q's 8 bytes of piece 0, then of piece 1
//   code plane [N, K / 2] bytes, per 64-byte span (four pieces): lane q's 4 bytes of each piece; byte i holds the
//                         codes of the lane's weights i (low nibble) and i + 4 (high nibble)
// and 12 integer operations per 8 weights (2 shifts, 6 logic / add, 4 byte permutes) rebuild the four BF16 pairs
// the plain kernel would have loaded: the MMAs, their order and the results for weights inside the window are the
// same bit for bit.
//
// Measured on B200 (cold weights, us per call, 12288 x 4096 / 4096 x 4096, 1..8 tokens): 18.1-18.4 / 8.9-9.0 against
// 18.1-18.4 / 8.3-8.4 for the plain walk: the 25 % fewer bytes buy nothing, because a round of the walk costs the
// same 1.5 us either way: memory latency plus, here, 0.35 us in which all 32 warps decode at once (48 integer
// operations per lane and round). Tried and slower: two packed groups per lane in registers (no gain: 19.2-20.4),
// the packed bytes through a per-lane cp.async ring 2-4 groups deep (22-30, worse with depth), 16 rows per round
// (21.6-25), the A fragments in shared memory (22-36), one CTA-wide reduction per two or four groups (18.3 /
// 21.3). The planner therefore never selects this kernel; it is an entry point with its numbers beside it.
#include <cstring>

#include "common.cuh"

namespace muse {

__device__ __forceinline__ void zip_mma_16816(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t zip_prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

constexpr int ZIP_MAX_CAP = 64;           // most table entries of a row group
constexpr int ZIP_TABLE_SMEM = 48 * 1024;  // most shared memory for one CTA's table entries (groups of the CTA x cap x 8 bytes)

// The 8 weights of one lane-piece: raw low bytes l0 (weights 0..3) and l1 (4..7), code word nb -> four BF16 pairs.
__device__ __forceinline__ void zip_decode8(uint32_t l0, uint32_t l1, uint32_t nb, uint32_t base4, uint32_t (&w)[4]) {
  const uint32_t ha = ((nb & 0x07070707u) + base4) | ((nb << 4) & 0x80808080u);
  const uint32_t hb = (((nb >> 4) & 0x07070707u) + base4) | (nb & 0x80808080u);
  w[0] = zip_prmt(l0, ha, 0x5140u);
  w[1] = zip_prmt(l0, ha, 0x7362u);
  w[2] = zip_prmt(l1, hb, 0x5140u);
  w[3] = zip_prmt(l1, hb, 0x7362u);
}

template <int U>
struct ZipRegs {
  uint4 lo[U / 2];
  uint4 nb[U / 4];
};

// NW warps x U pieces of 32 weights cover a row: K <= 32 NW U, K % 128 == 0. R = row groups between two CTA-wide
// reductions (1 or 2): a lane keeps its partial sums of R groups in registers, so the warps synchronise once per
// R groups and drift apart in between: while one warp decodes, another's loads are in flight. (With R = 1 every warp
// decodes at the same time and the decode adds to every round what the smaller weight saves.)
template <int NW, int U, bool VEC, int R>
__global__ void __launch_bounds__(NW * 32) fewtok_zip_kernel(const uint8_t* __restrict__ lo, const uint8_t* __restrict__ nib,
                                                             const int2* __restrict__ exc, int cap, uint32_t base4, float coded,
                                                             const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                             int m, int N, int K, int ld_x, int ld_out) {
  static_assert(U % 4 == 0, "a lane loads whole 16-byte vectors of the code plane: four pieces at a time");
  static_assert(R == 1 || R == 2, "row groups per reduction");
  // Dynamic shared memory: the partial sums red[2][R][NW][64] FP32, then the table entries of ALL of this CTA's row
  // groups ([groups][cap] int2) and the activations they multiply ([entry][8 tokens] FP32), fetched once at the start.
  extern __shared__ __align__(16) uint8_t zip_smem[];
  float* const red = reinterpret_cast<float*>(zip_smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int C = static_cast<int>(gridDim.x), c = static_cast<int>(blockIdx.x);
  const int kblocks = K >> 5, groups = (N + 7) >> 3;
  const int my_groups = c < groups ? (groups - c + C - 1) / C : 0;
  const int first = warp * U;
  int2* const exc_s = reinterpret_cast<int2*>(red + 2 * R * NW * 64);
  float* const xe_s = reinterpret_cast<float*>(exc_s + my_groups * cap);   // [entry][8 tokens]

  ZipRegs<U> p;
  auto load = [&](int i) {
    int row = (c + i * C) * 8 + g;
    row = row < N ? row : N - 1;
    const uint8_t* pl = lo + static_cast<size_t>(row) * K + first * 32 + q * 16;
    const uint8_t* pn = nib + static_cast<size_t>(row) * (K >> 1) + first * 16 + q * 16;
#pragma unroll
    for (int j = 0; j < U / 4; ++j) {
      const bool in = first + 4 * j < kblocks;
      p.lo[2 * j] = in ? ldg_stream16(pl + j * 128) : make_uint4(0u, 0u, 0u, 0u);
      p.lo[2 * j + 1] = in ? ldg_stream16(pl + j * 128 + 64) : make_uint4(0u, 0u, 0u, 0u);
      p.nb[j] = in ? ldg_stream16(pn + j * 64) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  if (my_groups > 0) load(0);
  griddep_launch_dependents();   // only the weights so far; the table is the weight's too, x and out are not
  griddep_wait();
  // One thread per (entry, token): the entry and the activation it multiplies, both fetched now, under the first
  // group's weight loads, so that no epilogue waits for a load.
  for (int v = threadIdx.x; v < my_groups * cap * 8; v += NW * 32) {
    const int en_i = v >> 3, t = v & 7;
    const int i = en_i / cap, e = en_i - i * cap;
    const int2 en = __ldg(exc + static_cast<size_t>(c + i * C) * cap + e);
    if (t == 0) exc_s[en_i] = en;
    xe_s[v] = (en.x >= 0 && t < m)
                  ? __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(x) + static_cast<size_t>(t) * ld_x + (en.x & 0xffff))))
                  : 0.f;
  }
  uint4 xr[U];   // the A fragments: lane (g, q) holds token g's 8 activations of each of its pieces
  {
    const uint4* px = reinterpret_cast<const uint4*>(x + static_cast<size_t>(g < m ? g : 0) * ld_x) + q;
#pragma unroll
    for (int u = 0; u < U; ++u) xr[u] = (g < m && first + u < kblocks) ? __ldcg(px + (first + u) * 4) : make_uint4(0u, 0u, 0u, 0u);
  }
  for (int i0 = 0; i0 < my_groups; i0 += R) {
    float2 part[R];
#pragma unroll
    for (int k = 0; k < R; ++k) {
      part[k] = make_float2(0.f, 0.f);
      const int i = i0 + k;
      if (i < my_groups) {   // CTA-uniform
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < U / 4; ++j) {
          const uint32_t nbw[4] = {p.nb[j].x, p.nb[j].y, p.nb[j].z, p.nb[j].w};
          const uint32_t low[8] = {p.lo[2 * j].x, p.lo[2 * j].y, p.lo[2 * j].z, p.lo[2 * j].w,
                                   p.lo[2 * j + 1].x, p.lo[2 * j + 1].y, p.lo[2 * j + 1].z, p.lo[2 * j + 1].w};
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t w[4];
            zip_decode8(low[2 * v], low[2 * v + 1], nbw[v], base4, w);
            const uint4 xa = xr[4 * j + v];
            zip_mma_16816(acc, xa.x, xa.y, w[0], w[1]);
            zip_mma_16816(acc, xa.z, xa.w, w[2], w[3]);
          }
        }
        if (i + 1 < my_groups) load(i + 1);   // the buffer is free: the next group leaves now
        part[k] = make_float2(acc[0], acc[1]);
      }
    }
    float* const rb = red + ((i0 / R) & 1) * (R * NW * 64);
#pragma unroll
    for (int k = 0; k < R; ++k) *reinterpret_cast<float2*>(rb + (k * NW + warp) * 64 + g * 8 + 2 * q) = part[k];
    __syncthreads();   // the buffer written two reductions ago is free again once every warp passed this
    for (int o = threadIdx.x; o < 64 * R; o += NW * 32) {   // NW * 32 >= 256: one pass; whole warps
      const int k = o >> 6, t = (o >> 3) & 7, r = o & 7;
      const int i = i0 + k;
      float sum = 0.f;
#pragma unroll 8
      for (int wv = 0; wv < NW; ++wv) sum += rb[(k * NW + wv) * 64 + (o & 63)];
      const int row0 = (c + i * C) * 8;
      // Weights outside the window: x * true - x * coded, both products exact in FP32 (entries are sorted: the
      // first empty one ends the list).
      if (i < my_groups) {
        for (int e = 0; e < cap; ++e) {
          const int2 en = exc_s[i * cap + e];
          if (en.x < 0) break;
          if ((en.x >> 16) == r) {
            const float xv = xe_s[(i * cap + e) * 8 + t];
            const float tv = __int_as_float(en.y);
            sum += xv * tv;
            sum -= xv * copysignf(coded, tv);
          }
        }
      }
      if constexpr (VEC) {
        const uint32_t v = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(sum)));
        const uint32_t p01 = v | (__shfl_down_sync(0xffffffffu, v, 1) << 16);
        const uint32_t p23 = __shfl_down_sync(0xffffffffu, p01, 2);
        const uint32_t p45 = __shfl_down_sync(0xffffffffu, p01, 4), p67 = __shfl_down_sync(0xffffffffu, p23, 4);
        if (r == 0 && t < m && i < my_groups) *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * ld_out + row0) = make_uint4(p01, p23, p45, p67);
      } else {
        if (t < m && i < my_groups && row0 + r < N) out[static_cast<size_t>(t) * ld_out + row0 + r] = __float2bfloat16_rn(sum);
      }
    }
  }
}

template <int NW, int U, bool VEC, int R>
static cudaError_t launch_zip(const void* lo, const void* nib, const void* exc, int cap, unsigned base4, float coded, const void* x,
                              void* out, int m, int N, int K, int ld_x, int ld_out, cudaStream_t s) {
  auto kern = fewtok_zip_kernel<NW, U, VEC, R>;
  constexpr size_t RED = static_cast<size_t>(2) * R * NW * 64 * sizeof(float);
  static int per_sm[64] = {0}, sms[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!per_sm[dev]) {
    if ((e = cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    int resident = 0;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(RED + ZIP_TABLE_SMEM))) != cudaSuccess)
      return e;
    if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, NW * 32, RED + 4096)) != cudaSuccess) return e;
    if (resident < 1) return cudaErrorInvalidConfiguration;
    per_sm[dev] = resident;
  }
  int walkers = sms[dev] * per_sm[dev];
  const int groups = (N + 7) / 8;
  if (walkers > groups) walkers = groups;
  const size_t table = static_cast<size_t>((groups + walkers - 1) / walkers) * cap * (sizeof(int2) + 8 * sizeof(float));
  if (table > ZIP_TABLE_SMEM) return cudaErrorInvalidConfiguration;
  return launch_dependent(kern, dim3(walkers), dim3(NW * 32), RED + table, s, reinterpret_cast<const uint8_t*>(lo),
                          reinterpret_cast<const uint8_t*>(nib), reinterpret_cast<const int2*>(exc), cap, base4, coded,
                          reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(out), m, N, K, ld_x, ld_out);
}

// 1..8 tokens; warps x unroll in {32 x 4, 16 x 8, 16 x 4}; `reduce_every` = row groups per CTA-wide reduction, 1 or 2. `exc`: per 8-row
// group `cap` entries {row in group << 16 | column, FP32 bits of the true weight}, the unused ones {-1, 0} last;
// base = the window's first high-byte value (0..120); the coded magnitude follows from it. Negative = argument error.
int fewtok_zip_dispatch(const void* lo, const void* nib, const void* exc, int cap, int base, const void* x, void* out, int m, int N,
                        int K, int ld_x, int ld_out, int warps, int unroll, int reduce_every, cudaStream_t stream) {
  if (!lo || !nib || !x || !out || N <= 0 || K <= 0) return -1;
  if (cap < 0 || cap > ZIP_MAX_CAP || (cap > 0 && !exc) || base < 0 || base > 120) return -1;
  if (m < 1 || m > 8) return -9;
  if (K % 128 != 0 || K > 32 * warps * unroll || ld_x % 8 != 0 || ld_x < K || ld_out < N || K > 65535) return -2;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(lo) | reinterpret_cast<uintptr_t>(nib)) & 15) return -2;
  if (exc && (reinterpret_cast<uintptr_t>(exc) & 7)) return -2;
  if (reduce_every != 1 && reduce_every != 2) return -9;
  const unsigned base4 = static_cast<unsigned>(base) * 0x01010101u;
  // The coded value of an out-of-window weight: high byte = base, low byte = 0 (exponent field 2 base, no mantissa).
  const unsigned coded_bits = static_cast<unsigned>(base) << 24;
  float coded;
  memcpy(&coded, &coded_bits, sizeof(coded));
  const bool vec = N % 8 == 0 && ((reinterpret_cast<uintptr_t>(out) | (static_cast<uintptr_t>(ld_out) * 2)) & 15) == 0;
  cudaError_t e = cudaErrorInvalidValue;
#define MUSE_ZIP(NW_, U_, R_)                                                                                          \
  if (warps == NW_ && unroll == U_ && reduce_every == R_)                                                                   \
    e = vec ? launch_zip<NW_, U_, true, R_>(lo, nib, exc, cap, base4, coded, x, out, m, N, K, ld_x, ld_out, stream)     \
            : launch_zip<NW_, U_, false, R_>(lo, nib, exc, cap, base4, coded, x, out, m, N, K, ld_x, ld_out, stream);
  MUSE_ZIP(32, 4, 1) MUSE_ZIP(32, 4, 2) MUSE_ZIP(16, 8, 1) MUSE_ZIP(16, 8, 2) MUSE_ZIP(16, 4, 1) MUSE_ZIP(16, 4, 2)
#undef MUSE_ZIP
  if (e == cudaErrorInvalidValue) return -9;
  return static_cast<int>(e);
}

}  // namespace muse
