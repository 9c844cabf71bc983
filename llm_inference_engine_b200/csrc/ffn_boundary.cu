// The post-FFN boundary of the reference's decode layer, the consumer of the unpooler projection
// (_ffn_boundary_kernel, best_submissions/muse_decode_layer.py:715-730; math of decode_layer/reference.py:466-476),
// per token over the hidden width D, with f the unpooler's output of nf <= D columns (up to 8 tokens a GPU computes
// only its slice of the unpooler's rows and the other columns are the all-gather's zeros):
//     f' = f * (1 + w_post)                                      (zero beyond nf)
//     s2 = alpha * s1 + beta * f' * rsqrt(mean(f'^2) + 1e-8)      s1, s2: FP32 residual stream
//     hidden = s2 * rsqrt(mean(s2^2) + 1e-5) * (1 + w_next)       the next layer's attention input, BF16
// Two forms: a stand-alone kernel (one CTA per token, f in BF16 as the projection stores it), and the unpooler
// projection and the boundary as ONE launch for up to 8 tokens: the register-MMA walk writes f in FP32 to a scratch,
// every CTA counts itself done, and CTA t < m then waits (bounded) for the count and computes token t.
#include "boundary.cuh"
#include "common.cuh"

namespace muse {

struct FfnBoundaryArgs {
  const float* stream1;           // [m, D] FP32
  const float* alpha;             // [D]
  const float* beta;              // [D]
  const __nv_bfloat16* post_w;    // [D] BF16
  const __nv_bfloat16* next_w;    // [D] BF16
  float* stream2;                 // [m, D] FP32 out (may be null)
  __nv_bfloat16* hidden;          // [m, D] BF16 out
};

__device__ __forceinline__ uint4 ffn_ld_cg16(const void* p) {   // L2 load of data another CTA of this launch wrote
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ffn_mma_16816(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

// Token t's boundary by a whole CTA of NT threads, CH chunks of 8 elements per thread (D <= 8 NT CH), in two steps
// so that the one-launch form can fetch what does not depend on f while f is still being computed.
template <int CH>
struct FfnTokenRegs {
  float v[CH][8];    // alpha * s1, later s2
  float be[CH][8];   // beta
  float wp[CH][8];   // 1 + w_post
};

template <int NT, int CH>
__device__ __forceinline__ void ffn_token_fetch(const FfnBoundaryArgs& a, int t, int D, FfnTokenRegs<CH>& r) {
  const int cpt = D >> 3;
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + j * NT;
    if (c < cpt) {
      float wp[8];
      bf16x8_to_f32(__ldg(reinterpret_cast<const uint4*>(a.post_w) + c), wp);
      const float4 s0 = __ldcg(reinterpret_cast<const float4*>(a.stream1 + static_cast<size_t>(t) * D) + 2 * c);
      const float4 s1 = __ldcg(reinterpret_cast<const float4*>(a.stream1 + static_cast<size_t>(t) * D) + 2 * c + 1);
      const float4 a0 = __ldg(reinterpret_cast<const float4*>(a.alpha) + 2 * c), a1 = __ldg(reinterpret_cast<const float4*>(a.alpha) + 2 * c + 1);
      const float4 b0 = __ldg(reinterpret_cast<const float4*>(a.beta) + 2 * c), b1 = __ldg(reinterpret_cast<const float4*>(a.beta) + 2 * c + 1);
      const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      const float al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float be[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        r.v[j][i] = al[i] * sv[i];
        r.be[j][i] = be[i];
        r.wp[j][i] = 1.f + wp[i];
      }
    }
  }
}

// F32F: f is FP32 written earlier in this launch (read through L2); otherwise BF16. `red`: NT / 32 floats, `bc`:
// one float.
template <int NT, int CH, bool F32F>
__device__ __forceinline__ void ffn_token_finish(const FfnBoundaryArgs& a, const void* f, int nf, int t, int D, FfnTokenRegs<CH>& r,
                                                 float* red, float* bc) {
  const int cpt = D >> 3, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  auto block_inv = [&](float v, float eps) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();   // red and bc are free again
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
      float s = lane < NT / 32 ? red[lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0) *bc = rsqrtf(s / static_cast<float>(D) + eps);
    }
    __syncthreads();
    return *bc;
  };
  float fv[CH][8];
  uint4 wn[CH];   // the next layer's norm weight: asked for now, needed after the two sums
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + j * NT;
    wn[j] = make_uint4(0u, 0u, 0u, 0u);
    if (c < cpt) {
      wn[j] = __ldg(reinterpret_cast<const uint4*>(a.next_w) + c);
      if (c * 8 < nf) {   // nf % 8 == 0: a chunk is inside f or outside
        if constexpr (F32F) {
          const uint4 f0 = ffn_ld_cg16(reinterpret_cast<const float*>(f) + static_cast<size_t>(t) * nf + c * 8);
          const uint4 f1 = ffn_ld_cg16(reinterpret_cast<const float*>(f) + static_cast<size_t>(t) * nf + c * 8 + 4);
          fv[j][0] = __uint_as_float(f0.x); fv[j][1] = __uint_as_float(f0.y); fv[j][2] = __uint_as_float(f0.z); fv[j][3] = __uint_as_float(f0.w);
          fv[j][4] = __uint_as_float(f1.x); fv[j][5] = __uint_as_float(f1.y); fv[j][6] = __uint_as_float(f1.z); fv[j][7] = __uint_as_float(f1.w);
        } else {
          bf16x8_to_f32(__ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(f) + static_cast<size_t>(t) * nf) + c), fv[j]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) fv[j][i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        fv[j][i] *= r.wp[j][i];
        ss = fmaf(fv[j][i], fv[j][i], ss);
        fv[j][i] *= r.be[j][i];
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
        r.v[j][i] = fmaf(fv[j][i], r1, r.v[j][i]);
        ss = fmaf(r.v[j][i], r.v[j][i], ss);
      }
      if (a.stream2) {
        float4* gp = reinterpret_cast<float4*>(a.stream2 + static_cast<size_t>(t) * D) + 2 * c;
        gp[0] = make_float4(r.v[j][0], r.v[j][1], r.v[j][2], r.v[j][3]);
        gp[1] = make_float4(r.v[j][4], r.v[j][5], r.v[j][6], r.v[j][7]);
      }
    }
  }
  const float r2 = block_inv(ss, BND_RMS_EPS);
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + j * NT;
    if (c < cpt) {
      float w[8], h[8];
      bf16x8_to_f32(wn[j], w);
#pragma unroll
      for (int i = 0; i < 8; ++i) h[i] = r.v[j][i] * r2 * (1.f + w[i]);
      reinterpret_cast<uint4*>(a.hidden + static_cast<size_t>(t) * D)[c] =
          make_uint4(pack_bf16x2(h[0], h[1]), pack_bf16x2(h[2], h[3]), pack_bf16x2(h[4], h[5]), pack_bf16x2(h[6], h[7]));
    }
  }
}

// Stand-alone: one CTA of 256 threads per token, D <= 8192, f BF16 [m, nf].
__global__ void __launch_bounds__(256) ffn_boundary_kernel(const __grid_constant__ FfnBoundaryArgs a, const __nv_bfloat16* __restrict__ f,
                                                           int nf, int D) {
  __shared__ float red[8];
  __shared__ float bc;
  griddep_launch_dependents();   // everything here depends on the kernels ahead: only the launch itself overlaps them
  griddep_wait();
  FfnTokenRegs<4> r;
  ffn_token_fetch<256, 4>(a, static_cast<int>(blockIdx.x), D, r);
  ffn_token_finish<256, 4, false>(a, f, nf, static_cast<int>(blockIdx.x), D, r, red, &bc);
}

// The unpooler projection (W [NF, K] BF16, x [m, K] BF16, m <= 8) and the boundary in one launch. 16 warps x U
// pieces of 32 weights cover a row (K <= 512 U). f: FP32 scratch [m, NF]. cnt[0] counts the CTAs whose rows of f
// are stored, cnt[1] the token CTAs that are done; the last of those puts both back to zero.
template <int U>
__global__ void __launch_bounds__(512, 1) unpooler_ffn_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ x,
                                                              float* __restrict__ f, const __grid_constant__ FfnBoundaryArgs a, int m,
                                                              int NF, int K, int ld_x, int D, int* __restrict__ cnt,
                                                              int* __restrict__ status) {
  constexpr int NW = 16;
  __shared__ __align__(16) float red[2][NW][64];
  __shared__ float bred[NW];
  __shared__ float bc;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  const int C = static_cast<int>(gridDim.x), c = static_cast<int>(blockIdx.x);
  const int kblocks = K >> 5, groups = NF >> 3;
  const int my_groups = c < groups ? (groups - c + C - 1) / C : 0;
  const int first = warp * U;
  uint4 w[U], xr[U];
  auto load = [&](int i) {
    const int r = (c + i * C) * 8 + g;
    const uint4* p = reinterpret_cast<const uint4*>(W + static_cast<size_t>(r) * K) + q;
#pragma unroll
    for (int u = 0; u < U; ++u) w[u] = first + u < kblocks ? ldg_stream16(p + (first + u) * 4) : make_uint4(0u, 0u, 0u, 0u);
  };
  if (my_groups > 0) load(0);
  griddep_launch_dependents();   // only the weights so far: x, stream1, the scratch and the counters wait for the kernels ahead
  griddep_wait();
  FfnTokenRegs<2> tok;   // CTA t < m: what token t's boundary needs besides f, asked for now
  if (c < m) ffn_token_fetch<512, 2>(a, c, D, tok);
  {
    const uint4* px = reinterpret_cast<const uint4*>(x + static_cast<size_t>(g < m ? g : 0) * ld_x) + q;
#pragma unroll
    for (int u = 0; u < U; ++u) xr[u] = (g < m && first + u < kblocks) ? __ldcg(px + (first + u) * 4) : make_uint4(0u, 0u, 0u, 0u);
  }
  for (int i = 0; i < my_groups; ++i) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int u = 0; u < U; ++u) {
      ffn_mma_16816(acc, xr[u].x, xr[u].y, w[u].x, w[u].y);
      ffn_mma_16816(acc, xr[u].z, xr[u].w, w[u].z, w[u].w);
    }
    if (i + 1 < my_groups) load(i + 1);
    *reinterpret_cast<float2*>(&red[i & 1][warp][g * 8 + 2 * q]) = make_float2(acc[0], acc[1]);
    __syncthreads();   // the buffer written two groups ago is free again once every warp passed this
    if (threadIdx.x < 64) {
      float sum = 0.f;
#pragma unroll 8
      for (int wv = 0; wv < NW; ++wv) sum += red[i & 1][wv][threadIdx.x];
      const int t = threadIdx.x >> 3, r = (c + i * C) * 8 + (threadIdx.x & 7);
      if (t < m) f[static_cast<size_t>(t) * NF + r] = sum;
    }
  }
  // This CTA's rows of f are stored: count it (the barrier orders every thread's stores before thread 0's fence).
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(cnt, 1);
  }
  if (c >= m) return;
  // CTA t < m: token t's boundary once every CTA has counted itself (bounded wait).
  bool ready = true;
  if (threadIdx.x == 0) {
    const unsigned long long t0 = global_ns();
    while (ld_acquire_gpu(cnt) < C) {
      if (global_ns() - t0 > WAIT_LIMIT_NS) {
        ready = false;
        break;
      }
    }
  }
  const bool ok = __syncthreads_and(ready ? 1 : 0) != 0;
  if (ok) ffn_token_finish<512, 2, true>(a, f, NF, c, D, tok, bred, &bc);
  else if (threadIdx.x == 0) atomicOr(status, ST_X_TIMEOUT);
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(cnt + 1, 1) == m - 1) {   // the last token CTA re-arms the counters
    cnt[0] = 0;
    cnt[1] = 0;
  }
}

static int ffn_args_ok(const FfnBoundaryArgs& a, int m, int D, int nf) {
  if (!a.stream1 || !a.alpha || !a.beta || !a.post_w || !a.next_w || !a.hidden || m < 1 || D < 8 || D % 8 || nf < 8 || nf % 8 || nf > D)
    return -1;
  const uintptr_t all = reinterpret_cast<uintptr_t>(a.stream1) | reinterpret_cast<uintptr_t>(a.alpha) | reinterpret_cast<uintptr_t>(a.beta) |
                        reinterpret_cast<uintptr_t>(a.post_w) | reinterpret_cast<uintptr_t>(a.next_w) |
                        reinterpret_cast<uintptr_t>(a.stream2) | reinterpret_cast<uintptr_t>(a.hidden);
  return (all & 15) ? -2 : 0;
}

// Stand-alone: any m, D <= 8192, f BF16 [m, nf] contiguous.
int ffn_boundary_dispatch(const FfnBoundaryArgs& a, const void* f, int m, int D, int nf, cudaStream_t stream) {
  const int bad = ffn_args_ok(a, m, D, nf);
  if (bad) return bad;
  if (!f || D > 8192) return -2;
  if (reinterpret_cast<uintptr_t>(f) & 15) return -2;
  return static_cast<int>(launch_dependent(ffn_boundary_kernel, dim3(m), dim3(256), 0, stream, a, reinterpret_cast<const __nv_bfloat16*>(f), nf, D));
}

// One launch: m <= 8, K <= 4096 in whole 32-element pieces, NF % 8 == 0 with at least m row groups, D <= 8192.
// f_scratch: FP32 [m, NF]; cnt: 2 ints, zero before the first call and again after every call.
int unpooler_ffn_dispatch(const void* W, const void* x, void* f_scratch, const FfnBoundaryArgs& a, int m, int NF, int K, int ld_x, int D,
                          int* cnt, int* status, cudaStream_t stream) {
  if (!W || !x || !f_scratch || !cnt || !status) return -1;
  const int bad = ffn_args_ok(a, m, D, NF);
  if (bad) return bad;
  if (m > BND_TOKENS || NF / 8 < m) return -9;
  if (K % 32 != 0 || K > 4096 || ld_x % 8 != 0 || ld_x < K || D > 8192) return -2;
  if ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(f_scratch)) & 15) return -2;
  static int sms[64] = {0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return static_cast<int>(cudaErrorInvalidDevice);
  if (!sms[dev] && (e = cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return static_cast<int>(e);
  const int groups = NF / 8;
  const int ctas = groups < sms[dev] ? groups : sms[dev];   // at most one CTA per SM: the token CTAs wait for all the others
  const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(W);
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  float* fs = reinterpret_cast<float*>(f_scratch);
  if (K <= 1024) e = launch_dependent(unpooler_ffn_kernel<2>, dim3(ctas), dim3(512), 0, stream, w, xb, fs, a, m, NF, K, ld_x, D, cnt, status);
  else if (K <= 2048) e = launch_dependent(unpooler_ffn_kernel<4>, dim3(ctas), dim3(512), 0, stream, w, xb, fs, a, m, NF, K, ld_x, D, cnt, status);
  else e = launch_dependent(unpooler_ffn_kernel<8>, dim3(ctas), dim3(512), 0, stream, w, xb, fs, a, m, NF, K, ld_x, D, cnt, status);
  return static_cast<int>(e);
}

}  // namespace muse
