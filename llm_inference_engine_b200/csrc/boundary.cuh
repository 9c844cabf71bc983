// The post-attention boundary that produces the pooler's and the router's input in the reference's decode
// layer (_attn_boundary_kernel, best_submissions/muse_decode_layer.py:694-712; math of
// decode_layer/reference.py:452-454), per token over the hidden width D:
//     s1 = alpha * s + beta * a * rsqrt(mean(a^2) + 1e-8)          s: FP32 residual stream, a: BF16 attention output
//     h  = s1 * rsqrt(mean(s1^2) + 1e-5) * (1 + w)                 w: BF16 norm weight; alpha, beta: FP32 vectors
// Two forms: a stand-alone kernel (one CTA per token), and a CTA-wide prologue that the register-MMA projection
// kernels run in place of loading x, for up to 8 tokens: every CTA rebuilds all of h (it needs whole rows for its
// x fragments), keeps s1 in shared memory, and CTA t also writes token t's s1 / h to global memory for the
// layer's other consumers.
#pragma once

#include "common.cuh"

namespace muse {

struct BoundaryArgs {
  const float* stream;            // [m, D] FP32
  const __nv_bfloat16* attn;      // [m, D] BF16
  const float* alpha;             // [D]
  const float* beta;              // [D]
  const __nv_bfloat16* norm_w;    // [D] BF16
  float* stream1;                 // [m, D] FP32 out (may be null in the fused form)
  __nv_bfloat16* h;               // [m, D] BF16 out (may be null)
  float* h_f32;                   // [m, D] FP32 out (may be null)
};

constexpr int BND_TOKENS = 8;      // most tokens of the fused form
constexpr int BND_PAD = 4;         // floats added to a row of s1 in shared memory (conflict-free fragment reads)
constexpr float BND_POST_EPS = 1e-8f, BND_RMS_EPS = 1e-5f;

__device__ __forceinline__ void bf16x8_to_f32(const uint4& v, float (&f)[8]) {
  f[0] = bf16lo_f32(v.x); f[1] = bf16hi_f32(v.x); f[2] = bf16lo_f32(v.y); f[3] = bf16hi_f32(v.y);
  f[4] = bf16lo_f32(v.z); f[5] = bf16hi_f32(v.z); f[6] = bf16lo_f32(v.w); f[7] = bf16hi_f32(v.w);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  const __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&p);
}

// Sum of eight per-token partials over the CTA; `inv[t] = rsqrt(total[t] / D + eps)` lands in shared memory.
// All NT threads call it (NT >= 256, a multiple of 32); red is [NT / 32][8].
template <int NT>
__device__ __forceinline__ void bnd_reduce8(float (&ss)[BND_TOKENS], float (*red)[BND_TOKENS], float* inv, int D, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int t = 0; t < BND_TOKENS; ++t) {
    float v = ss[t];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[warp][t] = v;
  }
  __syncthreads();
  if (warp < BND_TOKENS) {   // warp t adds up token t
    float v = 0.f;
    for (int w = lane; w < NT / 32; w += 32) v += red[w][warp];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) inv[warp] = rsqrtf(v / static_cast<float>(D) + eps);
  }
  __syncthreads();
}

// Shared memory of the prologue for m tokens of width D: s1 rows (FP32, padded), the attention rows (BF16) and
// 1 + w (FP32).
struct BoundarySmem {
  float* s1;            // [m][D + BND_PAD]
  __nv_bfloat16* a;     // [m][D]
  float* onew;          // [D]
};
__host__ __device__ inline size_t boundary_smem_bytes(int D, int m) {
  return static_cast<size_t>(m) * (D + BND_PAD) * sizeof(float) + static_cast<size_t>(m) * D * 2 + static_cast<size_t>(D) * sizeof(float);
}
__device__ __forceinline__ BoundarySmem boundary_smem_carve(float* base, int D, int m) {
  BoundarySmem b;
  b.s1 = base;
  b.a = reinterpret_cast<__nv_bfloat16*>(base + static_cast<size_t>(m) * (D + BND_PAD));
  b.onew = reinterpret_cast<float*>(b.a + static_cast<size_t>(m) * D);
  return b;
}

// The prologue. One thread starts a bulk copy of every token's stream row (into its s1 row, rewritten in place)
// and attention row, so that all of a CTA's input is in flight at once without holding registers (loads behind
// a per-token branch would be waited for one token at a time); the threads meanwhile fetch alpha, beta and the
// norm weight for their own 8-element chunks. On return (true) b.s1[t * (D + BND_PAD) + d] holds s1 for t < m,
// b.onew[d] = 1 + w[d] and inv2[t] the second norm's factor, so that h[t][d] = s1 * inv2[t] * onew[d]; CTA t
// has written token t's stream1 / h / h_f32 where those pointers are given. False (every thread alike): the
// copies did not arrive within the wait limit, ST_X_TIMEOUT has been raised in *status where given, and the
// caller returns. `bar` is a shared-memory mbarrier not used otherwise. D % 8 == 0; 1 <= m <= BND_TOKENS.
template <int NT>
__device__ __forceinline__ bool boundary_prologue(const BoundaryArgs& bd, int m, int D, const BoundarySmem& b, uint64_t* bar,
                                                  float (*red)[BND_TOKENS], float* inv1, float* inv2, int* status) {
  const int cpt = D >> 3, row = D + BND_PAD;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(bar), 1);
    fence_mbar_init();
    mbar_expect_tx(smem_u32(bar), static_cast<uint32_t>(m) * static_cast<uint32_t>(D) * 6u);
    for (int t = 0; t < m; ++t) {
      bulk_load_1d(smem_u32(b.s1 + t * row), bd.stream + static_cast<size_t>(t) * D, static_cast<uint32_t>(D) * 4u, smem_u32(bar));
      bulk_load_1d(smem_u32(b.a + static_cast<size_t>(t) * D), bd.attn + static_cast<size_t>(t) * D, static_cast<uint32_t>(D) * 2u,
                   smem_u32(bar));
    }
  }
  for (int c = threadIdx.x; c < cpt; c += NT) {
    float w[8];
    bf16x8_to_f32(__ldg(reinterpret_cast<const uint4*>(bd.norm_w) + c), w);
    float4* ow = reinterpret_cast<float4*>(b.onew + c * 8);
    ow[0] = make_float4(1.f + w[0], 1.f + w[1], 1.f + w[2], 1.f + w[3]);
    ow[1] = make_float4(1.f + w[4], 1.f + w[5], 1.f + w[6], 1.f + w[7]);
  }
  __syncthreads();   // the barrier's initialisation is visible to every waiter
  if (!__syncthreads_and(mbar_wait(smem_u32(bar), 0) ? 1 : 0)) {
    if (threadIdx.x == 0 && status) atomicOr(status, ST_X_TIMEOUT);
    return false;
  }
  float ss[BND_TOKENS];
#pragma unroll
  for (int t = 0; t < BND_TOKENS; ++t) ss[t] = 0.f;
  for (int c = threadIdx.x; c < cpt; c += NT) {
    const float4 a0 = __ldg(reinterpret_cast<const float4*>(bd.alpha) + 2 * c), a1 = __ldg(reinterpret_cast<const float4*>(bd.alpha) + 2 * c + 1);
#pragma unroll
    for (int t = 0; t < BND_TOKENS; ++t) {
      if (t < m) {
        float a[8];
        bf16x8_to_f32(reinterpret_cast<const uint4*>(b.a + static_cast<size_t>(t) * D)[c], a);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss[t] = fmaf(a[i], a[i], ss[t]);
        float4* p = reinterpret_cast<float4*>(b.s1 + t * row + c * 8);
        const float4 s0 = p[0], s1 = p[1];
        p[0] = make_float4(a0.x * s0.x, a0.y * s0.y, a0.z * s0.z, a0.w * s0.w);
        p[1] = make_float4(a1.x * s1.x, a1.y * s1.y, a1.z * s1.z, a1.w * s1.w);
      }
    }
  }
  bnd_reduce8<NT>(ss, red, inv1, D, BND_POST_EPS);
#pragma unroll
  for (int t = 0; t < BND_TOKENS; ++t) ss[t] = 0.f;
  for (int c = threadIdx.x; c < cpt; c += NT) {
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(bd.beta) + 2 * c), b1 = __ldg(reinterpret_cast<const float4*>(bd.beta) + 2 * c + 1);
#pragma unroll
    for (int t = 0; t < BND_TOKENS; ++t) {
      if (t < m) {
        float a[8];
        bf16x8_to_f32(reinterpret_cast<const uint4*>(b.a + static_cast<size_t>(t) * D)[c], a);
        float4* p = reinterpret_cast<float4*>(b.s1 + t * row + c * 8);
        const float r = inv1[t];
        float4 v0 = p[0], v1 = p[1];
        v0.x = fmaf(b0.x * a[0], r, v0.x); v0.y = fmaf(b0.y * a[1], r, v0.y); v0.z = fmaf(b0.z * a[2], r, v0.z); v0.w = fmaf(b0.w * a[3], r, v0.w);
        v1.x = fmaf(b1.x * a[4], r, v1.x); v1.y = fmaf(b1.y * a[5], r, v1.y); v1.z = fmaf(b1.z * a[6], r, v1.z); v1.w = fmaf(b1.w * a[7], r, v1.w);
        p[0] = v0;
        p[1] = v1;
        ss[t] += v0.x * v0.x + v0.y * v0.y + v0.z * v0.z + v0.w * v0.w + v1.x * v1.x + v1.y * v1.y + v1.z * v1.z + v1.w * v1.w;
        if (bd.stream1 && static_cast<int>(blockIdx.x) == t) {   // CTA t publishes token t
          float4* g = reinterpret_cast<float4*>(bd.stream1 + static_cast<size_t>(t) * D) + 2 * c;
          g[0] = v0;
          g[1] = v1;
        }
      }
    }
  }
  bnd_reduce8<NT>(ss, red, inv2, D, BND_RMS_EPS);
  const int t = static_cast<int>(blockIdx.x);
  if (t < m && (bd.h || bd.h_f32)) {
    const float r = inv2[t];
    for (int c = threadIdx.x; c < cpt; c += NT) {
      const float4* p = reinterpret_cast<const float4*>(b.s1 + t * row + c * 8);
      const float4* ow = reinterpret_cast<const float4*>(b.onew + c * 8);
      const float4 v0 = p[0], v1 = p[1], o0 = ow[0], o1 = ow[1];
      const float h[8] = {v0.x * r * o0.x, v0.y * r * o0.y, v0.z * r * o0.z, v0.w * r * o0.w,
                          v1.x * r * o1.x, v1.y * r * o1.y, v1.z * r * o1.z, v1.w * r * o1.w};
      if (bd.h)
        reinterpret_cast<uint4*>(bd.h + static_cast<size_t>(t) * D)[c] =
            make_uint4(pack_bf16x2(h[0], h[1]), pack_bf16x2(h[2], h[3]), pack_bf16x2(h[4], h[5]), pack_bf16x2(h[6], h[7]));
      if (bd.h_f32) {
        float4* g = reinterpret_cast<float4*>(bd.h_f32 + static_cast<size_t>(t) * D) + 2 * c;
        g[0] = make_float4(h[0], h[1], h[2], h[3]);
        g[1] = make_float4(h[4], h[5], h[6], h[7]);
      }
    }
  }
  return true;
}

// Eight consecutive values of h for token g starting at element k0 (a multiple of 8), from the prologue's buffers.
__device__ __forceinline__ void boundary_h8(const BoundarySmem& b, const float* inv2, int D, int g, int k0, float (&h)[8]) {
  const float4* p = reinterpret_cast<const float4*>(b.s1 + g * (D + BND_PAD) + k0);
  const float4* ow = reinterpret_cast<const float4*>(b.onew + k0);
  const float4 v0 = p[0], v1 = p[1], o0 = ow[0], o1 = ow[1];
  const float r = inv2[g];
  h[0] = v0.x * r * o0.x; h[1] = v0.y * r * o0.y; h[2] = v0.z * r * o0.z; h[3] = v0.w * r * o0.w;
  h[4] = v1.x * r * o1.x; h[5] = v1.y * r * o1.y; h[6] = v1.z * r * o1.z; h[7] = v1.w * r * o1.w;
}

}  // namespace muse
