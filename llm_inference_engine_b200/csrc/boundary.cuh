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

// The prologue. On return s1buf[t * (D + BND_PAD) + d] holds s1 (FP32) for t < m and inv2[t] the second norm's
// factor, so that h[t][d] = s1 * inv2[t] * (1 + w[d]). D % 8 == 0; m <= BND_TOKENS.
template <int NT>
__device__ __forceinline__ void boundary_prologue(const BoundaryArgs& bd, int m, int D, float* s1buf,
                                                  float (*red)[BND_TOKENS], float* inv1, float* inv2) {
  const int cpt = D >> 3, row = D + BND_PAD;
  float ss[BND_TOKENS];
#pragma unroll
  for (int t = 0; t < BND_TOKENS; ++t) ss[t] = 0.f;
  for (int c = threadIdx.x; c < cpt; c += NT) {
    const float4 a0 = __ldg(reinterpret_cast<const float4*>(bd.alpha) + 2 * c), a1 = __ldg(reinterpret_cast<const float4*>(bd.alpha) + 2 * c + 1);
#pragma unroll
    for (int t = 0; t < BND_TOKENS; ++t) {
      if (t < m) {
        float a[8];
        bf16x8_to_f32(__ldcg(reinterpret_cast<const uint4*>(bd.attn + static_cast<size_t>(t) * D) + c), a);
        const float4 s0 = __ldcg(reinterpret_cast<const float4*>(bd.stream + static_cast<size_t>(t) * D) + 2 * c);
        const float4 s1 = __ldcg(reinterpret_cast<const float4*>(bd.stream + static_cast<size_t>(t) * D) + 2 * c + 1);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss[t] = fmaf(a[i], a[i], ss[t]);
        float4* dst = reinterpret_cast<float4*>(s1buf + t * row + c * 8);
        dst[0] = make_float4(a0.x * s0.x, a0.y * s0.y, a0.z * s0.z, a0.w * s0.w);
        dst[1] = make_float4(a1.x * s1.x, a1.y * s1.y, a1.z * s1.z, a1.w * s1.w);
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
        bf16x8_to_f32(__ldcg(reinterpret_cast<const uint4*>(bd.attn + static_cast<size_t>(t) * D) + c), a);
        float4* p = reinterpret_cast<float4*>(s1buf + t * row + c * 8);
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
      float w[8];
      bf16x8_to_f32(__ldg(reinterpret_cast<const uint4*>(bd.norm_w) + c), w);
      const float4* p = reinterpret_cast<const float4*>(s1buf + t * row + c * 8);
      const float4 v0 = p[0], v1 = p[1];
      const float h[8] = {v0.x * r * (1.f + w[0]), v0.y * r * (1.f + w[1]), v0.z * r * (1.f + w[2]), v0.w * r * (1.f + w[3]),
                          v1.x * r * (1.f + w[4]), v1.y * r * (1.f + w[5]), v1.z * r * (1.f + w[6]), v1.w * r * (1.f + w[7])};
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
}

// Eight consecutive values of h for token g starting at element k0 (a multiple of 8), from the prologue's buffers.
__device__ __forceinline__ void boundary_h8(const BoundaryArgs& bd, const float* s1buf, const float* inv2, int D, int g, int k0,
                                            float (&h)[8]) {
  float w[8];
  bf16x8_to_f32(__ldg(reinterpret_cast<const uint4*>(bd.norm_w + k0)), w);
  const float4* p = reinterpret_cast<const float4*>(s1buf + g * (D + BND_PAD) + k0);
  const float4 v0 = p[0], v1 = p[1];
  const float r = inv2[g];
  h[0] = v0.x * r * (1.f + w[0]); h[1] = v0.y * r * (1.f + w[1]); h[2] = v0.z * r * (1.f + w[2]); h[3] = v0.w * r * (1.f + w[3]);
  h[4] = v1.x * r * (1.f + w[4]); h[5] = v1.y * r * (1.f + w[5]); h[6] = v1.z * r * (1.f + w[6]); h[7] = v1.w * r * (1.f + w[7]);
}

inline size_t boundary_smem_bytes(int D) { return static_cast<size_t>(BND_TOKENS) * (D + BND_PAD) * sizeof(float); }

}  // namespace muse
