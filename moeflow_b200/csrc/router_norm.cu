// Router top-k (noaux_tc) and RMSNorm for sm_100a.
//
// router_topk: one warp per token.  score = sigmoid(logit) (or softmax over the experts); the
// selection runs on score + bias, optionally restricted to the `topk_group` best expert groups
// (group score = sum of the two best biased scores when a bias is given, else the best one); ties
// go to the lower expert id; the returned weights are the unbiased scores of the selected experts,
// renormalised by (sum + 1e-20) and multiplied by the routed scaling factor.  Slot order is
// descending biased score.  Semantics follow moeflow/reference.py:21-62 and moeflow/router.py:10-42.
#include "common.cuh"
#include "moeflow_b200.h"
#include "router.cuh"

namespace mf {

constexpr int kRouterWarps = 4;

__global__ void __launch_bounds__(kRouterWarps * 32)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, float* __restrict__ weights,
                   int* __restrict__ ids, int tokens, RouteParams p) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* score = sm + (size_t)warp * 2 * p.E;
  const int t = blockIdx.x * kRouterWarps + warp;
  if (t >= tokens) return;
  float w;
  int id;
  route_token_warp(logits + (size_t)t * p.E, bias, score, score + p.E, p, lane, w, id);
  if (lane < p.K) {
    weights[(size_t)t * p.K + lane] = w;
    ids[(size_t)t * p.K + lane] = id;
  }
}

// out[r, :] = x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * gamma, bf16 in/out, fp32 math.
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
               __nv_bfloat16* __restrict__ out, int hidden, float eps) {
  __shared__ float red[8];
  const int r = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)r * hidden);
  const uint4* gr = reinterpret_cast<const uint4*>(gamma);
  uint4* orow = reinterpret_cast<uint4*>(out + (size_t)r * hidden);
  const int chunks = hidden / 8;
  float ss = 0.f;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const uint4 v = xr[c];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)hidden + eps);
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const uint4 v = xr[c];
    const uint4 g = gr[c];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      const float2 gf = __bfloat1622float2(gh[i]);
      // everything in fp32, one rounding at the end
      oh[i] = __floats2bfloat162_rn(f.x * inv * gf.x, f.y * inv * gf.y);
    }
    orow[c] = o;
  }
}

}  // namespace mf

extern "C" {

int mf_router_topk(const float* logits, const float* bias, float* weights, int* ids, int tokens, int experts,
                   int top_k, int n_group, int topk_group, int sigmoid, int renorm, float scale,
                   mf_stream_t stream) {
  if (tokens == 0) return 0;
  if (top_k > 32 || top_k < 1 || n_group < 1 || n_group > 32 || experts % n_group != 0 || top_k > experts) return -1;
  const size_t smem = (size_t)mf::kRouterWarps * 2 * experts * sizeof(float);
  if (smem > 48 * 1024) return -2;
  const int blocks = (tokens + mf::kRouterWarps - 1) / mf::kRouterWarps;
  const mf::RouteParams p{experts, top_k, n_group, topk_group, sigmoid, renorm, scale};
  mf::router_topk_kernel<<<blocks, mf::kRouterWarps * 32, smem, static_cast<cudaStream_t>(stream)>>>(
      logits, bias, weights, ids, tokens, p);
  return (int)cudaGetLastError();
}

int mf_rmsnorm(const void* x, const void* gamma, void* out, int rows, int hidden, float eps, mf_stream_t stream) {
  if (rows == 0) return 0;
  if (hidden % 8 != 0) return -1;
  mf::rmsnorm_kernel<<<rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gamma),
      static_cast<__nv_bfloat16*>(out), hidden, eps);
  return (int)cudaGetLastError();
}

}  // extern "C"
