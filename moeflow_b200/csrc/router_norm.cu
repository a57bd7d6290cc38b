// Router top-k (noaux_tc) and RMSNorm for sm_100a.
//
// router_topk: one warp per token.  score = sigmoid(logit) (or softmax over the experts); the
// selection runs on score + bias, optionally restricted to the `topk_group` best expert groups
// (group score = sum of the two best biased scores when a bias is given, else the best one); ties
// go to the lower expert id; the returned weights are the unbiased scores of the selected experts,
// renormalised by (sum + 1e-20) and multiplied by the routed scaling factor.  Slot order is
// descending biased score.  Semantics follow moeflow/reference.py:21-62 and moeflow/router.py:10-42.
#include <math_constants.h>

#include "common.cuh"
#include "moeflow_b200.h"

namespace mf {

constexpr int kRouterWarps = 4;

struct Best {
  float v;
  int id;
};

__device__ __forceinline__ bool better(float v, int id, float bv, int bid) {
  // descending value, ascending id; id < 0 means "nothing yet"
  if (bid < 0) return true;
  if (id < 0) return false;
  return v > bv || (v == bv && id < bid);
}

__device__ __forceinline__ Best warp_argmax(Best b) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, b.v, off);
    const int oi = __shfl_xor_sync(0xffffffffu, b.id, off);
    if (better(ov, oi, b.v, b.id)) {
      b.v = ov;
      b.id = oi;
    }
  }
  return b;
}

__global__ void __launch_bounds__(kRouterWarps * 32)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, float* __restrict__ weights,
                   int* __restrict__ ids, int tokens, int E, int K, int n_group, int topk_group, int sigmoid,
                   int renorm, float scale) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* score = sm + (size_t)warp * 2 * E;
  float* biased = score + E;
  const int t = blockIdx.x * kRouterWarps + warp;
  if (t >= tokens) return;
  const float* lg = logits + (size_t)t * E;

  if (sigmoid) {
    for (int e = lane; e < E; e += 32) score[e] = 1.f / (1.f + expf(-lg[e]));
  } else {
    float m = -CUDART_INF_F;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, lg[e]);
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    float s = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float x = expf(lg[e] - m);
      score[e] = x;
      s += x;
    }
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    for (int e = lane; e < E; e += 32) score[e] = score[e] / s;
  }
  for (int e = lane; e < E; e += 32) biased[e] = bias ? score[e] + bias[e] : score[e];
  __syncwarp();

  if (n_group > 1) {
    // One lane per group (n_group <= 32): score the group, then rank the groups.
    const int gs = E / n_group;
    float gscore = -CUDART_INF_F;
    if (lane < n_group) {
      float b1 = -CUDART_INF_F, b2 = -CUDART_INF_F;
      for (int i = 0; i < gs; ++i) {
        const float v = biased[lane * gs + i];
        if (v > b1) {
          b2 = b1;
          b1 = v;
        } else if (v > b2) {
          b2 = v;
        }
      }
      gscore = bias ? b1 + b2 : b1;
    }
    // rank = number of groups that come before this one (higher score, or equal score and lower id)
    int rank = 0;
    for (int g = 0; g < n_group; ++g) {
      const float og = __shfl_sync(0xffffffffu, gscore, g);
      if (lane < n_group && (og > gscore || (og == gscore && g < lane))) ++rank;
    }
    const unsigned keep = __ballot_sync(0xffffffffu, lane < n_group && rank < topk_group);
    for (int e = lane; e < E; e += 32)
      if (!((keep >> (e / gs)) & 1u)) biased[e] = -CUDART_INF_F;
    __syncwarp();
  }

  float wsum = 0.f;
  float my_w = 0.f;  // lane k keeps the weight of slot k (K <= 32)
  int my_id = 0;
  for (int k = 0; k < K; ++k) {
    Best b{-CUDART_INF_F, -1};
    for (int e = lane; e < E; e += 32) {
      const float v = biased[e];
      if (better(v, e, b.v, b.id)) {
        b.v = v;
        b.id = e;
      }
    }
    b = warp_argmax(b);
    const float w = score[b.id];
    wsum += w;
    if (lane == k) {
      my_w = w;
      my_id = b.id;
    }
    if (lane == (b.id & 31)) biased[b.id] = -CUDART_INF_F;
    // ids below -inf (already taken) can never win again because `better` needs v > bv or an equal
    // value with a lower id, and every remaining candidate has a finite score.
    __syncwarp();
  }
  if (lane < K) {
    float w = my_w;
    if (renorm) w = w / (wsum + 1e-20f);
    weights[(size_t)t * K + lane] = w * scale;
    ids[(size_t)t * K + lane] = my_id;
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
      // normalise in fp32, round once, then scale by gamma as the usual bf16 module does
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
  mf::router_topk_kernel<<<blocks, mf::kRouterWarps * 32, smem, static_cast<cudaStream_t>(stream)>>>(
      logits, bias, weights, ids, tokens, experts, top_k, n_group, topk_group, sigmoid, renorm, scale);
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
