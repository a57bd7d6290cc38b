// Per-token noaux_tc routing executed by one warp (shared by the stand-alone router kernel and the
// fused route + dispatch kernel).  Semantics: moeflow/reference.py:21-62, moeflow/router.py:10-42.
#pragma once

#include <math_constants.h>

#include "common.cuh"

namespace mf {

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

constexpr int kRouteRegs = 16;  // experts per lane kept in registers (E <= 512); larger E selects from shared memory

// Maps a float to an unsigned key with the same order (-inf lowest, +inf highest among non-NaN values).
__device__ __forceinline__ unsigned float_order_key(float x) {
  const unsigned u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct RouteParams {
  int E, K, n_group, topk_group, sigmoid, renorm;
  float scale;
};

// One warp routes one token.  `score` and `biased` are E floats of shared memory each, private to
// the warp.  On return lane k (< K) holds slot k: its final weight and expert id.
__device__ __forceinline__ void route_token_warp(const float* __restrict__ lg, const float* __restrict__ bias,
                                                 float* score, float* biased, const RouteParams& p, int lane,
                                                 float& out_w, int& out_id) {
  const int E = p.E;
  if (p.sigmoid) {
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

  if (p.n_group > 1) {
    // One lane per group (n_group <= 32): score the group, then rank the groups.
    const int gs = E / p.n_group;
    float gscore = -CUDART_INF_F;
    if (lane < p.n_group) {
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
    for (int g = 0; g < p.n_group; ++g) {
      const float og = __shfl_sync(0xffffffffu, gscore, g);
      if (lane < p.n_group && (og > gscore || (og == gscore && g < lane))) ++rank;
    }
    const unsigned keep = __ballot_sync(0xffffffffu, lane < p.n_group && rank < p.topk_group);
    for (int e = lane; e < E; e += 32)
      if (!((keep >> (e / gs)) & 1u)) biased[e] = -CUDART_INF_F;
    __syncwarp();
  }

  float wsum = 0.f;
  float my_w = 0.f;  // lane k keeps the weight of slot k (K <= 32)
  int my_id = 0;
  if (E <= 32 * kRouteRegs) {
    // Selection out of registers: lane l holds experts l, l + 32, ...; a round is a scan of the lane's own
    // values, one warp-wide max over order-preserving integer keys and one warp-wide min over the ids that
    // carry that maximum (ties go to the lower id), instead of ten dependent shuffles.
    float v[kRouteRegs];
#pragma unroll
    for (int j = 0; j < kRouteRegs; ++j) {
      const int e = lane + 32 * j;
      v[j] = e < E ? biased[e] : -CUDART_INF_F;
    }
    for (int k = 0; k < p.K; ++k) {
      unsigned bk = 0u;
      int bj = 0;
#pragma unroll
      for (int j = 0; j < kRouteRegs; ++j) {
        const unsigned key = (lane + 32 * j < E) ? float_order_key(v[j]) : 0u;  // padding never beats a real entry
        if (key > bk) {  // strictly greater: the lowest index (lowest id of this lane) keeps a tie
          bk = key;
          bj = j;
        }
      }
      const unsigned wmax = __reduce_max_sync(0xffffffffu, bk);
      const unsigned cand = (bk == wmax && bk != 0u) ? (unsigned)(lane + 32 * bj) : 0xffffffffu;
      const int id = (int)__reduce_min_sync(0xffffffffu, cand);
      const float w = score[id];
      wsum += w;
      if (lane == k) {
        my_w = w;
        my_id = id;
      }
#pragma unroll
      for (int j = 0; j < kRouteRegs; ++j)
        if (lane == (id & 31) && j == (id >> 5)) v[j] = -CUDART_INF_F;
    }
  } else {
    for (int k = 0; k < p.K; ++k) {
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
      __syncwarp();
    }
  }
  if (p.renorm) my_w = my_w / (wsum + 1e-20f);
  out_w = my_w * p.scale;
  out_id = my_id;
}

}  // namespace mf
