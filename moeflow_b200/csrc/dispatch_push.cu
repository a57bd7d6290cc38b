// Dispatch: pack + all-to-all in one kernel, over peer memory.
//
// Token t of source rank s bound for owner rank d always lands in row recv_d[s, t] (fixed position,
// no count exchange).  A row is
//     [ H bf16 hidden lanes | K int32 local expert ids | K fp32 routing weights | int32 valid ]
// with a row pitch padded to a multiple of 16 bytes.  Slots whose expert lives on another rank carry
// id -1 and weight 0; valid = 1 iff at least one slot is on d and t is a live token (t < T and
// t < *num_valid).  Rows t >= T get valid = 0 and all-empty slots; their hidden lanes stay stale.
//
// The kernel writes every row straight into the owner's receive buffer with plain 16-byte stores
// through the peer mapping (NVLink).  Every CTA (one per token position) then fences once at system
// scope and adds one to flag word [s] of every owner: the flags count arrivals, a forward brings exactly
// C of them per source, and the owner's metadata kernel waits for epoch * C.  No CTA has to be the last
// one, so no second fence and no local counter sit between the rows and the flag.  No NCCL call, no
// staging buffer.
//
// Replaces the reference's pack kernel plus its dispatch all_to_all_single
// (moeflow/kernels/dispatch_pack.py:10-95, moeflow/fixed.py:95-125,234).
#include "common.cuh"
#include "moeflow_b200.h"
#include "router.cuh"

namespace mf {

// Threads per CTA: 256 at decode sizes (the hidden row is loaded and stored by many lanes at once); 128 from 1024
// token positions on, where the kernel is bound by how many CTAs (one token each: a routing warp and its latency)
// an SM holds at a time, and half-size CTAs double that number.
constexpr int kMaxTopK = 32;
constexpr int kMaxRanks = 256;

template <int kDispatchThreads>
__global__ void __launch_bounds__(kDispatchThreads) dispatch_push_kernel(const mf_dispatch_args a) {
  __shared__ int s_id[kMaxTopK];
  __shared__ float s_w[kMaxTopK];
  __shared__ unsigned char s_present[kMaxRanks];

  const int t = blockIdx.x;
  const int tid = threadIdx.x;
  unsigned long long* trace = (a.trace != nullptr && blockIdx.x == 0 && tid == 0) ? a.trace : nullptr;
  if (trace) trace[0] = global_timer_ns();
  grid_dep_launch();  // the metadata kernel may get resident now; it waits for this grid to complete
  {
    // First touches in parallel instead of one after the other (see touch() in common.cuh): every page this CTA
    // reads or writes, one lane each; warp 1 also touches this token's row in every destination's receive buffer.
    if (tid < 12) {
      const void* warm[12] = {a.epoch, a.num_valid, a.logits ? (const void*)(a.logits + (size_t)min(t, a.T > 0 ? a.T - 1 : 0) * a.E) : nullptr,
                              a.bias, a.x, a.peer_recv, a.peer_flag, a.hit + (size_t)t * a.R, a.route_w, a.route_ids,
                              a.done_counter, a.weights};
      touch(warm[tid]);
    } else if (tid >= 32 && tid < 32 + a.R && tid < 64) {
      const int d = tid - 32;
      touch(reinterpret_cast<const uint8_t*>(a.peer_recv[d]) + ((size_t)a.rank * a.C + t) * a.pitch);
      touch(reinterpret_cast<const unsigned*>(a.peer_flag[d]) + a.rank);
    }
  }
  const unsigned epoch_next = *a.epoch + 1u;
  const bool has_token = t < a.T;
  const bool live = has_token && (a.num_valid == nullptr || t < *a.num_valid);

  if (a.logits != nullptr) {
    // Fused routing: warp 0 routes this CTA's token; the other warps go on to load the hidden row.
    extern __shared__ float s_route[];
    if (tid < 32) {
      float w = 0.f;
      int id = -1;
      if (has_token) {
        const RouteParams p{a.E, a.K, a.n_group, a.topk_group, a.sigmoid, a.renorm, a.scale};
        route_token_warp(a.logits + (size_t)t * a.E, a.bias, s_route, s_route + a.E, p, tid, w, id);
      }
      if (tid < a.K) {
        s_id[tid] = has_token ? id : -1;
        s_w[tid] = has_token ? w : 0.f;
        if (has_token) {
          a.route_w[(size_t)t * a.K + tid] = w;
          a.route_ids[(size_t)t * a.K + tid] = id;
        }
      }
    }
  } else if (tid < a.K) {
    s_id[tid] = has_token ? a.ids[(size_t)t * a.K + tid] : -1;
    s_w[tid] = has_token ? a.weights[(size_t)t * a.K + tid] : 0.f;
  }

  // The hidden row is read once and kept in registers for all destinations.
  const int chunks = a.H / 8;  // 16-byte chunks
  constexpr int kMaxPerThread = 4;  // H <= 8192
  uint4 xv[kMaxPerThread];
  if (has_token) {
    const uint4* xr = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.x) + (size_t)t * a.H);
#pragma unroll
    for (int i = 0; i < kMaxPerThread; ++i) {
      const int c = tid + i * kDispatchThreads;
      if (c < chunks) xv[i] = xr[c];
    }
  }
  __syncthreads();
  if (trace) trace[1] = global_timer_ns();  // routed, hidden row loaded

  // Which destinations does this token hit?  One thread per destination, once; the copy loop below then
  // needs no barrier, so the stores to all peers are in flight together.
  for (int d = tid; d < a.R; d += kDispatchThreads) {
    int present = 0;
    if (live)
      for (int k = 0; k < a.K; ++k) present |= (s_id[k] >= 0 && s_id[k] / a.L == d) ? 1 : 0;
    s_present[d] = (unsigned char)present;
    a.hit[(size_t)t * a.R + d] = (unsigned char)present;
  }
  __syncthreads();

  for (int d = 0; d < a.R; ++d) {
    const int present = s_present[d];
    uint8_t* row = reinterpret_cast<uint8_t*>(a.peer_recv[d]) + ((size_t)a.rank * a.C + t) * a.pitch;
    if (has_token && (present || !a.skip_payload)) {
      uint4* dst = reinterpret_cast<uint4*>(row);
#pragma unroll
      for (int i = 0; i < kMaxPerThread; ++i) {
        const int c = tid + i * kDispatchThreads;
        if (c < chunks) dst[c] = xv[i];
      }
    }
    int* meta = reinterpret_cast<int*>(row + (size_t)a.H * 2);
    if (tid < a.K) {
      const bool on = present && s_id[tid] >= 0 && s_id[tid] / a.L == d;
      meta[tid] = on ? s_id[tid] - d * a.L : -1;
      meta[a.K + tid] = on ? __float_as_int(s_w[tid]) : 0;
    } else if (tid == a.K) {
      meta[2 * a.K] = present;
    }
  }

  // Publish: the barrier orders every thread's stores before the system fence of warp 0's lanes (cumulative);
  // then one arrival per destination, issued by different lanes so that they travel together.
  __syncthreads();
  if (trace) trace[2] = global_timer_ns();  // rows stored
  if (tid < 32) {
    fence_before_arrival(a.R);
    if (trace) trace[3] = global_timer_ns();  // fenced
    for (int d = tid; d < a.R; d += 32) red_add_relaxed_sys_u32(reinterpret_cast<unsigned*>(a.peer_flag[d]) + a.rank, 1u);
    if (tid == 0) {
      // the local epoch (read by this rank's later kernels after this grid has completed)
      const unsigned done = atomicAdd(a.done_counter, 1u);
      if (done == gridDim.x - 1) {
        *a.done_counter = 0u;
        *a.epoch = epoch_next;
        if (a.trace) a.trace[5] = global_timer_ns();  // last CTA done
      }
    }
    if (trace) trace[4] = global_timer_ns();  // arrivals sent
  }
}

}  // namespace mf

extern "C" int mf_dispatch_push(const mf_dispatch_args* a, mf_stream_t stream) {
  const int threads = (a && a->C >= 1024 && a->H / 8 <= 128 * 4 && a->R <= 32) ? 128 : 256;
  if (!a || a->C < 1 || a->T > a->C || a->K > mf::kMaxTopK || a->R > mf::kMaxRanks || a->H % 8 != 0 ||
      a->H / 8 > threads * 4 || (a->pitch & 15) != 0 || a->pitch < (long long)a->H * 2 + (2 * a->K + 1) * 4)
    return -1;
  size_t smem = 0;
  if (a->logits != nullptr) {
    if (a->E < a->K || a->n_group < 1 || a->n_group > 32 || a->E % a->n_group != 0 || !a->route_w || !a->route_ids) return -2;
    smem = 2 * (size_t)a->E * sizeof(float);
    if (smem > 40 * 1024) return -3;
  }
  if (threads == 128)
    mf::dispatch_push_kernel<128><<<a->C, 128, smem, static_cast<cudaStream_t>(stream)>>>(*a);
  else
    mf::dispatch_push_kernel<256><<<a->C, 256, smem, static_cast<cudaStream_t>(stream)>>>(*a);
  return (int)cudaGetLastError();
}
