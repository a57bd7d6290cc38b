// Owner-side reduce fused with the return all-to-all, and the source-side combine.
//
// owner_reduce_push: for every received row (s, t) that is valid,
//     partial = bf16( sum_{k = 0..K-1, inv[row*K+k] >= 0} fp32(y[inv[row*K+k]]) )        (+0.0 start)
// is stored straight into the source rank's combine buffer ret_recv_s[this rank, t] through the peer
// mapping; every CTA (one per received row) then fences once and adds one to the source's return flag
// [this rank].  The flags count arrivals: a forward brings C of them per owner, the combine waits for
// epoch * C.
// `y` already holds bf16(routing weight * fp32 accumulator) from the down GEMM.
//
// combine: waits (bounded) for the return flags of all R owners, then
//     out[t] = bf16( sum_{d = 0..R-1, hit[t, d]} fp32(ret[d, t]) )                        (+0.0 start)
// in ascending owner order; rows without any hit are written as zeros.  The optional "ring" order
// starts at the owner after this rank and rounds to bf16 after every add, which reproduces a bf16
// ring reduce-scatter.
//
// Replaces moeflow/kernels/reduce.py:16-81 and the return all_to_all_single (moeflow/fixed.py:237).
#include "common.cuh"
#include "moeflow_b200.h"

namespace mf {

constexpr int kRowThreads = 256;

__device__ __forceinline__ void acc_bf16x8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&acc)[8]) {
  uint4 o;
  __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  return o;
}

__global__ void __launch_bounds__(kRowThreads) owner_reduce_push_kernel(const mf_reduce_push_args a) {
  __shared__ int s_pos[32];
  const int row = blockIdx.x;  // = s*C + t
  const int s = row / a.C, t = row - s * a.C;
  const int tid = threadIdx.x;
  unsigned long long* trace = (a.trace != nullptr && blockIdx.x == 0 && tid == 0) ? a.trace : nullptr;
  if (trace) trace[0] = global_timer_ns();
  grid_dep_launch();
  // The valid flag and the inverse map were final before the GEMMs started (this grid can only be resident
  // once the down GEMM is, which follows the gate/up GEMM's wait for the metadata pass), so they are fetched
  // ahead of the wait: two dependent cold loads less after the GEMM's last store.
  const int* meta = reinterpret_cast<const int*>(static_cast<const uint8_t*>(a.recv) + (size_t)row * a.pitch +
                                                 (size_t)a.H * 2);
  const bool valid = __ldcg(meta + a.valid_word) != 0;
  if (valid && tid < a.K) s_pos[tid] = __ldcg(a.inv + (size_t)row * a.K + tid);
  if (tid == 0) {
    // touch the pages of the return path ahead of the wait: the pointer tables, this row's destination
    touch(a.peer_ret + s);
    touch(a.peer_flag + s);
    touch(a.done_counter);
    touch(a.push_epoch);
  }
  grid_dep_wait_cta();  // the down GEMM has completed: y is final
  if (trace) trace[1] = global_timer_ns();
  if (valid) {
    __syncthreads();
    const int chunks = a.H / 8;
    const uint4* y = static_cast<const uint4*>(a.y);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.peer_ret[s]) +
                                          ((size_t)a.rank * a.C + t) * a.H * 2);
    for (int c = tid; c < chunks; c += kRowThreads) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      // Issue the loads of up to 8 slots together (they are independent), then add in slot order.
      for (int k0 = 0; k0 < a.K; k0 += 8) {
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int p = (k0 + j < a.K) ? s_pos[k0 + j] : -1;
          if (p >= 0) v[j] = __ldcg(&y[(size_t)p * chunks + c]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int p = (k0 + j < a.K) ? s_pos[k0 + j] : -1;
          if (p >= 0) acc_bf16x8(acc, v[j]);
        }
      }
      dst[c] = pack_bf16x8(acc);
    }
  }
  // The barrier orders every thread's stores before thread 0's fence, which is cumulative: one system
  // fence per CTA instead of one per thread; then this row's arrival at its source rank.
  __syncthreads();
  if (trace) trace[2] = global_timer_ns();  // row stored
  if (tid == 0) {
    fence_before_arrival(a.R);
    if (trace) trace[3] = global_timer_ns();  // fenced
    red_add_relaxed_sys_u32(reinterpret_cast<unsigned*>(a.peer_flag[s]) + a.rank, 1u);
    // Off the critical path: the last CTA counts this push locally.  The combine of this rank expects
    // push_epoch * C arrivals from every owner (all ranks run the same sequence of launches, so their push
    // counts agree), which stays right when some forwards are cut short before the return path.
    const unsigned done = atomicAdd(a.done_counter, 1u);
    if (done == gridDim.x - 1) {
      *a.done_counter = 0u;
      if (a.push_epoch != nullptr) *a.push_epoch += 1u;
      if (a.trace) a.trace[5] = global_timer_ns();  // last CTA done
    }
  }
}

// kThreads: kRowThreads at decode sizes, 128 from 1024 token positions on (one CTA per token: more CTAs per SM).
template <int kThreads>
__global__ void __launch_bounds__(kThreads) combine_kernel(const mf_combine_args a) {
  __shared__ unsigned char s_hit[256];
  const int t = blockIdx.x;
  const int tid = threadIdx.x;
  // hit[t, :] was written by this rank's dispatch kernel: pull its line into L2 ahead of the wait (a hint only,
  // the values are read after the wait), so that the read below does not go to DRAM.
  unsigned long long* trace = (a.trace != nullptr && blockIdx.x == 0 && tid == 0) ? a.trace : nullptr;
  if (trace) trace[0] = global_timer_ns();
  if (tid == 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.hit + (size_t)t * a.R));
  // touch the pages read after the wait: flags, push count, this token's row in every owner's return block
  if (tid < a.R) {
    touch(a.flags != nullptr ? a.flags + tid : nullptr);
    touch(static_cast<const uint8_t*>(a.ret) + ((size_t)tid * a.C + t) * a.H * 2);
  }
  if (tid == 32) touch(a.epoch);
  if (tid == 33) touch(static_cast<const uint8_t*>(a.out) + (size_t)t * a.H * 2);
  grid_dep_wait_cta();
  if (trace) trace[1] = global_timer_ns();
  if (tid < a.R) s_hit[tid] = __ldcg(a.hit + (size_t)t * a.R + tid);
  const unsigned epoch = a.epoch ? __ldcg(a.epoch) : 0u;
  // counting flags: every owner adds one per received row of this rank (C of them) in every forward
  if (a.flags != nullptr && tid < a.R) {
    if (!wait_flag_ge(a.flags + tid, epoch * (unsigned)a.C, a.wait_ns)) report_status(a.status, kReturnFlagTimeout, tid, t, epoch);
  }
  __syncthreads();
  if (trace) trace[2] = global_timer_ns();  // return flags seen
  const int chunks = a.H / 8;
  const uint4* ret = static_cast<const uint4*>(a.ret);
  uint4* out = static_cast<uint4*>(a.out) + (size_t)t * chunks;
  const unsigned char* hit = s_hit;
  for (int c = tid; c < chunks; c += kThreads) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (!a.ring) {
      for (int d0 = 0; d0 < a.R; d0 += 8) {
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (d0 + j < a.R && hit[d0 + j]) v[j] = __ldcg(&ret[((size_t)(d0 + j) * a.C + t) * chunks + c]);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (d0 + j < a.R && hit[d0 + j]) acc_bf16x8(acc, v[j]);
      }
    } else {
      for (int step = 1; step <= a.R; ++step) {
        const int d = (a.rank + step) % a.R;
        if (hit[d]) {
          acc_bf16x8(acc, __ldcg(&ret[((size_t)d * a.C + t) * chunks + c]));
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = bf16_round(acc[i]);
        }
      }
    }
    out[c] = pack_bf16x8(acc);
  }
  if (trace) trace[3] = global_timer_ns();  // row written
}

// Peer ping used by the runtime tests: store a value into every peer's word [rank], then wait
// (bounded) for all local words.  With skip_store nothing is stored, so the wait runs out and the
// status word receives kPingTimeout: the time-out path is exercised without hanging anything.
__global__ void peer_ping_kernel(const unsigned long long* peer_words, unsigned* local_words, int R, int rank,
                                 unsigned value, int skip_store, unsigned long long* status,
                                 unsigned long long wait_ns) {
  const int d = threadIdx.x;
  if (d >= R) return;
  if (!skip_store) st_release_sys_u32(reinterpret_cast<unsigned*>(peer_words[d]) + rank, value);
  if (!wait_flag_ge(local_words + d, value, wait_ns)) report_status(status, kPingTimeout, d, 0, value);
}

}  // namespace mf

extern "C" {

int mf_owner_reduce_push(const mf_reduce_push_args* a, mf_stream_t stream) {
  if (!a || a->K > 32 || a->H % 8 != 0 || a->R < 1 || a->C < 1) return -1;
  return (int)mf::launch_kernel(mf::owner_reduce_push_kernel, dim3(a->R * a->C), dim3(mf::kRowThreads), 0,
                                static_cast<cudaStream_t>(stream), true, *a);
}

int mf_combine(const mf_combine_args* a, mf_stream_t stream) {
  if (!a || a->H % 8 != 0 || a->R < 1 || a->R > mf::kRowThreads || a->C < 1) return -1;
  if (a->C >= 1024 && a->R <= 32)
    return (int)mf::launch_kernel(mf::combine_kernel<128>, dim3(a->C), dim3(128), 0, static_cast<cudaStream_t>(stream),
                                  true, *a);
  return (int)mf::launch_kernel(mf::combine_kernel<mf::kRowThreads>, dim3(a->C), dim3(mf::kRowThreads), 0,
                                static_cast<cudaStream_t>(stream), true, *a);
}

int mf_peer_ping(const unsigned long long* peer_words, unsigned* local_words, int R, int rank, unsigned value,
                 int skip_store, unsigned long long* status, unsigned long long wait_ns, mf_stream_t stream) {
  if (R < 1 || R > 64) return -1;
  mf::peer_ping_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(peer_words, local_words, R, rank, value,
                                                                         skip_store, status, wait_ns);
  return (int)cudaGetLastError();
}

}  // extern "C"

// -------------------------------------------------------------------------------------------------
// Received-row unpacking for external expert kernels: rows [N, pitch] -> contiguous hidden [N, H],
// global expert ids [N, K] (filler expert where the slot is empty or the row is not valid) and
// fp32 weights [N, K] (0 there).  One CTA per row.  Counterpart of the reference's
// moeflow/kernels/expert_prepare.py:10-75.
// -------------------------------------------------------------------------------------------------
namespace mf {
__global__ void __launch_bounds__(kRowThreads)
expert_prepare_kernel(const uint8_t* rows, long long pitch, int H, int K, int rank_offset, int filler, uint4* hidden,
                      int* ids32, long long* ids64, float* weights) {
  // No __restrict__ / read-only loads here: this kernel may become resident (programmatic launch) before its
  // predecessors have written the rows, and loads through the non-coherent path are only defined for data that
  // does not change during the kernel's lifetime.  Every input produced earlier in the stream is read from L2.
  grid_dep_wait_cta();
  const int r = blockIdx.x, tid = threadIdx.x;
  const uint8_t* row = rows + (size_t)r * pitch;
  const int* meta = reinterpret_cast<const int*>(row + (size_t)H * 2);
  const bool valid = __ldcg(meta + 2 * K) != 0;
  if (tid < K) {
    const int local = __ldcg(meta + tid);
    const bool live = valid && local >= 0;
    const int gid = live ? local + rank_offset : filler;
    if (ids32) ids32[(size_t)r * K + tid] = gid;
    if (ids64) ids64[(size_t)r * K + tid] = gid;
    weights[(size_t)r * K + tid] = live ? __int_as_float(__ldcg(meta + K + tid)) : 0.f;
  }
  const int chunks = H / 8;
  const uint4* src = reinterpret_cast<const uint4*>(row);
  uint4* dst = hidden + (size_t)r * chunks;
  // Rows that are not valid may hold stale payload (even NaN): copy them as they are; their slots all
  // point at the filler expert with weight 0, so nothing of them reaches an output.
  for (int c = tid; c < chunks; c += kRowThreads) dst[c] = __ldcg(src + c);
}
}  // namespace mf

extern "C" int mf_expert_prepare(const void* rows, long long pitch, int n_rows, int H, int K, int rank_offset, int filler,
                                 void* hidden, int* ids32, long long* ids64, float* weights, mf_stream_t stream) {
  if (n_rows == 0) return 0;
  if (H % 8 != 0 || K > 32 || (pitch & 15) != 0 || (ids32 == nullptr) == (ids64 == nullptr)) return -1;
  return (int)mf::launch_kernel(mf::expert_prepare_kernel, dim3(n_rows), dim3(mf::kRowThreads), 0,
                                static_cast<cudaStream_t>(stream), true, static_cast<const uint8_t*>(rows), pitch, H, K,
                                rank_offset, filler, static_cast<uint4*>(hidden), ids32, ids64, weights);
}

// -------------------------------------------------------------------------------------------------
// Expert-major copy of the received hidden rows: xg[pos] = hidden lanes of received row entry_row[pos]
// for every expert-major position pos < n_entries (plan word).  With it the gate/up GEMM can fetch its
// token tiles by TMA like the down GEMM does (prefill sizes, where the 16-byte gather is the limiter);
// the copy costs one extra read and write of the gathered rows.  No counterpart in the reference, whose
// Triton GEMM gathers through its row index.
// -------------------------------------------------------------------------------------------------
namespace mf {
__global__ void __launch_bounds__(kRowThreads)
permute_rows_kernel(const uint8_t* recv, long long pitch, const int* entry_row, const int* plan, uint4* xg, int H,
                    int n_rows) {
  // The pointers are deliberately not __restrict__ and every input is read with ld.global.cg: this kernel is
  // resident (programmatic launch) while the dispatch and metadata kernels are still writing recv, entry_row
  // and the plan, and a load through the non-coherent read-only path (which the compiler may pick for
  // const __restrict__ data) is only defined for memory that does not change during the kernel's lifetime.
  // With such loads the copy returned rows of an earlier forward on the same addresses.
  grid_dep_launch();
  grid_dep_wait_cta();  // the metadata pass has completed: entry_row and the plan are final
  const int n_entries = __ldcg(plan + MF_PLAN_N_ENTRIES);
  const int chunks = H / 8;
  for (int pos = blockIdx.x; pos < n_entries; pos += gridDim.x) {
    const int r = __ldcg(entry_row + pos);
    if (r < 0 || r >= n_rows) continue;  // never taken for a consistent layout; keeps a bad index from being followed
    const uint4* src = reinterpret_cast<const uint4*>(recv + (size_t)r * pitch);
    uint4* dst = xg + (size_t)pos * chunks;
    for (int c = threadIdx.x; c < chunks; c += kRowThreads) dst[c] = __ldcg(src + c);
  }
}
}  // namespace mf

extern "C" int mf_permute_rows(const void* recv, long long pitch, const int* entry_row, const int* plan, void* xg, int H,
                               int n_rows, int grid, mf_stream_t stream) {
  if (!recv || !entry_row || !plan || !xg || H % 8 != 0 || (pitch & 15) != 0 || grid < 1 || n_rows < 1) return -1;
  return (int)mf::launch_kernel(mf::permute_rows_kernel, dim3(grid), dim3(mf::kRowThreads), 0,
                                static_cast<cudaStream_t>(stream), true, static_cast<const uint8_t*>(recv), pitch,
                                entry_row, plan, static_cast<uint4*>(xg), H, n_rows);
}

