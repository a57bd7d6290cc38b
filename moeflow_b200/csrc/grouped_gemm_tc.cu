// Grouped expert GEMMs on the 5th-generation tensor cores (tcgen05) for sm_100a.
//
// The expert GEMMs of a decode step are weight-streaming bound: a few (1..64) token rows per expert
// against tens of MB of expert weights.  The kernels below are therefore written "swap-AB": the
// 128 weight rows of a block are the UMMA M dimension, the token rows are the UMMA N dimension
// (16..n_max), accumulators live in tensor memory, and the weight stream is a deep TMA pipeline.
//
//   gate/up  : acc_gate[128, n] = W13[e, mb*128 + r, :] . X[n, :]     (and acc_up for rows I + ...)
//              out[entry, mb*128 + r] = bf16( silu(min(gate, lim)) * clamp(up, +-lim) )
//   down     : acc[128, n] = W2[e, mb*128 + r, :] . ACT[n, :]
//              out[entry, mb*128 + r] = bf16( row_scale[entry] * acc )
//              (two_blocks: a unit covers two adjacent weight blocks with two accumulators, like gate/up,
//               so a token tile is fetched from L2 once per 256 output columns: the long-prefill form)
//
// A unit is (token tile, 128-row weight block); it needs k_blocks K steps.  The token tiles and the way
// the units are cut along K come from a device-side plan (see expert_meta.cu), so nothing is read back
// to the host.  Two cuts exist:
//   * K split S in {1, 2, 4, 8} (plan word = S): every unit is cut into S equal segments, segments are
//     dealt to the CTAs round-robin;
//   * stream-K (plan word = 0): the units' K steps are laid end to end and every CTA takes one contiguous
//     share of that line, so all CTAs stream the same number of weight bytes whatever the unit count
//     (no partly filled last round); a unit that straddles CTA boundaries is cut there.
// A segment that is not a whole unit stores its fp32 partial sums; the last segment to arrive (per
// 32-row quarter) adds the segments in K order, so the result does not depend on arrival order.
//
// Warp roles (256 threads, one CTA per SM, persistent over units blockIdx.x, +gridDim.x, ...):
//   warp 0      TMA producer for the weight tiles (lane 0 issues)
//   warp 1      UMMA issuer (lane 0 issues); owns the tensor-memory allocation
//   warps 2-3   token-operand producers: gather rows by index with cp.async into the swizzled tile
//   warps 4-7   epilogue: tcgen05.ld -> registers -> activation / scale -> global
//
// Replaces the reference's Triton grouped GEMM, unfused SwiGLU and expert-input gather
// (moeflow/kernels/grouped_gemm.py:15-80, moeflow/experts.py:10-17, moeflow/kernels/expert_prepare.py:10-38).
#include <cuda.h>

#include <cstring>

#include "common.cuh"
#include "moeflow_b200.h"
#include "work_iter.cuh"

namespace mf {

constexpr int kBlockM = 128;          // weight rows per block (UMMA M)
constexpr int kTileBytesA = 128 * 128;  // 128 rows x 128 bytes
constexpr int kThreads = 256;
constexpr int kThreadsWithReturn = 384;  // + 4 return warps (fused owner reduce + return push)
// Epilogue warp groups.  Tiles of 256 token columns fill all 512 tensor-memory columns with one accumulator stage
// (two accumulators of 256 columns), so their epilogue is not hidden behind the next unit's main loop: two groups of
// four warps then take half of the token columns each.  The variant with return warps keeps one group.
template <int N_MAX, bool kReturn>
constexpr int kEpiGroups = (N_MAX >= 256 && !kReturn) ? 2 : 1;
constexpr int kRetDepth = 4;            // queued unit descriptors per quarter
constexpr int kGatherThreads = 64;
constexpr int kMaxAccStages = 2;
constexpr int kOutStageBytes = 1024;   // 16 token columns x 32 weight rows of 16-bit outputs, per epilogue warp
constexpr int kMaxDevices = 64;        // devices one process may drive (per-device launch configuration)

template <bool kGateUp, int N_MAX>
struct GemmCfg {
  static constexpr int kATiles = kGateUp ? 2 : 1;
  static constexpr int kStageA = kATiles * kTileBytesA;
  static constexpr int kStageB = N_MAX * 128;
  static constexpr int kStageBytes = kStageA + kStageB;
  // As many stages as fit in 216 KB of the 227 KB a CTA may use (2 KB more go to alignment slack and
  // barriers): the bytes in flight per SM, not the tensor pipe, bound these weight-streaming kernels.
  static constexpr int kStages = (216 * 1024) / kStageBytes > 10 ? 10 : (216 * 1024) / kStageBytes;
  static constexpr int kAccCols = kATiles * N_MAX;
  // Two accumulator stages (the epilogue of unit i overlaps the main loop of unit i + 1) wherever the 512
  // tensor-memory columns allow it; the gate/up GEMM with 256-row token tiles needs all 512 for one stage.
  static constexpr int kAccStages = 2 * kAccCols <= 512 ? 2 : 1;
  static constexpr int kTmemCols = kAccStages * kAccCols;  // power of two for N_MAX in {32, 64, 128, 256}
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 1024 /*barriers, return queue*/ +
                                    (N_MAX >= 256 ? 8 : 4) * kOutStageBytes /*one transposing store buffer per epilogue warp*/;
};

struct PipeState {
  int stage = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void advance(int n_stages) {
    if (++stage == n_stages) {
      stage = 0;
      phase ^= 1u;
    }
  }
};

// Fused owner reduce + return push, called by one epilogue warp after it has written the final y values
// of `n_rows` entries (first entry `row_start`) for its 32 columns `col0 .. col0+31` of block `mb`.
// For every entry the warp counts one arrival on (received row, block, quarter); the arrival that
// completes a row's hit count sums that row's slots in slot order (fp32, +0.0 start), rounds once to
// bf16 and stores the 32 values into the source rank's combine buffer.  Completed quarters are counted
// on `ret_done`; the warp that brings it to valid_rows * m_blocks * 4 publishes the return flags.
// Returns the number of (row, block, quarter) reductions this call completed; the caller adds them up and
// reports them once with return_finish (one system-scope fence per warp, not per unit).
__device__ __forceinline__ int return_rows(const mf_gemm_args& a, int n_rows, int row_start, int mb, int wq, int lane) {
  const __nv_bfloat16* y = static_cast<const __nv_bfloat16*>(a.out);
  const long long col0 = (long long)mb * kBlockM + wq * 32;  // this quarter's 32 columns (64 bytes, 64-byte aligned)
  int completed = 0;
  for (int n0 = 0; n0 < n_rows; n0 += 32) {
    // One lane per entry: count the arrival; the lane whose arrival completes the row does the whole row
    // (all its slots, 32 columns) by itself, so the rows of a unit are reduced in parallel, not in turn.
    const int n = n0 + lane;
    int r = -1;
    bool last = false;
    if (n < n_rows) {
      r = a.entry_row[row_start + n];
      int* cnt = a.row_cnt + ((long long)r * a.m_blocks + mb) * 4 + wq;
      const int old = atomicAdd(cnt, 1);
      last = (old + 1 == a.row_hits[r]);
      if (last) *cnt = 0;  // self-cleaning: nobody else touches this counter again in this forward
    }
    const unsigned todo = __ballot_sync(0xffffffffu, last);
    if (todo == 0u) continue;
    __threadfence();  // the other slots' y values (written by other CTAs) are visible now
    if (last) {
      float acc[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = 0.f;
      for (int k = 0; k < a.ret_K; ++k) {
        const int p = a.inv[(long long)r * a.ret_K + k];
        if (p < 0) continue;
        const uint4* src = reinterpret_cast<const uint4*>(y + (long long)p * a.out_pitch + col0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 v = __ldcg(src + q);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            acc[q * 8 + 2 * i] += f.x;
            acc[q * 8 + 2 * i + 1] += f.y;
          }
        }
      }
      const int src_rank = r / a.ret_C, t = r - src_rank * a.ret_C;
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.ret_peer[src_rank]) +
                                            ((long long)a.ret_rank * a.ret_C + t) * a.out_pitch + col0);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(acc[q * 8 + 2 * i], acc[q * 8 + 2 * i + 1]);
        dst[q] = o;
      }
    }
    completed += __popc(todo);
  }
  return completed;
}

// Report `completed` reductions of this warp; the warp that brings the layer's counter to
// valid_rows * m_blocks * 4 publishes the return flags to every source rank.
__device__ __forceinline__ void return_finish(const mf_gemm_args& a, int completed, int lane) {
  if (completed == 0) return;
  __threadfence_system();  // the peer stores of all lanes precede the count (and so the flags)
  __syncwarp();
  if (lane == 0) {
    const unsigned total = (unsigned)a.plan[MF_PLAN_VALID_ROWS] * (unsigned)a.m_blocks * 4u;
    const unsigned before = atomicAdd(a.ret_done, (unsigned)completed);
    if (before + (unsigned)completed == total) {
      *a.ret_done = 0u;
      const unsigned pushes = *a.ret_epoch + 1u;  // counting flags: C arrivals per return push
      *a.ret_epoch = pushes;
      publish_flags(a.ret_flag, a.ret_R, a.ret_rank, pushes * (unsigned)a.ret_C);
    }
  }
}

// One output element: bf16 (one rounding of the fp32 value), or fp32 as it is when the caller asked for it
// (router logits from the down-projection kernel).
// Last step of the epilogue for C token columns of one weight row: the activation (gate/up), or the routing
// weight (down), then the stores.  The arithmetic of all C columns comes first and has no branch that depends on
// the column, so that the C dependency chains (exp, reciprocal) overlap: the epilogue warps are alone on their
// scheduler and a column-by-column loop ran at one chain's latency (about 300 cycles per column).
// v: first accumulator (gate, or the only one); w: second accumulator (up; with two_blocks the second weight block).
// With a staging buffer (`stage`, 1 KB of shared memory owned by the calling warp; C == 16; 16-bit outputs, all
// columns stored) the 16 x 32 block is transposed through it, and every lane stores 16 bytes (8 weight rows of one
// token): two store instructions per block instead of sixteen 64-byte ones.
template <bool kTwoAcc, int C>
__device__ __forceinline__ void finish_store(const mf_gemm_args& a, float (&v)[C], float (&w)[C], const float (&sc)[C],
                                             int n0, int n_rows, int row_start, long long out_col, bool col_ok,
                                             uint8_t* stage = nullptr, int lane = 0) {
  if (kTwoAcc && !a.two_blocks) {
    if (a.round_h) {
#pragma unroll
      for (int j = 0; j < C; ++j) {
        v[j] = bf16_round(v[j]);
        w[j] = bf16_round(w[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < C; ++j) v[j] = swiglu_clamped(v[j], w[j], a.limit);
  } else if (a.row_scale) {
#pragma unroll
    for (int j = 0; j < C; ++j) {
      v[j] *= sc[j];
      if (kTwoAcc) w[j] *= sc[j];
    }
  }
  const bool second = kTwoAcc && a.two_blocks;  // the other weight block's outputs, 128 columns further
  if (C == 16 && stage != nullptr && !a.out_fp32 && a.out_cols <= 0 && (a.out_pitch & 7) == 0 &&
      (reinterpret_cast<uintptr_t>(a.out) & 15) == 0) {  // 16-byte stores need rows that start on 16 bytes
    __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(stage);
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(a.out) + (long long)(row_start + n0) * a.out_pitch + (out_col - lane) +
                         (lane & 3) * 8;
    const uint4* src = reinterpret_cast<const uint4*>(stage) + lane;  // token lane / 4 (+ 8), rows 8 (lane & 3) ..
#pragma unroll
    for (int pass = 0; pass < (kTwoAcc ? 2 : 1); ++pass) {
      if (pass == 1 && !second) break;
      __syncwarp();  // the previous block's reads are done
#pragma unroll
      for (int j = 0; j < C; ++j) st[j * 32 + lane] = __float2bfloat16_rn(pass == 0 ? v[j] : w[j]);
      __syncwarp();
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int t = 8 * h + (lane >> 2);
        const uint4 x = src[32 * h];
        if (n0 + t < n_rows)
          *reinterpret_cast<uint4*>(out + (long long)t * a.out_pitch + (pass == 1 ? kBlockM : 0)) = x;
      }
    }
    return;
  }
  const bool all = n0 + C <= n_rows;
  const long long first = (long long)(row_start + n0) * a.out_pitch + out_col;
  if (a.out_fp32) {
    float* p = static_cast<float*>(a.out) + first;
#pragma unroll
    for (int j = 0; j < C; ++j) {
      if (all || n0 + j < n_rows) {
        if (col_ok) p[(long long)j * a.out_pitch] = v[j];
        if (second) p[(long long)j * a.out_pitch + kBlockM] = w[j];
      }
    }
  } else {
    __nv_bfloat16* p = static_cast<__nv_bfloat16*>(a.out) + first;
#pragma unroll
    for (int j = 0; j < C; ++j) {
      if (all || n0 + j < n_rows) {
        if (col_ok) p[(long long)j * a.out_pitch] = __float2bfloat16_rn(v[j]);
        if (second) p[(long long)j * a.out_pitch + kBlockM] = __float2bfloat16_rn(w[j]);
      }
    }
  }
}

template <bool kGateUp, int N_MAX, bool kReturn = false>
__global__ void __launch_bounds__(kReturn ? kThreadsWithReturn : 128 + 128 * kEpiGroups<N_MAX, kReturn>, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_b,
                    const mf_gemm_args a) {
  using Cfg = GemmCfg<kGateUp, N_MAX>;
  constexpr int STAGES = Cfg::kStages;
  constexpr int kGroups = kEpiGroups<N_MAX, kReturn>;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                                 // STAGES x kStageA
  uint8_t* sB = smem + STAGES * Cfg::kStageA;         // STAGES x kStageB
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::kStageBytes);
  uint64_t* full_bar = bars;                          // [STAGES]
  uint64_t* empty_bar = bars + STAGES;                // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;             // [kMaxAccStages]
  uint64_t* acc_empty = acc_full + kMaxAccStages;     // [kMaxAccStages]
  uint64_t* ret_full = acc_empty + kMaxAccStages;        // [4][kRetDepth] epilogue warp -> return warp
  uint64_t* ret_empty = ret_full + 4 * kRetDepth;     // [4][kRetDepth]
  int* ret_desc = reinterpret_cast<int*>(ret_empty + 4 * kRetDepth);  // [4][kRetDepth][4]: n_rows, row_start, mb
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ret_desc + 4 * kRetDepth * 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* out_stage = smem + STAGES * Cfg::kStageBytes + 1024;  // [4 epilogue warps][kOutStageBytes]
  // The fused return path runs on four extra warps (the kernel is then launched with 384 threads).
  constexpr bool with_return = kReturn;  // the down GEMM with four extra warps for the fused return path

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  // Token operand by TMA (contiguous rows) instead of the cp.async gather: warp 2 issues one bulk copy per
  // stage, warp 3 has nothing to do.
  const bool b_tma = a.b_tmap != nullptr;
  // Optional per-CTA time stamps: 0 entry, 1 dependencies met, 2 first weight tile requested, 3 first
  // operand stage complete, 4 first accumulator complete, 5 last epilogue done, 6 exit.
  unsigned long long* trace = a.trace ? a.trace + (size_t)blockIdx.x * 16 : nullptr;
  // Once-only stamps of the epilogue keep their "already written" bit in a per-thread word (reading the trace word
  // back would be a global load per 16-column group).  The two stamps inside the per-K-block loops of the producer
  // and the MMA issuer test the trace word itself instead: with the per-thread word live in those loops the
  // streaming kernels measured 0.7 us slower per unit (15 us per layer at 72 local experts), tracing off.
  uint32_t stamped = 0;
#define MF_STAMP_ONCE(i)                                   \
  do {                                                     \
    if (trace != nullptr && !(stamped & (1u << (i)))) {    \
      stamped |= 1u << (i);                                \
      trace[(i)] = global_timer_ns();                      \
    }                                                      \
  } while (0)
  if (trace && tid == 0) trace[0] = global_timer_ns();

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      // weight TMA expect_tx arrive + (one per gather thread | the token TMA expect_tx arrive)
      mbar_init(&full_bar[s], b_tma ? 2 : 1 + kGatherThreads);
      mbar_init(&empty_bar[s], 1);                  // tcgen05.commit
    }
    for (int s = 0; s < Cfg::kAccStages; ++s) {
      mbar_init(&acc_full[s], 1);   // tcgen05.commit
      mbar_init(&acc_empty[s], 4 * kGroups);  // one per epilogue warp
    }
    for (int s = 0; s < 4 * kRetDepth; ++s) {
      mbar_init(&ret_full[s], 1);
      mbar_init(&ret_empty[s], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_w);
    if (b_tma) tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Everything above overlaps the tail of the previous kernel.  The gate/up GEMM needs the plan
  // of the metadata kernel right away, so it waits first and only then lets the next kernel start:
  // when the down GEMM starts, the plan is therefore complete and it may stream weight tiles while
  // the gate/up GEMM is still finishing; only its token-operand producers wait for the activations.
  if (tid < 8) {
    // While the predecessor runs: touch the pages read right after the wait (see touch() in common.cuh).
    const void* p = tid == 0 ? (const void*)a.plan : tid == 1 ? (const void*)a.tile_e : tid == 2 ? (const void*)a.tile_s
                  : tid == 3 ? (const void*)a.tile_n : tid == 4 ? (const void*)a.b_index : tid == 5 ? (const void*)a.row_scale
                  : tid == 6 ? (const void*)a.counters : (const void*)a.tile_wait;
    touch(p);
  }
  if (kGateUp && !a.two_blocks) {
    grid_dep_wait_cta();
    grid_dep_launch();
  } else {
    grid_dep_launch();
    // token-operand producers (act rows) and epilogue: after the whole gate/up grid, unless the activations
    // are handed over tile by tile (tile_wait), in which case nothing here depends on that grid's completion
    if (warp >= 2 && a.tile_wait == nullptr) {
      if (lane == 0) grid_dep_wait();  // one waiting thread per warp (see grid_dep_wait_cta)
      __syncwarp();
    }
  }

  if (trace && tid == 0) trace[1] = global_timer_ns();
  if (kReturn && blockIdx.x == 0 && tid == 64) {
    // Fused return path with nothing to return: the flags must still be published (thread 64 belongs to
    // the warps that waited for the previous kernel).
    if (a.plan[MF_PLAN_VALID_ROWS] == 0) {
      const unsigned pushes = *a.ret_epoch + 1u;
      *a.ret_epoch = pushes;
      publish_flags(a.ret_flag, a.ret_R, a.ret_rank, pushes * (unsigned)a.ret_C);
    }
  }
  // ---- the plan: tile count and the K cut, checked against what the caller's buffers can hold -----------
  int n_tiles = __ldcg(a.plan + MF_PLAN_N_TILES);
  const int cut = __ldcg(a.plan + a.split_word);  // 0 = stream-K, else the K split
  int slot_cols = __ldcg(a.plan + MF_PLAN_SLOT_COLS);
  if (slot_cols <= 0 || slot_cols > N_MAX) slot_cols = N_MAX;
  const long long slot_floats = (long long)Cfg::kATiles * slot_cols * kBlockM;
  const unsigned long long wait_ns = a.wait_ns;
  WorkIter work;
  work.init(a, N_MAX, n_tiles, cut, blockIdx.x, gridDim.x);
  {
    // A plan that does not fit the buffers it indexes (a tile count or a cut larger than what the caller
    // sized the scratch for) is refused here, on the device, before anything is stored: every thread of
    // every CTA sees the same words and takes the same branch.
    bool bad = n_tiles < 0 || !(cut == 0 || cut == 1 || cut == 2 || cut == 4 || cut == 8) ||
               (cut > 1 && a.k_blocks % cut != 0);
    bad = bad || (a.max_tiles > 0 && n_tiles > a.max_tiles);
    bad = bad || (a.n_counters > 0 && (long long)n_tiles * a.m_blocks * 4 * kGroups > (long long)a.n_counters);
    bad = bad || (a.partial_floats > 0 && work.slots_needed() * slot_floats > a.partial_floats);
    if (bad) {
      if (tid == 0) report_status(a.status, kBadArgument, 6, blockIdx.x, 0);
      n_tiles = 0;
      work.init(a, N_MAX, 0, 1, blockIdx.x, gridDim.x);
    }
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ weight TMA producer
    PipeState st;
    bool ok = true;
    WorkIter it = work;
    Seg sg;
    while (ok && it.next(sg)) {
      const int row0 = sg.e * a.rows_per_expert + sg.mb * (a.two_blocks ? 2 * kBlockM : kBlockM);
      for (int j = 0; j < sg.nkb; ++j) {
        const int kb = sg.kb0 + j;
        ok = mbar_wait_bounded(&empty_bar[st.stage], st.phase ^ 1u, abort_flag, wait_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) report_status(a.status, kGemmEmptyTimeout, 0, blockIdx.x, 0);
          break;
        }
        if (lane == 0) {
          mbar_arrive_expect_tx(&full_bar[st.stage], Cfg::kStageA);
          uint8_t* dst = sA + st.stage * Cfg::kStageA;
          if (trace && trace[2] == 0) trace[2] = global_timer_ns();  // see the note at MF_STAMP_ONCE
          tma_load_2d(dst, &tmap_w, &full_bar[st.stage], kb * 64, row0);
          if (kGateUp) tma_load_2d(dst + kTileBytesA, &tmap_w, &full_bar[st.stage], kb * 64, row0 + a.up_row_offset);
        }
        __syncwarp();
        st.advance(STAGES);
      }
    }
    if (!ok) {
      // Give copies that are still in flight a moment to land before the CTA goes away.
      const unsigned long long t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 100000ull) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer
    PipeState st, acc;
    bool ok = true;
    WorkIter it = work;
    Seg sg;
    while (ok && it.next(sg)) {
      const uint32_t n_tile = (uint32_t)((sg.n_rows + 15) & ~15);
      const uint32_t idesc = umma_idesc(1, 1, kBlockM, n_tile < 16 ? 16 : n_tile);
      ok = mbar_wait_bounded(&acc_empty[acc.stage], acc.phase ^ 1u, abort_flag, wait_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report_status(a.status, kGemmAccTimeout, 1, blockIdx.x, 0);
        break;
      }
      tc_fence_after_sync();
      const uint32_t d0 = tmem_base + acc.stage * Cfg::kAccCols;
      for (int j = 0; j < sg.nkb; ++j) {
        ok = mbar_wait_bounded(&full_bar[st.stage], st.phase, abort_flag, wait_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (trace && lane == 0 && trace[3] == 0) trace[3] = global_timer_ns();
        if (!ok) {
          if (lane == 0) report_status(a.status, kGemmFullTimeout, 1, blockIdx.x, 0);
          break;
        }
        tc_fence_after_sync();
        if (lane == 0) {
          fence_proxy_async_smem();
          const uint32_t a_addr = smem_u32(sA + st.stage * Cfg::kStageA);
          const uint32_t b_addr = smem_u32(sB + st.stage * Cfg::kStageB);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t bdesc = umma_desc_sw128(b_addr + k * 32);
            const uint32_t accum = (j > 0 || k > 0) ? 1u : 0u;
            umma_f16(d0, umma_desc_sw128(a_addr + k * 32), bdesc, idesc, accum);
            if (kGateUp) umma_f16(d0 + N_MAX, umma_desc_sw128(a_addr + kTileBytesA + k * 32), bdesc, idesc, accum);
          }
          umma_commit(&empty_bar[st.stage]);
        }
        __syncwarp();
        st.advance(STAGES);
      }
      if (!ok) break;
      if (lane == 0) umma_commit(&acc_full[acc.stage]);
      __syncwarp();
      acc.advance(Cfg::kAccStages);
    }
  } else if (warp < 4 && b_tma) {
    // ------------------------------------------------------------------ token-operand producer (TMA)
    if (warp == 2) {
      PipeState st;
      bool ok = true;
      WorkIter it = work;
      Seg sg;
      int ready_tile = -1;
      while (ok && it.next(sg)) {
        if (a.tile_wait != nullptr && sg.tt != ready_tile) {
          // the tile's activations are final once every gate/up unit of the tile has reported its four quarters
          bool got = true;
          if (lane == 0) {
            got = wait_count_ge_gpu(a.tile_wait + sg.tt, a.tile_wait_target, wait_ns);
            fence_proxy_async_all();  // the TMA reads below come after the acquire
          }
          ok = __all_sync(0xffffffffu, got);
          if (!ok) {
            if (lane == 0) {
              *abort_flag = 1;
              report_status(a.status, kGemmFullTimeout, 6, blockIdx.x, 0);
            }
            break;
          }
          ready_tile = sg.tt;
        }
        for (int j = 0; j < sg.nkb; ++j) {
          const int kb = sg.kb0 + j;
          ok = mbar_wait_bounded(&empty_bar[st.stage], st.phase ^ 1u, abort_flag, wait_ns);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            if (lane == 0) report_status(a.status, kGemmEmptyTimeout, 2, blockIdx.x, 0);
            break;
          }
          if (lane == 0) {
            // the box is N_MAX rows whatever the tile's row count: rows past the tile (the next expert's
            // entries, or zero fill past the end of the buffer) land in smem rows the MMA does not read
            // or in accumulator columns the epilogue skips
            mbar_arrive_expect_tx(&full_bar[st.stage], Cfg::kStageB);
            tma_load_2d(sB + st.stage * Cfg::kStageB, &tmap_b, &full_bar[st.stage], kb * 64, sg.row_start);
          }
          __syncwarp();
          st.advance(STAGES);
        }
      }
      if (!ok) {
        const unsigned long long t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 100000ull) __nanosleep(1000);
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ token-operand producers (gather)
    const int gt = tid - 64;       // 0..63
    const int r_in = gt >> 3;      // row inside an 8-row group == swizzle phase
    const int chunk = gt & 7;      // 16-byte chunk inside the 128-byte row
    const uint32_t sw_off = (uint32_t)((chunk ^ r_in) << 4);
    PipeState st;
    bool ok = true;
    WorkIter it = work;
    Seg sg;
    int ready_tile = -1;
    while (ok && it.next(sg)) {
      if (a.tile_wait != nullptr && sg.tt != ready_tile) {
        bool got = wait_count_ge_gpu(a.tile_wait + sg.tt, a.tile_wait_target, wait_ns);
        ok = __all_sync(0xffffffffu, got);
        if (!ok) {
          if (lane == 0) {
            *abort_flag = 1;
            report_status(a.status, kGemmFullTimeout, 6, blockIdx.x, 0);
          }
          break;
        }
        ready_tile = sg.tt;
      }
      const int n_rows = sg.n_rows;
      int n_tile = (n_rows + 15) & ~15;
      if (n_tile < 16) n_tile = 16;
      const uint8_t* rp[N_MAX / 8];
#pragma unroll
      for (int i = 0; i < N_MAX / 8; ++i) {
        const int n = r_in + 8 * i;
        rp[i] = nullptr;
        if (n < n_rows) {
          const long long idx = a.b_index ? (long long)a.b_index[sg.row_start + n] : (long long)(sg.row_start + n);
          rp[i] = static_cast<const uint8_t*>(a.b_base) + idx * a.b_pitch + chunk * 16;
        }
      }
      for (int j = 0; j < sg.nkb; ++j) {
        const int kb = sg.kb0 + j;
        ok = mbar_wait_bounded(&empty_bar[st.stage], st.phase ^ 1u, abort_flag, wait_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) report_status(a.status, kGemmEmptyTimeout, 2, blockIdx.x, 0);
          break;
        }
        const uint32_t b_stage = smem_u32(sB + st.stage * Cfg::kStageB);
#pragma unroll
        for (int i = 0; i < N_MAX / 8; ++i) {
          const int n = r_in + 8 * i;
          if (n < n_tile) {
            const bool live = rp[i] != nullptr;
            cp_async_16(b_stage + n * 128 + sw_off, live ? (const void*)(rp[i] + (long long)kb * 128) : a.b_base,
                        live ? 16u : 0u);
          }
        }
        cp_async_mbar_arrive_noinc(&full_bar[st.stage]);
        st.advance(STAGES);
      }
    }
    // Drain this thread's cp.async operations before the CTA may exit.
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (warp < 4 + 4 * kGroups) {
    // ------------------------------------------------------------------ epilogue
    const int wq = warp & 3;                 // TMEM lane quarter this warp may read
    const int grp = (warp - 4) >> 2;         // column group (0 unless kGroups == 2)
    const int row = wq * 32 + lane;          // weight row inside the block
    PipeState acc;
    PipeState rq;                            // position in this quarter's return queue
    bool ok = true;
    // Hand a finished unit (final y values stored) to this quarter's return warp.  n_rows < 0 ends it.
    auto enqueue_return = [&](int n_rows_, int row_start_, int mb_) -> bool {
      __threadfence();  // the y stores of all lanes are visible device-wide before the hand-over
      __syncwarp();
      const int slot = wq * kRetDepth + rq.stage;
      bool k = mbar_wait_bounded(&ret_empty[slot], rq.phase ^ 1u, abort_flag, wait_ns);
      k = __all_sync(0xffffffffu, k);
      if (!k) return false;
      if (lane == 0) {
        int* d = ret_desc + slot * 4;
        d[0] = n_rows_;
        d[1] = row_start_;
        d[2] = mb_;
        mbar_arrive(&ret_full[slot]);
      }
      __syncwarp();
      rq.advance(kRetDepth);
      return true;
    };
    WorkIter it = work;
    Seg sg;
    while (ok && it.next(sg)) {
      const int mb = sg.mb;
      const int n_rows = sg.n_rows;
      const int row_start = sg.row_start;
      int n_tile = (n_rows + 15) & ~15;
      if (n_tile < 16) n_tile = 16;
      ok = mbar_wait_bounded(&acc_full[acc.stage], acc.phase, abort_flag, wait_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (warp == 4 && lane == 0) MF_STAMP_ONCE(4);
      if (!ok) {
        if (lane == 0) report_status(a.status, kGemmAccTimeout, 3, blockIdx.x, 0);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(wq * 32) << 16) + acc.stage * Cfg::kAccCols;
      const long long out_col = (long long)mb * (a.two_blocks ? 2 * kBlockM : kBlockM) + row;
      const bool col_ok = a.out_cols <= 0 || out_col < a.out_cols;  // weight rows padded up to a block are not stored

      const bool scaled = a.row_scale != nullptr && (!kGateUp || a.two_blocks);
      // this warp group's share of the token columns (whole 16-column groups)
      const int c_half = kGroups == 2 ? ((n_tile / 16 + 1) / 2) * 16 : n_tile;
      const int c_begin = grp * c_half;
      const int c_end = (kGroups == 2 && grp == 0) ? c_half : n_tile;
      const int counter_ix = (sg.unit * 4 + wq) * kGroups + grp;
      if (sg.nseg == 1) {
        // A real loop over 16-column groups (one copy of the code: unrolled over the whole tile it no longer fits
        // the instruction cache, and every group is executed once per unit).  Lane l fetches the routing weight of
        // column c0 + (l & 15) one group ahead.
        auto scale_of = [&](int c0) {
          const int n = c0 + (lane & 15);
          return (scaled && n < n_rows) ? __ldcg(a.row_scale + row_start + n) : 1.f;
        };
        float s_next = scale_of(c_begin);
#pragma unroll 1
        for (int c0 = c_begin; c0 < c_end; c0 += 16) {
          uint32_t g[16], up[16];
          tmem_ld_16(taddr + c0, g);
          if (kGateUp) tmem_ld_16(taddr + N_MAX + c0, up);
          const float s_cur = s_next;
          s_next = scale_of(c0 + 16);
          tmem_ld_wait();
          if (warp == 4 && lane == 0) MF_STAMP_ONCE(8);
          float v[16], w[16], sc[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            v[j] = __uint_as_float(g[j]);
            w[j] = kGateUp ? __uint_as_float(up[j]) : 0.f;
            sc[j] = scaled ? __shfl_sync(0xffffffffu, s_cur, j) : 1.f;
          }
          finish_store<kGateUp, 16>(a, v, w, sc, c0, n_rows, row_start, out_col, col_ok, out_stage + (warp - 4) * kOutStageBytes, lane);
          if (warp == 4 && lane == 0) MF_STAMP_ONCE(9);
        }
        if (warp == 4 && lane == 0) MF_STAMP_ONCE(10);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc.stage]);
        if (a.tile_done != nullptr) {
          __threadfence();  // every lane's stores are visible device-wide before the count
          __syncwarp();
          if (lane == 0) atomicAdd(a.tile_done + sg.tt, 1);
        }
        if (with_return) ok = enqueue_return(n_rows, row_start, mb);
      } else {
        // The unit is cut along K: park the fp32 partial sums, then the last quarter-warp to arrive adds
        // the segments in K order.
        float* mine = a.partial + (long long)it.slot_of(sg, sg.seg) * slot_floats;
        for (int c0 = c_begin; c0 < c_end; c0 += 16) {
          uint32_t g[16], up[16];
          tmem_ld_16(taddr + c0, g);
          if (kGateUp) tmem_ld_16(taddr + N_MAX + c0, up);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int n = c0 + j;
            if (n < n_rows) {
              __stcg(&mine[(long long)n * kBlockM + row], __uint_as_float(g[j]));
              if (kGateUp) __stcg(&mine[(long long)(slot_cols + n) * kBlockM + row], __uint_as_float(up[j]));
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc.stage]);
        __threadfence();
        __syncwarp();
        int old = 0;
        if (lane == 0) old = atomicAdd(&a.counters[counter_ix], 1);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old == sg.nseg - 1) {
          __threadfence();
          // Eight token columns at a time: their loads are independent and issued together (a loop that
          // took one column per L2 round trip cost tens of microseconds on 64-column tiles); the sums
          // still run over the segments in K order for every column.
          constexpr int kFix = 8;
          const int n_stop = n_rows < c_end ? n_rows : c_end;  // this group's columns that hold rows
          for (int n0 = c_begin; n0 < n_stop; n0 += kFix) {
            float v[kFix], w[kFix];
#pragma unroll
            for (int j = 0; j < kFix; ++j) v[j] = w[j] = 0.f;
            for (int s = 0; s < sg.nseg; ++s) {
              const float* p = a.partial + (long long)it.slot_of(sg, s) * slot_floats;
              float pv[kFix], pw[kFix];
#pragma unroll
              for (int j = 0; j < kFix; ++j) {
                const int n = n0 + j;
                pv[j] = n < n_rows ? __ldcg(&p[(long long)n * kBlockM + row]) : 0.f;
                pw[j] = (kGateUp && n < n_rows) ? __ldcg(&p[(long long)(slot_cols + n) * kBlockM + row]) : 0.f;
              }
#pragma unroll
              for (int j = 0; j < kFix; ++j) {
                v[j] += pv[j];
                w[j] += pw[j];
              }
            }
            float sc[kFix];
#pragma unroll
            for (int j = 0; j < kFix; ++j) sc[j] = (scaled && n0 + j < n_rows) ? __ldcg(a.row_scale + row_start + n0 + j) : 1.f;
            finish_store<kGateUp, kFix>(a, v, w, sc, n0, n_rows, row_start, out_col, col_ok);
          }
          if (lane == 0) a.counters[counter_ix] = 0;
          if (a.tile_done != nullptr) {
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(a.tile_done + sg.tt, 1);
          }
          if (with_return) ok = enqueue_return(n_rows, row_start, mb);
        }
      }
      acc.advance(Cfg::kAccStages);
      if (trace && warp == 4 && lane == 0) {
        const unsigned long long now = global_timer_ns();
        trace[5] = now;
        if (!(stamped & (1u << 7))) {
          stamped |= 1u << 7;
          trace[7] = now;
        }
      }
    }
    if (it.bad_tile && warp == 4 && lane == 0) report_status(a.status, kBadArgument, 7, blockIdx.x, 0);
    if (with_return) enqueue_return(-1, 0, 0);  // tell the return warp that nothing more will come
  } else {
    // ------------------------------------------------------------------ return warps (fused owner reduce + push)
    const int wq = warp & 3;
    PipeState rq;
    int completed = 0;
    while (true) {
      const int slot = wq * kRetDepth + rq.stage;
      bool k = mbar_wait_bounded(&ret_full[slot], rq.phase, abort_flag, wait_ns);
      k = __all_sync(0xffffffffu, k);
      if (!k) {
        if (lane == 0) report_status(a.status, kGemmAccTimeout, 5, blockIdx.x, 0);
        break;
      }
      const int* d = ret_desc + slot * 4;
      const int n_rows = d[0], row_start = d[1], mb = d[2];
      __syncwarp();
      if (lane == 0) mbar_arrive(&ret_empty[slot]);
      rq.advance(kRetDepth);
      if (n_rows < 0) break;
      completed += return_rows(a, n_rows, row_start, mb, wq, lane);
    }
    return_finish(a, completed, lane);
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (trace && tid == 0) trace[6] = global_timer_ns();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// -------------------------------------------------------------------------------------------------
// host side
// -------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

#undef MF_STAMP_ONCE

template <bool kGateUp, int N_MAX, bool kReturn = false>
static int launch(const void* tmap, const mf_gemm_args* args, int grid, cudaStream_t stream) {
  using Cfg = GemmCfg<kGateUp, N_MAX>;
  // The shared-memory attribute belongs to (function, device): set it once per device this process drives.
  static bool configured[kMaxDevices] = {};
  auto kern = grouped_gemm_kernel<kGateUp, N_MAX, kReturn>;
  int dev = 0;
  cudaError_t de = cudaGetDevice(&dev);
  if (de != cudaSuccess) return (int)de;
  if (dev < 0 || dev >= kMaxDevices || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < kMaxDevices) configured[dev] = true;
  }
  CUtensorMap tm, tb;
  memcpy(&tm, tmap, sizeof(tm));
  memcpy(&tb, args->b_tmap ? args->b_tmap : tmap, sizeof(tb));
  const int threads = kReturn ? kThreadsWithReturn : 128 + 128 * kEpiGroups<N_MAX, kReturn>;
  return (int)launch_kernel(kern, dim3(grid), dim3(threads), Cfg::kSmemBytes, stream, true, tm, tb, *args);
}

static int check_args(const mf_gemm_args* a, int n_max, int grid) {
  if (!a || grid < 1) return -1;
  if (n_max != 32 && n_max != 64 && n_max != 128 && n_max != 256) return -2;
  if (a->m_blocks < 1 || a->k_blocks < 1) return -3;
  if ((a->b_pitch & 15) != 0 || (reinterpret_cast<uintptr_t>(a->b_base) & 15) != 0) return -4;
  if (a->b_tmap != nullptr && a->b_index != nullptr) return -5;  // TMA token tiles need contiguous rows
  if (a->ret_peer != nullptr && (a->out_fp32 || a->out_cols > 0)) return -6;  // the fused return path reads bf16 rows of full width
  return 0;
}

}  // namespace mf

extern "C" {

int mf_make_tile_tmap(void* out_tmap, const void* base, long long rows, long long k_elems, int elem_bytes,
                      int box_rows) {
  auto fn = mf::get_encode_fn();
  if (!fn) return -10;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ((k_elems * elem_bytes) & 15) != 0) return -11;
  if (box_rows < 1 || box_rows > 256 || rows < 1) return -13;
  CUtensorMap tm;
  cuuint64_t dims[2] = {(cuuint64_t)k_elems, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(k_elems * elem_bytes)};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(&tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -12 - (int)r * 100;
  memcpy(out_tmap, &tm, sizeof(tm));
  return 0;
}

int mf_make_weight_tmap(void* out_tmap, const void* w, long long rows, long long k_elems, int elem_bytes) {
  return mf_make_tile_tmap(out_tmap, w, rows, k_elems, elem_bytes, 128);
}

int mf_gemm_smem_bytes(int gate_up, int n_max) {
  if (gate_up) {
    if (n_max == 32) return mf::GemmCfg<true, 32>::kSmemBytes;
    if (n_max == 64) return mf::GemmCfg<true, 64>::kSmemBytes;
    if (n_max == 128) return mf::GemmCfg<true, 128>::kSmemBytes;
    if (n_max == 256) return mf::GemmCfg<true, 256>::kSmemBytes;
  } else {
    if (n_max == 32) return mf::GemmCfg<false, 32>::kSmemBytes;
    if (n_max == 64) return mf::GemmCfg<false, 64>::kSmemBytes;
    if (n_max == 128) return mf::GemmCfg<false, 128>::kSmemBytes;
    if (n_max == 256) return mf::GemmCfg<false, 256>::kSmemBytes;
  }
  return -1;
}

int mf_gemm_gate_up(const void* tmap, const mf_gemm_args* args, int n_max, int grid, mf_stream_t stream) {
  int c = mf::check_args(args, n_max, grid);
  if (c) return c;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n_max == 32) return mf::launch<true, 32>(tmap, args, grid, s);
  if (n_max == 64) return mf::launch<true, 64>(tmap, args, grid, s);
  if (n_max == 128) return mf::launch<true, 128>(tmap, args, grid, s);
  return mf::launch<true, 256>(tmap, args, grid, s);
}

int mf_gemm_down(const void* tmap, const mf_gemm_args* args, int n_max, int grid, mf_stream_t stream) {
  int c = mf::check_args(args, n_max, grid);
  if (c) return c;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (args->two_blocks) {
    // two adjacent weight blocks per unit: the kernel form with two operand tiles and two accumulators
    if (args->ret_peer != nullptr || args->out_cols > 0 || args->up_row_offset != mf::kBlockM) return -7;
    if (n_max == 32) return mf::launch<true, 32>(tmap, args, grid, s);
    if (n_max == 64) return mf::launch<true, 64>(tmap, args, grid, s);
    if (n_max == 128) return mf::launch<true, 128>(tmap, args, grid, s);
    return mf::launch<true, 256>(tmap, args, grid, s);
  }
  if (args->ret_peer != nullptr) {  // owner reduce + return push fused into the epilogue (four extra warps)
    if (n_max == 32) return mf::launch<false, 32, true>(tmap, args, grid, s);
    if (n_max == 64) return mf::launch<false, 64, true>(tmap, args, grid, s);
    if (n_max == 128) return mf::launch<false, 128, true>(tmap, args, grid, s);
    return mf::launch<false, 256, true>(tmap, args, grid, s);
  }
  if (n_max == 32) return mf::launch<false, 32>(tmap, args, grid, s);
  if (n_max == 64) return mf::launch<false, 64>(tmap, args, grid, s);
  if (n_max == 128) return mf::launch<false, 128>(tmap, args, grid, s);
  return mf::launch<false, 256>(tmap, args, grid, s);
}

}  // extern "C"

// -------------------------------------------------------------------------------------------------
// Down projection without any allocation (declared in moeflow_b200.h, MF_STATIC_SCRATCH_* limits).
//
// The split-K scratch (fp32 partial sums, then the arrival counters) lives in the file-scope device
// array below instead of a caller-provided buffer.  Every GPU that loads this library holds the array
// until the process exits.  In host code the array's name is only a stand-in for the symbol; the
// device address comes from cudaGetSymbolAddress, taken once per device with that device current.
// -------------------------------------------------------------------------------------------------
namespace mf {

constexpr int kStaticNMax = 64;                                             // token rows per tile
constexpr size_t kStaticSlotFloats = (size_t)kStaticNMax * kBlockM;         // one accumulator tile
constexpr size_t kStaticPartialBytes = (size_t)MF_STATIC_SCRATCH_MAX_SLOTS * kStaticSlotFloats * sizeof(float);
constexpr size_t kStaticCounterBytes = (size_t)MF_STATIC_SCRATCH_MAX_COUNTERS * sizeof(int);

static __device__ __align__(256) unsigned char g_static_scratch[kStaticPartialBytes + kStaticCounterBytes];

// One host thread at a time per device is assumed for the first call (the table is written without a lock;
// two threads racing here would both store the same address).
static void* g_static_scratch_addr[kMaxDevices] = {nullptr};

}  // namespace mf

extern "C" int mf_gemm_down_static_scratch(const void* tmap, const mf_gemm_args* args, int max_tiles, int split,
                                           int grid, mf_stream_t stream) {
  using namespace mf;
  if (!tmap || !args || grid < 1 || max_tiles < 1) return -1;
  if (split != 1 && split != 2 && split != 4 && split != 8) return -2;
  if (args->m_blocks < 1 || args->k_blocks < 1 || args->k_blocks % split != 0) return -3;
  if ((args->b_pitch & 15) != 0 || (reinterpret_cast<uintptr_t>(args->b_base) & 15) != 0) return -4;
  // Sizes beyond the static array are refused, never truncated.
  const long long slots = (long long)max_tiles * args->m_blocks * split;
  const long long counters = (long long)max_tiles * args->m_blocks * 4;
  if (slots > MF_STATIC_SCRATCH_MAX_SLOTS) return -20;     // too many (tile, block, split) partial tiles
  if (counters > MF_STATIC_SCRATCH_MAX_COUNTERS) return -21;

  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return -22;
  if (g_static_scratch_addr[dev] == nullptr) {
    // First call on this device: resolve the symbol and size the kernel's shared memory.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(grouped_gemm_kernel<false, kStaticNMax>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             GemmCfg<false, kStaticNMax>::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    g_static_scratch_addr[dev] = p;
  }
  unsigned char* base = static_cast<unsigned char*>(g_static_scratch_addr[dev]);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left: the arrival counters must start at zero.
  e = cudaMemsetAsync(base + kStaticPartialBytes, 0, (size_t)counters * sizeof(int), s);
  if (e != cudaSuccess) return (int)e;

  mf_gemm_args a = *args;
  a.partial = reinterpret_cast<float*>(base);
  a.counters = reinterpret_cast<int*>(base + kStaticPartialBytes);
  a.max_split_slots = MF_STATIC_SCRATCH_MAX_SLOTS;
  a.b_tmap = nullptr;  // this entry always gathers the token rows
  // What the kernel may index, for its own check of the plan words (they live in device memory and can
  // disagree with max_tiles / split): the whole partial area, the counters cleared above, the declared tiles.
  a.partial_floats = (long long)(kStaticPartialBytes / sizeof(float));
  a.n_counters = (int)counters;
  a.max_tiles = max_tiles;
  CUtensorMap tm;
  memcpy(&tm, tmap, sizeof(tm));
  grouped_gemm_kernel<false, kStaticNMax>
      <<<grid, kThreads, GemmCfg<false, kStaticNMax>::kSmemBytes, s>>>(tm, tm, a);
  return (int)cudaGetLastError();
}
