// Expert metadata: from the received rows build, on the device and in one launch,
//   * offsets[L+1]: entries of local expert e are [offsets[e], offsets[e+1]) in expert-major order,
//     stable in (row, slot);
//   * entry_row / entry_slot / entry_w for every expert-major position, and the inverse map
//     inv[row*K + slot] = position (or -1 when the slot is empty or the row is not valid);
//   * the token tiles (expert, first entry, entry count <= block_m) the grouped GEMMs iterate over;
//   * the plan words: tile count, K-split factors for both GEMMs, entry count.
// It first waits (bounded) for every source rank's dispatch flag of this forward, so the receive
// buffer is complete when it is read, and clears the split-K arrival counters.
//
// The stable expert-major order is a counting sort: every warp owns a contiguous range of the flat
// (row, slot) index space, counts its keys per expert, a scan over (expert, warp) turns the counts
// into start positions, and a second sweep places the entries.  No atomics, so the layout is the
// same on every run.
//
// Replaces moeflow/kernels/metadata.py:24-137 (single-CTA Triton sort), the torch
// sort/scatter_add/cumsum chain in moeflow/fixed.py:179-186 and build_tile_schedule
// (moeflow/kernels/grouped_gemm.py:83-98).
#include "common.cuh"
#include "moeflow_b200.h"

namespace mf {

constexpr int kMetaThreads = 1024;
constexpr int kMetaWarps = kMetaThreads / 32;
constexpr int kMetaBatch = 8;  // warp-wide steps whose loads are issued together

// Exclusive scan of one int per thread over the whole block; `total` gets the sum.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += o;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = lane < kMetaWarps ? warp_sums[lane] : 0;
    int wi = w;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, wi, off);
      if (lane >= off) wi += o;
    }
    warp_sums[lane] = wi - w;            // exclusive prefix of the warp sums
    if (lane == 31) warp_sums[32] = wi;  // grand total
  }
  __syncthreads();
  const int res = warp_sums[warp] + incl - v;
  total = warp_sums[32];
  __syncthreads();
  return res;
}

// Pick the K split S in {1,2,4,8}.  Cost model in units of one K block of streaming: a unit costs its
// K blocks plus a fixed overhead (pipeline fill, epilogue, and for S > 1 the partial-sum round trip);
// the kernel takes ceil(units * S / SMs) rounds of such units.  Ties go to the smaller S.
__host__ __device__ __forceinline__ int choose_split(int units, int k_blocks, int n_sms, int max_slots,
                                                     int overhead_kb, int cols) {
  if (units <= 0) return 1;
  int best = 1;
  long long best_cost = (long long)((units + n_sms - 1) / n_sms) * (k_blocks + overhead_kb);
  // the partial-sum round trip of a split unit grows with the tile's token columns (measured: splitting
  // 64-column tiles in two cost more than the idle SMs of an uneven last round)
  const int wide = cols > 16 ? (cols - 16) / 8 : 0;
  for (int s = 2; s <= 8; s <<= 1) {
    if (k_blocks % s != 0 || k_blocks / s < 2) break;
    if ((long long)units * s > max_slots) break;
    const long long rounds = ((long long)units * s + n_sms - 1) / n_sms;
    const long long cost = rounds * (k_blocks / s + overhead_kb + 1 + wide);
    if (cost < best_cost) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

// The K cut of one GEMM: stream-K (0) when asked for, the units do not fill many rounds of the persistent CTAs
// (below 8 units per CTA an uneven last round costs more than the partial tiles of the cut units) and the
// scratch holds the two partial tiles a CTA may need; else the K split of choose_split.
__device__ __forceinline__ int choose_cut(const mf_meta_args& a, int units, int k_blocks, int slots, int overhead_kb,
                                          int cols) {
  if (a.stream_k && units > 0 && units < 8 * a.n_sms && units % a.n_sms != 0 && slots >= 2 * a.n_sms) return 0;
  return choose_split(units, k_blocks, a.n_sms, slots, overhead_kb, cols);
}

__global__ void __launch_bounds__(kMetaThreads) expert_meta_kernel(const mf_meta_args a) {
  extern __shared__ int sm[];
  const int L = a.L, K = a.K;
  int* hist = sm;                       // [kMetaWarps][L]
  int* cnt = hist + kMetaWarps * L;     // [L]
  int* offs = cnt + L;                  // [L]
  int* warp_sums = offs + L;            // [33]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned long long* trace = (a.trace != nullptr && tid == 0) ? a.trace : nullptr;
  if (trace) trace[0] = global_timer_ns();
  grid_dep_launch();
  for (int i = tid; i < kMetaWarps * L; i += kMetaThreads) hist[i] = 0;
  grid_dep_wait_cta();  // the dispatch kernel of this forward has completed (epoch, local rows)
  if (trace) trace[1] = global_timer_ns();
  const unsigned epoch = a.epoch ? *a.epoch : 0u;

  // counting flags: every source adds one per token position (rows / R of them) in every forward
  if (a.flags != nullptr && tid < a.R) {
    if (!wait_flag_ge(a.flags + tid, epoch * (unsigned)(a.rows / a.R), a.wait_ns))
      report_status(a.status, kDispatchFlagTimeout, tid, 0, epoch);
  }
  for (int i = tid; i < a.n_counters1; i += kMetaThreads) a.counters1[i] = 0;
  for (int i = tid; i < a.n_counters2; i += kMetaThreads) a.counters2[i] = 0;
  __syncthreads();
  if (trace) trace[2] = global_timer_ns();  // flags seen, counters cleared

  const int N = a.rows * K;
  int per = (N + kMetaWarps - 1) / kMetaWarps;
  per = (per + 31) & ~31;
  const int begin = min(N, warp * per), end = min(N, (warp + 1) * per);
  const uint8_t* recv = static_cast<const uint8_t*>(a.recv);
  const size_t meta_off = (size_t)a.H * 2;
  int* my_hist = hist + warp * L;

  // Keys of a batch of kMetaBatch warp-wide steps are loaded together (independent loads in flight at
  // once) before the dependent match/count steps: the received rows are cold in cache when this kernel
  // starts, and one load latency per step would dominate it.
  auto load_keys = [&](int i0, int (&key)[kMetaBatch], int (&wbits)[kMetaBatch], bool want_w) {
#pragma unroll
    for (int b = 0; b < kMetaBatch; ++b) {
      const int i = i0 + b * 32 + lane;
      key[b] = -1;
      wbits[b] = 0;
      if (i < end) {
        const int row = i / K, slot = i - row * K;
        const int* meta = reinterpret_cast<const int*>(recv + (size_t)row * a.pitch + meta_off);
        const int id = meta[slot];
        const int valid = meta[2 * K];
        const int wb = want_w ? meta[K + slot] : 0;
        if (valid != 0 && id >= 0 && id < L) {
          key[b] = id;
          wbits[b] = wb;
        }
      }
    }
  };

  // sweep 1: per-warp histogram
  for (int i0 = begin; i0 < end; i0 += 32 * kMetaBatch) {
    int key[kMetaBatch], wbits[kMetaBatch];
    load_keys(i0, key, wbits, false);
#pragma unroll
    for (int b = 0; b < kMetaBatch; ++b) {
      const unsigned same = __match_any_sync(0xffffffffu, key[b]);
      if (key[b] >= 0 && lane == __ffs(same) - 1) my_hist[key[b]] += __popc(same);
      __syncwarp();
    }
  }
  __syncthreads();
  if (trace) trace[3] = global_timer_ns();  // histogram sweep done

  // per expert: prefix over warps, total count
  for (int e = tid; e < L; e += kMetaThreads) {
    int run = 0;
    for (int w = 0; w < kMetaWarps; ++w) {
      const int c = hist[w * L + e];
      hist[w * L + e] = run;
      run += c;
    }
    cnt[e] = run;
  }
  __syncthreads();

  // scans over experts (L <= 1024: one expert per thread): entry offsets and tile bases
  const int my_cnt = tid < L ? cnt[tid] : 0;
  int n_entries, n_tiles;
  const int my_off = block_exclusive_scan(my_cnt, warp_sums, n_entries);
  const int my_nt = (my_cnt + a.block_m - 1) / a.block_m;
  const int my_tb = block_exclusive_scan(my_nt, warp_sums, n_tiles);
  if (tid < L) {
    offs[tid] = my_off;
    a.offsets[tid] = my_off;
    for (int j = 0; j < my_nt; ++j) {
      const int idx = my_tb + j;
      if (idx < a.max_tiles) {
        a.tile_e[idx] = tid;
        a.tile_s[idx] = my_off + j * a.block_m;
        a.tile_n[idx] = min(a.block_m, my_cnt - j * a.block_m);
      }
    }
  }
  // per received row: number of slots that live here (the fused return path of the down GEMM needs it),
  // and the number of rows with at least one
  if (tid == 0) warp_sums[35] = 0;
  __syncthreads();
  if (a.row_hits != nullptr) {
    int mine = 0;
    for (int r = tid; r < a.rows; r += kMetaThreads) {
      const int* meta = reinterpret_cast<const int*>(recv + (size_t)r * a.pitch + meta_off);
      int hits = 0;
      if (meta[2 * K] != 0)
        for (int k = 0; k < K; ++k) hits += (meta[k] >= 0 && meta[k] < L) ? 1 : 0;
      a.row_hits[r] = hits;
      mine += hits > 0 ? 1 : 0;
    }
    if (mine) atomicAdd(&warp_sums[35], mine);
  }
  // widest token tile: the split-K partial slots are sized for it, so a decode step (few rows per
  // expert) can afford many more, smaller K splits than the worst case would allow
  if (tid == 0) warp_sums[34] = 0;
  __syncthreads();
  if (tid < L && my_cnt > 0) atomicMax(&warp_sums[34], min(my_cnt, a.block_m));
  __syncthreads();
  if (tid == 0) {
    a.offsets[L] = n_entries;
    const int nt = min(n_tiles, a.max_tiles);
    int cols = (warp_sums[34] + 15) & ~15;
    if (cols < 16) cols = 16;
    const int wide_cols = cols;
    int slots1 = a.max_split_slots, slots2 = a.max_split_slots;
    if (a.partial_floats > 0) {
      slots1 = (int)min((long long)0x7fffffff, a.partial_floats / (2ll * cols * 128));
      slots2 = (int)min((long long)0x7fffffff, a.partial_floats / (1ll * cols * 128));
    } else {
      cols = 0;  // fixed slots of the kernel's n_max columns
    }
    a.plan[MF_PLAN_N_TILES] = nt;
    a.plan[MF_PLAN_SPLIT1] = choose_cut(a, nt * a.m_blocks1, a.k_blocks1, slots1, 4, wide_cols);
    a.plan[MF_PLAN_SPLIT2] = choose_cut(a, nt * a.m_blocks2, a.k_blocks2, slots2, 8, wide_cols);
    a.plan[MF_PLAN_N_ENTRIES] = n_entries;
    a.plan[MF_PLAN_SLOT_COLS] = cols;
    a.plan[MF_PLAN_VALID_ROWS] = warp_sums[35];
  }
  __syncthreads();
  if (trace) trace[4] = global_timer_ns();  // offsets, tiles and plan written

  // sweep 2: place the entries
  for (int i0 = begin; i0 < end; i0 += 32 * kMetaBatch) {
    int key[kMetaBatch], wbits[kMetaBatch];
    load_keys(i0, key, wbits, true);
#pragma unroll
    for (int b = 0; b < kMetaBatch; ++b) {
      const int i = i0 + b * 32 + lane;
      const unsigned same = __match_any_sync(0xffffffffu, key[b]);
      if (key[b] >= 0) {
        // pos < N always holds when the rows did not change between the two sweeps; the guard keeps a
        // racing writer (a peer that runs ahead in a truncated stage-timing run) from causing a stray store.
        const int pos = offs[key[b]] + my_hist[key[b]] + __popc(same & ((1u << lane) - 1u));
        if (pos < N) {
          const int row = i / K;
          a.entry_row[pos] = row;
          a.entry_slot[pos] = i - row * K;
          a.entry_w[pos] = __int_as_float(wbits[b]);
        }
        a.inv[i] = pos < N ? pos : -1;
      } else if (i < end) {
        a.inv[i] = -1;
      }
      __syncwarp();
      if (key[b] >= 0 && lane == __ffs(same) - 1) my_hist[key[b]] += __popc(same);
      __syncwarp();
    }
  }
  if (trace) trace[5] = global_timer_ns();  // entries placed
}


// ---------------------------------------------------------------------------------------------------
// Decode sizes (rows * K <= kMetaThreads * kMetaBatch = 8192 slot words): the same layout in one pass.
// Every thread keeps its (at most kMetaBatch) keys and weight bits in registers: the received rows are
// read once, with all loads of a thread in flight together; the position of an entry inside its warp's
// range is recorded while the warp histogram is built, so that after the scans the placement is pure
// arithmetic and stores (no second sweep over the rows, no second round of matching).  The prefix over
// the warps runs as warp scans (one expert per warp at a time) instead of one thread per expert.
// Identical output to expert_meta_kernel; about a quarter of its latency.
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kMetaThreads) expert_meta_small_kernel(const mf_meta_args a) {
  extern __shared__ int sm[];
  const int L = a.L, K = a.K;
  int* hist = sm;                       // [kMetaWarps][L]
  int* cnt = hist + kMetaWarps * L;     // [L]
  int* offs = cnt + L;                  // [L]
  int* warp_sums = offs + L;            // [40]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned long long* trace = (a.trace != nullptr && tid == 0) ? a.trace : nullptr;
  if (trace) trace[0] = global_timer_ns();
  if (!a.late_launch) grid_dep_launch();
  for (int i = tid; i < kMetaWarps * L; i += kMetaThreads) hist[i] = 0;
  if (tid == 0) warp_sums[34] = warp_sums[35] = 0;
  const int N = a.rows * K;
  int per = (N + kMetaWarps - 1) / kMetaWarps;
  per = (per + 31) & ~31;               // <= 32 * kMetaBatch by the launcher's choice of this kernel
  const int begin = min(N, warp * per), end = min(N, (warp + 1) * per);
  const uint8_t* recv = static_cast<const uint8_t*>(a.recv);
  const size_t meta_off = (size_t)a.H * 2;
  int* my_hist = hist + warp * L;
  {
    // While the dispatch kernel runs: touch every page this kernel reads or writes after the wait.
    if (tid == 0) {
      touch(a.epoch);
      touch(a.flags);
      touch(a.plan);
      touch(a.offsets);
      touch(a.tile_e);
      touch(a.tile_s);
      touch(a.tile_n);
      touch(a.row_hits);
    }
    const int i = begin + lane;
    if (i < end) {
      touch(recv + (size_t)(i / K) * a.pitch + meta_off);
      touch(a.inv + i);
      touch(a.entry_row + i);
      touch(a.entry_slot + i);
      touch(a.entry_w + i);
    }
    if (tid < a.n_counters1) touch(a.counters1 + tid);
    if (tid < a.n_counters2) touch(a.counters2 + tid);
  }
  grid_dep_wait_cta();  // the dispatch kernel of this forward has completed (epoch, local rows)
  if (trace) trace[1] = global_timer_ns();
  const unsigned epoch = a.epoch ? __ldcg(a.epoch) : 0u;
  if (a.flags != nullptr && tid < a.R) {
    if (!wait_flag_ge(a.flags + tid, epoch * (unsigned)(a.rows / a.R), a.wait_ns))
      report_status(a.status, kDispatchFlagTimeout, tid, 0, epoch);
  }
  __syncthreads();
  if (trace) trace[2] = global_timer_ns();  // flags seen

  // the only reads of the received rows: id, valid flag and weight bits of every slot word of this thread
  int key[kMetaBatch], wbits[kMetaBatch], pre[kMetaBatch];
#pragma unroll
  for (int b = 0; b < kMetaBatch; ++b) {
    const int i = begin + b * 32 + lane;
    key[b] = -1;
    wbits[b] = 0;
    if (i < end) {
      const int row = i / K, slot = i - row * K;
      const int* meta = reinterpret_cast<const int*>(recv + (size_t)row * a.pitch + meta_off);
      const int id = __ldcg(meta + slot);
      const int valid = __ldcg(meta + 2 * K);
      const int wb = __ldcg(meta + K + slot);
      if (valid != 0 && id >= 0 && id < L) {
        key[b] = id;
        wbits[b] = wb;
      }
    }
  }
  // the split-K arrival counters are cleared while those loads are in flight
  for (int i = tid; i < a.n_counters1; i += kMetaThreads) a.counters1[i] = 0;
  for (int i = tid; i < a.n_counters2; i += kMetaThreads) a.counters2[i] = 0;
  if (trace) trace[6] = global_timer_ns();  // counter stores issued

  // warp histogram; pre[b] = entries of the same expert earlier in this warp's range
  const unsigned lt_mask = (1u << lane) - 1u;
  int rows_hit = 0;
  const bool k_pow2 = (K & (K - 1)) == 0 && K <= 32;
#pragma unroll
  for (int b = 0; b < kMetaBatch; ++b) {
    if (begin + b * 32 < end) {  // warp-uniform
      const unsigned same = __match_any_sync(0xffffffffu, key[b]);
      int before = 0;
      if (key[b] >= 0) before = my_hist[key[b]];
      pre[b] = before + __popc(same & lt_mask);
      __syncwarp();
      if (key[b] >= 0 && lane == __ffs(same) - 1) my_hist[key[b]] = before + __popc(same);
      __syncwarp();
      if (k_pow2) {
        // a received row is K consecutive slot words of one warp step: its hit count is a ballot away
        const unsigned live = __ballot_sync(0xffffffffu, key[b] >= 0);
        const int g0 = lane & ~(K - 1);
        const unsigned gmask = (K == 32 ? 0xffffffffu : ((1u << K) - 1u)) << g0;
        const int hits = __popc(live & gmask);
        const int i = begin + b * 32 + lane;
        if (lane == g0 && i < end) {
          if (a.row_hits != nullptr) a.row_hits[i / K] = hits;
          rows_hit += hits > 0 ? 1 : 0;
        }
      }
    }
  }
  if (k_pow2) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) rows_hit += __shfl_xor_sync(0xffffffffu, rows_hit, off);
    if (lane == 0 && rows_hit) atomicAdd(&warp_sums[35], rows_hit);
  }
  if (trace) trace[7] = global_timer_ns();  // this warp's histogram done (its loads have landed)
  __syncthreads();
  if (trace) trace[3] = global_timer_ns();  // histogram done

  // per expert: exclusive prefix over the warps (lane = source warp), total count
  for (int e = warp; e < L; e += kMetaWarps) {
    const int c = hist[lane * L + e];
    int incl = c;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += o;
    }
    hist[lane * L + e] = incl - c;
    if (lane == 31) cnt[e] = incl;
  }
  if (!k_pow2) {
    // general K: rows do not line up with warp steps; count their hits from the rows (cache hits by now)
    int mine = 0;
    for (int r = tid; r < a.rows; r += kMetaThreads) {
      const int* meta = reinterpret_cast<const int*>(recv + (size_t)r * a.pitch + meta_off);
      int hits = 0;
      if (__ldcg(meta + 2 * K) != 0)
        for (int k = 0; k < K; ++k) {
          const int id = __ldcg(meta + k);
          hits += (id >= 0 && id < L) ? 1 : 0;
        }
      if (a.row_hits != nullptr) a.row_hits[r] = hits;
      mine += hits > 0 ? 1 : 0;
    }
    if (mine) atomicAdd(&warp_sums[35], mine);
  }
  __syncthreads();

  // scans over experts (L <= 1024: one expert per thread): entry offsets and tile bases
  const int my_cnt = tid < L ? cnt[tid] : 0;
  int n_entries, n_tiles;
  const int my_off = block_exclusive_scan(my_cnt, warp_sums, n_entries);
  const int my_nt = (my_cnt + a.block_m - 1) / a.block_m;
  const int my_tb = block_exclusive_scan(my_nt, warp_sums, n_tiles);
  if (tid < L) {
    offs[tid] = my_off;
    a.offsets[tid] = my_off;
    for (int j = 0; j < my_nt; ++j) {
      const int idx = my_tb + j;
      if (idx < a.max_tiles) {
        a.tile_e[idx] = tid;
        a.tile_s[idx] = my_off + j * a.block_m;
        a.tile_n[idx] = min(a.block_m, my_cnt - j * a.block_m);
      }
    }
    if (my_cnt > 0) atomicMax(&warp_sums[34], min(my_cnt, a.block_m));
  }
  __syncthreads();
  if (tid == kMetaThreads - 1) {
    // the plan words, by a thread of the last warp (its range of slot words is the shortest, often empty)
    a.offsets[L] = n_entries;
    const int nt = min(n_tiles, a.max_tiles);
    int cols = (warp_sums[34] + 15) & ~15;
    if (cols < 16) cols = 16;
    const int wide_cols = cols;
    int slots1 = a.max_split_slots, slots2 = a.max_split_slots;
    if (a.partial_floats > 0) {
      slots1 = (int)min((long long)0x7fffffff, a.partial_floats / (2ll * cols * 128));
      slots2 = (int)min((long long)0x7fffffff, a.partial_floats / (1ll * cols * 128));
    } else {
      cols = 0;
    }
    a.plan[MF_PLAN_N_TILES] = nt;
    a.plan[MF_PLAN_SPLIT1] = choose_cut(a, nt * a.m_blocks1, a.k_blocks1, slots1, 4, wide_cols);
    a.plan[MF_PLAN_SPLIT2] = choose_cut(a, nt * a.m_blocks2, a.k_blocks2, slots2, 8, wide_cols);
    a.plan[MF_PLAN_N_ENTRIES] = n_entries;
    a.plan[MF_PLAN_SLOT_COLS] = cols;
    a.plan[MF_PLAN_VALID_ROWS] = warp_sums[35];
  }
  if (trace) trace[4] = global_timer_ns();  // offsets and tiles written

  // placement: arithmetic and stores only
#pragma unroll
  for (int b = 0; b < kMetaBatch; ++b) {
    const int i = begin + b * 32 + lane;
    if (i < end) {
      int pos = -1;
      if (key[b] >= 0) {
        pos = offs[key[b]] + my_hist[key[b]] + pre[b];
        // pos < N always holds for a consistent buffer; the guard keeps a racing writer (a peer that runs ahead
        // in a truncated stage-timing run) from causing a stray store
        if (pos < N) {
          const int row = i / K;
          a.entry_row[pos] = row;
          a.entry_slot[pos] = i - row * K;
          a.entry_w[pos] = __int_as_float(wbits[b]);
        } else {
          pos = -1;
        }
      }
      a.inv[i] = pos;
    }
  }
  if (trace) trace[5] = global_timer_ns();  // entries placed
}


// ---------------------------------------------------------------------------------------------------
// Multi-CTA variant for prefill sizes: the flat (row, slot) index space is cut into one contiguous
// chunk per CTA (and inside a CTA into one contiguous range per warp, as above).  Launch 1 counts:
// per-CTA expert histograms go to cta_hist.  Launch 2 recomputes its own per-warp histograms, adds the
// counts of the CTAs before it (a plain loop over cta_hist: no atomics, no waiting between CTAs, so the
// layout is again the same on every run and equal to the single-CTA kernel's) and places its entries.
// ---------------------------------------------------------------------------------------------------
struct MetaRange {
  int begin, end;
};
__device__ __forceinline__ MetaRange meta_range(int N, int n_ctas, int cta, int warp) {
  int chunk = (N + n_ctas - 1) / n_ctas;
  chunk = (chunk + 31) & ~31;
  const int cb = min(N, cta * chunk), ce = min(N, (cta + 1) * chunk);
  int per = (ce - cb + kMetaWarps - 1) / kMetaWarps;
  per = (per + 31) & ~31;
  MetaRange r;
  r.begin = min(ce, cb + warp * per);
  r.end = min(ce, cb + (warp + 1) * per);
  return r;
}

// keys (local expert id or -1) and weight bits of kMetaBatch warp-wide steps starting at i0
__device__ __forceinline__ void meta_load_keys(const mf_meta_args& a, int i0, int end, int lane, bool want_w,
                                               int (&key)[kMetaBatch], int (&wbits)[kMetaBatch]) {
  const uint8_t* recv = static_cast<const uint8_t*>(a.recv);
  const size_t meta_off = (size_t)a.H * 2;
#pragma unroll
  for (int b = 0; b < kMetaBatch; ++b) {
    const int i = i0 + b * 32 + lane;
    key[b] = -1;
    wbits[b] = 0;
    if (i < end) {
      const int row = i / a.K, slot = i - row * a.K;
      const int* meta = reinterpret_cast<const int*>(recv + (size_t)row * a.pitch + meta_off);
      const int id = meta[slot];
      const int valid = meta[2 * a.K];
      const int wb = want_w ? meta[a.K + slot] : 0;
      if (valid != 0 && id >= 0 && id < a.L) {
        key[b] = id;
        wbits[b] = wb;
      }
    }
  }
}

__device__ __forceinline__ void meta_histogram(const mf_meta_args& a, MetaRange r, int lane, int* my_hist) {
  for (int i0 = r.begin; i0 < r.end; i0 += 32 * kMetaBatch) {
    int key[kMetaBatch], wbits[kMetaBatch];
    meta_load_keys(a, i0, r.end, lane, false, key, wbits);
#pragma unroll
    for (int b = 0; b < kMetaBatch; ++b) {
      const unsigned same = __match_any_sync(0xffffffffu, key[b]);
      if (key[b] >= 0 && lane == __ffs(same) - 1) my_hist[key[b]] += __popc(same);
      __syncwarp();
    }
  }
}

__global__ void __launch_bounds__(kMetaThreads) expert_meta_count_kernel(const mf_meta_args a) {
  extern __shared__ int sm[];
  const int L = a.L, K = a.K;
  int* hist = sm;                    // [kMetaWarps][L]
  int* warp_sums = hist + kMetaWarps * L;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cta = blockIdx.x, n_ctas = gridDim.x;
  grid_dep_launch();
  for (int i = tid; i < kMetaWarps * L; i += kMetaThreads) hist[i] = 0;
  if (tid == 0) warp_sums[0] = 0;
  grid_dep_wait_cta();  // the dispatch kernel of this forward has completed (epoch, local rows)
  const unsigned epoch = a.epoch ? *a.epoch : 0u;
  if (a.flags != nullptr && tid < a.R) {
    if (!wait_flag_ge(a.flags + tid, epoch * (unsigned)(a.rows / a.R), a.wait_ns))
      report_status(a.status, kDispatchFlagTimeout, tid, cta, epoch);
  }
  for (int i = cta * kMetaThreads + tid; i < a.n_counters1; i += n_ctas * kMetaThreads) a.counters1[i] = 0;
  for (int i = cta * kMetaThreads + tid; i < a.n_counters2; i += n_ctas * kMetaThreads) a.counters2[i] = 0;
  __syncthreads();

  const int N = a.rows * K;
  meta_histogram(a, meta_range(N, n_ctas, cta, warp), lane, hist + warp * L);
  __syncthreads();
  for (int e = tid; e < L; e += kMetaThreads) {
    int total = 0;
    for (int w = 0; w < kMetaWarps; ++w) total += hist[w * L + e];
    a.cta_hist[(size_t)cta * L + e] = total;
  }
  // slots per received row, and the number of rows with at least one
  const uint8_t* recv = static_cast<const uint8_t*>(a.recv);
  const size_t meta_off = (size_t)a.H * 2;
  int mine = 0;
  for (int r = cta * kMetaThreads + tid; r < a.rows; r += n_ctas * kMetaThreads) {
    const int* meta = reinterpret_cast<const int*>(recv + (size_t)r * a.pitch + meta_off);
    int hits = 0;
    if (meta[2 * K] != 0)
      for (int k = 0; k < K; ++k) hits += (meta[k] >= 0 && meta[k] < L) ? 1 : 0;
    if (a.row_hits != nullptr) a.row_hits[r] = hits;
    mine += hits > 0 ? 1 : 0;
  }
  if (mine) atomicAdd(&warp_sums[0], mine);
  __syncthreads();
  if (tid == 0 && warp_sums[0] != 0) atomicAdd(&a.acc[0], warp_sums[0]);  // a count: the order does not matter
}

__global__ void __launch_bounds__(kMetaThreads) expert_meta_place_kernel(const mf_meta_args a) {
  extern __shared__ int sm[];
  const int L = a.L, K = a.K;
  int* hist = sm;                       // [kMetaWarps][L]
  int* cnt = hist + kMetaWarps * L;     // [L] entries of the expert over all CTAs
  int* offs = cnt + L;                  // [L] first position of this CTA's entries of the expert
  int* warp_sums = offs + L;            // [40]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cta = blockIdx.x, n_ctas = gridDim.x;
  grid_dep_launch();
  for (int i = tid; i < kMetaWarps * L; i += kMetaThreads) hist[i] = 0;
  if (tid == 0) warp_sums[34] = 0;
  grid_dep_wait_cta();  // the count launch has completed (and with it the dispatch kernel)
  __syncthreads();

  const int N = a.rows * K;
  const MetaRange range = meta_range(N, n_ctas, cta, warp);
  int* my_hist = hist + warp * L;
  meta_histogram(a, range, lane, my_hist);
  __syncthreads();

  for (int e = tid; e < L; e += kMetaThreads) {
    int run = 0;
    for (int w = 0; w < kMetaWarps; ++w) {
      const int c = hist[w * L + e];
      hist[w * L + e] = run;
      run += c;
    }
    int before = 0, total = 0;
    for (int c = 0; c < n_ctas; ++c) {
      const int v = a.cta_hist[(size_t)c * L + e];
      before += c < cta ? v : 0;
      total += v;
    }
    cnt[e] = total;
    offs[e] = before;
  }
  __syncthreads();

  const int my_cnt = tid < L ? cnt[tid] : 0;
  int n_entries, n_tiles;
  const int my_off = block_exclusive_scan(my_cnt, warp_sums, n_entries);
  const int my_nt = (my_cnt + a.block_m - 1) / a.block_m;
  const int my_tb = block_exclusive_scan(my_nt, warp_sums, n_tiles);
  if (tid < L) {
    offs[tid] += my_off;
    if (cta == 0) {
      a.offsets[tid] = my_off;
      for (int j = 0; j < my_nt; ++j) {
        const int idx = my_tb + j;
        if (idx < a.max_tiles) {
          a.tile_e[idx] = tid;
          a.tile_s[idx] = my_off + j * a.block_m;
          a.tile_n[idx] = min(a.block_m, my_cnt - j * a.block_m);
        }
      }
      if (my_cnt > 0) atomicMax(&warp_sums[34], min(my_cnt, a.block_m));
    }
  }
  __syncthreads();
  if (cta == 0 && tid == 0) {
    a.offsets[L] = n_entries;
    const int nt = min(n_tiles, a.max_tiles);
    int cols = (warp_sums[34] + 15) & ~15;
    if (cols < 16) cols = 16;
    const int wide_cols = cols;
    int slots1 = a.max_split_slots, slots2 = a.max_split_slots;
    if (a.partial_floats > 0) {
      slots1 = (int)min((long long)0x7fffffff, a.partial_floats / (2ll * cols * 128));
      slots2 = (int)min((long long)0x7fffffff, a.partial_floats / (1ll * cols * 128));
    } else {
      cols = 0;
    }
    a.plan[MF_PLAN_N_TILES] = nt;
    a.plan[MF_PLAN_SPLIT1] = choose_cut(a, nt * a.m_blocks1, a.k_blocks1, slots1, 4, wide_cols);
    a.plan[MF_PLAN_SPLIT2] = choose_cut(a, nt * a.m_blocks2, a.k_blocks2, slots2, 8, wide_cols);
    a.plan[MF_PLAN_N_ENTRIES] = n_entries;
    a.plan[MF_PLAN_SLOT_COLS] = cols;
    a.plan[MF_PLAN_VALID_ROWS] = a.acc[0];
    a.acc[0] = 0;  // ready for the next forward (its count launch runs after this one)
  }

  for (int i0 = range.begin; i0 < range.end; i0 += 32 * kMetaBatch) {
    int key[kMetaBatch], wbits[kMetaBatch];
    meta_load_keys(a, i0, range.end, lane, true, key, wbits);
#pragma unroll
    for (int b = 0; b < kMetaBatch; ++b) {
      const int i = i0 + b * 32 + lane;
      const unsigned same = __match_any_sync(0xffffffffu, key[b]);
      if (key[b] >= 0) {
        const int pos = offs[key[b]] + my_hist[key[b]] + __popc(same & ((1u << lane) - 1u));
        if (pos < N) {
          const int row = i / K;
          a.entry_row[pos] = row;
          a.entry_slot[pos] = i - row * K;
          a.entry_w[pos] = __int_as_float(wbits[b]);
        }
        a.inv[i] = pos < N ? pos : -1;
      } else if (i < range.end) {
        a.inv[i] = -1;
      }
      __syncwarp();
      if (key[b] >= 0 && lane == __ffs(same) - 1) my_hist[key[b]] += __popc(same);
      __syncwarp();
    }
  }
}

}  // namespace mf

extern "C" int mf_plan_split(int units, int k_blocks, int n_sms, int max_slots, int overhead_kb, int cols) {
  return mf::choose_split(units, k_blocks, n_sms, max_slots, overhead_kb, cols);
}

extern "C" int mf_expert_meta(const mf_meta_args* a, mf_stream_t stream) {
  if (!a || a->L < 1 || a->L > mf::kMetaThreads || a->R > mf::kMetaThreads || a->block_m < 1) return -1;
  const size_t smem = ((size_t)mf::kMetaWarps * a->L + 2 * (size_t)a->L + 40) * sizeof(int);
  static size_t configured_all[64] = {};  // per device: the attribute belongs to (function, device)
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  size_t& configured = configured_all[dev];
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e =
        cudaFuncSetAttribute(mf::expert_meta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(mf::expert_meta_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(mf::expert_meta_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(mf::expert_meta_place_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a->n_ctas > 1) {
    if (!a->cta_hist || !a->acc || a->n_ctas > 1024) return -2;
    cudaError_t e = mf::launch_kernel(mf::expert_meta_count_kernel, dim3(a->n_ctas), dim3(mf::kMetaThreads), smem, s,
                                      !a->plain_launch, *a);
    if (e != cudaSuccess) return (int)e;
    return (int)mf::launch_kernel(mf::expert_meta_place_kernel, dim3(a->n_ctas), dim3(mf::kMetaThreads), smem, s, true,
                                  *a);
  }
  // one CTA: the register-resident one-pass kernel when every warp's range fits one batch of steps
  const long long n_words = (long long)a->rows * a->K;
  if (n_words <= (long long)mf::kMetaThreads * mf::kMetaBatch)
    return (int)mf::launch_kernel(mf::expert_meta_small_kernel, dim3(1), dim3(mf::kMetaThreads), smem, s, !a->plain_launch, *a);
  return (int)mf::launch_kernel(mf::expert_meta_kernel, dim3(1), dim3(mf::kMetaThreads), smem, s, !a->plain_launch, *a);
}
