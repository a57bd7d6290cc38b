// Block-scaled FP8 (e4m3) grouped expert GEMMs on tcgen05, and the 1x128 activation quantiser.
//
// Checkpoint format: weights are float8_e4m3fn with one fp32 scale per 128x128 block
// (weight_scale_inv); activations are quantised on the fly to e4m3 with one fp32 scale per row and
// 128-wide K group.  These scales are arbitrary fp32 numbers, not the power-of-two per-32 scales the
// hardware block-scaling mode wants, so the kernel accumulates in two levels:
//
//   per 128-wide K block:  tmp[128, n]  = W_q[128 rows, 128 k] . X_q[n, 128 k]^T      (tcgen05 kind::f8f6f4,
//                                                                                     fp32 in tensor memory)
//                          acc[r, n]   += w_scale[block(r), kb] * x_scale[n, kb] * tmp[r, n]     (registers)
//
// The weight block of a unit (128 rows) is exactly one scale-block row, and one K block of 128 bytes is
// one TMA box row and one scale-block column, so a unit needs one weight scale per K block (two for
// gate/up) and one activation scale per token and K block; the epilogue warps preload them into
// shared memory per unit.  Tensor-memory accumulators are double-buffered per K block so that the
// promotion of block kb overlaps the MMAs of block kb+1.
//
// Everything else (swap-AB, persistent CTAs, device-side plan, split-K with ordered fix-up, bounded
// waits, warp roles) is as in grouped_gemm_tc.cu.  Output is bf16: SwiGLU activations for gate/up,
// routing-weighted rows for the down projection.
//
// The reference has no FP8 kernel of its own: it dequantises to bf16 (moeflow/weights.py:23-27) or calls
// the serving engine's fused experts and moe_kernel_quantize_input (moeflow/integrations/vllm_pf.py:97).
#include <cuda.h>
#include <cuda_fp8.h>

#include <cstring>

#include "common.cuh"
#include "moeflow_b200.h"
#include "work_iter.cuh"

namespace mf {

constexpr int kF8BlockM = 128;
constexpr int kF8TileA = 128 * 128;
constexpr int kF8Gather = 64;
constexpr int kF8Tables = 2;  // scale tables: the unit being promoted and the prefetched next one
constexpr int kF8MaxKb = 32;  // K <= 4096 (one unit never spans more K blocks than this)

template <bool kGateUp, int N_MAX>
struct F8Cfg {
  static constexpr int kATiles = kGateUp ? 2 : 1;
  static constexpr int kStageA = kATiles * kF8TileA;
  static constexpr int kStageB = N_MAX * 128;
  static constexpr int kStageBytes = kStageA + kStageB;
  // Promotion warps: one group of four warps (one per tensor-memory lane quarter) takes N_MAX / kGroups token
  // columns: 32 columns per group for tiles of up to 64 rows (a K block's promotion is then one tensor-memory
  // round trip per warp), 64 for 128-row tiles (a thread keeps at most 2 x 64 running sums in registers).
  static constexpr int kGroups = N_MAX > 32 ? 2 : 1;
  static constexpr int kCols = N_MAX / kGroups;
  static constexpr int kThreads = 128 + 128 * kGroups;
  static constexpr int kTableFloats = N_MAX * kF8MaxKb + 2 * kF8MaxKb;  // x scales [kb][n], weight scales [2][kb]
  static constexpr int kTableBytes = kF8Tables * kTableFloats * 4;
  static constexpr int kStages = (222 * 1024 - kTableBytes) / kStageBytes > 8 ? 8 : (222 * 1024 - kTableBytes) / kStageBytes;
  static constexpr int kTmpCols = kATiles * N_MAX;
  // One tensor-memory accumulator per K block in flight: the MMA -> promotion -> MMA round trip is about a
  // microsecond, so two stages cannot keep up with the weight stream; use all 512 columns (at most 8 stages).
  static constexpr int kTmpStages = 512 / kTmpCols > 8 ? 8 : 512 / kTmpCols;
  static constexpr int kTmemCols = kTmpStages * kTmpCols;
  static constexpr int kSmemBytes = kStages * kStageBytes + kTableBytes + 1024 + 512;
};

struct F8Pipe {
  int stage = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void advance(int n) {
    if (++stage == n) {
      stage = 0;
      phase ^= 1u;
    }
  }
};

template <bool kGateUp, int N_MAX>
__global__ void __launch_bounds__(F8Cfg<kGateUp, N_MAX>::kThreads, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_b,
                        const mf_gemm_args a) {
  using Cfg = F8Cfg<kGateUp, N_MAX>;
  constexpr int STAGES = Cfg::kStages;
  constexpr int GROUPS = Cfg::kGroups;
  constexpr int COLS = Cfg::kCols;
  constexpr int PROMO_WARPS = 4 * GROUPS;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * Cfg::kStageA;
  float* sTable = reinterpret_cast<float*>(smem + STAGES * Cfg::kStageBytes);  // [kF8Tables][kTableFloats]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::kStageBytes + Cfg::kTableBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmp_full = bars + 2 * STAGES;
  uint64_t* tmp_empty = tmp_full + Cfg::kTmpStages;
  uint64_t* tbl_bar = tmp_empty + Cfg::kTmpStages;  // [kF8Tables] table filled
  uint64_t* tbl_free = tbl_bar + kF8Tables;         // [kF8Tables] table no longer read
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tbl_free + kF8Tables);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool b_tma = a.b_tmap != nullptr;  // token tiles by TMA (contiguous rows) instead of the 16-byte gather
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], b_tma ? 2 : 1 + kF8Gather);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < Cfg::kTmpStages; ++s) {
      mbar_init(&tmp_full[s], 1);
      mbar_init(&tmp_empty[s], PROMO_WARPS);
    }
    for (int s = 0; s < kF8Tables; ++s) {
      mbar_init(&tbl_bar[s], PROMO_WARPS);
      mbar_init(&tbl_free[s], PROMO_WARPS);
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

  grid_dep_wait_cta();
  grid_dep_launch();

  int n_tiles = a.plan[MF_PLAN_N_TILES];
  const int cut = a.plan[a.split_word];  // 0 = stream-K, else the K split
  int slot_cols = a.plan[MF_PLAN_SLOT_COLS];
  if (slot_cols <= 0 || slot_cols > N_MAX) slot_cols = N_MAX;
  const long long slot_floats = (long long)Cfg::kATiles * slot_cols * kF8BlockM;
  const unsigned long long wait_ns = a.wait_ns;
  WorkIter work;
  work.init(a, N_MAX, n_tiles, cut, blockIdx.x, gridDim.x);
  {
    // the plan is checked against the buffers it indexes before anything is stored (same rule as the bf16 kernel)
    bool bad = n_tiles < 0 || !(cut == 0 || cut == 1 || cut == 2 || cut == 4 || cut == 8) ||
               (cut > 1 && a.k_blocks % cut != 0);
    bad = bad || (a.max_tiles > 0 && n_tiles > a.max_tiles);
    bad = bad || (a.n_counters > 0 && (long long)n_tiles * a.m_blocks * 4 * GROUPS > (long long)a.n_counters);
    bad = bad || (a.partial_floats > 0 && work.slots_needed() * slot_floats > a.partial_floats);
    if (bad) {
      if (tid == 0) report_status(a.status, kBadArgument, 6, blockIdx.x, 0);
      n_tiles = 0;
      work.init(a, N_MAX, 0, 1, blockIdx.x, gridDim.x);
    }
  }

  if (warp == 0) {
    // ---------------------------------------------------------------- weight TMA producer
    F8Pipe st;
    bool ok = true;
    WorkIter it = work;
    Seg sg;
    while (ok && it.next(sg)) {
      const int row0 = sg.e * a.rows_per_expert + sg.mb * kF8BlockM;
      for (int j = 0; j < sg.nkb; ++j) {
        const int kb = sg.kb0 + j;
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&empty_bar[st.stage], st.phase ^ 1u, abort_flag, wait_ns));
        if (!ok) {
          if (lane == 0) report_status(a.status, kGemmEmptyTimeout, 0, blockIdx.x, 0);
          break;
        }
        if (lane == 0) {
          mbar_arrive_expect_tx(&full_bar[st.stage], Cfg::kStageA);
          uint8_t* dst = sA + st.stage * Cfg::kStageA;
          tma_load_2d(dst, &tmap_w, &full_bar[st.stage], kb * 128, row0);
          if (kGateUp) tma_load_2d(dst + kF8TileA, &tmap_w, &full_bar[st.stage], kb * 128, row0 + a.up_row_offset);
        }
        __syncwarp();
        st.advance(STAGES);
      }
    }
    if (!ok) {
      const unsigned long long t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 100000ull) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- UMMA issuer (one K block per tmp stage)
    F8Pipe st, tmp;
    bool ok = true;
    WorkIter it = work;
    Seg sg;
    while (ok && it.next(sg)) {
      uint32_t n_tile = (uint32_t)((sg.n_rows + 15) & ~15);
      if (n_tile < 16) n_tile = 16;
      const uint32_t idesc = umma_idesc(0, 0, kF8BlockM, n_tile);  // e4m3 x e4m3 -> fp32
      for (int j = 0; j < sg.nkb; ++j) {
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&tmp_empty[tmp.stage], tmp.phase ^ 1u, abort_flag, wait_ns));
        if (!ok) {
          if (lane == 0) report_status(a.status, kGemmAccTimeout, 1, blockIdx.x, 0);
          break;
        }
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&full_bar[st.stage], st.phase, abort_flag, wait_ns));
        if (!ok) {
          if (lane == 0) report_status(a.status, kGemmFullTimeout, 1, blockIdx.x, 0);
          break;
        }
        tc_fence_after_sync();
        if (lane == 0) {
          fence_proxy_async_smem();
          const uint32_t d0 = tmem_base + tmp.stage * Cfg::kTmpCols;
          const uint32_t a_addr = smem_u32(sA + st.stage * Cfg::kStageA);
          const uint32_t b_addr = smem_u32(sB + st.stage * Cfg::kStageB);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t bdesc = umma_desc_sw128(b_addr + k * 32);
            umma_f8(d0, umma_desc_sw128(a_addr + k * 32), bdesc, idesc, k > 0 ? 1u : 0u);
            if (kGateUp) umma_f8(d0 + N_MAX, umma_desc_sw128(a_addr + kF8TileA + k * 32), bdesc, idesc, k > 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[st.stage]);
          umma_commit(&tmp_full[tmp.stage]);
        }
        __syncwarp();
        st.advance(STAGES);
        tmp.advance(Cfg::kTmpStages);
      }
    }
  } else if (warp < 4 && b_tma) {
    // ---------------------------------------------------------------- token-operand producer (TMA)
    if (warp == 2) {
      F8Pipe st;
      bool ok = true;
      WorkIter it = work;
      Seg sg;
      while (ok && it.next(sg)) {
        for (int j = 0; j < sg.nkb; ++j) {
          const int kb = sg.kb0 + j;
          ok = __all_sync(0xffffffffu, mbar_wait_bounded(&empty_bar[st.stage], st.phase ^ 1u, abort_flag, wait_ns));
          if (!ok) {
            if (lane == 0) report_status(a.status, kGemmEmptyTimeout, 2, blockIdx.x, 0);
            break;
          }
          if (lane == 0) {
            mbar_arrive_expect_tx(&full_bar[st.stage], Cfg::kStageB);
            tma_load_2d(sB + st.stage * Cfg::kStageB, &tmap_b, &full_bar[st.stage], kb * 128, sg.row_start);
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
    // ---------------------------------------------------------------- token-operand producers (e4m3 rows)
    const int gt = tid - 64, r_in = gt >> 3, chunk = gt & 7;
    const uint32_t sw_off = (uint32_t)((chunk ^ r_in) << 4);
    F8Pipe st;
    bool ok = true;
    WorkIter it = work;
    Seg sg;
    while (ok && it.next(sg)) {
      const int n_rows = sg.n_rows, row_start = sg.row_start;
      int n_tile = (n_rows + 15) & ~15;
      if (n_tile < 16) n_tile = 16;
      const uint8_t* rp[N_MAX / 8];
#pragma unroll
      for (int i = 0; i < N_MAX / 8; ++i) {
        const int n = r_in + 8 * i;
        rp[i] = nullptr;
        if (n < n_rows) {
          const long long idx = a.b_index ? (long long)a.b_index[row_start + n] : (long long)(row_start + n);
          rp[i] = static_cast<const uint8_t*>(a.b_base) + idx * a.b_pitch + chunk * 16;
        }
      }
      for (int j = 0; j < sg.nkb; ++j) {
        const int kb = sg.kb0 + j;
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&empty_bar[st.stage], st.phase ^ 1u, abort_flag, wait_ns));
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
            cp_async_16(b_stage + n * 128 + sw_off, live ? (const void*)(rp[i] + (long long)kb * 128) : a.b_base, live ? 16u : 0u);
          }
        }
        cp_async_mbar_arrive_noinc(&full_bar[st.stage]);
        st.advance(STAGES);
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else {
    // ---------------------------------------------------------------- promotion + epilogue
    const int pw = warp - 4;                 // 0 .. PROMO_WARPS-1
    const int wq = pw & 3;                   // tensor-memory lane quarter
    const int grp = pw >> 2;                 // column group
    const int col0 = grp * COLS;
    const int row = wq * 32 + lane;
    F8Pipe tmp;
    bool ok = true;
    const int row_blocks = a.rows_per_expert / kF8BlockM;
    // Scale table of one segment into buffer `buf`: x scales [j][n] and weight scales [t][j], j = kb - kb0.
    // Every promotion warp fills its share (token columns n = pw, pw + PROMO_WARPS, ... in blocks of 32 lanes)
    // and arrives once on the buffer's barrier.
    auto load_table = [&](const Seg& s_, int buf) {
      int n_tile_ = (s_.n_rows + 15) & ~15;
      if (n_tile_ < 16) n_tile_ = 16;
      float* t = sTable + buf * Cfg::kTableFloats;
      for (int n0 = pw * 32; n0 < n_tile_; n0 += PROMO_WARPS * 32) {
        const int n = n0 + lane;
        if (n < n_tile_) {
          const bool live = n < s_.n_rows;
          long long idx = 0;
          if (live) idx = a.b_index ? (long long)a.b_index[s_.row_start + n] : (long long)(s_.row_start + n);
          // all of the row's scales are requested before the first one is stored: one memory round trip per
          // token instead of one per K block (a dependent load-store loop here cost as much as the unit's
          // whole weight stream)
          const float* src = a.b_scale + idx * a.b_scale_pitch + s_.kb0;
          float v[kF8MaxKb];
#pragma unroll
          for (int j = 0; j < kF8MaxKb; ++j) v[j] = (live && j < s_.nkb) ? __ldcg(src + j) : 0.f;
#pragma unroll
          for (int j = 0; j < kF8MaxKb; ++j)
            if (j < s_.nkb) t[j * N_MAX + n] = v[j];
        }
      }
      if (pw < (kGateUp ? 2 : 1)) {
        const int rb = (pw == 0 ? 0 : a.up_row_offset / kF8BlockM) + s_.mb;
        const float* ws = a.w_scale + ((long long)s_.e * row_blocks + rb) * a.k_blocks + s_.kb0;
        for (int j = lane; j < s_.nkb; j += 32) t[N_MAX * kF8MaxKb + pw * kF8MaxKb + j] = ws[j];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&tbl_bar[buf]);
    };
    WorkIter it = work;    // the segment being promoted
    WorkIter ahead = work; // one segment ahead, for the table prefetch
    Seg sg, nx;
    bool have_next = ahead.next(nx);
    if (have_next) load_table(nx, 0);
    int n_it = 0;  // index of this CTA's segment
    while (ok && it.next(sg)) {
      const int mb = sg.mb, n_rows = sg.n_rows, row_start = sg.row_start;
      int n_tile = (n_rows + 15) & ~15;
      if (n_tile < 16) n_tile = 16;
      const int buf = n_it % kF8Tables;
      const float* tbl = sTable + buf * Cfg::kTableFloats;
      const float* tblW = tbl + N_MAX * kF8MaxKb;
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(&tbl_bar[buf], (uint32_t)(n_it / kF8Tables) & 1u, abort_flag, wait_ns));
      if (!ok) {
        if (lane == 0) report_status(a.status, kGemmAccTimeout, 4, blockIdx.x, 0);
        break;
      }
      // Prefetch the next segment's table into the other buffer, once every warp has stopped reading what
      // that buffer held (the table of the previous segment).
      have_next = ahead.next(nx);
      if (have_next) {
        const int nb = (n_it + 1) % kF8Tables;
        if (n_it >= 1) {
          ok = __all_sync(0xffffffffu, mbar_wait_bounded(&tbl_free[nb], (uint32_t)((n_it - 1) / kF8Tables) & 1u, abort_flag, wait_ns));
          if (!ok) {
            if (lane == 0) report_status(a.status, kGemmAccTimeout, 6, blockIdx.x, 0);
            break;
          }
        }
        load_table(nx, nb);
      }

      float acc_g[COLS], acc_u[kGateUp ? COLS : 1];
#pragma unroll
      for (int i = 0; i < COLS; ++i) acc_g[i] = 0.f;
      if (kGateUp) {
#pragma unroll
        for (int i = 0; i < COLS; ++i) acc_u[i] = 0.f;
      }

      for (int j = 0; j < sg.nkb; ++j) {
        if (!kGateUp && COLS == 32 && Cfg::kTmpStages >= 2 && j + 1 < sg.nkb) {
          // Down projection, 32-column groups: two K blocks per round trip.  A K block is only 16 KB of weights
          // here, so the fixed cost of a promotion step (barrier, tensor-memory load, fence, arrival) has to be
          // shared between two of them to keep up with the weight stream.
          F8Pipe nxt = tmp;
          nxt.advance(Cfg::kTmpStages);
          ok = __all_sync(0xffffffffu, mbar_wait_bounded(&tmp_full[tmp.stage], tmp.phase, abort_flag, wait_ns));
          if (ok) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&tmp_full[nxt.stage], nxt.phase, abort_flag, wait_ns));
          if (!ok) {
            if (lane == 0) report_status(a.status, kGemmAccTimeout, 3, blockIdx.x, 0);
            break;
          }
          tc_fence_after_sync();
          if (col0 < n_tile) {
            const uint32_t lane_base = tmem_base + ((uint32_t)(wq * 32) << 16) + col0;
            uint32_t r0[32], r1[32];
            tmem_ld_32(lane_base + tmp.stage * Cfg::kTmpCols, r0);
            tmem_ld_32(lane_base + nxt.stage * Cfg::kTmpCols, r1);
            tmem_ld_wait();
            const float w0 = tblW[j], w1 = tblW[j + 1];
            const float4* x0 = reinterpret_cast<const float4*>(tbl + j * N_MAX + col0);
            const float4* x1 = reinterpret_cast<const float4*>(tbl + (j + 1) * N_MAX + col0);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 a0 = x0[q], a1 = x1[q];
              acc_g[4 * q] = fmaf(__uint_as_float(r0[4 * q]), w0 * a0.x, acc_g[4 * q]);
              acc_g[4 * q + 1] = fmaf(__uint_as_float(r0[4 * q + 1]), w0 * a0.y, acc_g[4 * q + 1]);
              acc_g[4 * q + 2] = fmaf(__uint_as_float(r0[4 * q + 2]), w0 * a0.z, acc_g[4 * q + 2]);
              acc_g[4 * q + 3] = fmaf(__uint_as_float(r0[4 * q + 3]), w0 * a0.w, acc_g[4 * q + 3]);
              acc_g[4 * q] = fmaf(__uint_as_float(r1[4 * q]), w1 * a1.x, acc_g[4 * q]);
              acc_g[4 * q + 1] = fmaf(__uint_as_float(r1[4 * q + 1]), w1 * a1.y, acc_g[4 * q + 1]);
              acc_g[4 * q + 2] = fmaf(__uint_as_float(r1[4 * q + 2]), w1 * a1.z, acc_g[4 * q + 2]);
              acc_g[4 * q + 3] = fmaf(__uint_as_float(r1[4 * q + 3]), w1 * a1.w, acc_g[4 * q + 3]);
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(&tmp_empty[tmp.stage]);
            mbar_arrive(&tmp_empty[nxt.stage]);
          }
          tmp.advance(Cfg::kTmpStages);
          tmp.advance(Cfg::kTmpStages);
          ++j;
          continue;
        }
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&tmp_full[tmp.stage], tmp.phase, abort_flag, wait_ns));
        if (!ok) {
          if (lane == 0) report_status(a.status, kGemmAccTimeout, 3, blockIdx.x, 0);
          break;
        }
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + ((uint32_t)(wq * 32) << 16) + tmp.stage * Cfg::kTmpCols + col0;
        const float wsg = tblW[j];
        const float wsu = kGateUp ? tblW[kF8MaxKb + j] : 0.f;
        const float4* xs4 = reinterpret_cast<const float4*>(tbl + j * N_MAX + col0);
        // Thirty-two token columns per tensor-memory round trip (the load latency, not the arithmetic, bounds a
        // K block's promotion); with 32-column groups the gate and the up values travel together.
        constexpr bool kBoth = kGateUp && COLS == 32;
#pragma unroll
        for (int c0 = 0; c0 < COLS; c0 += 32) {
          if (col0 + c0 < n_tile) {
            uint32_t g[32], u2[kBoth ? 32 : 1];
            tmem_ld_32(taddr + c0, g);
            if (kBoth) tmem_ld_32(taddr + N_MAX + c0, reinterpret_cast<uint32_t(&)[32]>(u2));
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 xs = xs4[c0 / 4 + q];
              acc_g[c0 + 4 * q] = fmaf(__uint_as_float(g[4 * q]), wsg * xs.x, acc_g[c0 + 4 * q]);
              acc_g[c0 + 4 * q + 1] = fmaf(__uint_as_float(g[4 * q + 1]), wsg * xs.y, acc_g[c0 + 4 * q + 1]);
              acc_g[c0 + 4 * q + 2] = fmaf(__uint_as_float(g[4 * q + 2]), wsg * xs.z, acc_g[c0 + 4 * q + 2]);
              acc_g[c0 + 4 * q + 3] = fmaf(__uint_as_float(g[4 * q + 3]), wsg * xs.w, acc_g[c0 + 4 * q + 3]);
            }
            if (kGateUp) {
              if (!kBoth) {
                tmem_ld_32(taddr + N_MAX + c0, g);
                tmem_ld_wait();
              }
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 xs = xs4[c0 / 4 + q];
                const uint32_t* r = kBoth ? u2 : g;
                acc_u[c0 + 4 * q] = fmaf(__uint_as_float(r[4 * q]), wsu * xs.x, acc_u[c0 + 4 * q]);
                acc_u[c0 + 4 * q + 1] = fmaf(__uint_as_float(r[4 * q + 1]), wsu * xs.y, acc_u[c0 + 4 * q + 1]);
                acc_u[c0 + 4 * q + 2] = fmaf(__uint_as_float(r[4 * q + 2]), wsu * xs.z, acc_u[c0 + 4 * q + 2]);
                acc_u[c0 + 4 * q + 3] = fmaf(__uint_as_float(r[4 * q + 3]), wsu * xs.w, acc_u[c0 + 4 * q + 3]);
              }
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmp_empty[tmp.stage]);
        tmp.advance(Cfg::kTmpStages);
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(&tbl_free[buf]);  // this warp is done with the segment's table

      __nv_bfloat16* out = static_cast<__nv_bfloat16*>(a.out);
      const long long out_col = (long long)mb * kF8BlockM + row;
      if (sg.nseg == 1) {
        // 16 columns at a time: their arithmetic first (independent chains overlap), then their stores
        __nv_bfloat16* p = out + (long long)(row_start + col0) * a.out_pitch + out_col;
        const bool all = col0 + COLS <= n_rows;
#pragma unroll
        for (int c0 = 0; c0 < COLS; c0 += 16) {
          if (kGateUp) {
            if (a.round_h) {
#pragma unroll
              for (int c = c0; c < c0 + 16; ++c) {
                acc_g[c] = bf16_round(acc_g[c]);
                acc_u[c] = bf16_round(acc_u[c]);
              }
            }
#pragma unroll
            for (int c = c0; c < c0 + 16; ++c) acc_g[c] = swiglu_clamped(acc_g[c], acc_u[c], a.limit);
          } else if (a.row_scale) {
#pragma unroll
            for (int c = c0; c < c0 + 16; ++c)
              acc_g[c] *= col0 + c < n_rows ? __ldcg(a.row_scale + row_start + col0 + c) : 1.f;
          }
#pragma unroll
          for (int c = c0; c < c0 + 16; ++c)
            if (all || col0 + c < n_rows) p[(long long)c * a.out_pitch] = __float2bfloat16_rn(acc_g[c]);
        }
      } else {
        float* mine = a.partial + (long long)it.slot_of(sg, sg.seg) * slot_floats;
#pragma unroll
        for (int c = 0; c < COLS; ++c) {
          const int n = col0 + c;
          if (n < n_rows) {
            __stcg(&mine[(long long)n * kF8BlockM + row], acc_g[c]);
            if (kGateUp) __stcg(&mine[(long long)(slot_cols + n) * kF8BlockM + row], acc_u[c]);
          }
        }
        __threadfence();
        __syncwarp();
        int* counter = a.counters + ((long long)sg.unit * 4 + wq) * GROUPS + grp;
        int old = 0;
        if (lane == 0) old = atomicAdd(counter, 1);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old == sg.nseg - 1) {
          __threadfence();
          constexpr int kFix = 8;
          const int n_end = n_rows < col0 + COLS ? n_rows : col0 + COLS;
          for (int n0 = col0; n0 < n_end; n0 += kFix) {
            float v[kFix], w[kFix];
#pragma unroll
            for (int jx = 0; jx < kFix; ++jx) v[jx] = w[jx] = 0.f;
            for (int s_ = 0; s_ < sg.nseg; ++s_) {
              const float* p = a.partial + (long long)it.slot_of(sg, s_) * slot_floats;
              float pv[kFix], pw_[kFix];
#pragma unroll
              for (int jx = 0; jx < kFix; ++jx) {
                const int n = n0 + jx;
                pv[jx] = n < n_end ? __ldcg(&p[(long long)n * kF8BlockM + row]) : 0.f;
                pw_[jx] = (kGateUp && n < n_end) ? __ldcg(&p[(long long)(slot_cols + n) * kF8BlockM + row]) : 0.f;
              }
#pragma unroll
              for (int jx = 0; jx < kFix; ++jx) {
                v[jx] += pv[jx];
                w[jx] += pw_[jx];
              }
            }
#pragma unroll
            for (int jx = 0; jx < kFix; ++jx) {
              const int n = n0 + jx;
              if (n < n_end) {
                float r = v[jx];
                if (kGateUp) {
                  float u = w[jx];
                  if (a.round_h) {
                    r = bf16_round(r);
                    u = bf16_round(u);
                  }
                  r = swiglu_clamped(r, u, a.limit);
                } else if (a.row_scale) {
                  r *= a.row_scale[row_start + n];
                }
                out[(long long)(row_start + n) * a.out_pitch + out_col] = __float2bfloat16_rn(r);
              }
            }
          }
          if (lane == 0) *counter = 0;
        }
      }
      ++n_it;
    }
    if (it.bad_tile && pw == 0 && lane == 0) report_status(a.status, kBadArgument, 7, blockIdx.x, 0);
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// -------------------------------------------------------------------------------------------------
// 1x128 activation quantisation: x[row, :] (bf16) -> q[row, :] (e4m3) and scales[row, g] = amax_g / 448.
// One CTA per output row; 16 threads share a 128-wide group.  Rows can be gathered (row_index), skipped
// when an int32 flag inside the source row is zero (valid_off >= 0: the received-row valid flag), and
// bounded by a device-side row count (n_rows_dev, e.g. the plan's entry count).
// -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
quant_rows_kernel(const uint8_t* x, long long x_pitch, const int* row_index, int hidden, uint8_t* q, float* scales,
                  long long valid_off, const int* n_rows_dev) {
  // Inputs are produced by kernels that may still run while this one is resident (programmatic launch), so
  // they are read from L2 (ld.global.cg), never through the non-coherent read-only path.
  grid_dep_launch();
  grid_dep_wait_cta();
  const int r = blockIdx.x;
  if (n_rows_dev != nullptr && r >= __ldcg(n_rows_dev)) return;
  const long long src = row_index ? (long long)__ldcg(row_index + r) : (long long)r;
  const uint8_t* row = x + src * x_pitch;
  if (valid_off >= 0 && __ldcg(reinterpret_cast<const int*>(row + valid_off)) == 0) return;
  const int chunks = hidden / 8;
  const int groups = hidden / 128;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(row) + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    float f[8];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
      amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
    }
    // 16 consecutive threads hold one 128-wide group (chunks is a multiple of 16, so a group is either
    // fully active or fully idle in the last sweep)
    const unsigned active = __activemask();
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(active, amax, off));
    const float scale = fmaxf(amax, 1e-10f) / 448.f;
    const float inv = 1.f / scale;
    uint2 packed;
    uint8_t* pb = reinterpret_cast<uint8_t*>(&packed);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      pb[i] = (uint8_t)__nv_cvt_float_to_fp8(f[i] * inv, __NV_SATFINITE, __NV_E4M3);
    reinterpret_cast<uint2*>(q + (long long)r * hidden)[c] = packed;
    if ((c & 15) == 0) scales[(long long)r * groups + (c >> 4)] = scale;
  }
}

typedef CUresult (*F8EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

template <bool kGateUp, int N_MAX>
static int launch_f8(const void* tmap, const mf_gemm_args* args, int grid, cudaStream_t stream) {
  using Cfg = F8Cfg<kGateUp, N_MAX>;
  static bool configured[64] = {};  // per device: the attribute belongs to (function, device)
  auto kern = grouped_gemm_fp8_kernel<kGateUp, N_MAX>;
  int dev = 0;
  cudaError_t de = cudaGetDevice(&dev);
  if (de != cudaSuccess) return (int)de;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  CUtensorMap tm, tb;
  memcpy(&tm, tmap, sizeof(tm));
  memcpy(&tb, args->b_tmap ? args->b_tmap : tmap, sizeof(tb));
  return (int)launch_kernel(kern, dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, true, tm, tb, *args);
}

static int check_f8(const mf_gemm_args* a, int n_max, int grid) {
  if (!a || grid < 1) return -1;
  if (n_max != 32 && n_max != 64 && n_max != 128) return -2;
  if (a->b_tmap != nullptr && a->b_index != nullptr) return -6;  // TMA token tiles need contiguous rows
  if (a->m_blocks < 1 || a->k_blocks < 1 || a->k_blocks > kF8MaxKb) return -3;
  if ((a->b_pitch & 15) != 0 || (reinterpret_cast<uintptr_t>(a->b_base) & 15) != 0) return -4;
  if (!a->w_scale || !a->b_scale) return -5;
  return 0;
}

}  // namespace mf

extern "C" {

int mf_gemm_gate_up_fp8(const void* tmap, const mf_gemm_args* args, int n_max, int grid, mf_stream_t stream) {
  int c = mf::check_f8(args, n_max, grid);
  if (c) return c;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n_max == 32) return mf::launch_f8<true, 32>(tmap, args, grid, s);
  if (n_max == 64) return mf::launch_f8<true, 64>(tmap, args, grid, s);
  return mf::launch_f8<true, 128>(tmap, args, grid, s);
}

int mf_gemm_down_fp8(const void* tmap, const mf_gemm_args* args, int n_max, int grid, mf_stream_t stream) {
  int c = mf::check_f8(args, n_max, grid);
  if (c) return c;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n_max == 32) return mf::launch_f8<false, 32>(tmap, args, grid, s);
  if (n_max == 64) return mf::launch_f8<false, 64>(tmap, args, grid, s);
  return mf::launch_f8<false, 128>(tmap, args, grid, s);
}

int mf_quant_rows_1x128(const void* x, long long x_pitch, const int* row_index, int rows, int hidden, void* q,
                        float* scales, long long valid_off, const int* n_rows_dev, mf_stream_t stream) {
  if (rows == 0) return 0;
  if (hidden % 128 != 0 || (x_pitch & 15) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) return -1;
  return (int)mf::launch_kernel(mf::quant_rows_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), true,
                                static_cast<const uint8_t*>(x), x_pitch, row_index, hidden, static_cast<uint8_t*>(q),
                                scales, valid_off, n_rows_dev);
}

}  // extern "C"
