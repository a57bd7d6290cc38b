// C ABI of libmoeflow_b200: every kernel launcher and runtime call the Python layer uses.
// All launchers are asynchronous on the given stream, allocate nothing, and return a cudaError_t
// value (0 = success) or a negative library error for bad arguments.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* mf_stream_t;

// ---- plan words written by mf_expert_meta and read by the grouped GEMMs -------------------------
enum {
  MF_PLAN_N_TILES = 0,    // number of (expert, row range) token tiles
  MF_PLAN_SPLIT1 = 1,     // K cut of the gate/up GEMM: 1, 2, 4 or 8 equal segments per unit, or 0 = stream-K
  MF_PLAN_SPLIT2 = 2,     // K cut of the down GEMM
  MF_PLAN_N_ENTRIES = 3,  // valid (row, slot) entries = offsets[L]
  MF_PLAN_SLOT_COLS = 4,  // token columns per split-K partial slot (multiple of 16; 0 = the kernel's n_max)
  MF_PLAN_VALID_ROWS = 5, // received rows with at least one hit on this rank
  MF_PLAN_WORDS = 8
};

// ---- grouped GEMM -------------------------------------------------------------------------------
typedef struct {
  const void* b_base;        // token-side operand, rows of K elements (bf16) or K bytes (e4m3)
  long long b_pitch;         // bytes between rows of b_base
  const int* b_index;        // optional: entry -> row of b_base (gather); NULL = identity
  const int* tile_e;         // per tile: local expert
  const int* tile_s;         // per tile: first entry
  const int* tile_n;         // per tile: number of entries (<= n_max)
  const int* plan;           // MF_PLAN_* words
  int split_word;            // MF_PLAN_SPLIT1 or MF_PLAN_SPLIT2
  int m_blocks;              // 128-row weight blocks per expert
  int k_blocks;              // K / 64 (bf16) or K / 128 (e4m3)
  int rows_per_expert;       // weight rows per expert in the tensor map
  int up_row_offset;         // gate/up only: row distance from a gate row to its up row
  void* out;                 // bf16 [entries, out_pitch]
  long long out_pitch;       // elements
  const float* row_scale;    // down only, optional: per-entry multiplier applied to the fp32 sum
  float* partial;            // split-K scratch, fp32
  int* counters;             // split-K arrival counters (zero between launches)
  int max_split_slots;       // capacity of `partial` in (tile, m-block, split) slots
  float limit;               // SwiGLU clamp (<= 0: none)
  int round_h;               // gate/up only: round gate and up to bf16 before the activation
  unsigned long long* status;
  unsigned long long wait_ns;
  // block-scaled e4m3 only
  const float* w_scale;      // [experts, rows_per_expert/128, K/128] fp32 (weight_scale_inv)
  const float* b_scale;      // [b rows, K/128] fp32 activation scales (1x128 groups)
  long long b_scale_pitch;   // floats between rows of b_scale
  float* out_scale;          // reserved
  unsigned long long* trace; // optional [grid, 16] globaltimer stamps per CTA (profiling aid), or NULL
  // Down GEMM only, optional (ret_peer != NULL): owner reduce + return all-to-all fused into the epilogue.
  // When the last of a received row's slots has been written for a 32-column quarter of a block, that
  // warp sums the row's slots in slot order (fp32, from +0.0) and stores the bf16 partial straight into
  // the source rank's ret_recv[this rank, t]; the warp that completes the last quarter publishes the
  // return flags.  Needs the plan word MF_PLAN_VALID_ROWS and row_hits from mf_expert_meta.
  const unsigned long long* ret_peer;   // [R] base addresses of every rank's ret_recv [R, C, H]
  const unsigned long long* ret_flag;   // [R] base addresses of every rank's return flags [R]
  unsigned* ret_epoch;       // this rank's count of return pushes (incremented by the warp that publishes)
  unsigned* ret_done;        // completion counter, zero between launches
  int* row_cnt;              // [rows * m_blocks * 4] arrival counters, zero between launches (self-cleaning)
  const int* row_hits;       // [rows] valid slots of each received row on this rank
  const int* entry_row;      // [entries] received row of every expert-major entry
  const int* inv;            // [rows * top_k] (row, slot) -> entry, -1 = none
  int ret_rank, ret_R, ret_C, ret_K;
  // Optional: host pointer to a 128-byte tensor map over the token operand viewed as [rows, K] with a box of
  // n_max rows x 128 bytes (mf_make_tile_tmap).  When set, b_index must be NULL (entry n reads row
  // b_base + n * b_pitch): token tiles are then fetched by TMA, one bulk copy per pipeline stage, instead of
  // being gathered 16 bytes at a time.  Rows past a tile's end are fetched too and ignored.
  const void* b_tmap;
  // Capacities the kernel checks the plan against before it stores anything (0 = not checked).  A plan whose
  // tile count or K cut needs more than this is refused on the device: status word kBadArgument, no store.
  long long partial_floats;  // floats in `partial`
  int n_counters;            // ints in `counters`
  int max_tiles;             // entries in tile_e / tile_s / tile_n
  int out_fp32;              // bf16 kernels: 1 = `out` is fp32 [entries, out_pitch] (no rounding); not with ret_peer
  int out_cols;              // bf16 kernels: > 0 = only output columns below this are stored (weight rows padded to 128)
  // Tile-level hand-over from the gate/up GEMM to the down GEMM (bf16 kernels, both optional).  The gate/up
  // kernel adds one to tile_done[tile] whenever a 32-row quarter of one of the tile's units has its final
  // activations stored; the down kernel, given the same array as tile_wait, fetches a tile's activations as
  // soon as the count reaches tile_wait_target (= 4 * the gate/up GEMM's m_blocks) instead of waiting for the
  // whole gate/up grid, so SMs that the gate/up GEMM has left go straight on with down-projection units.
  // The array must be zero before the gate/up kernel starts (mf_expert_meta clears it with the counters).
  int* tile_done;
  const int* tile_wait;
  int tile_wait_target;
  // mf_gemm_down only: 1 = a unit is two adjacent 128-row weight blocks (m_blocks counts pairs, up_row_offset
  // must be 128): the token tile is shared by both, which halves its L2 traffic per output column.
  int two_blocks;
} mf_gemm_args;

// Encode a 2-D tiled tensor map (K innermost) for a weight matrix [rows, k_elems]; box = 128 bytes x
// 128 rows with the 128-byte swizzle.  `out_tmap` receives 128 bytes.
// General form of mf_make_weight_tmap: boxes of box_rows rows x 128 bytes, 128-byte swizzle.
int mf_make_tile_tmap(void* out_tmap, const void* base, long long rows, long long k_elems, int elem_bytes,
                      int box_rows);
int mf_make_weight_tmap(void* out_tmap, const void* w, long long rows, long long k_elems, int elem_bytes);

int mf_gemm_gate_up(const void* tmap, const mf_gemm_args* args, int n_max, int grid, mf_stream_t stream);
int mf_gemm_down(const void* tmap, const mf_gemm_args* args, int n_max, int grid, mf_stream_t stream);
int mf_gemm_smem_bytes(int gate_up, int n_max);


// ---- down projection for callers that cannot allocate -------------------------------------------------
// No counterpart in the reference.
//
// Some callers of this library have no way to get device memory at call time: a C or C++ host that
// does not link a tensor framework, or serving code that runs after the engine has handed every
// free byte of the GPU to its KV-cache pool, where a cudaMalloc can fail or stall the whole device.
// mf_gemm_down needs split-K scratch (fp32 partial tiles and arrival counters) that somebody has to
// own; this variant owns it itself, in a device array that is part of the loaded library.
//
//  * It computes exactly what mf_gemm_down computes with n_max = 64 (token tiles of up to 64 rows):
//    same kernel, same summation order, so the results are identical.  The caller still passes the
//    inputs and outputs in `args` (operand rows, tile arrays, plan words, out, row_scale, status);
//    args->partial, args->counters and args->max_split_slots are ignored.
//  * `max_tiles` is the largest tile count the plan word MF_PLAN_N_TILES may hold and `split` the value
//    of the plan word args->split_word (1, 2, 4 or 8).  The call is refused with a negative code, and
//    nothing is launched, when max_tiles * m_blocks * split exceeds MF_STATIC_SCRATCH_MAX_SLOTS (-20)
//    or max_tiles * m_blocks * 4 exceeds MF_STATIC_SCRATCH_MAX_COUNTERS (-21).
//  * The plan itself lives in device memory, so the kernel checks it again before it stores anything:
//    a tile count above `max_tiles`, a K cut whose partial tiles do not fit the array, or a tile wider
//    than 64 rows makes the kernel report "bad argument" in args->status and leave the output, the
//    array and its neighbours untouched (a wide tile is skipped, the rest of the plan still runs).
//  * It calls no cudaMalloc / cudaFree and no allocating library routine.  The scratch array
//    (MF_STATIC_SCRATCH_MAX_SLOTS * 32 KiB + MF_STATIC_SCRATCH_MAX_COUNTERS * 4 bytes, about 4.1 MiB) is
//    held by every GPU that loads the library until the process exits.
//  * The first call on a device resolves the array's device address and sets the kernel's shared-memory
//    attribute; make that first call with the device current and before any stream capture begins.
//  * All calls share the one array per device.  It keeps the previous call's contents; the entry point
//    clears the arrival counters on `stream` before the launch.  Two calls that overlap on the same GPU
//    (different streams, or different host threads) race on the array: serialise them.
#define MF_STATIC_SCRATCH_MAX_SLOTS 128
#define MF_STATIC_SCRATCH_MAX_COUNTERS 4096
int mf_gemm_down_static_scratch(const void* tmap, const mf_gemm_args* args, int max_tiles, int split, int grid,
                                mf_stream_t stream);

// ---- router / norm --------------------------------------------------------------------------------
int mf_router_topk(const float* logits, const float* bias, float* weights, int* ids, int tokens, int experts,
                   int top_k, int n_group, int topk_group, int sigmoid, int renorm, float scale,
                   mf_stream_t stream);
int mf_rmsnorm(const void* x, const void* gamma, void* out, int rows, int hidden, float eps, mf_stream_t stream);

// ---- dispatch (pack + peer stores + flags) ----------------------------------------------------------
typedef struct {
  const void* x;             // [T, H] bf16
  const float* weights;      // [T, K] fp32
  const int* ids;            // [T, K] int32 global expert ids
  const int* num_valid;      // optional device scalar: rows >= *num_valid are padding
  const unsigned long long* peer_recv;  // [R] base addresses of every rank's recv buffer
  const unsigned long long* peer_flag;  // [R] base addresses of every rank's dispatch flags [R]
  unsigned char* hit;        // [C, R] local
  unsigned* epoch;           // device-resident forward counter of this layer
  unsigned* done_counter;    // zero between launches
  int T, C, H, K, R, L, rank;
  long long pitch;           // bytes per recv row
  int skip_payload;          // 1: hidden lanes are stored only on rows with valid = 1
  // Optional fused routing: with logits != NULL the kernel routes every token itself (one warp per
  // token, same arithmetic as mf_router_topk), writes the result to `route_w` / `route_ids` ([T, K]) and
  // ignores `weights` / `ids`.
  const float* logits;       // [T, E] fp32
  const float* bias;         // [E] fp32 or NULL
  float* route_w;
  int* route_ids;
  int E, n_group, topk_group, sigmoid, renorm;
  float scale;
  unsigned long long* trace; // optional [8] globaltimer stamps of CTA 0 (profiling aid), or NULL
} mf_dispatch_args;
int mf_dispatch_push(const mf_dispatch_args* args, mf_stream_t stream);

// ---- expert metadata ------------------------------------------------------------------------------------
typedef struct {
  const void* recv;          // [R*C rows] local receive buffer
  long long pitch;           // bytes per row
  int H, K, L, rows;         // rows = R*C
  int R;
  const unsigned* flags;     // [R] dispatch flags (local), may be NULL (no wait)
  const unsigned* epoch;     // expected flag value
  int* offsets;              // [L+1]
  int* entry_row;            // [rows*K]
  int* entry_slot;           // [rows*K]
  float* entry_w;            // [rows*K]
  int* inv;                  // [rows*K]
  int* tile_e;               // [max_tiles]
  int* tile_s;
  int* tile_n;
  int* plan;                 // MF_PLAN_WORDS
  int* counters1;            // split-K counters to clear
  int n_counters1;
  int* counters2;
  int n_counters2;
  int block_m;               // tokens per tile (= n_max of the GEMMs)
  int max_tiles;
  int m_blocks1, k_blocks1, m_blocks2, k_blocks2;
  int n_sms;
  int max_split_slots;       // unused when partial_floats > 0
  unsigned long long* status;
  unsigned long long wait_ns;
  long long partial_floats;  // capacity of the split-K scratch in floats: bounds slots = floats / (tiles * cols * 128)
  int* row_hits;             // optional [rows]: valid slots per received row (for the fused return path)
  // Multi-CTA variant (prefill sizes): with n_ctas > 1 the work is split over n_ctas CTAs in two chained
  // launches (count, then scan + place); cta_hist [n_ctas * L] and acc [2] are its scratch (acc zeroed once
  // by the caller, left zero by every call).  Results are identical to the single-CTA kernel.
  int n_ctas;
  int* cta_hist;
  int* acc;
  // 1: GEMMs with fewer than 8 units per CTA get the stream-K cut (plan word 0) when the scratch holds two
  // partial tiles per CTA; 0: always a K split from mf_plan_split.
  int stream_k;
  unsigned long long* trace; // optional [8] globaltimer stamps of CTA 0 (profiling aid), or NULL
  int late_launch;           // 1: the kernels that follow may only start when this one exits (no early launch)
  int plain_launch;          // 1: launched without programmatic serialization (starts when its predecessor has completed)
} mf_meta_args;
int mf_expert_meta(const mf_meta_args* args, mf_stream_t stream);
// The K-split rule of the metadata kernels, callable on the host (no device needed): the split in {1,2,4,8}
// for `units` (token tile, 128-row block) work items of `k_blocks` K blocks on `n_sms` persistent CTAs, given
// `max_slots` partial-sum slots, the fixed per-unit overhead in K-block units (4 for gate/up, 8 for down) and
// the tile's token columns `cols`.
int mf_plan_split(int units, int k_blocks, int n_sms, int max_slots, int overhead_kb, int cols);

// ---- owner reduce + return push, combine -------------------------------------------------------------
typedef struct {
  const void* y;             // [entries, H] bf16 weighted expert outputs
  const int* inv;            // [rows*K]
  const void* recv;          // local receive buffer (valid flags)
  long long pitch;
  const unsigned long long* peer_ret;   // [R] base addresses of every rank's ret_recv [R, C, H]
  const unsigned long long* peer_flag;  // [R] base addresses of every rank's return flags [R]
  const unsigned* epoch;
  unsigned* done_counter;
  int R, C, H, K, rank;
  int valid_word;            // index of the valid flag among a row's int32 metadata words (2 * top_k)
  unsigned* push_epoch;      // local count of return pushes; the last CTA adds one (the combine's expectation)
  unsigned long long* trace; // optional [8] globaltimer stamps of CTA 0 (profiling aid), or NULL
} mf_reduce_push_args;
int mf_owner_reduce_push(const mf_reduce_push_args* args, mf_stream_t stream);

typedef struct {
  const void* ret;           // local ret_recv [R, C, H] bf16
  const unsigned char* hit;  // [C, R]
  void* out;                 // [C, H] bf16
  const unsigned* flags;     // [R] return flags (local), may be NULL: counting flags, C arrivals per return push
  const unsigned* epoch;     // this rank's count of return pushes (every rank runs the same launch sequence)
  int R, C, H, rank;
  int ring;                  // 1: order (rank+1 .. rank+R) % R with bf16 rounding after every add
  unsigned long long* status;
  unsigned long long wait_ns;
  unsigned long long* trace; // optional [8] globaltimer stamps of CTA 0 (profiling aid), or NULL
} mf_combine_args;
int mf_combine(const mf_combine_args* args, mf_stream_t stream);

// ---- received-row unpacking for external expert kernels ------------------------------------------------
// rows [n_rows, pitch bytes] -> hidden [n_rows, H] bf16, ids [n_rows, K] (exactly one of ids32 / ids64) and
// weights [n_rows, K] fp32; empty slots and rows with valid = 0 get `filler` and weight 0.
int mf_expert_prepare(const void* rows, long long pitch, int n_rows, int H, int K, int rank_offset, int filler,
                      void* hidden, int* ids32, long long* ids64, float* weights, mf_stream_t stream);

// Expert-major copy of the received hidden rows: xg[pos, :H] = recv row entry_row[pos] for pos < plan[N_ENTRIES]
// (so that the gate/up GEMM can read token tiles by TMA; see mf_gemm_args.b_tmap).  `grid` CTAs loop over the entries.
int mf_permute_rows(const void* recv, long long pitch, const int* entry_row, const int* plan, void* xg, int H,
                    int n_rows, int grid, mf_stream_t stream);

// ---- activation quantisation (1x128 groups -> e4m3 + fp32 scales) --------------------------------------
// q[r, :] = e4m3(x[src(r), :] / scale), scales[r, g] = max(amax_g, 1e-10) / 448 for every 128-wide group g.
// src(r) = row_index ? row_index[r] : r.  With valid_off >= 0 a source row whose int32 at that byte offset is
// zero is skipped; with n_rows_dev != NULL rows r >= *n_rows_dev are skipped.
int mf_quant_rows_1x128(const void* x, long long x_pitch, const int* row_index, int rows, int hidden, void* q,
                        float* scales, long long valid_off, const int* n_rows_dev, mf_stream_t stream);
// Block-scaled e4m3 variants of the grouped GEMMs (args->w_scale, b_scale, b_scale_pitch are required;
// b_base rows are e4m3 bytes, k_blocks = K / 128, the tensor map is built with elem_bytes = 1; n_max 32 or 64).
int mf_gemm_gate_up_fp8(const void* tmap, const mf_gemm_args* args, int n_max, int grid, mf_stream_t stream);
int mf_gemm_down_fp8(const void* tmap, const mf_gemm_args* args, int n_max, int grid, mf_stream_t stream);

// ---- peer-memory runtime ------------------------------------------------------------------------------------
int mf_peer_alloc(void** ptr, unsigned long long bytes);
int mf_peer_free(void* ptr);
int mf_peer_export(void* ptr, void* handle64);
int mf_peer_open(const void* handle64, void** ptr);
int mf_peer_close(void* ptr);
int mf_peer_can_access(int dev, int peer_dev, int* ok);
// Ping: store `value` into every peer's word [rank] then wait (bounded) until the local words all
// reach `value`; `skip_store` leaves the stores out so that the wait runs out (status test).
int mf_peer_ping(const unsigned long long* peer_words, unsigned* local_words, int R, int rank, unsigned value,
                 int skip_store, unsigned long long* status, unsigned long long wait_ns, mf_stream_t stream);
const char* mf_error_string(int code);
// Programmatic dependent launch between the kernels of one forward (default on; MOEFLOW_PDL=0 turns it off).
int mf_pdl_enabled(void);
void mf_set_pdl(int on);
int mf_device_sm_count(int* out);

#ifdef __cplusplus
}
#endif
