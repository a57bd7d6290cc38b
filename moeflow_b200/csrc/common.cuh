// Shared device helpers for the sm_100a kernels: status words, bounded waits, PTX wrappers for
// mbarrier / TMA / tcgen05 (UMMA) / cp.async, and a few small math utilities.
//
// Conventions
//  * Every wait in this library is bounded.  A wait that runs out records a status code in the
//    layer's status word, raises the CTA-local abort flag where there is one, and returns; it never
//    traps and never spins forever, so the CUDA context stays usable and the host can read the code.
//  * Nothing here issues a TMA load with cluster multicast.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mf {

// ---------------------------------------------------------------------------------------------
// Status word (one int64 per layer, device memory, read lazily by the host outside graphs).
// layout: bits [0,8) code, [8,16) peer/stage, [16,32) detail, [32,64) epoch.
// ---------------------------------------------------------------------------------------------
enum StatusCode : int {
  kOk = 0,
  kDispatchFlagTimeout = 1,   // expert_meta gave up waiting for a source rank's dispatch flag
  kReturnFlagTimeout = 2,     // combine gave up waiting for an owner rank's return flag
  kGemmFullTimeout = 3,       // MMA issuer gave up waiting for operand tiles
  kGemmEmptyTimeout = 4,      // a producer gave up waiting for a free pipeline stage
  kGemmAccTimeout = 5,        // accumulator hand-off (MMA <-> epilogue) timed out
  kGemmTmemTimeout = 6,       // (reserved)
  kBadArgument = 7,
  kPingTimeout = 8,           // peer ping test
};

__device__ __forceinline__ void report_status(unsigned long long* status, int code, int who, int detail,
                                              unsigned epoch) {
  if (status == nullptr) return;
  unsigned long long v = (unsigned long long)(code & 0xff) | ((unsigned long long)(who & 0xff) << 8) |
                         ((unsigned long long)(detail & 0xffff) << 16) | ((unsigned long long)epoch << 32);
  // First error wins: only replace a zero word.
  atomicCAS(status, 0ull, v);
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
  uint32_t l;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
  return l;
}

// ---------------------------------------------------------------------------------------------
// Warm-up touches.  A kernel launched with programmatic serialization sits idle until its predecessor is
// done; the first access it then makes to every page costs an address-translation miss, and with a cold
// L2 the page-table walk itself goes to DRAM (measured on B200: microseconds per first touch, one after
// the other on a dependent chain).  touch() reads one word before the wait, so the translation is
// in place and the line is in L2 when the real access comes.  The value read is never used (it may be stale).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void touch(const void* p) {
  if (p == nullptr) return;
  p = reinterpret_cast<const void*>(reinterpret_cast<uintptr_t>(p) & ~uintptr_t(3));  // a 4-byte load: align down (byte arrays)
  asm volatile(
      "{\n\t"
      ".reg .u32 unused;\n\t"
      "ld.volatile.global.u32 unused, [%0];\n\t"
      "}" ::"l"(p)
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched with the programmatic-serialization attribute
// may start while its predecessor in the stream is still running; it must call grid_dep_wait()
// before it touches anything the predecessor writes (the wait returns when the predecessor has
// completed and its writes are visible).  grid_dep_launch() lets the *next* kernel start early.
// Both are no-ops in a kernel launched the ordinary way.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// The whole CTA waits for the predecessor, but only one thread executes the wait instruction; the others sit
// at the CTA barrier.  The wait makes the predecessor's writes visible to the grid, and the barrier orders the
// other threads after it.  Measured on B200: with every thread of every early-resident CTA in
// griddepcontrol.wait (148 GEMM CTAs of 256 threads, a thousand reduce CTAs), the kernels that were still
// running took three times longer per phase; with one waiting thread per CTA they run at full speed.
// All threads of the CTA must call this (it contains a __syncthreads()).
__device__ __forceinline__ void grid_dep_wait_cta() {
  if (threadIdx.x == 0) grid_dep_wait();
  __syncthreads();
}
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// System-scope flag access (peer-visible memory).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_u32(unsigned* p, unsigned v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Publish one value in word [rank] of every peer's flag array.  A release store carries a full
// system-scope fence each; with R peers that is R fences in a row, so fence once and store relaxed.
__device__ __forceinline__ void publish_flags(const unsigned long long* peer_flag, int n_peers, int rank, unsigned value) {
  __threadfence_system();
  for (int d = 0; d < n_peers; ++d) st_relaxed_sys_u32(reinterpret_cast<unsigned*>(peer_flag[d]) + rank, value);
}
// Fence between a CTA's row stores and its arrival: system scope when the rows went to peers' memory, device
// scope when the only rank is this GPU (the system-scope fence costs microseconds even without a peer).
__device__ __forceinline__ void fence_before_arrival(int n_ranks) {
  if (n_ranks > 1)
    __threadfence_system();
  else
    __threadfence();
}

// Counting flags: every CTA that has finished its share of a transfer adds one to word [rank] of the
// destination's flag array, after a system-scope fence that orders the CTA's peer stores before it.  The
// waiter knows how many arrivals a forward brings (epoch * arrivals per forward), so no CTA has to be the
// last one and no second fence or local counter sits between the data and the flag.
__device__ __forceinline__ void red_add_relaxed_sys_u32(unsigned* p, unsigned v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_relaxed_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ int ld_acquire_gpu_s32(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Orders later async-proxy accesses (TMA) of this thread after its earlier generic-proxy accesses: needed when
// data written with ordinary stores by another CTA is fetched by TMA after a flag handshake.
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
// Bounded wait for a device-scope counter to reach `want`.
__device__ __forceinline__ bool wait_count_ge_gpu(const int* counter, int want, unsigned long long limit_ns) {
  if (ld_acquire_gpu_s32(counter) >= want) return true;
  const unsigned long long t0 = global_timer_ns();
  unsigned spins = 0;
  while (true) {
    if (ld_acquire_gpu_s32(counter) >= want) return true;
    if ((++spins & 63u) == 0u) {
      if (global_timer_ns() - t0 > limit_ns) return false;
    }
    __nanosleep(32);
  }
}

// Spin until *flag >= want (wrap-safe signed difference) or until `limit_ns` has passed.
// Returns true on success.
__device__ __forceinline__ bool wait_flag_ge(const unsigned* flag, unsigned want, unsigned long long limit_ns) {
  if ((int)(ld_acquire_sys_u32(flag) - want) >= 0) return true;
  const unsigned long long t0 = global_timer_ns();
  unsigned spins = 0;
  while (true) {
    if ((int)(ld_acquire_sys_u32(flag) - want) >= 0) return true;
    if ((++spins & 63u) == 0u) {
      if (global_timer_ns() - t0 > limit_ns) return false;
      __nanosleep(64);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded mbarrier wait.  `abort_flag` is a CTA-shared int: once any role has given up, every other
// wait in the CTA returns quickly so that the CTA can tear down (free TMEM, exit).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                  unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  unsigned spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 255u) == 0u) {
      if (*abort_flag != 0) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// TMA (tiled bulk tensor copy, global -> this CTA's shared memory, no multicast)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// ---------------------------------------------------------------------------------------------
// cp.async (16-byte, L2-only) with zero fill, completion reported to an mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void* gmem_src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gmem_src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05 (5th-generation tensor core, accumulators in tensor memory)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]^T, bf16/f16 inputs, fp32 accumulate.  One thread issues.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same, 8-bit float inputs (e4m3/e5m2 selected in idesc), K = 32 per instruction.
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival when every tcgen05 operation issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// 32 lanes x 16 consecutive fp32 columns: thread i of the warp gets lane (base_lane + i).
__device__ __forceinline__ void tmem_ld_16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 32 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld_32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (the layout a TMA box of 64 bf16 x rows with SWIZZLE_128B produces): 8-row groups
// are 1024 bytes apart.  The tile base must be 1024-byte aligned; a K step of 32 bytes inside the
// 128-byte row is taken by adding 2 to the encoded start address.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);   // start address, 16-byte units
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024u >> 4) << 32;             // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                        // descriptor version for sm_100
  d |= (uint64_t)2 << 61;                        // layout: 128-byte swizzle
  return d;
}
// Instruction descriptor, dense, fp32 accumulate, both operands K-major.
// fmt: 0 = f16, 1 = bf16 (kind::f16); 0 = e4m3, 1 = e5m2 (kind::f8f6f4).
__device__ __forceinline__ uint32_t umma_idesc(uint32_t fmt_a, uint32_t fmt_b, uint32_t m, uint32_t n) {
  return (1u << 4) | (fmt_a << 7) | (fmt_b << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------
// Small math
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// SwiGLU with the asymmetric clamp: gate clamped from above only, up clamped to [-limit, limit].
// limit <= 0 means "no clamp".
__device__ __forceinline__ float swiglu_clamped(float gate, float up, float limit) {
  if (limit > 0.f) {
    gate = fminf(gate, limit);
    up = fminf(fmaxf(up, -limit), limit);
  }
  return __fdividef(gate, 1.f + __expf(-gate)) * up;  // reciprocal + multiply: 2 ulp, far inside the 16-bit output
}

struct alignas(16) U4 {
  uint32_t x, y, z, w;
};

}  // namespace mf

// Host side: launch with or without the programmatic-serialization attribute.
extern "C" int mf_pdl_enabled(void);

namespace mf {
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 bool dependent, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (dependent && mf_pdl_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
}  // namespace mf
