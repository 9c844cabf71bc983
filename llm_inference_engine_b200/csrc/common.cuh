// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk[.tensor], no cluster
// multicast anywhere), tcgen05 (TMEM alloc, UMMA, commit, ld) and the UMMA descriptors.
//
// Every wait in this file is bounded: it gives up after WAIT_LIMIT_NS of wall time and reports
// failure to the caller, which records a status code and leaves through its normal teardown.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace muse {

// Status codes a kernel may OR into its status word (0 = clean).
enum : int {
  ST_PRODUCER_TIMEOUT = 1,  // TMA producer: a stage was never released
  ST_MMA_TIMEOUT = 2,       // MMA issuer: a stage never filled
  ST_EPILOGUE_TIMEOUT = 4,  // epilogue: the accumulator-ready barrier never completed
  ST_X_TIMEOUT = 8,         // GEMV: the bulk copy of x never completed
  ST_DRAIN_TIMEOUT = 16,    // teardown: an issued TMA copy did not land within the limit
};

constexpr unsigned long long WAIT_LIMIT_NS = 500ull * 1000ull * 1000ull;  // 0.5 s

// Phase stamps are a diagnostic of -DMUSE_TRACE builds only. There every translation unit carries a device
// pointer (set through muse_trace_set, which only such builds export) to a buffer of 16 unsigned 64-bit
// slots per CTA; in an ordinary build the base is a compile-time null and every stamp site folds away.
#ifdef MUSE_TRACE
static __device__ unsigned long long* g_trace_dev = nullptr;
#define MUSE_TRACE_BASE() (g_trace_dev)
#define MUSE_TRACE_SETTER(name) \
  cudaError_t name(unsigned long long* p) { return cudaMemcpyToSymbol(g_trace_dev, &p, sizeof(p)); }
#else
#define MUSE_TRACE_BASE() (static_cast<unsigned long long*>(nullptr))
#define MUSE_TRACE_SETTER(name)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Returns false if the phase did not complete within WAIT_LIMIT_NS.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_ns() - t0 > WAIT_LIMIT_NS) return false;
  }
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// 2-D tiled load global -> shared, completion counted in bytes on `bar`. c0 = innermost coordinate
// (elements; c0 * elem_size must be a multiple of 16 bytes), c1 = row coordinate.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, int c0, int c1, uint32_t bar,
                                            uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(c0), "r"(c1), "r"(bar), "l"(policy)
      : "memory");
}
// 1-D bulk copy global -> shared (both 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {  // whole warp
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; BF16 inputs, FP32 accumulate; one thread issues.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives once on `bar` when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor for a K-major BF16 tile whose rows are 128 bytes (64 elements)
// laid out with the 128-byte swizzle (what a TMA box of {64, rows} with SWIZZLE_128B writes):
// 8-row groups are 1024 bytes apart (stride byte offset), the leading byte offset is unused.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (ignored for swizzled K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version: Blackwell
  d |= static_cast<uint64_t>(2) << 61;                      // layout: SWIZZLE_128B
  return d;
}

// Instruction descriptor: BF16 x BF16 -> FP32, both operands K-major, dense, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N) {
  return (1u << 4)                                  // D format: F32
         | (1u << 7)                                // A format: BF16
         | (1u << 10)                               // B format: BF16
         | (static_cast<uint32_t>(N >> 3) << 17)    // N / 8
         | (static_cast<uint32_t>(M >> 4) << 24);   // M / 16
}

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with launch_dependent() below may become resident while the kernel before it in the stream is
// still running (as that kernel's CTAs leave their SMs). Until griddep_wait() returns it may touch only what no
// kernel ever writes -- the weights -- so its first weight loads, its launch latency and its set-up run under the
// previous kernel's tail; activations, outputs, workspaces, counters and the status word come after the wait, which
// returns once every kernel ahead in the stream has completed and its writes are visible. A kernel says with
// griddep_launch_dependents() that the next one may be brought in; without it that happens when the kernel ends.
// Both are no-ops for a kernel launched the ordinary way. One more rule follows from the overlap: anything another
// kernel writes (activations, residual streams) is read with L2-coherent loads (__ldcg, TMA, bulk copies), never
// through the non-coherent path (__ldg / ld.global.nc): that path is for data that is read-only for the kernel's
// whole lifetime, which here begins before the predecessor's ends, so such a load may be scheduled above the wait
// or served from an L1 line cached calls ago.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

extern bool g_programmatic_launch;   // capi.cu; muse_set_programmatic_launch()

template <typename... P, typename... A>
inline cudaError_t launch_dependent(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_programmatic_launch ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}

// ---------------------------------------------------------------- plain memory helpers
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ float ldg_cg_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void stg_cg_f32(float* p, float v) {
  asm volatile("st.global.cg.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ void red_add_f32(float* p, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ float bf16lo_f32(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16hi_f32(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// ---------------------------------------------------------------- column-parallel output exchange
//
// With the weight sharded by output rows over `world` GPUs (one process each), a kernel writes its
// [m, n] slice straight into the [m, N] output of EVERY rank (plain stores through peer-mapped
// pointers over NVLink; no multimem, no TMA to or from peer memory), at column `col0`, so the
// all-gather is part of the kernel. Two rounds of flags, living in a small peer-mapped int array per
// rank, order it against the neighbours:
//   enter[r]   written to every peer when rank r's kernel of call e starts. A rank stores into a
//              peer only after that peer has entered call e: the peer's consumers of call e-1's
//              output ran earlier on its stream. The wait sits in the epilogue, long after the flag
//              was raised, and normally returns at once.
//   done[r]    written to every peer by rank r's last CTA after all its stores (system-scope fence).
//              The same CTA then waits for every peer's done[.] >= e, so when the kernel completes
//              the local [m, N] holds every rank's slice.
// The register-MMA kernel exchanges without fences or flags: its CTAs send 16-byte lines {data, call
// number, data, call number} into a staging area on each peer (ll[.], two halves used by odd and even
// calls, one block per sending rank) and finish by unpacking what the peers sent them into their own
// gathered output, polling each line until both of its 8-byte halves carry this call's number. Nothing
// is written into a peer's gathered output, so that path needs no enter round either. A half is reused
// two calls later; between the two uses lies a whole call in which both ranks had to receive each
// other's lines, i.e. the receiver had finished unpacking the earlier use.
// Layout of a rank's flag array (int32): [0, 8) enter, [8, 16) done, [16] epoch of the last finished
// call, [17] CTA arrival counter. All waits are bounded and report through the status word.
constexpr int MAX_WORLD = 8;
enum : int { ST_PEER_ENTER_TIMEOUT = 32, ST_PEER_DONE_TIMEOUT = 64 };

struct PeerSync {
  int world;   // 0 or 1: single GPU, nothing below is used
  int rank;
  int col0;    // first output column of this rank's slice in the gathered [m, N]
  int pad_;
  void* out[MAX_WORLD];    // every rank's gathered output (same shape and row stride everywhere)
  int* flags[MAX_WORLD];   // every rank's flag array
  void* ll[MAX_WORLD];     // every rank's staging for self-validating lines (register-MMA kernel; may be null)
};
constexpr int LL_TOKENS = 32;   // most tokens of a call exchanged through the staging

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_volatile_s32(const int* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool peer_active(const PeerSync& ps) { return ps.world > 1; }
// The call number this launch represents (every rank makes the same sequence of calls). The word was
// written by this GPU's previous kernel, so a plain load sees it. ONE thread per CTA reads it and
// hands it to the others through shared memory: system-scope operations are kept to a handful per CTA.
__device__ __forceinline__ int peer_epoch(const PeerSync& ps) { return ld_volatile_s32(ps.flags[ps.rank] + 16) + 1; }
// One thread of the grid: tell every peer that this rank has entered call `e`. Nothing is released by
// this flag (the kernels that consumed the previous output completed before this one started), so the
// stores are relaxed and leave back to back: a release per peer would cost one NVLink round trip each.
__device__ __forceinline__ void peer_announce_enter(const PeerSync& ps, int e) {
  for (int p = 0; p < ps.world; ++p) st_relaxed_sys(ps.flags[p] + ps.rank, e);
}
__device__ __forceinline__ bool peer_wait_flag(const int* flag, int e) {
  if (ld_acquire_sys(flag) >= e) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (ld_volatile_s32(flag) >= e) return ld_acquire_sys(flag) >= e;
    if (global_ns() - t0 > WAIT_LIMIT_NS) return false;
  }
}
// All threads of a CTA, before its first store to a peer: threads 0..world-1 each wait for one peer
// to have entered call `e` (one acquire per peer per CTA), then the CTA synchronises.
__device__ __forceinline__ void peer_wait_all_entered(const PeerSync& ps, int e, int* status) {
  if (threadIdx.x < ps.world && !peer_wait_flag(ps.flags[ps.rank] + threadIdx.x, e))
    atomicOr(status, ST_PEER_ENTER_TIMEOUT);
  __syncthreads();
}
// All threads of every CTA call this after their last store (to peers or to the local output).
// `s_flag` is a shared int. A CTA orders its stores before its arrival with a GPU-scope fence;
// returns true (CTA-uniform) in the last CTA to arrive, which is then ordered after every other
// CTA's stores.
__device__ __forceinline__ bool peer_last_cta(const PeerSync& ps, int total_ctas, int* s_flag) {
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int last = atomicAdd(ps.flags[ps.rank] + 17, 1) == total_ctas - 1;
    if (last) __threadfence();
    *s_flag = last;
  }
  __syncthreads();
  return *s_flag != 0;
}
// All threads of the last CTA, after any stores of its own: one system-scope fence, then done[rank]
// goes to every peer (release/acquire chains are cumulative across scopes, so the peers see every
// CTA's stores), then wait for every peer's done flag: the kernel completes only when the local
// gathered output is complete. Finally the epoch advances and the arrival counter is reset.
__device__ __forceinline__ void peer_publish(const PeerSync& ps, int e, int* status) {
  int* mine = ps.flags[ps.rank];
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) mine[17] = 0;
  if (threadIdx.x < ps.world) {
    // One thread per peer, all in parallel: a system-scope fence (it covers the whole CTA's stores, which
    // the barrier above ordered before it), the flag, then the wait for that peer's flag.
    __threadfence_system();
    st_relaxed_sys(ps.flags[threadIdx.x] + 8 + ps.rank, e);
    if (!peer_wait_flag(mine + 8 + threadIdx.x, e)) atomicOr(status, ST_PEER_DONE_TIMEOUT);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    mine[16] = e;
    __threadfence();
  }
}
__device__ __forceinline__ void peer_finish(const PeerSync& ps, int e, int total_ctas, int* status, int* s_flag) {
  if (peer_last_cta(ps, total_ctas, s_flag)) peer_publish(ps, e, status);
}

// ---- self-validating lines (see above)
__device__ __forceinline__ void st_volatile_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// Byte offset, inside a rank's staging, of the lines that `src` sends for token t of call e (n = slice width).
__device__ __forceinline__ size_t ll_row_offset(int e, int world, int src, int t, int n) {
  return ((static_cast<size_t>(e & 1) * world + src) * LL_TOKENS + t) * static_cast<size_t>(n) * 4;
}
// 16 bytes of payload (8 BF16 outputs) as two lines tagged with the call number.
__device__ __forceinline__ void ll_send16(void* dst, uint4 v, int e) {
  st_volatile_v4(dst, v.x, static_cast<uint32_t>(e), v.y, static_cast<uint32_t>(e));
  st_volatile_v4(static_cast<char*>(dst) + 16, v.z, static_cast<uint32_t>(e), v.w, static_cast<uint32_t>(e));
}
// Poll two lines until all four halves carry call number e (bounded); false on time-out.
__device__ __forceinline__ bool ll_recv16(const void* src, int e, uint4& v) {
  const uint32_t want = static_cast<uint32_t>(e);
  const unsigned long long t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      const uint4 a = ld_volatile_v4(src), b = ld_volatile_v4(static_cast<const char*>(src) + 16);
      if (a.y == want && a.w == want && b.y == want && b.w == want) {
        v = make_uint4(a.x, a.z, b.x, b.z);
        return true;
      }
    }
    if (global_ns() - t0 > WAIT_LIMIT_NS) return false;
  }
}

}  // namespace muse
