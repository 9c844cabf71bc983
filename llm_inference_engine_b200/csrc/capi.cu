// extern "C" boundary of libmuse_proj.so: argument checks, tensor-map encoding, launches.
// Declarations and the contract of every entry point are in include/muse_proj.h.
#include <cudaTypedefs.h>
#include <string.h>

#include "../../include/muse_proj.h"
#include "boundary.cuh"
#include "common.cuh"

namespace muse {
bool g_programmatic_launch = true;
int gemv1_dispatch(const void* W, const void* x, void* out, int N, int K, int w_is_f32, int wpr, int unroll,
                   int persistent, int* status, const PeerSync* peers, cudaStream_t stream);
int skinny_tc_dispatch(const CUtensorMap* tw, const CUtensorMap* twlo, const CUtensorMap* tx, void* out, float* ws,
                       int* cnt, int* status, int m, int n, int k, int ld_out, int ntok, int cluster, int groups,
                       int stages, int out_f32, const PeerSync* peers, cudaStream_t stream);
int skinny_stage_bytes(int ntok, int hilo);
int skinny_smem_bytes(int ntok, int hilo, int stages, int cluster, int m);
int skinny_max_clusters(int ntok, int hilo, int m, int stages, int cluster);
int skinny_tc_static_dispatch(const CUtensorMap* tw, const CUtensorMap* twlo, const CUtensorMap* tx, void* out,
                              int* status, int m, int n, int k, int ld_out, int ntok, int cluster, int groups,
                              int stages, int out_f32, cudaStream_t stream);
int fewtok_mma_dispatch(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out, int warps,
                        int unroll, int tok_split, int* status, const PeerSync* peers, cudaStream_t stream);
size_t fewtok_smem_bytes(int m, int K, int warps);
int fewtok_f32_dispatch(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out, int unroll,
                        int tok_split, int x_is_f32, cudaStream_t stream);
int fewtok_rowpar_dispatch(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out, int* status,
                           const PeerSync* peers, cudaStream_t stream);
int attn_boundary_dispatch(const BoundaryArgs& bd, int m, int D, cudaStream_t stream);
int fewtok_boundary_dispatch(const void* W, int w_is_f32, const BoundaryArgs& bd, void* out, int m, int N, int K, int ld_out,
                             int* status, cudaStream_t stream);
int fused_boundary_dispatch(const void* Wp, const void* Wr_hi, const void* Wr_lo, const BoundaryArgs& bd, void* h_lo, void* outp,
                            void* outr, int m, int Np, int Nr, int K, int ld_outp, int ld_outr, int* cnt, int* status,
                            cudaStream_t stream);
int fewtok_zip_dispatch(const void* lo, const void* nib, const void* exc, int cap, int base, const void* x, void* out, int m, int N,
                        int K, int ld_x, int ld_out, int warps, int unroll, int reduce_every, cudaStream_t stream);
struct FfnBoundaryArgs;
int ffn_boundary_dispatch(const FfnBoundaryArgs& a, const void* f, int m, int D, int nf, cudaStream_t stream);
int unpooler_ffn_dispatch(const void* W, const void* x, void* f_scratch, const FfnBoundaryArgs& a, int m, int NF, int K, int ld_x, int D,
                          int* cnt, int* status, cudaStream_t stream);
int gemm_tc_dispatch(const CUtensorMap* tw, const CUtensorMap* tx, void* out, float* ws, int* cnt, int* status, int m, int n,
                     int k, int ld_out, int ntok, int pair, int cluster, int split, int stages, int warpgroups, int tile_rows,
                     int katoms, const PeerSync* peers, cudaStream_t stream);
long long gemm_tc_ws_floats(int m, int n, int ntok, int pair, int split, int tile_rows);
int gemm_tc_cnt_ints(int m, int n, int ntok, int pair, int split, int tile_rows);
int gemm_tc_smem_bytes(int ntok, int pair, int stages, int cluster, int m, int warpgroups, int tile_rows, int katoms);
int gemm_tc_max_clusters(int ntok, int pair, int stages, int cluster, int m, int warpgroups, int tile_rows, int katoms);
#ifdef MUSE_TRACE
cudaError_t skinny_trace_set(unsigned long long* p);
cudaError_t fewtok_trace_set(unsigned long long* p);
cudaError_t gemm_trace_set(unsigned long long* p);
#endif
long long skinny_static_ws_floats();
int skinny_static_cnt_ints();

// cuTensorMapEncodeTiled is a driver entry point; fetching it through the runtime keeps the
// library free of a link-time dependency on libcuda (it must load on machines without a driver).
static PFN_cuTensorMapEncodeTiled encode_fn() {
  static PFN_cuTensorMapEncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
  }
  return fn;
}

static int encode_2d(CUtensorMap* tm, const void* base, long long rows, long long cols, long long row_stride_bytes,
                     int box_rows) {
  if (!tm || !base || rows <= 0 || cols <= 0 || box_rows <= 0 || box_rows > 256) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15) || row_stride_bytes < cols * 2) return -2;
  PFN_cuTensorMapEncodeTiled fn = encode_fn();
  if (!fn) return -8;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_stride_bytes)};
  const cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return static_cast<int>(r);
}
__global__ void nop_kernel() {}

// Copies `vecs` 16-byte vectors from page-locked host memory (device-addressable) into device memory with
// plain loads: for a few KB this is a kernel-to-kernel dependency for the consumer instead of a copy-engine
// hand-off.
__global__ void fetch_host_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long vecs) {
  griddep_launch_dependents();   // the projection behind this kernel may start its weight loads now; it waits for x itself
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < vecs;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = __ldcg(src + i);   // never through the non-coherent path: the source is rewritten between launches
}
}  // namespace muse

extern "C" {

int muse_nop(void* stream) {
  muse::nop_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>();
  return static_cast<int>(cudaGetLastError());
}

int muse_abi_version(void) { return MUSE_PROJ_ABI_VERSION; }

int muse_set_programmatic_launch(int enabled) {
  const int was = muse::g_programmatic_launch ? 1 : 0;
  muse::g_programmatic_launch = enabled != 0;
  return was;
}

#ifdef MUSE_TRACE
// Diagnostic builds only (not part of the ABI in muse_proj.h): the device buffer that the kernels' phase
// stamps go to, 16 unsigned 64-bit slots per CTA of the largest grid; NULL turns stamping off.
int muse_trace_set(void* device_buffer) {
  cudaError_t e = muse::skinny_trace_set(static_cast<unsigned long long*>(device_buffer));
  if (e == cudaSuccess) e = muse::fewtok_trace_set(static_cast<unsigned long long*>(device_buffer));
  if (e == cudaSuccess) e = muse::gemm_trace_set(static_cast<unsigned long long*>(device_buffer));
  return static_cast<int>(e);
}
#endif

int muse_query(int what) {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  cudaError_t e = cudaSuccess;
  switch (what) {
    case 0: e = cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev); break;
    case 1: e = cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev); break;
    case 2: {
      int mj = 0, mn = 0;
      e = cudaDeviceGetAttribute(&mj, cudaDevAttrComputeCapabilityMajor, dev);
      if (e == cudaSuccess) e = cudaDeviceGetAttribute(&mn, cudaDevAttrComputeCapabilityMinor, dev);
      v = mj * 10 + mn;
      break;
    }
    case 3: e = cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, dev); break;
    default: return -2;
  }
  return e == cudaSuccess ? v : -1;
}

static_assert(sizeof(muse_peer_sync_t) == sizeof(muse::PeerSync), "muse_peer_sync_t must mirror PeerSync");
static_assert(sizeof(muse_boundary_t) == sizeof(muse::BoundaryArgs), "muse_boundary_t must mirror BoundaryArgs");

int muse_attn_boundary(const muse_boundary_t* bd, int m, int d, void* stream) {
  if (!bd) return -1;
  return muse::attn_boundary_dispatch(*reinterpret_cast<const muse::BoundaryArgs*>(bd), m, d, static_cast<cudaStream_t>(stream));
}

int muse_fewtok_boundary(const void* W, int w_is_f32, const muse_boundary_t* bd, void* out, int m, int N, int K, int ld_out,
                         int* status, void* stream) {
  if (!bd) return -1;
  return muse::fewtok_boundary_dispatch(W, w_is_f32, *reinterpret_cast<const muse::BoundaryArgs*>(bd), out, m, N, K, ld_out, status,
                                        static_cast<cudaStream_t>(stream));
}

int muse_boundary_pooler_router(const void* W_pooler, const void* W_router_hi, const void* W_router_lo, const muse_boundary_t* bd,
                                void* h_lo, void* out_pooler, void* out_router, int m, int n_pooler, int n_router, int K,
                                int ld_out_pooler, int ld_out_router, int* cnt, int* status, void* stream) {
  if (!bd) return -1;
  return muse::fused_boundary_dispatch(W_pooler, W_router_hi, W_router_lo, *reinterpret_cast<const muse::BoundaryArgs*>(bd), h_lo,
                                       out_pooler, out_router, m, n_pooler, n_router, K, ld_out_pooler, ld_out_router, cnt, status,
                                       static_cast<cudaStream_t>(stream));
}

int muse_fewtok_zip(const void* low, const void* code, const void* table, int cap, int base, const void* x, void* out, int m, int N,
                    int K, int ld_x, int ld_out, int warps, int unroll, int reduce_every, void* stream) {
  return muse::fewtok_zip_dispatch(low, code, table, cap, base, x, out, m, N, K, ld_x, ld_out, warps, unroll, reduce_every,
                                   static_cast<cudaStream_t>(stream));
}

int muse_ffn_boundary(const muse_ffn_boundary_t* bd, const void* f, int m, int d, int nf, void* stream) {
  if (!bd) return -1;
  return muse::ffn_boundary_dispatch(*reinterpret_cast<const muse::FfnBoundaryArgs*>(bd), f, m, d, nf, static_cast<cudaStream_t>(stream));
}

int muse_unpooler_ffn_boundary(const void* W, const void* x, void* f_scratch, const muse_ffn_boundary_t* bd, int m, int nf, int K, int ld_x,
                               int d, int* cnt, int* status, void* stream) {
  if (!bd) return -1;
  return muse::unpooler_ffn_dispatch(W, x, f_scratch, *reinterpret_cast<const muse::FfnBoundaryArgs*>(bd), m, nf, K, ld_x, d, cnt, status,
                                     static_cast<cudaStream_t>(stream));
}

int muse_gemv1(const void* W, const void* x, void* out, int N, int K, int w_is_f32, int wpr, int unroll, int persistent,
               int* status, const muse_peer_sync_t* peers, void* stream) {
  return muse::gemv1_dispatch(W, x, out, N, K, w_is_f32, wpr, unroll, persistent, status,
                              reinterpret_cast<const muse::PeerSync*>(peers), static_cast<cudaStream_t>(stream));
}

int muse_copy_h2d_async(void* dst_device, const void* src_host, long long bytes, void* stream) {
  if (!dst_device || !src_host || bytes < 0) return -1;
  return static_cast<int>(cudaMemcpyAsync(dst_device, src_host, static_cast<size_t>(bytes), cudaMemcpyHostToDevice,
                                          static_cast<cudaStream_t>(stream)));
}

int muse_fetch_host(void* dst_device, const void* src_host, long long bytes, void* stream) {
  if (!dst_device || !src_host || bytes < 0 || bytes % 16 ||
      ((reinterpret_cast<uintptr_t>(dst_device) | reinterpret_cast<uintptr_t>(src_host)) & 15))
    return -1;
  if (bytes == 0) return 0;
  const long long vecs = bytes / 16;
  const int grid = static_cast<int>(vecs / 256 + 1 < 148 ? vecs / 256 + 1 : 148);
  muse::fetch_host_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint4*>(dst_device), static_cast<const uint4*>(src_host), vecs);
  return static_cast<int>(cudaGetLastError());
}

int muse_copy_d2h_sync(void* dst_host, const void* src_device, long long bytes, void* stream) {
  if (!dst_host || !src_device || bytes < 0) return -1;
  cudaError_t e = cudaMemcpyAsync(dst_host, src_device, static_cast<size_t>(bytes), cudaMemcpyDeviceToHost,
                                  static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
}

int muse_fewtok_mma(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out, int warps,
                    int unroll, int tok_split, int* status, const muse_peer_sync_t* peers, void* stream) {
  return muse::fewtok_mma_dispatch(W, x, out, m, N, K, ld_x, ld_out, warps, unroll, tok_split, status,
                                   reinterpret_cast<const muse::PeerSync*>(peers), static_cast<cudaStream_t>(stream));
}

int muse_fewtok_rowpar(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out, int* status,
                       const muse_peer_sync_t* peers, void* stream) {
  return muse::fewtok_rowpar_dispatch(W, x, out, m, N, K, ld_x, ld_out, status, reinterpret_cast<const muse::PeerSync*>(peers),
                                      static_cast<cudaStream_t>(stream));
}

int muse_fewtok_mma_host(const void* W, const void* x_host, void* x_device, void* out_device, void* out_host, int m, int N,
                         int K, int warps, int unroll, int tok_split, int* status, void* stream) {
  if (!x_host || !x_device || !out_device || !out_host || m < 1 || N < 1 || K < 1) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(x_device, x_host, static_cast<size_t>(m) * K * 2, cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int rc = muse::fewtok_mma_dispatch(W, x_device, out_device, m, N, K, K, N, warps, unroll, tok_split, status, nullptr, s);
  if (rc != 0) return rc;
  e = cudaMemcpyAsync(out_host, out_device, static_cast<size_t>(m) * N * 2, cudaMemcpyDeviceToHost, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaStreamSynchronize(s));
}

int muse_fewtok_f32(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out, int unroll,
                    int tok_split, int x_is_f32, void* stream) {
  return muse::fewtok_f32_dispatch(W, x, out, m, N, K, ld_x, ld_out, unroll, tok_split, x_is_f32,
                                   static_cast<cudaStream_t>(stream));
}

long long muse_fewtok_smem_bytes(int m, int K, int warps) {
  return static_cast<long long>(muse::fewtok_smem_bytes(m, K, warps));
}

int muse_tmap_encode_2d(void* tmap_out128, const void* base, long long rows, long long cols,
                        long long row_stride_bytes, int box_rows) {
  CUtensorMap tm;
  const int r = muse::encode_2d(&tm, base, rows, cols, row_stride_bytes, box_rows);
  if (r == 0) memcpy(tmap_out128, &tm, sizeof(tm));
  return r;
}

int muse_skinny_tiles(int m, int n, int ntok) {
  if (m <= 0 || n <= 0 || ntok <= 0) return -1;
  return ((n + 127) / 128) * ((m + ntok - 1) / ntok);
}

long long muse_skinny_ws_floats(int m, int n, int ntok) {
  const int t = muse_skinny_tiles(m, n, ntok);
  return t < 0 ? -1 : static_cast<long long>(t) * 128 * ntok;
}

int muse_skinny_stage_bytes(int ntok, int hilo) { return muse::skinny_stage_bytes(ntok, hilo); }

int muse_skinny_smem_bytes(int ntok, int hilo, int stages, int cluster, int m) {
  return muse::skinny_smem_bytes(ntok, hilo, stages, cluster, m);
}

int muse_skinny_max_clusters(int ntok, int hilo, int m, int stages, int cluster) {
  return muse::skinny_max_clusters(ntok, hilo, m, stages, cluster);
}

int muse_skinny_tc(const void* tmap_w, const void* tmap_w_lo, const void* x, void* out, float* ws, int* cnt,
                   int* status, int m, int n, int k, int ld_x, int ld_out, int ntok, int cluster, int groups, int stages,
                   int out_is_f32, const muse_peer_sync_t* peers, void* stream) {
  if (!tmap_w || !x) return -1;
  if (ld_x < k || ld_x % 8 != 0) return -2;
  // x moves between calls (a fresh activation tensor each time), so its map is encoded per call; the
  // map travels in the kernel's parameters, which is what makes a captured launch replayable.
  CUtensorMap tx;
  const int r = muse::encode_2d(&tx, x, m, k, static_cast<long long>(ld_x) * 2, ntok);
  if (r != 0) return r;
  CUtensorMap tw, twlo;
  memcpy(&tw, tmap_w, sizeof(tw));
  if (tmap_w_lo) memcpy(&twlo, tmap_w_lo, sizeof(twlo));
  return muse::skinny_tc_dispatch(&tw, tmap_w_lo ? &twlo : nullptr, &tx, out, ws, cnt, status, m, n, k, ld_out, ntok,
                                  cluster, groups, stages, out_is_f32, reinterpret_cast<const muse::PeerSync*>(peers),
                                  static_cast<cudaStream_t>(stream));
}

static bool gemm_tile_rows_ok(int pair, int tile_rows) {
  return tile_rows >= 8 && tile_rows <= 128 && tile_rows % 8 == 0 && (!pair || tile_rows == 128);
}

int muse_gemm_tc_smem_bytes(int ntok, int pair, int stages, int cluster, int m, int warpgroups, int tile_rows, int k_atoms) {
  if (ntok < 16 || ntok > 256 || ntok % 16 || stages < 1 || cluster < 1 || m < 1 || warpgroups < 1 || warpgroups > 4 ||
      !gemm_tile_rows_ok(pair, tile_rows) || k_atoms < 1 || k_atoms > 8)
    return -1;
  return muse::gemm_tc_smem_bytes(ntok, pair, stages, cluster, m, warpgroups, tile_rows, k_atoms);
}

int muse_gemm_tc_max_clusters(int ntok, int pair, int stages, int cluster, int m, int warpgroups, int tile_rows, int k_atoms) {
  if (!gemm_tile_rows_ok(pair, tile_rows)) return -1;
  return muse::gemm_tc_max_clusters(ntok, pair, stages, cluster, m, warpgroups, tile_rows, k_atoms);
}

long long muse_gemm_tc_ws_floats(int m, int n, int ntok, int pair, int split, int tile_rows) {
  if (m < 1 || n < 1 || ntok < 16 || ntok > 256 || ntok % 16 || split < 1 || !gemm_tile_rows_ok(pair, tile_rows)) return -1;
  return muse::gemm_tc_ws_floats(m, n, ntok, pair, split, tile_rows);
}
int muse_gemm_tc_cnt_ints(int m, int n, int ntok, int pair, int split, int tile_rows) {
  if (m < 1 || n < 1 || ntok < 16 || ntok > 256 || ntok % 16 || split < 1 || !gemm_tile_rows_ok(pair, tile_rows)) return -1;
  return muse::gemm_tc_cnt_ints(m, n, ntok, pair, split, tile_rows);
}

int muse_gemm_tc(const void* tmap_w, const void* x, void* out, float* ws, int* cnt, int* status, int m, int n, int k, int ld_x,
                 int ld_out, int ntok, int pair, int cluster, int split, int stages, int warpgroups, int tile_rows, int k_atoms,
                 const muse_peer_sync_t* peers, void* stream) {
  if (!tmap_w || !x) return -1;
  if (ld_x < k || ld_x % 8 != 0) return -2;
  if (ntok < 16 || ntok > 256 || ntok % 16) return -7;
  CUtensorMap tx;   // x moves between calls: its map is encoded per call and rides in the kernel parameters
  const int r = muse::encode_2d(&tx, x, m, k, static_cast<long long>(ld_x) * 2, ntok);
  if (r != 0) return r;
  CUtensorMap tw;
  memcpy(&tw, tmap_w, sizeof(tw));
  return muse::gemm_tc_dispatch(&tw, &tx, out, ws, cnt, status, m, n, k, ld_out, ntok, pair, cluster, split, stages, warpgroups, tile_rows, k_atoms,
                                reinterpret_cast<const muse::PeerSync*>(peers), static_cast<cudaStream_t>(stream));
}

long long muse_static_scratch_floats(void) { return muse::skinny_static_ws_floats(); }
int muse_static_scratch_tiles(void) { return muse::skinny_static_cnt_ints(); }

int muse_skinny_tc_noalloc(const void* tmap_w, const void* tmap_w_lo, const void* x, void* out, int* status, int m, int n,
                           int k, int ld_x, int ld_out, int ntok, int cluster, int groups, int stages, int out_is_f32,
                           void* stream) {
  if (!tmap_w || !x) return -1;
  if (ld_x < k || ld_x % 8 != 0) return -2;
  CUtensorMap tx;
  const int r = muse::encode_2d(&tx, x, m, k, static_cast<long long>(ld_x) * 2, ntok);
  if (r != 0) return r;
  CUtensorMap tw, twlo;
  memcpy(&tw, tmap_w, sizeof(tw));
  if (tmap_w_lo) memcpy(&twlo, tmap_w_lo, sizeof(twlo));
  return muse::skinny_tc_static_dispatch(&tw, tmap_w_lo ? &twlo : nullptr, &tx, out, status, m, n, k, ld_out, ntok,
                                         cluster, groups, stages, out_is_f32, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
