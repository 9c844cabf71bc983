/* C ABI of libmuse_proj.so: the sm_100a kernels behind the `muse_bf16_proj` hot path
 * (out = x @ W[:n].T for the qkv_gate / o / pooler / unpooler BF16 weights and the FP32 router).
 *
 * Conventions: every pointer named W, x, out, ws, cnt, status is a DEVICE pointer on the current
 * CUDA device; `stream` is a cudaStream_t passed as void*; tensor maps are 128-byte HOST blobs
 * (CUtensorMap) filled by muse_tmap_encode_2d. Every entry point returns 0 on success, a negative
 * value for an argument it rejects (nothing was launched) or a positive cudaError_t / CUresult.
 * Nothing here allocates device memory or synchronises; launches go to `stream` and can be
 * captured in a CUDA graph. Thread-compatible: concurrent calls are fine as long as they do not
 * share a workspace (ws / cnt), which belongs to one stream at a time. The first launch of a kernel
 * variant on a device sets that variant's function attributes (shared-memory opt-in, cluster size) and
 * caches a few device facts without locking: make the first call of each shape from one thread (a
 * warm-up pass, as prepare() of the Python host does) before calling from several.
 *
 * The reference for this path is a Python submission (best_submissions/muse_bf16_proj.py) whose
 * native boundary is a pybind function around gemv1_launch (bf16_proj/gemv1.cu:122-125) plus Triton
 * launchers; each entry point cites what it replaces.
 */
#ifndef MUSE_PROJ_H
#define MUSE_PROJ_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MUSE_PROJ_ABI_VERSION 18

/* Bits a kernel may OR into its status word when one of its bounded waits gives up. */
#define MUSE_ST_PRODUCER_TIMEOUT 1
#define MUSE_ST_MMA_TIMEOUT 2
#define MUSE_ST_EPILOGUE_TIMEOUT 4
#define MUSE_ST_X_TIMEOUT 8
#define MUSE_ST_DRAIN_TIMEOUT 16
#define MUSE_ST_PEER_ENTER_TIMEOUT 32
#define MUSE_ST_PEER_DONE_TIMEOUT 64

/* Column-parallel output exchange (optional last-but-one argument of muse_gemv1 / muse_skinny_tc;
 * NULL or world <= 1 = single GPU). The weight is sharded by output rows over `world` GPUs of one
 * node, one process per GPU. With this descriptor the kernel ignores its `out` argument and stores
 * its [m, n] slice at columns [col0, col0 + n) of EVERY rank's gathered output out[p] (row stride
 * ld_out, the same on all ranks) through peer-mapped pointers, then exchanges flags with the peers,
 * so that when the kernel completes the local out[rank] holds every rank's slice: the all-gather
 * is part of the kernel. out[p] and flags[p] are device pointers valid in THIS process (peer-mapped
 * memory, e.g. torch symmetric memory or CUDA IPC); flags[p] is rank p's array of 32 ints, zero
 * before the first call and owned by these kernels afterwards. All ranks must make the same sequence
 * of calls. Waits on peers are bounded (status bits above). Plain peer stores only: no multimem,
 * no TMA to or from peer memory. No counterpart in the reference, which runs on one GPU and leaves
 * the all-gather out (bf16_proj/baseline.py:11).
 *
 * muse_fewtok_mma exchanges differently (m <= MUSE_LL_TOKENS): it never writes into a peer's gathered
 * output. Every CTA sends its rows to each peer's staging area ll[p] as 16-byte lines
 * {data, call number, data, call number} -- 8 bytes of payload that validate themselves, so no fence
 * and no flag follow them -- and finishes by unpacking the lines the peers sent it into its own
 * out[rank], polling each line until it carries this call's number. ll[p] is rank p's zeroed staging
 * of 2 x world x MUSE_LL_TOKENS x n x 4 bytes (n = the slice width; two halves used by odd and even
 * calls, then one block per sending rank), peer-mapped like out[p]; it may be NULL when
 * muse_fewtok_mma is not used column-parallel. */
#define MUSE_MAX_WORLD 8
#define MUSE_LL_TOKENS 32
typedef struct muse_peer_sync {
  int world, rank, col0, reserved;
  void* out[MUSE_MAX_WORLD];
  int* flags[MUSE_MAX_WORLD];
  void* ll[MUSE_MAX_WORLD];
} muse_peer_sync_t;

/* ABI version of the loaded library (MUSE_PROJ_ABI_VERSION at build time). */
int muse_abi_version(void);

/* Programmatic dependent launch (on by default). The launches of every projection kernel (GEMV, register-MMA
 * walks, TMEM kernels, the fused boundary kernels; column- and row-parallel forms included) carry cudaLaunchAttributeProgrammaticStreamSerialization: such a kernel may become resident while the
 * kernel ahead of it in the stream is still running, and until its griddepcontrol.wait it touches only the weights
 * (which no kernel writes): its launch latency, set-up and first weight loads run under the previous kernel's tail;
 * activations, outputs, workspaces and the status word are touched only after every kernel ahead has completed.
 * Stream order is unchanged for the caller, also under stream capture (the graph gets a programmatic edge).
 * What this asks of the caller: a weight (and its hi / lo halves, 12-bit planes and tables) must not be the output
 * of work still in flight on the stream when a projection is launched; weights are static, so one synchronisation
 * after loading them is enough (the Python prepare() does it).
 * muse_set_programmatic_launch(0) makes every launch an ordinary one; returns the previous setting. Process-wide:
 * set it before launching from several threads. */
int muse_set_programmatic_launch(int enabled);

/* Device facts the host-side planner needs. what: 0 = SM count, 1 = opt-in shared memory per
 * block (bytes), 2 = compute capability major*10+minor, 3 = L2 size (bytes). Negative on error.
 * Replaces nothing in the reference (its configs are hard-coded for one H200,
 * best_submissions/muse_bf16_proj.py:56-62, :205-212). */
int muse_query(int what);

/* y[N] = W[N,K] . x[K], one token. W BF16 (out BF16) or FP32 when w_is_f32 (out FP32); x BF16,
 * 16-byte aligned; K % 8 == 0; wpr in {1,2,4,8} warps share a row, K % wpr == 0 and each K / wpr
 * segment a whole number of 16-byte vectors; unroll in {1,2,4,8} 16-byte loads in flight per lane
 * per batch. persistent != 0 (wpr must be 1): a grid that is resident all at once, each warp
 * walking rows g, g + G, ... with its loads double-buffered across row boundaries (tall weights).
 * Replaces gemv1_launch (bf16_proj/gemv1.cu:122-125; pybind wrapper
 * best_submissions/muse_bf16_proj.py:193-196). */
int muse_gemv1(const void* W, const void* x, void* out, int N, int K, int w_is_f32, int wpr, int unroll, int persistent,
               int* status, const muse_peer_sync_t* peers, void* stream);

/* out[m, N] = x[m, K] . W[N, K]^T for m = 1..16 * tok_split tokens against a BF16 weight, as a persistent
 * streaming walk over W with register-level tensor-core MMAs (no tensor memory, no split-K
 * workspace, bit-reproducible): the regime between muse_gemv1 and muse_skinny_tc. K % 32 == 0; x BF16 with ld_x
 * elements between rows (multiple of 8, 16-byte aligned base), out BF16 with ld_out elements
 * between rows; warps in {16, 32} per CTA, unroll in {1, 2, 4} (8 with 16 warps when K <= 4096).
 * When warps * unroll * 32 >= K the kernel keeps its x fragments in registers; only then may
 * tok_split be 2..4: the grid is that many interleaved copies of the walk, each multiplying its own
 * block of 8 or 16 tokens, and W is read from HBM once and a second time from L2. Otherwise
 * tok_split = 1. `peers` (NULL on one GPU) makes the call column-parallel (the self-validating
 * lines described at muse_peer_sync_t): only the register-resident form, m <= MUSE_LL_TOKENS,
 * N % 8 == 0 and col0 % 8 == 0 (-8 otherwise). Serves the smallest of the m <= 32
 * calls that the reference gives to _swab / _swab_kernel (best_submissions/muse_bf16_proj.py:323-337,
 * :236-257). -5 = x does not fit in shared memory (muse_fewtok_smem_bytes > 227 KB). */
int muse_fewtok_mma(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out, int warps,
                    int unroll, int tok_split, int* status, const muse_peer_sync_t* peers, void* stream);
long long muse_fewtok_smem_bytes(int m, int K, int warps);

/* Row-parallel form of muse_fewtok_mma for m = 1..MUSE_RP_TOKENS tokens: W [N, K] and x [m, K] are THIS RANK's
 * slice of the reduction dimension (the reference's tensor-parallel layout of the `o` projection,
 * bf16_proj/reference.py:17, whose all-reduce is the identity on its single GPU,
 * decode_layer/reference.py:451), and out[m, N] (BF16, in this rank's own memory) = the sum over all ranks.
 * The all-reduce is part of the kernel, one NVLink flight: every CTA sends its FP32 partial sums to every
 * rank's staging (its own included) as 16-byte lines {sum, call number, sum, call number} and, once its row
 * groups are done, adds up the lines of all ranks for those groups in rank order (every rank ends with the
 * same bits). Of `peers` the fields world, rank, flags[] and ll[] are used: ll[p] is rank p's zeroed staging
 * of 2 x world x MUSE_RP_TOKENS x N x 8 bytes, peer-mapped; out[] is ignored. K <= 4096, K % 32 == 0,
 * N % 8 == 0. All ranks must make the same sequence of calls; the wait for a peer's lines is bounded
 * (MUSE_ST_PEER_DONE_TIMEOUT). No counterpart in the reference beyond the layout it names. */
#define MUSE_RP_TOKENS 8
int muse_fewtok_rowpar(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out, int* status,
                       const muse_peer_sync_t* peers, void* stream);

/* The same walk over an FP32 weight with FP32 output (the MoE router) for m = 1..8 * tok_split tokens:
 * the kernel reads W as FP32 once and splits every element in registers into BF16 hi = bf16(w) and
 * lo = bf16(w - hi), both multiplied into one FP32 accumulator -- the arithmetic of the reference's
 * prepare() split and _router_kernel (best_submissions/muse_bf16_proj.py:346-349, :260-287) without
 * the pre-split copies. 16 warps per CTA, unroll in {2, 4, 8} with K <= 512 * unroll (x stays in
 * registers), K % 32 == 0; x BF16, or FP32 when x_is_f32: the FP32-input mode of the reference's decode
 * layer (X_F32, best_submissions/muse_decode_layer.py:165-200), x split like the weight and
 * out = x_hi (hi + lo) + x_lo hi. ld_x counts elements of x's type, ld_x % 8 == 0. */
int muse_fewtok_f32(const void* W, const void* x, void* out, int m, int N, int K, int ld_x, int ld_out, int unroll,
                    int tok_split, int x_is_f32, void* stream);

/* The post-FFN boundary of the reference's decode layer, the consumer of the unpooler's output
 * (_ffn_boundary_kernel, best_submissions/muse_decode_layer.py:715-730; decode_layer/reference.py:466-476), per
 * token over the hidden width d, f being the unpooler's output of nf <= d columns (zero beyond: up to 8 tokens a
 * GPU computes only its slice):
 *     f'      = f * (1 + post_w)
 *     stream2 = alpha * stream1 + beta * f' * rsqrt(mean(f'^2) + 1e-8)
 *     hidden  = stream2 * rsqrt(mean(stream2^2) + 1e-5) * (1 + next_w)         (the next layer's attention input)
 * stream1, stream2: FP32 [m, d]; hidden: BF16 [m, d]; alpha, beta: FP32 [d]; post_w, next_w: BF16 [d]. All
 * contiguous, 16-byte aligned; d % 8 == 0, d <= 8192, nf % 8 == 0. */
typedef struct muse_ffn_boundary {
  const float* stream1;
  const float* alpha;
  const float* beta;
  const void* post_w;
  const void* next_w;
  float* stream2;   /* output, may be NULL */
  void* hidden;     /* output */
} muse_ffn_boundary_t;
/* Stand-alone: one CTA per token, f BF16 [m, nf] contiguous (the projection's output). */
int muse_ffn_boundary(const muse_ffn_boundary_t* bd, const void* f, int m, int d, int nf, void* stream);
/* The unpooler projection and the boundary as ONE launch (lines 869-877 of the reference's layer, two launches
 * there): f = x . W[nf, K]^T by the register-MMA walk of muse_fewtok_mma, kept in FP32 in f_scratch [m, nf]; every
 * CTA counts itself done and CTA t < m then computes token t after a bounded wait for the count. m <= 8,
 * K <= 4096, K % 32 == 0, nf >= 8 m. cnt: 2 ints in device memory, zero before the first call and left zero by
 * every call (one per stream that may run such calls at once, and a scratch each). `status`: ST_X_TIMEOUT if the
 * count never completed. */
int muse_unpooler_ffn_boundary(const void* W, const void* x, void* f_scratch, const muse_ffn_boundary_t* bd, int m, int nf, int K, int ld_x,
                               int d, int* cnt, int* status, void* stream);

/* out[m, N] = x . W^T for 1..8 tokens with W in the LOSSLESS 12-bit form of the reference author's experiment
 * (bf16_proj/probe18.py:332-362 `_zip`; 25 % fewer bytes): `low` uint8 [N, K] raw low bytes, `code` uint8 [N, K/2]
 * 4-bit codes (sign, index of the high byte in the 8-value window starting at `base`), `table` int32
 * [ceil(N/8), cap, 2] = {row in group << 16 | column, FP32 bits of the true weight} for the weights outside the
 * window ({-1, 0} = unused, last; cap <= 64, NULL when cap == 0), in the lane-major layouts that
 * llm_inference_engine_b200/zip12.py documents and builds. The register-MMA walk of muse_fewtok_mma with the
 * decode in registers: the same MMAs on the same BF16 values, plus x * true - x * coded in FP32 for the listed
 * weights. K % 128 == 0, K <= 32 * warps * unroll, (warps, unroll) in {(32, 4), (16, 8), (16, 4)}, reduce_every = 1 or
 * 2 row groups per CTA-wide reduction. No waits (x is read with plain loads): no status word. */
int muse_fewtok_zip(const void* low, const void* code, const void* table, int cap, int base, const void* x, void* out, int m, int N,
                    int K, int ld_x, int ld_out, int warps, int unroll, int reduce_every, void* stream);

/* The post-attention boundary of the reference's decode layer, the producer of the pooler's and the router's
 * input (_attn_boundary_kernel, best_submissions/muse_decode_layer.py:694-712; decode_layer/reference.py:452-454),
 * per token over the hidden width d:
 *     stream1 = alpha * stream + beta * attn_out * rsqrt(mean(attn_out^2) + 1e-8)
 *     h       = stream1 * rsqrt(mean(stream1^2) + 1e-5) * (1 + norm_w)
 * stream, stream1, h_f32: FP32 [m, d]; attn_out, h: BF16 [m, d]; alpha, beta: FP32 [d] (the residual
 * coefficients of the gate); norm_w: BF16 [d]. All contiguous, 16-byte aligned, d % 8 == 0. */
typedef struct muse_boundary {
  const float* stream;
  const void* attn_out;
  const float* alpha;
  const float* beta;
  const void* norm_w;
  float* stream1;   /* outputs: any of the three may be NULL (not written) */
  void* h;
  float* h_f32;
} muse_boundary_t;
/* Stand-alone: one CTA per token, d <= 8192, at least one output. */
int muse_attn_boundary(const muse_boundary_t* bd, int m, int d, void* stream);
/* Fused: out[m, N] = h . W[N, K]^T with the boundary as the projection's prologue instead of a kernel of its
 * own (K = d <= 4096, K % 32 == 0, m <= 8, N >= 8 m): the register-MMA walk of muse_fewtok_mma (16 warps x 8
 * loads), where every CTA rebuilds h in shared memory while its first weight loads are in flight and takes its
 * x fragments from there; CTA t also writes token t's stream1 / h / h_f32 where those pointers are given.
 * w_is_f32 = 0: BF16 W, h rounded to BF16 as the MMA input, BF16 out (the pooler; `status` as for
 * muse_fewtok_mma). w_is_f32 != 0: FP32 W and out, h kept FP32 and split to BF16 hi + lo like the weight (the
 * router's FP32-input mode, muse_fewtok_f32 with x_is_f32). */
int muse_fewtok_boundary(const void* W, int w_is_f32, const muse_boundary_t* bd, void* out, int m, int N, int K, int ld_out,
                         int* status, void* stream);
/* The whole stretch between the `o` projection and the experts as ONE launch (the boundary, the pooler and the
 * router of best_submissions/muse_decode_layer.py:855-869, three launches on two streams there): one CTA per
 * token computes its boundary once and publishes stream1 (where given), h (REQUIRED: the BF16 h, which is also
 * the high half of the FP32 h), h_lo (REQUIRED scratch, BF16 [m, K]: bf16(h_fp32 - h)) and h_f32 (where given);
 * every CTA waits for the m tokens with a bounded wait, then most CTAs walk the pooler's BF16 rows with h and the
 * others the router's rows with h + h_lo against the router weight's BF16 hi + lo halves (W_router_hi / _lo:
 * hi = bf16(W), lo = bf16(W - hi), as muse_skinny_tc takes them): x_hi W_hi + x_hi W_lo + x_lo W_hi, the sums
 * muse_fewtok_f32 forms in its FP32-input mode. out_pooler: BF16 [m, n_pooler]; out_router: FP32 [m, n_router];
 * m <= 8, K = d <= 4096, K % 32 == 0, n_pooler >= 8 m. cnt: 9 ints in device memory, zero before the first call
 * and left zero by every call (calls that may overlap on the GPU need one each, and an h_lo each). `status`:
 * ST_X_TIMEOUT if a token never arrived. */
int muse_boundary_pooler_router(const void* W_pooler, const void* W_router_hi, const void* W_router_lo, const muse_boundary_t* bd,
                                void* h_lo, void* out_pooler, void* out_router, int m, int n_pooler, int n_router, int K,
                                int ld_out_pooler, int ld_out_router, int* cnt, int* status, void* stream);

/* Staging for callers whose activations live in HOST memory (page-locked for the copies to be
 * asynchronous): x goes host -> device on `stream` before the projection is launched there, and
 * muse_copy_d2h_sync brings the result back and returns once it has landed (it synchronises the
 * stream). Positive = CUDA error. No counterpart in the reference, whose harness hands kernel_fn
 * device tensors (best_submissions/muse_bf16_proj.py:369-372). */
int muse_copy_h2d_async(void* dst_device, const void* src_host, long long bytes, void* stream);
/* The same copy-in done by a small kernel that reads the page-locked host buffer directly (it must be
 * device-addressable: cudaHostAlloc / cudaHostRegister memory under unified addressing); bytes a
 * multiple of 16, both pointers 16-byte aligned. For a few KB the consumer then waits on a
 * kernel-to-kernel dependency instead of a copy-engine hand-off. The kernel is a plain 16-byte copy,
 * so with the pointers swapped (destination in page-locked host memory) it is the copy-out as well. */
int muse_fetch_host(void* dst_device, const void* src_host, long long bytes, void* stream);
int muse_copy_d2h_sync(void* dst_host, const void* src_device, long long bytes, void* stream);
/* The whole round trip of one muse_fewtok_mma call in one entry: x_host [m, K] -> x_device, the
 * kernel (contiguous x and out), out_device [m, N] -> out_host, stream synchronised. */
int muse_fewtok_mma_host(const void* W, const void* x_host, void* x_device, void* out_device, void* out_host, int m, int N,
                         int K, int warps, int unroll, int tok_split, int* status, void* stream);

/* Fill a 128-byte tensor map for a row-major BF16 matrix [rows, cols] at `base` (device pointer,
 * 16-byte aligned) with `row_stride_bytes` between rows (multiple of 16), delivering boxes of
 * [box_rows, 64 columns] with the 128-byte shared-memory swizzle and zero fill outside the matrix.
 * Replaces TensorDescriptor.from_tensor (best_submissions/muse_bf16_proj.py:334, :357). */
int muse_tmap_encode_2d(void* tmap_out128, const void* base, long long rows, long long cols,
                        long long row_stride_bytes, int box_rows);

/* Floats of workspace and ints of counters muse_skinny_tc needs for (m, n, ntok) when split > 1.
 * Replaces the capacity rule of _workspace (best_submissions/muse_bf16_proj.py:302-307). */
long long muse_skinny_ws_floats(int m, int n, int ntok);
int muse_skinny_tiles(int m, int n, int ntok);

/* Bytes of shared memory one pipeline stage takes (W box [+ lo box] + x box), and the dynamic shared
 * memory a launch with `stages` stages asks for (the ring, or the parked accumulator if larger). */
int muse_skinny_stage_bytes(int ntok, int hilo);
int muse_skinny_smem_bytes(int ntok, int hilo, int stages, int cluster, int m);

/* How many thread-block clusters of `cluster` CTAs of this launch shape the current device can hold
 * at once (0: the shape does not fit; negative: bad argument). The planner keeps a launch within one
 * wave with it. No counterpart in the reference. */
int muse_skinny_max_clusters(int ntok, int hilo, int m, int stages, int cluster);

/* out[m, n] = x[m, K] . W[n, K]^T through TMA + tcgen05 (swap-AB, split-K = cluster x groups).
 *   tmap_w      tensor map of W[:n] with box_rows = 128 (muse_tmap_encode_2d)
 *   tmap_w_lo   NULL for a BF16 weight; for the router the map of the "lo" half, in which case
 *               tmap_w is the "hi" half and both accumulate into one FP32 accumulator
 *   x           BF16 [m, K], 16-byte aligned, ld_x elements between rows (ld_x % 8 == 0)
 *   out         BF16, or FP32 when out_is_f32; ld_out elements between token rows (>= n)
 *   ws, cnt     zeroed workspace (muse_skinny_ws_floats floats) and counters (muse_skinny_tiles
 *               ints); left zeroed again when the kernel finishes; may be NULL when groups == 1
 *   ntok        tokens per tile = MMA N: 16, 32, 64, 128 or 256
 *   cluster     K slices reduced on chip: CTAs per thread-block cluster (1 .. 16), summed through
 *               distributed shared memory in a fixed order
 *   groups      clusters per tile (>= 1); their sums meet in ws through FP32 atomics, so results are
 *               bit-reproducible only when groups == 1. cluster * groups <= ceil(K/64)
 *   stages      pipeline depth 1 .. 12
 * Replaces _swab / _swab_kernel (best_submissions/muse_bf16_proj.py:323-337, :236-257), _router /
 * _router_kernel (:310-320, :260-287), _finish (:215-233) and the cuBLAS call for m > 32 (:390). */
int muse_skinny_tc(const void* tmap_w, const void* tmap_w_lo, const void* x, void* out, float* ws, int* cnt,
                   int* status, int m, int n, int k, int ld_x, int ld_out, int ntok, int cluster, int groups, int stages,
                   int out_is_f32, const muse_peer_sync_t* peers, void* stream);

/* out[m, n] = x[m, K] . W[n, K]^T, BF16 out, for many tokens (the m > 32 GEMM): TMA + tcgen05 as in
 * muse_skinny_tc, but a CTA multiplies a PAIR of 128-row weight tiles (pair != 0) against one copy of the
 * x chunk (two accumulators in tensor memory), which halves the L2 -> shared-memory traffic that bounds
 * these shapes; pair == 0 keeps one tile per CTA (small weights: more CTAs).
 *   tmap_w   tensor map of W[:n] with box_rows = tile_rows (muse_tmap_encode_2d)
 *   tile_rows  weight rows per CTA when pair == 0: a multiple of 8 up to 128 (must be 128 with pair). A short
 *            tile lets a weight of any height fill the SMs in one wave without any K split (12288 rows = 140
 *            CTAs of 88): the MMA stays M = 128 and the surplus accumulator lanes are not read. For few tokens.
 *   x, out   as for muse_skinny_tc; out is BF16
 *   ntok     tokens per tile = MMA N: any multiple of 16 up to 256 (m > ntok runs ceil(m / ntok) token tiles)
 *   cluster  K slices as the CTAs of one thread-block cluster (1 .. 16), summed through distributed shared
 *            memory; no workspace
 *   split    K slices as independent CTAs (1 .. 64) that exchange their partial sums through `ws` (plain
 *            16-byte stores and loads that stay in L2, no atomics) and count themselves in and out on `cnt`;
 *            they wait for one another, so the whole grid must be resident at once: row units x split x token
 *            tiles <= SM count (-10 otherwise). One of cluster, split must be 1; cluster * split <= ceil(K / 64).
 *            Either way the sum has a fixed order: bit-reproducible.
 *   ws, cnt  for split > 1: muse_gemm_tc_ws_floats floats (16-byte aligned, contents irrelevant) and
 *            muse_gemm_tc_cnt_ints counters, zero before the first call and left zero; else may be NULL
 *   stages   pipeline depth 1 .. 12
 *   k_atoms  64-wide pieces of K per pipeline stage, 1 .. 8 (each its own 128-byte-swizzled TMA box): one step then
 *            asks DRAM for k_atoms x 128 contiguous bytes of every weight row. K slices are whole steps:
 *            cluster * split <= ceil(ceil(K / 64) / k_atoms)
 *   warpgroups  1 .. 4: CTA size in units of 128 threads; all of them read the accumulators out, push and store
 * One CTA per SM (the launch asks for at least 116 KB of shared memory). muse_gemm_tc_smem_bytes = the
 * dynamic shared memory of a launch; muse_gemm_tc_max_clusters = how many of its clusters the current
 * device holds at once (0: does not fit). Replaces the cuBLAS call x @ W[:n].T of
 * best_submissions/muse_bf16_proj.py:390. */
int muse_gemm_tc_smem_bytes(int ntok, int pair, int stages, int cluster, int m, int warpgroups, int tile_rows, int k_atoms);
int muse_gemm_tc_max_clusters(int ntok, int pair, int stages, int cluster, int m, int warpgroups, int tile_rows, int k_atoms);
long long muse_gemm_tc_ws_floats(int m, int n, int ntok, int pair, int split, int tile_rows);
int muse_gemm_tc_cnt_ints(int m, int n, int ntok, int pair, int split, int tile_rows);
int muse_gemm_tc(const void* tmap_w, const void* x, void* out, float* ws, int* cnt, int* status, int m, int n, int k, int ld_x,
                 int ld_out, int ntok, int pair, int cluster, int split, int stages, int warpgroups, int tile_rows, int k_atoms,
                 const muse_peer_sync_t* peers, void* stream);

/* muse_skinny_tc for callers that must not allocate device memory (a server whose pool owns all of
 * HBM and bans cudaMalloc after start-up, a plug-in slot that passes inputs and outputs only). No
 * counterpart in the reference. The split-K scratch is a fixed array inside the library, present on every
 * GPU that loads it until the process exits: muse_static_scratch_floats() floats (1 Mi = 4 MiB) and
 * muse_static_scratch_tiles() counters (4096). A launch with groups > 1 needs
 * muse_skinny_ws_floats(m, n, ntok) floats and muse_skinny_tiles(m, n, ntok) counters; more than the
 * array holds is refused with MUSE_ERR_STATIC_SCRATCH. groups == 1 uses no scratch and runs at any size.
 * Every argument is checked before anything reaches the stream; the entry point calls no cudaMalloc,
 * cudaFree or allocating library routine. The first call on a device looks up the array's address
 * (once per device, that device current): make it outside a stream capture, and not concurrently with
 * another first call. All calls share the array, which keeps the last call's contents: with groups > 1
 * the part about to be used is cleared on the stream before the kernel. Calls that can overlap on the
 * GPU race on it: order them, or give one its own workspace through muse_skinny_tc. */
#define MUSE_ERR_STATIC_SCRATCH (-20)
long long muse_static_scratch_floats(void);
int muse_static_scratch_tiles(void);
int muse_skinny_tc_noalloc(const void* tmap_w, const void* tmap_w_lo, const void* x, void* out, int* status, int m, int n,
                           int k, int ld_x, int ld_out, int ntok, int cluster, int groups, int stages, int out_is_f32,
                           void* stream);

/* Launches an empty kernel on `stream`: the calibration point for the fixed cost of replaying a
 * one-kernel CUDA graph, which the benchmark reports beside every per-call time. Replaces the `nop`
 * graph of the reference's timing harness (bf16_proj/tune.py:79-98). */
int muse_nop(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MUSE_PROJ_H */
