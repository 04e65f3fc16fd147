// C ABI of the sm_100a kernel library.  Every function takes raw device pointers and
// a CUDA stream (as void*), launches asynchronously, allocates nothing unless stated,
// and returns a cudaError_t value as int (0 = launched).  Device-side problems
// (expired waits, failed bounds checks) are reported through the caller's 4-int
// `status` block: {code, kernel id, detail, observed value}; see common.cuh.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GEEPS_MAX_RANKS 8

enum GeepsTableMode { GEEPS_TABLE_ADDITIVE = 0, GEEPS_TABLE_SGD_MOMENTUM = 1 };

// ---------------- row ops (row = 128 fp32) ----------------
// index: array of {int64 id0, int64 id1} pairs ("double index": id0 = position in the
// application buffer, id1 = position in the cache / oplog).
int geeps_row_gather(float* dst, const float* src, const void* index, long long num_rows,
                     long long dst_off, long long src_off, long long num_vals_limit,
                     long long dst_rows, long long src_rows, int* status, void* stream);
int geeps_row_scatter(float* dst, const float* src, const void* index, long long num_rows,
                      long long dst_off, long long src_off, long long num_vals_limit,
                      long long dst_rows, long long src_rows, int* status, void* stream);
int geeps_row_scatter_add(float* dst, const float* src, const void* index, long long num_rows,
                          long long dst_off, long long src_off, long long num_vals_limit,
                          long long dst_rows, long long src_rows, int* status, void* stream);
// scatter-add with a scale: dst[id1 + dst_off] += alpha * src[id0 + src_off]
int geeps_row_scatter_axpy(float* dst, const float* src, const void* index, long long num_rows,
                           long long dst_off, long long src_off, long long num_vals_limit,
                           long long dst_rows, long long src_rows, float alpha, int* status, void* stream);
int geeps_axpy(float* y, const float* x, float alpha, long long n, void* stream);

// ---------------- parameter-server fabric ----------------
typedef struct GeepsPushApplyParams {
  const float* upd[GEEPS_MAX_RANKS];   // each worker's update buffer (full-table layout)
  float* cache[GEEPS_MAX_RANKS];       // each worker's fp32 parameter cache (full table) or NULL
  void* cache16[GEEPS_MAX_RANKS];      // each worker's bf16 compute copy (full table) or NULL
  int* data_age[GEEPS_MAX_RANKS];      // each worker's data_age[n_ranks] flag array or NULL
  float* master;                       // this shard's rows, compact [n_owned][128]
  float* momentum;                     // same shape; SGD tables only
  const int* push_ready;               // local flags [n_ranks] written by the workers, or NULL
  int* global_clock;                   // local flag: this shard applied clock_stamp (may be NULL)
  int* cta_counter;                    // one zero-initialised int of scratch
  int* status;                         // 4 ints or NULL
  long long n_owned, row_start, row_stride, total_rows;
  unsigned long long wait_budget_ns;
  int n_ranks, rank, clock_stamp, mode, publish;
  float lr, momentum_coef, weight_decay, grad_scale;
  long long fp32_from_row;             // rows below this id are published to the bf16 caches only (0: all in fp32 too)
  const int* clock_ref;                // NULL, or a device word added to clock_stamp when the kernel runs (stamps
                                       // relative to a device-resident clock: launches that a CUDA graph replays)
  void* master16;                      // NULL, or this shard's bf16 copy of its master rows, compact [n_owned][128]
                                       // (uncached tables: consumers read it in place over NVLink)
  // NVSwitch multicast view (all NULL: peer loads / stores).  upd_mc: the update buffer as seen through the
  // multicast mapping - one multimem.ld_reduce returns the sum over all workers, added inside the switch, instead
  // of one load per worker; cache_mc / cache16_mc: the caches through the mapping - one multimem.st publishes to
  // every worker instead of one store per worker.  Same table layout as upd / cache / cache16.
  const float* upd_mc;
  float* cache_mc;
  void* cache16_mc;
} GeepsPushApplyParams;
int geeps_ps_push_apply(const GeepsPushApplyParams* p, int max_ctas, void* stream);

typedef struct GeepsPullParams {
  const float* master[GEEPS_MAX_RANKS];  // each shard's compact master rows (peer pointers)
  const int* global_clock[GEEPS_MAX_RANKS];  // each shard's applied-clock flag or NULL (no wait)
  long long n_owned[GEEPS_MAX_RANKS], row_start[GEEPS_MAX_RANKS], row_stride[GEEPS_MAX_RANKS];
  float* cache;        // local fp32 cache or NULL
  void* cache16;       // local bf16 copy or NULL
  int* data_age_local; // local data_age[n_ranks] or NULL
  int* cta_counter;
  int* status;
  long long total_rows;
  unsigned long long wait_budget_ns;
  int n_ranks, rank, needed_stamp;
  long long row_from;  // only rows with id >= row_from are copied (0: all); cache / cache16 are indexed by
                       // (row id - row_base), so a buffer that holds just the tail of a table can be filled
  long long row_base;
} GeepsPullParams;
int geeps_ps_pull(const GeepsPullParams* p, int max_ctas, void* stream);

typedef struct GeepsFlagList { int* ptr[GEEPS_MAX_RANKS]; int n; } GeepsFlagList;
int geeps_flag_signal(const GeepsFlagList* list, int index, int stamp, void* stream);
int geeps_flag_wait(const int* flags, int n, int stamp, unsigned long long budget_ns, int* status,
                    void* stream);
// wait as geeps_flag_wait, then write `stamp` into slot `index` of each array of `then` (skipped when the wait
// expired): the shard's "publish of this clock begins" mark on every worker
int geeps_flag_wait_signal(const int* flags, int n, int stamp, unsigned long long budget_ns, int* status,
                           const GeepsFlagList* then, int index, void* stream);
int geeps_f32_to_bf16(const float* src, void* dst, long long n, void* stream);
// Forms whose stamp is relative to a device-resident clock word: the kernel uses stamp_rel + *clock_ref.  With them
// a step's launches carry no per-step immediate, so the step can be captured once in a CUDA graph and replayed.
int geeps_flag_signal_rel(const GeepsFlagList* list, int index, int stamp_rel, const int* clock_ref, void* stream);
int geeps_flag_wait_rel(const int* flags, int n, int stamp_rel, const int* clock_ref, unsigned long long budget_ns,
                        int* status, void* stream);
int geeps_flag_wait_signal_rel(const int* flags, int n, int stamp_rel, const int* clock_ref,
                               unsigned long long budget_ns, int* status, const GeepsFlagList* then, int index,
                               void* stream);
// *clock += 1 (one thread), at the end of a step
int geeps_clock_advance(int* clock, void* stream);

// Read with read-my-updates on the NVLINK transport: dst[id0] = cache[id1] + alpha * (sum of this worker's own ring
// slots whose clock the owning shard has not published yet).  Per row the owning shard's data_age stamp is read
// before and its publish_begin stamp after the copy; if a publish started in between, the row is read again
// (bounded; an exhausted budget reports GEEPS_ERR_TIMEOUT).  ring holds ring_slots copies of the table
// ([slot][total_rows][128], slot of clock k = k % ring_slots); clock is the reader's clock.
typedef struct GeepsRmwReadParams {
  float* dst; const float* cache; const float* ring; const void* index;
  const int* data_age; const int* publish_begin;   // local flag arrays [n_ranks]
  int* status;
  long long num_rows, num_vals_limit, dst_rows, total_rows;
  unsigned long long wait_budget_ns;
  int n_ranks, partition_kind, ring_slots, clock;
  int additive_below_clock;   // own updates of clocks below this are added as they are (initial values), not scaled
  float alpha;
  const int* clock_ref;       // NULL, or a device word added to `clock` when the kernel runs
  long long partition_per;    // rows per shard of the range partition (0: ceil(total_rows / n_ranks))
} GeepsRmwReadParams;
int geeps_row_gather_rmw(const GeepsRmwReadParams* p, void* stream);

// ---------------- GEMM (bf16 x bf16 -> fp32 accumulate) ----------------
// C[M,N] = alpha * A[M,K] * B[N,K]^T + beta * C + bias, optional ReLU.
//   a_mn_major = 0: A is stored [M][lda] (K contiguous); 1: stored [K][lda] (M contiguous)
//   b_mn_major = 0: B is stored [N][ldb] (K contiguous); 1: stored [K][ldb] (N contiguous)
//   out_fp32   = 0: C is bf16; 1: C is fp32.   ldc in elements.
//   bias_mode  = 0 none, 1 bias[n], 2 bias[m] (fp32)
//   split_k > 1: partial sums are added into fp32 C with red.global.add (C must hold the
//                beta-scaled initial value already; relu is not applied).
typedef struct GeepsGemmParams {
  const void* A; const void* B; void* C; const float* bias;
  long long M, N, K, lda, ldb, ldc;
  float alpha, beta;
  int a_mn_major, b_mn_major, out_fp32, bias_mode, relu, split_k;
  int block_n;     // 0 = auto, else 64 / 128 / 256
  int* status;
} GeepsGemmParams;
int geeps_gemm_bf16(const GeepsGemmParams* p, void* stream);       // tcgen05 + TMA + TMEM
int geeps_gemm_bf16_simt(const GeepsGemmParams* p, void* stream);  // plain SIMT fallback / cross-check
int geeps_gemm_tc_supported(const GeepsGemmParams* p);             // 1 if the tcgen05 path accepts p
// CTA-pair variant (tcgen05 cta_group::2, 256-row tiles): K-major A and B, no split-K, beta == 0, M >= 256
int geeps_gemm_bf16_pair(const GeepsGemmParams* p, void* stream);
int geeps_gemm_pair_supported(const GeepsGemmParams* p);
// C[m][n] = beta * C[m][n] (exactly 0 when beta == 0) over an M x N view with pitch ldc
int geeps_scale_matrix_f32(float* c, long long M, long long N, long long ldc, float beta, void* stream);

// ---------------- implicit-GEMM convolution, stride 1 (tcgen05 + 4-D TMA, no patch matrix) ----------------
// NHWC bf16 activations: x is [B][H][W] pixels of x_pitch channels of which this call uses the cg channels
// starting at x; y likewise [B][OH][OW] x y_pitch with og channels; OH = H + 2 pad - KH + 1.
// w is [og][ldw] with column (kh * KW + kw) * cg + ci.
//   mode 0 forward:        y = conv(x, w) + bias, optional ReLU   (w bf16, ldw % 8 == 0)
//   mode 1 data gradient:  x = conv^T(y, w)                        (y holds dY, x receives dX)
//   mode 2 weight gradient: w = dY^T * patches(x), fp32            (w fp32, ldw % 4 == 0; split_k 0 = auto)
// Pointers 16-byte aligned; cg, og and the pitches multiples of 8.
typedef struct GeepsConvTcParams {
  void* x; void* y; void* w; const float* bias; int* status;
  long long x_pitch, y_pitch, ldw;
  int B, H, W, cg, OH, OW, og, KH, KW, pad, relu, mode, split_k;
  int stride;   // 0 or 1: stride 1; 2 .. 8: forward and weight gradient only (the activation boxes are loaded with
                // that TMA element stride), the data gradient of a strided layer is not an implicit GEMM here
} GeepsConvTcParams;
int geeps_conv_tc(const GeepsConvTcParams* p, void* stream);
int geeps_conv_tc_supported(const GeepsConvTcParams* p);
// Halo-tile variant for forward / data gradient (conv_halo.cu): every activation is fetched once per 64-channel
// chunk and the filter taps are shifted MMA-descriptor starts.  geeps_conv_tc() routes to it when applicable
// (a negative split_k on a forward / data-gradient call keeps the call on the box kernel).
int geeps_conv_halo_applicable(const GeepsConvTcParams* p);
int geeps_conv_halo(const GeepsConvTcParams* p, void* stream);
// Weight gradient with the taps of a filter row served by one activation tile (conv_wgrad_halo.cu); same routing.
int geeps_conv_wgrad_halo_applicable(const GeepsConvTcParams* p);
int geeps_conv_wgrad_halo(const GeepsConvTcParams* p, void* stream);
// The geometry the two halo kernels would use for a call (host arithmetic only; for tests and tuning).  `ok` = 0 when
// the kernel does not accept the call.
typedef struct GeepsHaloPlanInfo {
  int ok, routed;                       // accepted; geeps_conv_tc() would route the call to this kernel
  int PW, R, row_tiles, m_tiles;        // flat pitch, image rows per block, row tiles per image, channel blocks
  int positions, ncols2, ncols1;        // positions per block; MMA N of a two-block / one-block tile (forward, dgrad)
  int TY, passes, split, n_blocks;      // weight gradient: filter rows per item, passes, position slices, blocks
  int stages_x, stages_w, x_stage_bytes, tmem_cols;
  long long smem_bytes;
  double util;
} GeepsHaloPlanInfo;
int geeps_conv_halo_plan(const GeepsConvTcParams* p, GeepsHaloPlanInfo* out);
int geeps_conv_wgrad_halo_plan(const GeepsConvTcParams* p, GeepsHaloPlanInfo* out);

// ---------------- parameter pull fused with the consuming GEMM ----------------
// Y[M,N] = X[M,K] * W[N,K]^T + bias (+ReLU), M <= 256, K a multiple of 64.  W's rows live on the server
// shards: shard s holds rows [n_start[s], n_start[s+1]) (n_start[n_shards] = N) as bf16 at w_shard[s]
// (a peer pointer, row pitch ldw elements).  ready[s] (local int flag or NULL) must reach needed_stamp
// before shard s is read.  w_local (or NULL) receives a full local copy [N][ldw] of what was pulled.
typedef struct GeepsPullGemmParams {
  const void* X; void* Y; const float* bias;
  const void* w_shard[GEEPS_MAX_RANKS];
  const int* ready[GEEPS_MAX_RANKS];
  long long n_start[GEEPS_MAX_RANKS + 1];
  void* w_local;
  int* status;
  long long M, N, K, ldx, ldw, ldy;
  unsigned long long wait_budget_ns;
  int n_shards, needed_stamp, relu, out_fp32, block_n;
} GeepsPullGemmParams;
int geeps_pull_gemm_bf16(const GeepsPullGemmParams* p, void* stream);

#ifdef __cplusplus
}
#endif
