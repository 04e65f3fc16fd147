// Implicit-GEMM convolution (stride 1, forward and data gradient) that fetches every activation ONCE per
// 64-channel chunk instead of once per filter tap, and issues the widest MMA the tensor core has.
//
// conv_tc.cu loads, for each (tap, chunk) k-step, the 128-pixel activation box shifted by the tap: a 5 x 5 filter
// reads the same activations 25 times out of L2.  Here a tile is up to 256 CONSECUTIVE positions of the zero-padded
// image flattened with pitch PW = out_width + KW - 1:
//
//     out_flat[m] = sum over taps (ty, tx) and channels of  in_flat[m + ty * PW + tx] * W[tap]
//
// (positions whose column is >= out_width are computed and dropped).  One TMA box load brings the halo tile -
// [rows + KH - 1][PW][64 channels], zero-filled outside the image - into shared memory as exactly that flat array,
// 128 bytes per position with the 128-byte swizzle.  The operand of tap (ty, tx) is then the SAME tile read through
// an MMA descriptor whose start address is advanced by (ty * PW + tx) whole 128-byte rows.  Such a start is no longer
// 1024-byte aligned, and that is fine: the 128-byte swizzle is a function of the absolute shared-memory address bits
// (chunk bits 4..6 xor row bits 7..9), for the TMA write and for the MMA read alike, so the descriptor's base-offset
// field stays 0 (measured: with (address >> 7) & 7 in that field the products are wrong, with 0 they match the fp32
// reference).  Only the weights stream per tap.
//
// The product is computed transposed: D[channel, position] = W[channel, k] * X[position, k]^T, weights as the M = 128
// operand (128 output channels per tile; input channels for the data gradient), positions as N <= 256.  One thread
// issues every MMA and spends a few hundred cycles of instructions per pipeline stage (measured: the issue loop, not
// the tensor pipe or L2, bounded the first version of this kernel, which had positions as M = 128 and 48 .. 128
// channels as N), so every MMA must carry as much work as the instruction allows: 128 x 256 x 16.  The roles run
// their loops with the whole warp converged and elect one lane for the TMA / MMA / commit instructions.
//
// The accumulator therefore holds channels in TMEM lanes and positions in columns.  Each epilogue thread owns one
// channel: it adds that channel's bias (one register), applies ReLU and writes bf16 into a [position][64 channels]
// slab with the 128-byte swizzle - the 32 lanes of a warp write 64 contiguous bytes of one position per store - and
// a 4-D TMA store (64 channels, PW, rows, 1) writes the slab to the NHWC tensor, clipping the dropped columns, the
// rows past the image and the channels past the layer's extent.  A tile is two store blocks of Rb image rows; the
// pitch PW is padded until a block has a multiple of 8 positions, which makes the swizzled chunk offsets of a
// thread's channel constants; each block has its own pair of slabs; eight epilogue warps (two per TMEM lane quarter,
// alternate column groups) share the conversion.
//
// conv_tc() routes a forward / data-gradient call here when the geometry wastes little (see
// geeps_conv_halo_applicable); GEEPS_HALO_CONV=0 keeps every call on the box kernel.  Bounded waits and TMEM
// double buffering as in conv_tc.cu.
#include <cuda.h>
#include <cuda_bf16.h>
#include <mutex>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "kernels.h"
#include "tc05.cuh"

namespace {

constexpr int BM = 128;                       // channels per tile (TMEM lanes)
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int PANEL_BYTES = 64 * BK * 2;
constexpr int W_STAGE_BYTES = BM * BK * 2;    // 128 channels x 64 k (forward) or two [64 k][64 channels] panels (dgrad)
constexpr int MAX_X_STAGES = 2;
constexpr int MAX_W_STAGES = 8;
constexpr uint64_t WAIT_BUDGET_NS = 2000000000ull;
constexpr int C_SLAB_BYTES = 128 * 128;       // 128 positions x 64 channels bf16
constexpr int ACC_COLS = 256;
constexpr int kEpilogueWarps = 8;             // two per TMEM lane quarter: they take alternate column groups
constexpr int kThreads = 64 + 32 * kEpilogueWarps;

enum { MODE_FWD = 0, MODE_DGRAD = 1 };

struct HaloDev {
  const float* bias; int* status;
  int KH, KW, taps, cchunks, k_last;   // k_last: MMA k-substeps (of 16) in the last chunk (zero channels are skipped)
  int PW, Rb, px, py;                  // padded pitch, image rows per store block (two blocks per tile), halo left / top
  int split, ncols2, ncols1;           // positions per block (Rb * PW); MMA N for a tile of two blocks / one block
  int GH;                              // output rows of the image
  int row_tiles, m_tiles, n_images;    // tiles = m_tiles * n_images * row_tiles
  int n_valid;                         // channels produced
  int x_stage_bytes, stages_x, stages_w;
  int relu;
};

struct SmemCtl {
  uint64_t full_x[MAX_X_STAGES], empty_x[MAX_X_STAGES];
  uint64_t full_w[MAX_W_STAGES], empty_w[MAX_W_STAGES];
  uint64_t tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct Tile { int b, y0, nb, mi; };
__device__ __forceinline__ Tile decode_tile(const HaloDev& d, int t) {
  Tile q;
  const int per_m = d.n_images * d.row_tiles;
  q.mi = t / per_m;
  const int r = t - q.mi * per_m;
  q.b = r / d.row_tiles;
  q.y0 = (r - q.b * d.row_tiles) * (2 * d.Rb);
  q.nb = d.GH - q.y0 > d.Rb ? 2 : 1;
  return q;
}

// tmX: the source activations (fwd: X, dgrad: dY) as (c, w, h, b) with box (64, PW, 2 Rb + KH - 1, 1);
// tmW: weights (ci, tap, co): fwd box (64 ci, 1, 128 co) K-major, dgrad box (64 ci, 1, 64 co) = one MN-major panel;
// tmC: the result (fwd: Y, dgrad: dX) with box (64, PW, Rb, 1).
template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
conv_halo_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                 const __grid_constant__ CUtensorMap tmC, const HaloDev d) {
  constexpr bool W_MN = MODE == MODE_DGRAD;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles_x = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* tiles_w = tiles_x + (size_t)d.stages_x * d.x_stage_bytes;
  uint8_t* cslab = tiles_w + (size_t)d.stages_w * W_STAGE_BYTES;
  SmemCtl* ctl = (SmemCtl*)(cslab + 4 * C_SLAB_BYTES);          // two sets (one per store block) of two slabs
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = d.m_tiles * d.n_images * d.row_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < d.stages_x; ++s) { tc05::mbar_init(&ctl->full_x[s], 1); tc05::mbar_init(&ctl->empty_x[s], 1); }
    for (int s = 0; s < d.stages_w; ++s) { tc05::mbar_init(&ctl->full_w[s], 1); tc05::mbar_init(&ctl->empty_w[s], 1); }
    for (int a = 0; a < 2; ++a) { tc05::mbar_init(&ctl->tmem_full[a], 1); tc05::mbar_init(&ctl->tmem_empty[a], kEpilogueWarps); }
    ctl->abort_flag = 0;
    tc05::mbar_fence_init();
  }
  {
    // an MMA reads N rows from a shifted start: the few rows past the halo tile feed dropped columns only, but
    // they must not hold NaN patterns left by an earlier kernel
    uint4* z = reinterpret_cast<uint4*>(tiles_x);
    const int n16 = d.stages_x * d.x_stage_bytes / 16;
    for (int i = threadIdx.x; i < n16; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
    tc05::fence_proxy_async_smem();
  }
  if (warp == 1) {
    tc05::tmem_alloc(&ctl->tmem_base, 2 * ACC_COLS);
    tc05::tmem_relinquish();
  }
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;
  const int NR = 2 * d.Rb + d.KH - 1;
  const uint32_t x_tx = (uint32_t)(NR * d.PW * 128);

  if (warp == 0) {
    // ---------------- TMA producer: one halo tile per chunk, one weight tile per (tap, chunk) ----------------
    const bool leader = tc05::elect_one();
    if (leader) { tc05::tma_prefetch_desc(&tmX); tc05::tma_prefetch_desc(&tmW); }
    int sx = 0, sw = 0;
    uint32_t phx = 0, phw = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const Tile q = decode_tile(d, t);
      for (int cc = 0; cc < d.cchunks && ok; ++cc) {
        if (!tc05::mbar_wait_warp(&ctl->empty_x[sx], phx ^ 1u, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
        if (leader) {
          tc05::mbar_expect_tx(&ctl->full_x[sx], x_tx);
          tc05::tma_load_4d(tiles_x + (size_t)sx * d.x_stage_bytes, &tmX, &ctl->full_x[sx], cc * 64, -d.px, q.y0 - d.py, q.b);
        }
        if (++sx == d.stages_x) { sx = 0; phx ^= 1u; }
        for (int tap = 0; tap < d.taps; ++tap) {
          if (!tc05::mbar_wait_warp(&ctl->empty_w[sw], phw ^ 1u, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
          if (leader) {
            uint8_t* dst = tiles_w + (size_t)sw * W_STAGE_BYTES;
            tc05::mbar_expect_tx(&ctl->full_w[sw], W_STAGE_BYTES);
            if (MODE == MODE_FWD) {
              tc05::tma_load_3d(dst, &tmW, &ctl->full_w[sw], cc * 64, tap, q.mi * BM);
            } else {
              // data gradient: the filter is applied mirrored; rows of the product are input channels
              const int wtap = d.taps - 1 - tap;
              tc05::tma_load_3d(dst, &tmW, &ctl->full_w[sw], q.mi * BM, wtap, cc * 64);
              tc05::tma_load_3d(dst + PANEL_BYTES, &tmW, &ctl->full_w[sw], q.mi * BM + 64, wtap, cc * 64);
            }
          }
          if (++sw == d.stages_w) { sw = 0; phw ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    const bool leader = tc05::elect_one();
    const uint32_t idesc2 = tc05::make_idesc_bf16(BM, d.ncols2, W_MN ? 1 : 0, 0);
    const uint32_t idesc1 = tc05::make_idesc_bf16(BM, d.ncols1, W_MN ? 1 : 0, 0);
    constexpr uint32_t d_hi = tc05::desc_hi(1024);
    constexpr uint32_t w_kstep = W_MN ? 128u : 2u;      // 16 k: two 8-row groups of 1024 bytes, or 32 bytes in the row
    const uint32_t row_wrap8 = (uint32_t)(d.PW - d.KW + 1) * 8u;
    uint32_t tile_i = 0;
    int sx = 0, sw = 0;
    uint32_t phx = 0, phw = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_i) {
      const Tile q = decode_tile(d, t);
      const uint32_t idesc = q.nb == 2 ? idesc2 : idesc1;
      const uint32_t acc = tile_i & 1u, acc_ph = (tile_i >> 1) & 1u;
      if (!tc05::mbar_wait_warp(&ctl->tmem_empty[acc], acc_ph ^ 1u, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
      tc05::fence_after_sync();
      const uint32_t tacc = tmem + acc * (uint32_t)ACC_COLS;
      uint32_t accumulate = 0;                          // the very first MMA of a tile overwrites the accumulator
      for (int cc = 0; cc < d.cchunks && ok; ++cc) {
        if (!tc05::mbar_wait_warp(&ctl->full_x[sx], phx, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
        // tap (ty, tx) reads the halo tile from row ty * PW + tx on: 8 descriptor units (128 bytes) per row
        uint32_t x_lo = tc05::desc_lo(tc05::smem_u32(tiles_x + (size_t)sx * d.x_stage_bytes), 16);
        const bool full_k = cc + 1 < d.cchunks || d.k_last == BK / UMMA_K;
        int tx = 0;
        for (int tap = 0; tap < d.taps; ++tap) {
          if (!tc05::mbar_wait_warp(&ctl->full_w[sw], phw, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
          tc05::fence_after_sync();
          if (leader) {
            const uint32_t w_lo = tc05::desc_lo(tc05::smem_u32(tiles_w + (size_t)sw * W_STAGE_BYTES), W_MN ? PANEL_BYTES : 16);
            if (full_k) {
              tc05::mma_bf16_ss_lohi(tacc, w_lo, d_hi, x_lo, d_hi, idesc, accumulate);
              tc05::mma_bf16_ss_lohi(tacc, w_lo + w_kstep, d_hi, x_lo + 2, d_hi, idesc, 1u);
              tc05::mma_bf16_ss_lohi(tacc, w_lo + 2 * w_kstep, d_hi, x_lo + 4, d_hi, idesc, 1u);
              tc05::mma_bf16_ss_lohi(tacc, w_lo + 3 * w_kstep, d_hi, x_lo + 6, d_hi, idesc, 1u);
            } else {
              tc05::mma_bf16_ss_lohi(tacc, w_lo, d_hi, x_lo, d_hi, idesc, accumulate);
              if (d.k_last > 1) tc05::mma_bf16_ss_lohi(tacc, w_lo + w_kstep, d_hi, x_lo + 2, d_hi, idesc, 1u);
              if (d.k_last > 2) tc05::mma_bf16_ss_lohi(tacc, w_lo + 2 * w_kstep, d_hi, x_lo + 4, d_hi, idesc, 1u);
            }
            tc05::mma_commit(&ctl->empty_w[sw]);
          }
          accumulate = 1u;
          if (++sw == d.stages_w) { sw = 0; phw ^= 1u; }
          if (++tx == d.KW) { tx = 0; x_lo += row_wrap8; } else { x_lo += 8u; }
        }
        if (ok && leader) tc05::mma_commit(&ctl->empty_x[sx]);
        if (++sx == d.stages_x) { sx = 0; phx ^= 1u; }
      }
      if (ok && leader) tc05::mma_commit(&ctl->tmem_full[acc]);
    }
  } else {
    // ---------------- epilogue: TMEM (channel lanes) -> bf16 [position][channel] slab -> TMA store ----------------
    const int q4 = warp & 3;                       // TMEM lane quarter this warp may access
    const int sub = (warp - 2) >> 2;               // which of the quarter's two warps
    const int half = q4 >> 1;                      // which 64-channel slab of a set
    const int chin = (q4 & 1) * 32 + lane;         // channel inside the slab
    const uint32_t chunk = (uint32_t)(chin >> 3), within = (uint32_t)((chin & 7) * 2);
    // Slab rows are positions (128 bytes, 128-byte swizzle: 16-byte chunk ^ row % 8).  A block has a multiple of
    // 8 positions and a column group starts at a multiple of 32, so the row of element e of a group is congruent
    // to e mod 8: the eight swizzled chunk offsets of this thread's channel are constants of the thread.
    uint32_t cb[8];
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) cb[jj] = ((chunk ^ (uint32_t)jj) << 4) + within;
    const uint32_t slab_base = tc05::smem_u32(cslab) + (uint32_t)(half * C_SLAB_BYTES);     // set p adds p * 2 slabs
    const bool storer = lane == 0 && (q4 & 1) == 0 && sub == 0;          // one thread per slab issues its stores
    const float floor_v = d.relu ? 0.f : -INFINITY;
    uint32_t tile_i = 0;
    int bias_mi = -1;
    float bias_v = 0.f;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++tile_i) {
      const Tile q = decode_tile(d, t);
      if (q.mi != bias_mi) {                       // tiles are ordered by channel block: this happens m_tiles times
        const int ch = q.mi * BM + q4 * 32 + lane;
        bias_v = (MODE == MODE_FWD && d.bias != nullptr && ch < d.n_valid) ? __ldg(d.bias + ch) : 0.f;
        bias_mi = q.mi;
      }
      const bool slab_valid = q.mi * BM + half * 64 < d.n_valid;           // same for every thread of the slab
      const uint32_t acc = tile_i & 1u, acc_ph = (tile_i >> 1) & 1u;
      if (!tc05::mbar_wait(&ctl->tmem_full[acc], acc_ph, abort_flag, WAIT_BUDGET_NS)) break;
      tc05::fence_after_sync();
      const uint32_t tacc = tmem + acc * (uint32_t)ACC_COLS + ((uint32_t)(q4 * 32) << 16);
      for (int p = 0; p < q.nb; ++p) {
        const uint32_t slab = slab_base + (uint32_t)(p * 2 * C_SLAB_BYTES);
        // block p of the previous tile was stored out of this slab: that store must have read it (the one store
        // issued since, out of the other set, may still be reading)
        if (storer) tc05::bulk_wait_read<1>();
        tc05::named_bar_sync(1, 32 * kEpilogueWarps);
        if (slab_valid) {
          const int c_begin = p * d.split, c_end = c_begin + d.split;
#pragma unroll 1
          for (int g = (c_begin & ~31) + 32 * sub; g < c_end; g += 64) {
            uint32_t r[32];
            tc05::tmem_ld_32x32(tacc + (uint32_t)g, r);
            tc05::tmem_ld_wait();
            const int row0 = g - c_begin;              // slab row of element 0: a multiple of 8, negative for a first
            const uint32_t rbase = slab + (uint32_t)(row0 * 128);     // group that starts in the previous block
            if (row0 >= 0 && row0 + 32 <= d.split) {
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                const float v = fmaxf(__uint_as_float(r[e]) + bias_v, floor_v);
                tc05::st_shared_bf16(rbase + cb[e & 7] + (uint32_t)(e * 128), v);
              }
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                const int row = row0 + e;
                if (row >= 0 && row < d.split) {
                  const float v = fmaxf(__uint_as_float(r[e]) + bias_v, floor_v);
                  tc05::st_shared_bf16(rbase + cb[e & 7] + (uint32_t)(e * 128), v);
                }
              }
            }
          }
        }
        tc05::fence_proxy_async_smem();
        tc05::named_bar_sync(1, 32 * kEpilogueWarps);
        if (storer && slab_valid) {
          // box (64 channels, PW, Rb, 1): columns past the image width, rows past its height and channels past
          // the extent are clipped by TMA
          tc05::tma_store_4d_addr(&tmC, slab, q.mi * BM + half * 64, 0, q.y0 + p * d.Rb, q.b);
          tc05::bulk_commit();
        }
      }
      tc05::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive(&ctl->tmem_empty[acc]);
    }
    if (storer) tc05::bulk_wait<0>();
  }

  tc05::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && ctl->abort_flag)
    geeps_report(d.status, GEEPS_ERR_TIMEOUT, KID_CONV_TC, (int)blockIdx.x, 1);
  if (warp == 1) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc(tmem, 2 * ACC_COLS);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}
bool make_map(CUtensorMap* map, const void* base, int rank, const long long* dims, const long long* strides_bytes,
              const int* box) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t gd[4], gs[3];
  cuuint32_t bx[4], es[4];
  for (int i = 0; i < rank; ++i) { gd[i] = (cuuint64_t)dims[i]; bx[i] = (cuuint32_t)box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = (cuuint64_t)strides_bytes[i];
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gd, gs, bx, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
bool make_act_map(CUtensorMap* map, const void* base, int ch, int W, int H, int B, long long pitch, int bw, int bh) {
  const long long dims[4] = {ch, W, H, B};
  const long long st[3] = {pitch * 2, pitch * 2 * W, pitch * 2 * W * H};
  const int box[4] = {64, bw, bh, 1};
  return make_map(map, base, 4, dims, st, box);
}
int round_up(long long v, int m) { return (int)((v + m - 1) / m * m); }

template <int MODE>
int launch(const CUtensorMap& tx, const CUtensorMap& tw, const CUtensorMap& tc, const HaloDev& d, int grid, size_t smem,
           cudaStream_t st) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(conv_halo_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  conv_halo_kernel<MODE><<<grid, kThreads, smem, st>>>(tx, tw, tc, d);
  return (int)cudaGetLastError();
}

// geometry shared by the applicability check and the launch
struct HaloPlan { HaloDev d; size_t smem; double util; bool ok; };

HaloPlan plan_halo(const GeepsConvTcParams* p) {
  HaloPlan hp;
  hp.ok = false;
  hp.smem = 0;
  hp.util = 0;
  HaloDev& d = hp.d;
  memset(&d, 0, sizeof(d));
  if ((p->mode != MODE_FWD && p->mode != MODE_DGRAD) || p->stride > 1) return hp;
  const bool fwd = p->mode == MODE_FWD;
  const int GW = fwd ? p->OW : p->W, GH = fwd ? p->OH : p->H;
  d.KH = p->KH; d.KW = p->KW; d.taps = p->KH * p->KW;
  d.px = fwd ? p->pad : p->KW - 1 - p->pad;
  d.py = fwd ? p->pad : p->KH - 1 - p->pad;
  if (d.px < 0 || d.py < 0 || d.taps < 2) return hp;
  d.GH = GH;
  // Two store blocks of Rb image rows per tile, at most 128 positions each; the rows are spread evenly over the
  // tiles so that the last tile is not mostly padding.  The pitch is the smallest one >= out_width + KW - 1 that
  // makes a block a multiple of 8 positions (the epilogue's constant swizzle offsets rely on it).
  bool found = false;
  for (int pw = GW + p->KW - 1; pw <= GW + p->KW + 6 && pw <= 128; ++pw) {
    const int rb_max = 128 / pw;
    const int row_tiles = (GH + 2 * rb_max - 1) / (2 * rb_max);
    const int rb = (GH + 2 * row_tiles - 1) / (2 * row_tiles);
    if ((rb * pw) % 8) continue;
    d.PW = pw; d.row_tiles = row_tiles; d.Rb = rb;
    found = true;
    break;
  }
  if (!found) return hp;
  d.split = d.Rb * d.PW;
  d.ncols2 = round_up(2 * d.split, 16);
  d.ncols1 = round_up(d.split, 16);
  const int kch = fwd ? p->cg : p->og, nch = fwd ? p->og : p->cg;
  d.cchunks = (kch + 63) / 64;
  const int tail = kch - (d.cchunks - 1) * 64;
  d.k_last = (tail + UMMA_K - 1) / UMMA_K;
  d.n_valid = nch;
  d.m_tiles = (nch + BM - 1) / BM;
  d.n_images = p->B;
  const int NR = 2 * d.Rb + p->KH - 1;
  const int over = d.ncols2 - 2 * d.split + p->KW;     // rows an MMA may read past the halo tile
  d.x_stage_bytes = round_up((long long)(NR * d.PW + over) * 128, 1024);
  d.stages_x = 2;
  const long long budget = 224 * 1024 - 4 * C_SLAB_BYTES - (long long)d.stages_x * d.x_stage_bytes;
  d.stages_w = (int)(budget / W_STAGE_BYTES);
  if (d.stages_w > MAX_W_STAGES) d.stages_w = MAX_W_STAGES;
  if (d.stages_w < 3) return hp;
  hp.smem = (size_t)d.stages_x * d.x_stage_bytes + (size_t)d.stages_w * W_STAGE_BYTES + 4 * C_SLAB_BYTES + sizeof(SmemCtl) + 1024;
  // share of the issued MMA work that lands in real outputs: positions x channels
  const double pos = (double)GH * GW / ((double)d.row_tiles * d.ncols2);
  const double chn = (double)nch / ((double)d.m_tiles * BM);
  hp.util = pos * chn;
  hp.ok = true;
  return hp;
}

int halo_mode() {
  static int m = -1;
  if (m < 0) { const char* e = getenv("GEEPS_HALO_CONV"); m = e ? atoi(e) : 1; }
  return m;
}

}  // namespace

extern "C" {

// 1 when conv_tc() should route this call here.  The rule is fitted to timings of both kernels on AlexNet and
// Inception layers at batch 128 .. 256 (python -m geeps_b200.utils.microbench conv): the activations must be re-read
// often enough by the box kernel (>= 9 taps), and the 128-channel row blocks must be mostly real channels - a 192- or
// 384-channel layer on 13 x 13 .. 56 x 56 maps is still faster on the box kernel, whose tile is exactly as wide as the
// layer.  A 5 x 5 data gradient always wins here (the box kernel runs it with N = 48 .. 64 MMAs).
int geeps_conv_halo_applicable(const GeepsConvTcParams* p) {
  if (!halo_mode()) return 0;
  if (!geeps_conv_tc_supported(p)) return 0;
  const HaloPlan hp = plan_halo(p);
  if (!hp.ok || hp.d.taps < 9) return 0;
  const HaloDev& d = hp.d;
  const int GW = p->mode == MODE_FWD ? p->OW : p->W;
  const double pos = (double)d.GH * GW / ((double)d.row_tiles * d.ncols2);
  const double chn = (double)d.n_valid / ((double)d.m_tiles * BM);
  if (pos < 0.6) return 0;
  // its tiles are large (up to 256 positions x 128 channels): with fewer than two per SM the box kernel's smaller
  // tiles spread better (Inception at batch 32 .. 100: 5.60 against 5.79 ms per step of the 22K net); a layer of one
  // channel block still wins from 1.7 tiles per SM on (AlexNet conv5 per group, 256 tiles: 0.030 against 0.038 ms)
  const long long tiles = (long long)d.m_tiles * d.n_images * d.row_tiles;
  if (tiles * 10 < (d.m_tiles == 1 ? 17LL : 20LL) * geeps_sm_count()) return 0;
  if (p->mode == MODE_FWD) return (d.m_tiles == 1 && d.n_valid >= 96) || (chn >= 0.85 && pos >= 0.8) ? 1 : 0;
  return d.taps >= 25 || (d.n_valid >= 64 && (d.n_valid <= 128 || chn >= 0.85)) ? 1 : 0;
}

int geeps_conv_halo_plan(const GeepsConvTcParams* p, GeepsHaloPlanInfo* out) {
  memset(out, 0, sizeof(*out));
  if (!geeps_conv_tc_supported(p)) return 0;
  const HaloPlan hp = plan_halo(p);
  if (!hp.ok) return 0;
  const HaloDev& d = hp.d;
  out->ok = 1;
  out->routed = geeps_conv_halo_applicable(p);
  out->PW = d.PW; out->R = d.Rb; out->row_tiles = d.row_tiles; out->m_tiles = d.m_tiles;
  out->positions = d.split; out->ncols2 = d.ncols2; out->ncols1 = d.ncols1;
  out->stages_x = d.stages_x; out->stages_w = d.stages_w; out->x_stage_bytes = d.x_stage_bytes;
  out->tmem_cols = 2 * ACC_COLS;
  out->smem_bytes = (long long)hp.smem;
  out->util = hp.util;
  return 1;
}

int geeps_conv_halo(const GeepsConvTcParams* p, void* stream) {
  if (!geeps_conv_tc_supported(p)) return (int)cudaErrorInvalidValue;
  HaloPlan hp = plan_halo(p);
  if (!hp.ok) return (int)cudaErrorInvalidValue;
  HaloDev& d = hp.d;
  const bool fwd = p->mode == MODE_FWD;
  d.bias = fwd ? p->bias : nullptr;
  d.status = p->status;
  d.relu = fwd ? p->relu : 0;
  const int NR = 2 * d.Rb + p->KH - 1;
  CUtensorMap tx, tw, tc;
  bool ok;
  const long long wdims[3] = {p->cg, d.taps, p->og};
  const long long wst[2] = {(long long)p->cg * 2, p->ldw * 2};
  if (fwd) {
    ok = make_act_map(&tx, p->x, p->cg, p->W, p->H, p->B, p->x_pitch, d.PW, NR);
    const int wbox[3] = {64, 1, BM};
    ok = ok && make_map(&tw, p->w, 3, wdims, wst, wbox);
    ok = ok && make_act_map(&tc, p->y, p->og, p->OW, p->OH, p->B, p->y_pitch, d.PW, d.Rb);
  } else {
    ok = make_act_map(&tx, p->y, p->og, p->OW, p->OH, p->B, p->y_pitch, d.PW, NR);
    const int wbox[3] = {64, 1, 64};
    ok = ok && make_map(&tw, p->w, 3, wdims, wst, wbox);
    ok = ok && make_act_map(&tc, p->x, p->cg, p->W, p->H, p->B, p->x_pitch, d.PW, d.Rb);
  }
  if (!ok) return (int)cudaErrorInvalidValue;
  const long long num_tiles = (long long)d.m_tiles * d.n_images * d.row_tiles;
  const int sms = geeps_sm_count();
  const int grid = (int)(num_tiles < sms ? num_tiles : sms);
  if (fwd) return launch<MODE_FWD>(tx, tw, tc, d, grid, hp.smem, (cudaStream_t)stream);
  return launch<MODE_DGRAD>(tx, tw, tc, d, grid, hp.smem, (cudaStream_t)stream);
}

}  // extern "C"
