// Implicit-GEMM convolution (stride 1) on the 5th-generation tensor cores: no patch matrix is ever
// written.  The activation operand of every k-tile is fetched straight from the NHWC tensor by one tiled
// 4-D TMA load whose (w, h) start is shifted by the filter tap; pixels that fall into the padding are
// outside the tensor's extent and arrive as zeros.  Three products share one persistent kernel:
//
//   forward        Y[pix, co]  = sum_{tap, ci} X[pix + tap, ci] * W[co, tap, ci]   (+ bias, ReLU)
//   data gradient  dX[pix, ci] = sum_{tap, co} dY[pix - tap, co] * W[co, tap, ci]
//   weight grad.   dW[co, tap, ci] = sum_{pix} dY[pix, co] * X[pix + tap, ci]      (fp32, split over pixels)
//
// The 128 accumulator rows of a tile are a box of bw x bh x bn output pixels (chosen per layer so that the
// box wastes few rows), so the same box shape serves the 4-D load and the 4-D store of the result, and
// ragged edges are clipped by TMA.  The weight matrix [co][tap][ci] is a 3-D tensor for TMA, so channel
// counts that are not multiples of 64 (48-channel groups) are zero-filled instead of reading the next tap.
// For the weight gradient the reduction runs over pixel boxes of 64, both operands are MN-major panels of
// [64 pixels x 64 channels], and one tile's N covers up to four (tap, channel-chunk) panels.
//
// Roles, pipeline, TMEM double buffering, bounded waits and the swizzled-slab TMA-store epilogue are those
// of the plain GEMM in gemm_tc.cu.
//
// The reference has no convolution of its own (its layers lived in a Caffe fork that is not in its tree);
// this replaces the im2col + GEMM + col2im formulation for stride-1 layers.
#include <cuda.h>
#include <mutex>
#include <stdio.h>

#include "kernels.h"
#include "tc05.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int PANEL_BYTES = 64 * BK * 2;     // one MN-major panel: 64 k-rows x 128 bytes
constexpr int MAX_STAGES = 8;
constexpr uint64_t WAIT_BUDGET_NS = 2000000000ull;
constexpr int C_SLAB_BYTES = BM * 128;

enum { MODE_FWD = 0, MODE_DGRAD = 1, MODE_WGRAD = 2 };

struct ConvDev {
  const float* bias; int* status;
  int taps, KW, pad, cchunks;     // k-tile (fwd, dgrad) or N panel (wgrad) = (tap, 64-channel chunk)
  int bw, bh, bnb, wt, ht;        // pixel box and number of boxes along W and H (batch boxes follow)
  int rows;                       // bw * bh * bnb
  int bn, n_valid;                // tile width; valid output columns (fwd: Og, dgrad: Cg, wgrad: panels * 64)
  int m_tiles, n_tiles, kt_total, split_k, stages, tmem_cols;
  int relu, zero_fill_c;          // wgrad: a channel coordinate outside X, for panels past the last one
  int ch_valid;                   // wgrad: channels per tap (cg)
  int narrow;                     // fwd / dgrad: result leaves in 32-channel (64-byte) slabs, see the host code
  int stride;                     // fwd / wgrad: pixel stride of the layer (the X boxes are loaded with this element stride)
  int pad_w, pad_h;               // dgrad: dY offset of tap (0, 0); equal to pad for a stride-1 layer
  int tap0, tap_dw, tap_dh;       // dgrad: weight tap of loop position (kh, kw) = tap0 + kh * tap_dh + kw * tap_dw
                                  // (a strided layer's data gradient runs one parity class of dX at a time, each
                                  // with the sub-filter of the taps that reach it)
};

struct SmemCtl {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct Box { int w0, h0, b0; };
__device__ __forceinline__ Box decode_box(const ConvDev& d, int i) {
  Box b;
  const int wi = i % d.wt;
  const int r = i / d.wt;
  b.w0 = wi * d.bw;
  b.h0 = (r % d.ht) * d.bh;
  b.b0 = (r / d.ht) * d.bnb;
  return b;
}

// tmA: activations of the M side (fwd: X, dgrad: dY, wgrad: dY); tmB: fwd/dgrad: W as (ci, tap, co),
// wgrad: X; tmC: fwd: Y, dgrad: dX (4-D bf16), wgrad: dW as (ci, tap, co) fp32.
template <int MODE>
__global__ void __launch_bounds__(192, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const ConvDev d) {
  constexpr bool A_MN = MODE == MODE_WGRAD;
  constexpr bool B_MN = MODE != MODE_FWD;
  extern __shared__ uint8_t smem_raw[];
  const int BN = d.bn;
  const int B_STAGE_BYTES = BN * BK * 2;
  const int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* cslab = tiles + (size_t)d.stages * STAGE_BYTES;
  SmemCtl* ctl = (SmemCtl*)(cslab + 2 * C_SLAB_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = d.stages;
  const int kt_per = (d.kt_total + d.split_k - 1) / d.split_k;
  const int tiles_mn = d.m_tiles * d.n_tiles;
  const int num_tiles = tiles_mn * d.split_k;
  const int acc_stride = d.tmem_cols >> 1;

  if (MODE == MODE_WGRAD && d.rows < 64) {
    // a pixel box with fewer than 64 pixels leaves the tail of every panel untouched: it must read as zero
    uint4* z = reinterpret_cast<uint4*>(tiles);
    const int n16 = d.stages * STAGE_BYTES / 16;
    for (int i = threadIdx.x; i < n16; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
    tc05::fence_proxy_async_smem();
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { tc05::mbar_init(&ctl->full[s], 1); tc05::mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { tc05::mbar_init(&ctl->tmem_full[a], 1); tc05::mbar_init(&ctl->tmem_empty[a], 4); }
    ctl->abort_flag = 0;
    tc05::mbar_fence_init();
  }
  if (warp == 1) {
    tc05::tmem_alloc(&ctl->tmem_base, (uint32_t)d.tmem_cols);
    tc05::tmem_relinquish();
  }
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    // the loop runs with the whole warp converged; the elected lane issues the copies
    {
      const bool leader = tc05::elect_one();
      if (leader) { tc05::tma_prefetch_desc(&tmA); tc05::tma_prefetch_desc(&tmB); }
      // every index below advances incrementally: this one thread's latency is the producer's throughput,
      // and an integer division costs more than the TMA issue itself
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      const uint32_t tx_bytes = MODE == MODE_WGRAD ? (uint32_t)((2 + BN / 64) * d.rows * 128)
                                                   : (uint32_t)(d.rows * 128 + BN * 128);
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int mn = t % tiles_mn, z = t / tiles_mn;
        const int mi = mn % d.m_tiles, ni = mn / d.m_tiles;
        const int kt_begin = z * kt_per, kt_end = min(d.kt_total, kt_begin + kt_per);
        Box mb = {0, 0, 0};
        if (MODE != MODE_WGRAD) mb = decode_box(d, mi);
        // fwd / dgrad: k-tile = (kh, kw, channel chunk), starting at 0 (no split)
        int kh = 0, kw = 0, cc = 0, tap = 0, wtap = d.tap0;
        // wgrad: k-tile = pixel box; the N panels of this tile are fixed
        Box kb = {0, 0, 0};
        int pc[4] = {0, 0, 0, 0}, pdw[4] = {0, 0, 0, 0}, pdh[4] = {0, 0, 0, 0};
        if (MODE == MODE_WGRAD) {
          kb = decode_box(d, kt_begin);
          for (int j = 0; j < BN / 64; ++j) {
            const int panel = ni * (BN / 64) + j;
            const bool valid = panel * 64 < d.n_valid;
            const int ptap = valid ? panel / d.cchunks : 0;
            const int pkh = ptap / d.KW;
            pc[j] = valid ? (panel - ptap * d.cchunks) * 64 : d.zero_fill_c;
            pdw[j] = ptap - pkh * d.KW - d.pad;
            pdh[j] = pkh - d.pad;
          }
        }
        for (int kt = kt_begin; kt < kt_end; ++kt) {
          if (!tc05::mbar_wait_warp(&ctl->empty[s], ph ^ 1u, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
          uint8_t* sa = tiles + (size_t)s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          uint64_t* bar = &ctl->full[s];
          if (leader) {
          tc05::mbar_expect_tx(bar, tx_bytes);
          if (MODE == MODE_FWD) {
            tc05::tma_load_4d(sa, &tmA, bar, cc * 64, mb.w0 * d.stride + kw - d.pad, mb.h0 * d.stride + kh - d.pad, mb.b0);
            tc05::tma_load_3d(sb, &tmB, bar, cc * 64, tap, ni * BN);
          } else if (MODE == MODE_DGRAD) {
            tc05::tma_load_4d(sa, &tmA, bar, cc * 64, mb.w0 + d.pad_w - kw, mb.h0 + d.pad_h - kh, mb.b0);
            for (int h = 0; h < BN / 64; ++h)
              tc05::tma_load_3d(sb + h * PANEL_BYTES, &tmB, bar, ni * BN + 64 * h, wtap, cc * 64);
          } else {
            for (int h = 0; h < 2; ++h)
              tc05::tma_load_4d(sa + h * PANEL_BYTES, &tmA, bar, mi * BM + 64 * h, kb.w0, kb.h0, kb.b0);
            for (int j = 0; j < BN / 64; ++j)
              tc05::tma_load_4d(sb + j * PANEL_BYTES, &tmB, bar, pc[j], kb.w0 * d.stride + pdw[j], kb.h0 * d.stride + pdh[j], kb.b0);
          }
          }
          if (MODE == MODE_WGRAD) {
            kb.w0 += d.bw;
            if (kb.w0 >= d.wt * d.bw) {
              kb.w0 = 0; kb.h0 += d.bh;
              if (kb.h0 >= d.ht * d.bh) { kb.h0 = 0; kb.b0 += d.bnb; }
            }
          } else if (++cc == d.cchunks) {
            cc = 0; ++tap; wtap += d.tap_dw;
            if (++kw == d.KW) { kw = 0; ++kh; wtap += d.tap_dh - d.KW * d.tap_dw; }
          }
          if (++s == S) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    {
      const bool leader = tc05::elect_one();
      const uint32_t idesc = tc05::make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t tile_i = 0, ph = 0;
      int s = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_i) {
        const int z = t / tiles_mn;
        const int kt_begin = z * kt_per, kt_end = min(d.kt_total, kt_begin + kt_per);
        const uint32_t acc = tile_i & 1u, acc_ph = (tile_i >> 1) & 1u;
        if (!tc05::mbar_wait_warp(&ctl->tmem_empty[acc], acc_ph ^ 1u, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
        tc05::fence_after_sync();
        const uint32_t tacc = tmem + acc * (uint32_t)acc_stride;
        for (int kt = kt_begin; kt < kt_end; ++kt) {
          if (!tc05::mbar_wait_warp(&ctl->full[s], ph, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
          tc05::fence_after_sync();
          const uint32_t sa = tc05::smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
          if (leader) {
          // descriptors as 32-bit halves: per MMA this one thread spends an add per operand, not a rebuild
          const uint32_t a_lo = tc05::desc_lo(sa, A_MN ? PANEL_BYTES : 16), b_lo = tc05::desc_lo(sb, B_MN ? PANEL_BYTES : 16);
          constexpr uint32_t d_hi = tc05::desc_hi(1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc05::mma_bf16_ss_lohi(tacc, a_lo + (A_MN ? 128 : 2) * k, d_hi, b_lo + (B_MN ? 128 : 2) * k, d_hi, idesc,
                                   (kt > kt_begin || k > 0) ? 1u : 0u);
          tc05::mma_commit(&ctl->empty[s]);
          }
          if (++s == S) { s = 0; ph ^= 1u; }
        }
        if (ok && leader) tc05::mma_commit(&ctl->tmem_full[acc]);
      }
    }
  } else {
    // ---------------- epilogue: TMEM -> registers -> swizzled slab -> TMA store ----------------
    const int q = warp & 3;
    uint32_t tile_i = 0, slab_i = 0;
    const int cols_per_slab = (MODE == MODE_WGRAD || d.narrow) ? 32 : 64;
    const bool issuer = threadIdx.x == 64;
    const int rloc = q * 32 + lane;
    // wide slab: 128-byte rows, 128-byte swizzle (16-byte chunk ^ row % 8); narrow slab: 64-byte rows, 64-byte
    // swizzle (chunk ^ (row / 2) % 4)
    const bool narrow = MODE != MODE_WGRAD && d.narrow;
    const uint32_t row_off = (uint32_t)rloc * (narrow ? 64u : 128u);
    const uint32_t rsw = narrow ? (uint32_t)((rloc >> 1) & 3) : (uint32_t)(rloc & 7);
    const bool relu = d.relu != 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++tile_i) {
      const int mn = t % tiles_mn;
      const int mi = mn % d.m_tiles, ni = mn / d.m_tiles;
      const int n0 = ni * BN;
      const uint32_t acc = tile_i & 1u, acc_ph = (tile_i >> 1) & 1u;
      if (!tc05::mbar_wait(&ctl->tmem_full[acc], acc_ph, abort_flag, WAIT_BUDGET_NS)) break;
      tc05::fence_after_sync();
      const uint32_t tacc = tmem + acc * (uint32_t)acc_stride + ((uint32_t)(q * 32) << 16);
      Box mb = {0, 0, 0};
      if (MODE != MODE_WGRAD) mb = decode_box(d, mi);
#pragma unroll 1
      for (int c = 0; c < BN; c += cols_per_slab) {
        if (n0 + c >= d.n_valid) break;
        uint8_t* slab = cslab + (size_t)(slab_i & 1u) * C_SLAB_BYTES;
        if (issuer) tc05::bulk_wait_read<1>();
        tc05::named_bar_sync(1, 128);
        for (int h = 0; h < cols_per_slab; h += 32) {
          if (n0 + c + h >= d.n_valid) break;      // columns past the tensor's extent are clipped by the store anyway
          uint32_t r[32];
          tc05::tmem_ld_32x32(tacc + (uint32_t)(c + h), r);
          tc05::tmem_ld_wait();
          if (MODE == MODE_WGRAD) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t off = row_off + (uint32_t)((j ^ rsw) << 4);
              *reinterpret_cast<uint4*>(slab + off) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            }
          } else {
            float v[32];
            const int col0 = n0 + c + h;
            if (MODE == MODE_FWD && d.bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                v[j] = __uint_as_float(r[j]) + (col0 + j < d.n_valid ? __ldg(d.bias + col0 + j) : 0.f);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            }
            if (relu) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t off = row_off + (uint32_t)((((h >> 3) + j) ^ rsw) << 4);
              *reinterpret_cast<uint4*>(slab + off) =
                  make_uint4(pack_bf16x2(v[8 * j], v[8 * j + 1]), pack_bf16x2(v[8 * j + 2], v[8 * j + 3]),
                             pack_bf16x2(v[8 * j + 4], v[8 * j + 5]), pack_bf16x2(v[8 * j + 6], v[8 * j + 7]));
            }
          }
        }
        tc05::fence_proxy_async_smem();
        tc05::named_bar_sync(1, 128);
        if (issuer) {
          if (MODE == MODE_WGRAD) {
            const int panel = (n0 + c) >> 6;
            const int tap = panel / d.cchunks, cc = panel - tap * d.cchunks;
            const int x = cc * 64 + (c & 32);
            if (x < d.ch_valid) {       // never start a store past the extent
              if (d.split_k > 1) tc05::tma_reduce_add_3d(&tmC, slab, x, tap, mi * BM);
              else tc05::tma_store_3d(&tmC, slab, x, tap, mi * BM);
            }
          } else {
            tc05::tma_store_4d(&tmC, slab, n0 + c, mb.w0, mb.h0, mb.b0);
          }
          tc05::bulk_commit();
        }
        ++slab_i;
      }
      tc05::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive(&ctl->tmem_empty[acc]);
    }
  }

  if (threadIdx.x == 64) tc05::bulk_wait<0>();
  tc05::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && ctl->abort_flag)
    geeps_report(d.status, GEEPS_ERR_TIMEOUT, KID_CONV_TC, (int)blockIdx.x, 0);
  if (warp == 1) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc(tmem, (uint32_t)d.tmem_cols);
  }
}

// ---------------- host side ----------------
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

// rank-N map (128-byte swizzle unless told otherwise); dims / box innermost first, strides (bytes) for dims 1..rank-1
bool make_map(CUtensorMap* map, const void* base, int rank, const long long* dims, const long long* strides_bytes,
              const int* box, bool fp32, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B,
              const int* elem_strides = nullptr) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t gd[4], gs[3];
  cuuint32_t bx[4], es[4];
  for (int i = 0; i < rank; ++i) {
    gd[i] = (cuuint64_t)dims[i]; bx[i] = (cuuint32_t)box[i];
    es[i] = elem_strides ? (cuuint32_t)elem_strides[i] : 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = (cuuint64_t)strides_bytes[i];
  return fn(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank,
            const_cast<void*>(base), gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// NHWC activation tensor as (channels, W, H, B) with a pixel pitch of `pitch` channels.  stride > 1: a box of
// bw x bh pixels takes every stride-th pixel (TMA element strides; the box extent is given in traversed elements,
// of which ceil(extent / stride) are loaded).
bool make_act_map(CUtensorMap* map, const void* base, int ch, int W, int H, int B, long long pitch, int bw, int bh,
                  int bnb, bool narrow = false, int stride = 1) {
  const long long dims[4] = {ch, W, H, B};
  const long long st[3] = {pitch * 2, pitch * 2 * W, pitch * 2 * W * H};
  const int box[4] = {narrow ? 32 : 64, bw * stride, bh * stride, bnb};
  const int es[4] = {1, stride, stride, 1};
  return make_map(map, base, 4, dims, st, box, false, narrow ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                  es);
}

// A parity class of an NHWC tensor: pixels (s * i + a, s * j + b) as a dense (channels, W2, H2, B) tensor
bool make_act_view(CUtensorMap* map, const void* base, int ch, int W, int H, int B, long long pitch, int s, int a,
                   int b, int W2, int H2, int bw, int bh, int bnb, bool narrow) {
  const long long dims[4] = {ch, W2, H2, B};
  const long long st[3] = {pitch * 2 * s, pitch * 2 * W * s, pitch * 2 * W * H};
  const int box[4] = {narrow ? 32 : 64, bw, bh, bnb};
  const char* origin = (const char*)base + ((long long)a * W + b) * pitch * 2;
  return make_map(map, origin, 4, dims, st, box, false, narrow ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
}

// Pick the pixel box (bw, bh, bnb) with at most `cap` pixels that covers the W x H x B grid with the fewest
// boxes; ties go to the wider box (longer contiguous runs).
void pick_box(int W, int H, int B, int cap, int* bw, int* bh, int* bnb) {
  long long best = -1;
  *bw = 1; *bh = 1; *bnb = 1;
  for (int w = 1; w <= W && w <= cap; ++w) {
    for (int h = 1; h <= H && w * h <= cap; ++h) {
      int n = cap / (w * h);
      if (n > B) n = B;
      if (n > 256 || w > 256 || h > 256) continue;
      const long long boxes = (long long)((W + w - 1) / w) * ((H + h - 1) / h) * ((B + n - 1) / n);
      if (best < 0 || boxes < best || (boxes == best && w > *bw)) { best = boxes; *bw = w; *bh = h; *bnb = n; }
    }
  }
}

int round_up(long long v, int m) { return (int)((v + m - 1) / m * m); }

// A result tensor whose pixel pitch is not a multiple of 128 bytes and whose channel count ends in a half
// slab (96 channels: 192-byte pixels) stores badly in 128-byte rows - they straddle lines and the last slab is
// clipped (the 96-channel conv1 output took 218 us where 64 / 128 channels took 144 / 182 us).  Such tensors
// leave in 32-channel slabs: 64-byte rows that never straddle a 128-byte line and are never clipped.
int narrow_store(int channels, long long pitch) {
  return (channels % 64 == 32 && (pitch * 2) % 128 != 0) ? 1 : 0;
}

template <int MODE>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const ConvDev& d, int grid,
           cudaStream_t st) {
  const int stage_bytes = A_STAGE_BYTES + d.bn * BK * 2;
  const size_t smem = (size_t)d.stages * stage_bytes + 2 * C_SLAB_BYTES + sizeof(SmemCtl) + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(conv_tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  conv_tc_kernel<MODE><<<grid, 192, smem, st>>>(ta, tb, tc, d);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

int geeps_conv_tc_supported(const GeepsConvTcParams* p) {
  if (p->B <= 0 || p->H <= 0 || p->W <= 0 || p->cg <= 0 || p->og <= 0 || p->KH <= 0 || p->KW <= 0) return 0;
  const int s = p->stride > 1 ? p->stride : 1;
  // a strided data gradient runs per parity class of dX; a class without taps (filter narrower than the stride)
  // would have to be zeroed instead and is left to the caller
  if (s > 8 || (s > 1 && p->mode == MODE_DGRAD && (p->KH < s || p->KW < s))) return 0;
  if (p->OH != (p->H + 2 * p->pad - p->KH) / s + 1 || p->OW != (p->W + 2 * p->pad - p->KW) / s + 1) return 0;
  if (p->OH <= 0 || p->OW <= 0) return 0;
  if (((uintptr_t)p->x & 15) || ((uintptr_t)p->y & 15) || ((uintptr_t)p->w & 15)) return 0;
  if ((p->x_pitch & 7) || (p->y_pitch & 7) || (p->cg & 7) || (p->og & 7)) return 0;
  if (p->mode == MODE_WGRAD ? (p->ldw & 3) : (p->ldw & 7)) return 0;
  if (p->ldw < (long long)p->KH * p->KW * p->cg) return 0;
  if (p->mode < 0 || p->mode > 2) return 0;
  return 1;
}

}  // extern "C"

namespace {
// one parity class (a, b) of a strided layer's data gradient, or {s = 1}: the whole problem
struct DgradClass { int s, a, b; };
int conv_tc_run(const GeepsConvTcParams* p, DgradClass cls, void* stream);
}  // namespace

extern "C" {

int geeps_conv_tc(const GeepsConvTcParams* p, void* stream) {
  if (!geeps_conv_tc_supported(p)) return (int)cudaErrorInvalidValue;
  if (p->mode != MODE_WGRAD && p->split_k >= 0 && geeps_conv_halo_applicable(p)) return geeps_conv_halo(p, stream);
  if (p->mode == MODE_WGRAD && p->split_k >= 0 && geeps_conv_wgrad_halo_applicable(p))
    return geeps_conv_wgrad_halo(p, stream);
  if (p->mode == MODE_DGRAD && p->stride > 1) {
    // dX[s i + a, s j + b] = sum over u, v of dY[i + oh0 - u, j + ow0 - v] * W[kh0 + s u, kw0 + s v]: s * s
    // stride-1 problems over dense views of dX, each with its sub-filter
    for (int a = 0; a < p->stride; ++a)
      for (int b = 0; b < p->stride; ++b) {
        if (a >= p->H || b >= p->W) continue;
        const int e = conv_tc_run(p, DgradClass{p->stride, a, b}, stream);
        if (e) return e;
      }
    return 0;
  }
  return conv_tc_run(p, DgradClass{1, 0, 0}, stream);
}

}  // extern "C"

namespace {

int conv_tc_run(const GeepsConvTcParams* p, DgradClass cls, void* stream) {
  const int kSMs = geeps_sm_count();
  cudaStream_t st = (cudaStream_t)stream;
  ConvDev d;
  d.bias = p->mode == MODE_FWD ? p->bias : nullptr;
  d.status = p->status;
  d.taps = p->KH * p->KW; d.KW = p->KW; d.pad = p->pad;
  d.relu = p->mode == MODE_FWD ? p->relu : 0;
  d.split_k = 1;
  d.zero_fill_c = 0;
  d.ch_valid = p->cg;
  d.narrow = 0;
  d.stride = p->stride > 1 ? p->stride : 1;
  d.pad_w = d.pad_h = p->pad;
  d.tap0 = 0; d.tap_dw = 1; d.tap_dh = p->KW;
  CUtensorMap ta, tb, tc;
  bool ok = true;
  const long long wdims[3] = {p->cg, d.taps, p->og};
  if (p->mode == MODE_FWD || p->mode == MODE_DGRAD) {
    const bool fwd = p->mode == MODE_FWD;
    // rows of the tile: pixels of the output (fwd) or of the input gradient (dgrad)
    int GW = fwd ? p->OW : p->W, GH = fwd ? p->OH : p->H;
    if (cls.s > 1) {
      const int sd = cls.s;
      GW = (p->W - cls.b + sd - 1) / sd; GH = (p->H - cls.a + sd - 1) / sd;
      const int kh0 = (cls.a + p->pad) % sd, kw0 = (cls.b + p->pad) % sd;
      const int khs = (p->KH - kh0 + sd - 1) / sd, kws = (p->KW - kw0 + sd - 1) / sd;    // >= 1: KH, KW >= s
      d.pad_h = (cls.a + p->pad - kh0) / sd; d.pad_w = (cls.b + p->pad - kw0) / sd;
      d.tap0 = kh0 * p->KW + kw0; d.tap_dw = sd; d.tap_dh = sd * p->KW;
      d.KW = kws; d.taps = khs * kws;
      d.stride = 1;
    }
    pick_box(GW, GH, p->B, BM, &d.bw, &d.bh, &d.bnb);
    d.rows = d.bw * d.bh * d.bnb;
    d.wt = (GW + d.bw - 1) / d.bw; d.ht = (GH + d.bh - 1) / d.bh;
    d.m_tiles = d.wt * d.ht * ((p->B + d.bnb - 1) / d.bnb);
    const int kch = fwd ? p->cg : p->og;          // reduced channels
    const int nch = fwd ? p->og : p->cg;          // produced channels
    d.cchunks = (kch + 63) / 64;
    d.kt_total = d.taps * d.cchunks;
    d.n_valid = nch;
    const int nt = (nch + 255) / 256;
    int bn = round_up((nch + nt - 1) / nt, (fwd && nt == 1) ? 32 : 64);
    if (bn > 256) bn = 256;
    d.bn = bn;
    d.n_tiles = (nch + bn - 1) / bn;
    const long long wst[2] = {(long long)p->cg * 2, p->ldw * 2};
    if (fwd) {
      ok = make_act_map(&ta, p->x, p->cg, p->W, p->H, p->B, p->x_pitch, d.bw, d.bh, d.bnb, false, d.stride);
      const int wbox[3] = {64, 1, bn};
      ok = ok && make_map(&tb, p->w, 3, wdims, wst, wbox, false);
      d.narrow = narrow_store(p->og, p->y_pitch);
      ok = ok && make_act_map(&tc, p->y, p->og, p->OW, p->OH, p->B, p->y_pitch, d.bw, d.bh, d.bnb, d.narrow != 0);
    } else {
      ok = make_act_map(&ta, p->y, p->og, p->OW, p->OH, p->B, p->y_pitch, d.bw, d.bh, d.bnb);
      const int wbox[3] = {64, 1, 64};
      ok = ok && make_map(&tb, p->w, 3, wdims, wst, wbox, false);
      d.narrow = narrow_store(p->cg, p->x_pitch);
      if (cls.s > 1)
        ok = ok && make_act_view(&tc, p->x, p->cg, p->W, p->H, p->B, p->x_pitch, cls.s, cls.a, cls.b, GW, GH, d.bw,
                                 d.bh, d.bnb, d.narrow != 0);
      else
        ok = ok && make_act_map(&tc, p->x, p->cg, p->W, p->H, p->B, p->x_pitch, d.bw, d.bh, d.bnb, d.narrow != 0);
    }
  } else {
    // reduction over output pixels in boxes of up to 64
    pick_box(p->OW, p->OH, p->B, 64, &d.bw, &d.bh, &d.bnb);
    d.rows = d.bw * d.bh * d.bnb;
    d.wt = (p->OW + d.bw - 1) / d.bw; d.ht = (p->OH + d.bh - 1) / d.bh;
    d.kt_total = d.wt * d.ht * ((p->B + d.bnb - 1) / d.bnb);
    d.m_tiles = (p->og + BM - 1) / BM;
    d.cchunks = (p->cg + 63) / 64;
    const int panels = d.taps * d.cchunks;
    d.n_valid = panels * 64;
    // panels per tile: fewest panel loads per pixel box over the whole product (2 dY panels + `per` patch panels
    // for each of ceil(panels / per) tiles); ties go to the wider tile
    int per = 1;
    long long best_cost = -1;
    for (int c = 1; c <= 4 && c <= panels; ++c) {
      const long long cost = (long long)((panels + c - 1) / c) * (2 + c);
      if (best_cost < 0 || cost <= best_cost) { best_cost = cost; per = c; }
    }
    d.bn = per * 64;
    d.n_tiles = (panels + per - 1) / per;
    d.zero_fill_c = d.cchunks * 64;
    ok = make_act_map(&ta, p->y, p->og, p->OW, p->OH, p->B, p->y_pitch, d.bw, d.bh, d.bnb);
    ok = ok && make_act_map(&tb, p->x, p->cg, p->W, p->H, p->B, p->x_pitch, d.bw, d.bh, d.bnb, false, d.stride);
    const long long wst[2] = {(long long)p->cg * 4, p->ldw * 4};
    const int wbox[3] = {32, 1, BM};
    ok = ok && make_map(&tc, p->w, 3, wdims, wst, wbox, true);
    int split = p->split_k;
    const long long tiles = (long long)d.m_tiles * d.n_tiles;
    if (split <= 0) {
      split = 1;
      if (tiles < kSMs && d.kt_total >= 8) {
        long long want = (2 * kSMs) / tiles;   // at most two full waves: one work item more would add a third round
        long long cap = d.kt_total / 4;
        split = (int)(want < cap ? want : cap);
        if (split < 1) split = 1;
      }
    }
    if (split > d.kt_total) split = d.kt_total;
    if (split > 1) {
      const int per_k = (d.kt_total + split - 1) / split;
      split = (d.kt_total + per_k - 1) / per_k;      // every k-slice non-empty
    }
    d.split_k = split;
    const long long kd = (long long)d.taps * p->cg;
    if (split > 1) {
      // partial sums are reduce-added: the whole [og][ldw] block starts at zero
      int e = geeps_scale_matrix_f32((float*)p->w, p->og, p->ldw, p->ldw, 0.f, stream);
      if (e) return e;
    } else if (p->ldw > kd) {
      // the pad columns past the last tap are never stored: keep them at zero
      int e = geeps_scale_matrix_f32((float*)p->w + kd, p->og, p->ldw - kd, p->ldw, 0.f, stream);
      if (e) return e;
    }
  }
  if (!ok) return (int)cudaErrorInvalidValue;
  int tmem_cols = 32;
  while (tmem_cols < 2 * d.bn) tmem_cols <<= 1;
  d.tmem_cols = tmem_cols;
  const int stage_bytes = A_STAGE_BYTES + d.bn * BK * 2;
  d.stages = (200 * 1024 - 2 * C_SLAB_BYTES) / stage_bytes;
  if (d.stages > MAX_STAGES) d.stages = MAX_STAGES;
  if (d.stages < 2) d.stages = 2;
  const long long num_tiles = (long long)d.m_tiles * d.n_tiles * d.split_k;
  const int grid = (int)(num_tiles < kSMs ? num_tiles : kSMs);
  if (p->mode == MODE_FWD) return launch<MODE_FWD>(ta, tb, tc, d, grid, st);
  if (p->mode == MODE_DGRAD) return launch<MODE_DGRAD>(ta, tb, tc, d, grid, st);
  return launch<MODE_WGRAD>(ta, tb, tc, d, grid, st);
}

}  // namespace
