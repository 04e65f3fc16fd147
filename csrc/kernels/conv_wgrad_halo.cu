// Weight gradient of a stride-1 convolution with the taps of one filter row served by ONE activation tile.
//
//     dW[co, (ty, tx), ci] = sum over positions m of  dY[m, co] * X[m + ty * PW + tx, ci]
//
// with the positions of the zero-padded image flattened at pitch PW >= out_width + KW - 1, as in conv_halo.cu (dY is
// loaded through a box that is wider than the image, so the padded positions arrive as zeros and add nothing).  The
// reduction runs over positions: both operands are MN-major tiles [position rows][64 channels x 2 bytes], straight
// from 4-D TMA box loads.  The box kernel (conv_tc.cu, weight-gradient mode) loads one activation panel per tap and
// asks L2 for about 94 bytes per clock per SM, twice what it delivers.  Here the B operand of an MMA is up to four
// N panels of 64 input channels whose leading-dimension byte offset is 128: panel j starts ONE ROW later than
// panel j - 1, which makes it the same tile shifted by one position - tap tx + j.  One 128 x 256 x 16 MMA therefore
// covers four taps of a filter row from a single tile in shared memory, and a 5 x 5 filter row costs one activation
// tile + one gradient tile per 128 positions instead of five + two.
//
// The accumulators of a work item - 128 output channels x (TY filter rows x KW taps x 64 input channels) - stay in
// TMEM while the item walks its slice of the positions (TY * KW * 64 <= 512 columns: one filter row of a 5 x 5 or
// 7 x 7 filter, two rows of a 3 x 3), and leave at the end through fp32 slabs and TMA reduce-add into dW (several
// items - slices, filter rows - add into the same rows, so dW is zeroed first).  Roles and bounded waits as in
// conv_halo.cu.  conv_tc() routes a weight-gradient call here when geeps_conv_wgrad_halo_applicable() says so;
// GEEPS_HALO_CONV=0 keeps everything on the box kernel.
#include <cuda.h>
#include <mutex>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "kernels.h"
#include "tc05.cuh"

namespace {

constexpr int BM = 128;                       // output channels per item (TMEM lanes)
constexpr int UMMA_K = 16;
constexpr int MAX_STAGES = 6;
constexpr uint64_t WAIT_BUDGET_NS = 2000000000ull;
constexpr int C_SLAB_BYTES = BM * 128;        // 128 output channels x 32 fp32
constexpr int MAX_COLS = 512;

struct WgDev {
  int* status;
  int KH, KW, taps, cchunks, m_tiles;
  int PW, R, pad, GH;                  // flat pitch, image rows per position block, padding, output rows
  int kpos;                            // positions per block = R * PW (a multiple of 16)
  int TY, passes;                      // filter rows per item, items per filter
  int row_tiles, n_blocks, split;      // position blocks = images * row_tiles, sliced `split` ways
  int panel_bytes, x_bytes, stage_bytes, stages, tmem_cols;
  int ch_valid;                        // input channels (dW's innermost extent)
};

struct SmemCtl {
  uint64_t full[MAX_STAGES], empty[MAX_STAGES];
  uint64_t tmem_full, tmem_empty;
  uint32_t tmem_base;
  int abort_flag;
};

struct Item { int mi, cc, ty0, nty, blk_begin, blk_end; };
__device__ __forceinline__ Item decode_item(const WgDev& d, int w) {
  Item it;
  const int z = w % d.split;
  int rest = w / d.split;
  const int pass = rest % d.passes; rest /= d.passes;
  it.cc = rest % d.cchunks;
  it.mi = rest / d.cchunks;
  it.ty0 = pass * d.TY;
  it.nty = min(d.TY, d.KH - it.ty0);
  const int per = (d.n_blocks + d.split - 1) / d.split;
  it.blk_begin = z * per;
  it.blk_end = min(d.n_blocks, it.blk_begin + per);
  return it;
}

// tmY: dY as (co, w, h, b) with box (64, PW, R, 1); tmX: X as (ci, w, h, b) with box (64, PW, R + TY - 1, 1);
// tmW: dW as (ci, tap, co) fp32 with box (32, 1, 128).
__global__ void __launch_bounds__(192, 1)
conv_wgrad_halo_kernel(const __grid_constant__ CUtensorMap tmY, const __grid_constant__ CUtensorMap tmX,
                       const __grid_constant__ CUtensorMap tmW, const WgDev d) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* cslab = tiles + (size_t)d.stages * d.stage_bytes;
  SmemCtl* ctl = (SmemCtl*)(cslab + 2 * C_SLAB_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_items = d.m_tiles * d.cchunks * d.passes * d.split;

  if (threadIdx.x == 0) {
    for (int s = 0; s < d.stages; ++s) { tc05::mbar_init(&ctl->full[s], 1); tc05::mbar_init(&ctl->empty[s], 1); }
    tc05::mbar_init(&ctl->tmem_full, 1);
    tc05::mbar_init(&ctl->tmem_empty, 4);
    ctl->abort_flag = 0;
    tc05::mbar_fence_init();
  }
  {
    // the shifted panels read a few rows past the activation tile: they meet zero rows of dY only, but must be finite
    uint4* z = reinterpret_cast<uint4*>(tiles);
    const int n16 = d.stages * d.stage_bytes / 16;
    for (int i = threadIdx.x; i < n16; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
    tc05::fence_proxy_async_smem();
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
    // ---------------- TMA producer: per position block two gradient panels and one activation tile ----------------
    const bool leader = tc05::elect_one();
    if (leader) { tc05::tma_prefetch_desc(&tmY); tc05::tma_prefetch_desc(&tmX); }
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
      const Item it = decode_item(d, w);
      // (a last pass with fewer filter rows than TY still loads the TY-row box: one tensor map serves all passes)
      const uint32_t tx_bytes = (uint32_t)(2 * d.panel_bytes + (d.R + d.TY - 1) * d.PW * 128);
      int b = it.blk_begin / d.row_tiles, rt = it.blk_begin - b * d.row_tiles;
      for (int blk = it.blk_begin; blk < it.blk_end; ++blk) {
        if (!tc05::mbar_wait_warp(&ctl->empty[s], ph ^ 1u, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
        if (leader) {
          uint8_t* st = tiles + (size_t)s * d.stage_bytes;
          const int y0 = rt * d.R;
          tc05::mbar_expect_tx(&ctl->full[s], tx_bytes);
          tc05::tma_load_4d(st, &tmY, &ctl->full[s], it.mi * BM, 0, y0, b);
          tc05::tma_load_4d(st + d.panel_bytes, &tmY, &ctl->full[s], it.mi * BM + 64, 0, y0, b);
          tc05::tma_load_4d(st + 2 * d.panel_bytes, &tmX, &ctl->full[s], it.cc * 64, -d.pad, y0 + it.ty0 - d.pad, b);
        }
        if (++s == d.stages) { s = 0; ph ^= 1u; }
        if (++rt == d.row_tiles) { rt = 0; ++b; }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    const bool leader = tc05::elect_one();
    constexpr uint32_t d_hi = tc05::desc_hi(1024);
    const uint32_t ksteps = (uint32_t)(d.kpos / UMMA_K);
    uint32_t item_i = 0, ph = 0;
    int s = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x, ++item_i) {
      const Item it = decode_item(d, w);
      // the epilogue must have drained the accumulators of the previous item
      if (!tc05::mbar_wait_warp(&ctl->tmem_empty, (item_i & 1u) ^ 1u, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
      tc05::fence_after_sync();
      uint32_t accumulate = 0;
      for (int blk = it.blk_begin; blk < it.blk_end; ++blk) {
        if (!tc05::mbar_wait_warp(&ctl->full[s], ph, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
        tc05::fence_after_sync();
        if (leader) {
          const uint32_t st = tc05::smem_u32(tiles + (size_t)s * d.stage_bytes);
          // A: dY^T, M = 128 output channels in two panels one panel apart, K = positions (16 rows = 2048 bytes)
          const uint32_t a_lo = tc05::desc_lo(st, (uint32_t)d.panel_bytes);
          // B: X, N = 64 input channels per tap, the panel of tap tx + 1 one row (128 bytes) after that of tap tx
          const uint32_t b_lo0 = tc05::desc_lo(st + 2 * d.panel_bytes, 128);
          uint32_t col = 0;
          for (int ty = 0; ty < it.nty; ++ty) {
            for (int tx0 = 0; tx0 < d.KW; tx0 += 4) {
              const int nt = min(4, d.KW - tx0);
              const uint32_t idesc = tc05::make_idesc_bf16(BM, nt * 64, 1, 1);
              const uint32_t b_lo = b_lo0 + (uint32_t)((ty * d.PW + tx0) * 8);
              const uint32_t tacc = tmem + col;
              for (uint32_t ks = 0; ks < ksteps; ++ks)
                tc05::mma_bf16_ss_lohi(tacc, a_lo + ks * 128u, d_hi, b_lo + ks * 128u, d_hi, idesc,
                                       (ks == 0) ? accumulate : 1u);
              col += (uint32_t)(nt * 64);
            }
          }
          tc05::mma_commit(&ctl->empty[s]);
        }
        accumulate = 1u;
        if (++s == d.stages) { s = 0; ph ^= 1u; }
      }
      if (ok && leader) tc05::mma_commit(&ctl->tmem_full);
    }
  } else {
    // ---------------- epilogue: one fp32 slab of 32 input channels per (tap, half chunk), reduce-added into dW ----------------
    const int q = warp & 3;
    const bool issuer = threadIdx.x == 64;
    const int rloc = q * 32 + lane;
    const uint32_t row_off = (uint32_t)rloc * 128u, rsw = (uint32_t)(rloc & 7);
    uint32_t item_i = 0, slab_i = 0;
    for (int w = blockIdx.x; w < num_items; w += gridDim.x, ++item_i) {
      const Item it = decode_item(d, w);
      if (!tc05::mbar_wait(&ctl->tmem_full, item_i & 1u, abort_flag, WAIT_BUDGET_NS)) break;
      tc05::fence_after_sync();
      const uint32_t tacc = tmem + ((uint32_t)(q * 32) << 16);
      const int ntap = it.nty * d.KW;
#pragma unroll 1
      for (int tp = 0; tp < ntap; ++tp) {
#pragma unroll 1
        for (int h = 0; h < 64; h += 32) {
          const int x = it.cc * 64 + h;
          if (x >= d.ch_valid) break;                      // never start a store past the extent
          uint8_t* slab = cslab + (size_t)(slab_i & 1u) * C_SLAB_BYTES;
          if (issuer) tc05::bulk_wait_read<1>();
          tc05::named_bar_sync(1, 128);
          uint32_t r[32];
          tc05::tmem_ld_32x32(tacc + (uint32_t)(tp * 64 + h), r);
          tc05::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t off = row_off + (uint32_t)((j ^ rsw) << 4);
            *reinterpret_cast<uint4*>(slab + off) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          }
          tc05::fence_proxy_async_smem();
          tc05::named_bar_sync(1, 128);
          if (issuer) {
            tc05::tma_reduce_add_3d(&tmW, slab, x, it.ty0 * d.KW + tp, it.mi * BM);
            tc05::bulk_commit();
          }
          ++slab_i;
        }
      }
      tc05::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive(&ctl->tmem_empty);
    }
    if (issuer) tc05::bulk_wait<0>();
  }

  tc05::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && ctl->abort_flag)
    geeps_report(d.status, GEEPS_ERR_TIMEOUT, KID_CONV_TC, (int)blockIdx.x, 2);
  if (warp == 1) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc(tmem, (uint32_t)d.tmem_cols);
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
bool make_map(CUtensorMap* map, const void* base, bool fp32, int rank, const long long* dims,
              const long long* strides_bytes, const int* box) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t gd[4], gs[3];
  cuuint32_t bx[4], es[4];
  for (int i = 0; i < rank; ++i) { gd[i] = (cuuint64_t)dims[i]; bx[i] = (cuuint32_t)box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = (cuuint64_t)strides_bytes[i];
  return fn(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank,
            const_cast<void*>(base), gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
bool make_act_map(CUtensorMap* map, const void* base, int ch, int W, int H, int B, long long pitch, int bw, int bh) {
  const long long dims[4] = {ch, W, H, B};
  const long long st[3] = {pitch * 2, pitch * 2 * W, pitch * 2 * W * H};
  const int box[4] = {64, bw, bh, 1};
  return make_map(map, base, false, 4, dims, st, box);
}
int round_up(long long v, int m) { return (int)((v + m - 1) / m * m); }

struct WgPlan { WgDev d; size_t smem; double util; bool ok; };

WgPlan plan_wgrad(const GeepsConvTcParams* p) {
  WgPlan wp;
  wp.ok = false;
  wp.smem = 0;
  wp.util = 0;
  WgDev& d = wp.d;
  memset(&d, 0, sizeof(d));
  if (p->mode != 2 || p->stride > 1) return wp;
  d.KH = p->KH; d.KW = p->KW; d.taps = p->KH * p->KW; d.pad = p->pad; d.GH = p->OH;
  if (d.KW * 64 > MAX_COLS || d.taps < 2) return wp;
  // positions per block: R image rows at a pitch that makes R * PW a multiple of 16 (the MMA's k step), <= 128
  bool found = false;
  for (int pw = p->OW + p->KW - 1; pw <= p->OW + p->KW + 14 && pw <= 128; ++pw) {
    const int r = 128 / pw;
    if (r < 1 || (r * pw) % 16) continue;
    d.PW = pw; d.R = r < p->OH ? r : p->OH;
    if ((d.R * pw) % 16) continue;
    found = true;
    break;
  }
  if (!found) return wp;
  d.kpos = d.R * d.PW;
  d.TY = MAX_COLS / (d.KW * 64);
  if (d.TY > d.KH) d.TY = d.KH;
  d.passes = (d.KH + d.TY - 1) / d.TY;
  d.cchunks = (p->cg + 63) / 64;
  d.m_tiles = (p->og + BM - 1) / BM;
  d.ch_valid = p->cg;
  d.row_tiles = (p->OH + d.R - 1) / d.R;
  d.n_blocks = p->B * d.row_tiles;
  d.panel_bytes = d.kpos * 128;
  // activation tile: (R + TY - 1) rows of PW positions, plus the rows the last taps read past it
  d.x_bytes = round_up((long long)((d.R + d.TY - 1) * d.PW + d.KW) * 128, 1024);
  d.stage_bytes = 2 * d.panel_bytes + d.x_bytes;
  d.stages = (int)((212 * 1024 - 2 * C_SLAB_BYTES) / d.stage_bytes);
  if (d.stages > MAX_STAGES) d.stages = MAX_STAGES;
  if (d.stages < 2) return wp;
  int tc = 32;
  while (tc < d.TY * d.KW * 64) tc <<= 1;
  d.tmem_cols = tc;
  // slices of the positions: at most two items per SM (one more would add a third round for a few SMs)
  const long long base_items = (long long)d.m_tiles * d.cchunks * d.passes;
  long long split = (2LL * geeps_sm_count()) / base_items;
  if (split > d.n_blocks) split = d.n_blocks;
  if (split < 1) split = 1;
  const int per = (int)((d.n_blocks + split - 1) / split);
  d.split = (d.n_blocks + per - 1) / per;            // every slice non-empty
  wp.smem = (size_t)d.stages * d.stage_bytes + 2 * C_SLAB_BYTES + sizeof(SmemCtl) + 1024;
  wp.util = (double)p->OH * p->OW / ((double)d.row_tiles * d.kpos);
  wp.ok = true;
  return wp;
}

int halo_mode() {
  static int m = -1;
  if (m < 0) { const char* e = getenv("GEEPS_HALO_CONV"); m = e ? atoi(e) : 1; }
  return m;
}

}  // namespace

extern "C" {

// 1 when conv_tc() should route this weight-gradient call here.  Fitted to timings of both kernels at batch 128 .. 256
// (python -m geeps_b200.utils.microbench conv): filter rows of 5 taps or more always win (AlexNet conv2 0.103 ->
// 0.087 ms per group, Inception 5 x 5 0.054 -> 0.050 ms); 3-tap rows only when the layer is one item wide (one block
// of output channels, one chunk of input channels: AlexNet conv1 0.120 -> 0.112 ms) - wider 3 x 3 layers are faster
// on the box kernel, which covers four (tap, chunk) panels per MMA whatever the filter's shape.
int geeps_conv_wgrad_halo_applicable(const GeepsConvTcParams* p) {
  if (!halo_mode()) return 0;
  if (!geeps_conv_tc_supported(p)) return 0;
  const WgPlan wp = plan_wgrad(p);
  if (!wp.ok) return 0;
  const int tail = p->cg - (wp.d.cchunks - 1) * 64;
  if (tail < 32 || wp.util < 0.6 || wp.d.n_blocks < 4 * geeps_sm_count()) return 0;
  return p->KW >= 5 || (p->KW >= 3 && wp.d.m_tiles == 1 && wp.d.cchunks == 1) ? 1 : 0;
}

int geeps_conv_wgrad_halo_plan(const GeepsConvTcParams* p, GeepsHaloPlanInfo* out) {
  memset(out, 0, sizeof(*out));
  if (!geeps_conv_tc_supported(p)) return 0;
  const WgPlan wp = plan_wgrad(p);
  if (!wp.ok) return 0;
  const WgDev& d = wp.d;
  out->ok = 1;
  out->routed = geeps_conv_wgrad_halo_applicable(p);
  out->PW = d.PW; out->R = d.R; out->row_tiles = d.row_tiles; out->m_tiles = d.m_tiles;
  out->positions = d.kpos;
  out->TY = d.TY; out->passes = d.passes; out->split = d.split; out->n_blocks = d.n_blocks;
  out->stages_x = d.stages; out->stages_w = d.stages; out->x_stage_bytes = d.x_bytes;
  out->tmem_cols = d.tmem_cols;
  out->smem_bytes = (long long)wp.smem;
  out->util = wp.util;
  return 1;
}

int geeps_conv_wgrad_halo(const GeepsConvTcParams* p, void* stream) {
  if (!geeps_conv_tc_supported(p)) return (int)cudaErrorInvalidValue;
  WgPlan wp = plan_wgrad(p);
  if (!wp.ok) return (int)cudaErrorInvalidValue;
  WgDev& d = wp.d;
  d.status = p->status;
  CUtensorMap ty, tx, tw;
  bool ok = make_act_map(&ty, p->y, p->og, p->OW, p->OH, p->B, p->y_pitch, d.PW, d.R);
  ok = ok && make_act_map(&tx, p->x, p->cg, p->W, p->H, p->B, p->x_pitch, d.PW, d.R + d.TY - 1);
  const long long wdims[3] = {p->cg, d.taps, p->og};
  const long long wst[2] = {(long long)p->cg * 4, p->ldw * 4};
  const int wbox[3] = {32, 1, BM};
  ok = ok && make_map(&tw, p->w, true, 3, wdims, wst, wbox);
  if (!ok) return (int)cudaErrorInvalidValue;
  // every item reduce-adds: the whole [og][ldw] block starts at zero (pad columns past the last tap included)
  int e = geeps_scale_matrix_f32((float*)p->w, p->og, p->ldw, p->ldw, 0.f, stream);
  if (e) return e;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t ce = cudaFuncSetAttribute(conv_wgrad_halo_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
    if (ce != cudaSuccess) return (int)ce;
    attr_set = true;
  }
  const long long items = (long long)d.m_tiles * d.cchunks * d.passes * d.split;
  const int sms = geeps_sm_count();
  const int grid = (int)(items < sms ? items : sms);
  conv_wgrad_halo_kernel<<<grid, 192, wp.smem, (cudaStream_t)stream>>>(ty, tx, tw, d);
  return (int)cudaGetLastError();
}

}  // extern "C"
