// Local response normalisation across channels fused with the max pooling that follows it (AlexNet pairs
// them after conv1 and conv2), forward and backward, on NHWC bf16 activations.
//
// Unfused, the pair moves the full-resolution tensor five times per direction: LRN forward writes y and
// 1/scale, pooling reads y; pooling backward writes the full-resolution gradient, LRN backward reads it together
// with x, y and 1/scale.  Here the normalised tensor and its gradient never reach global memory:
//
//   forward   one CTA per output row: the K input rows go to shared memory, LRN is evaluated there once per
//             element, the pooled row and the window codes leave.          traffic: x in, pooled + codes out
//   backward  one CTA per block of input rows: x rows, the covering pooled-gradient rows and their codes go to
//             shared memory; the pooling gradient, scale = k + alpha/n * window sum of x^2, scale^-beta and the
//             cross-channel term are recomputed from them; dx leaves with the ReLU mask of the producing
//             convolution applied and its per-channel sums (that convolution's bias gradient) accumulated.
//                                                                          traffic: x, pooled gradient, codes in, dx out
//
// Nothing of the forward pass is kept for the backward pass except the window codes (one byte per pooled
// element).  The reference has no layer kernels of its own (they lived in its Caffe application).
#include <math.h>
#include <stdlib.h>

#include "common.cuh"
#include "nn_ops.h"

namespace {

typedef __nv_bfloat16 bf16;

// ---- arithmetic of the normalisation ----
// scale = k + alpha/n * w = k * (1 + eps), w = window sum of x^2, eps = alpha / (n k) * w.  The two powers the
// kernels need are scale^-beta = k^-beta (1+eps)^-beta and scale^-(beta+1).  For eps <= kPolyEps both are
// evaluated as cubic Taylor polynomials, written directly in w (the coefficients carry the powers of alpha/(n k)),
// with a relative error below 4e-4 at the bound - far below the bf16 rounding of the results; only a vector with a
// larger eps takes the special-function path.  These kernels are bound by instruction issue, not by memory: the
// special-function unit runs at a quarter of the FMA rate and every avoided instruction per element counts.
constexpr float kPolyEps = 0.1f;
struct LrnCoef {
  float w_max;              // window sums up to this take the polynomial
  float p0, p1, p2, p3;     // scale^-beta     ~ p0 + w (p1 + w (p2 + w p3))
  float q0, q1, q2, q3;     // scale^-(beta+1) ~ q0 + w (q1 + w (q2 + w q3))
  float es, beta, k;        // exact path: scale = k * (1 + es * w)
};
__device__ __forceinline__ float max8(const float (&w)[8]) {
  return fmaxf(fmaxf(fmaxf(w[0], w[1]), fmaxf(w[2], w[3])), fmaxf(fmaxf(w[4], w[5]), fmaxf(w[6], w[7])));
}

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// The channels [c-4, c+12) of one pixel as floats (zero outside [0, C)): one 16-byte and two 8-byte loads.
// Works on global and shared pointers alike; c is a multiple of 8.
__device__ __forceinline__ void load16(const bf16* px, int c, int C, float (&v)[16]) {
  uint2 lo = make_uint2(0u, 0u), hi = make_uint2(0u, 0u);
  if (c > 0) lo = *reinterpret_cast<const uint2*>(px + c - 4);
  const uint4 mid = *reinterpret_cast<const uint4*>(px + c);
  if (c + 8 < C) hi = *reinterpret_cast<const uint2*>(px + c + 8);
  v[0] = bf_lo(lo.x); v[1] = bf_hi(lo.x); v[2] = bf_lo(lo.y); v[3] = bf_hi(lo.y);
  v[4] = bf_lo(mid.x); v[5] = bf_hi(mid.x); v[6] = bf_lo(mid.y); v[7] = bf_hi(mid.y);
  v[8] = bf_lo(mid.z); v[9] = bf_hi(mid.z); v[10] = bf_lo(mid.w); v[11] = bf_hi(mid.w);
  v[12] = bf_lo(hi.x); v[13] = bf_hi(hi.x); v[14] = bf_lo(hi.y); v[15] = bf_hi(hi.y);
}
// window sums of 2*HALF+1 consecutive entries around index 4+e, e = 0..7 (sliding)
template <int HALF>
__device__ __forceinline__ void window8(const float (&t)[16], float (&w)[8]) {
  float acc = 0.f;
#pragma unroll
  for (int j = 4 - HALF; j <= 4 + HALF; ++j) acc += t[j];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    w[e] = acc;
    if (e < 7) acc += t[4 + e + HALF + 1] - t[4 + e - HALF];
  }
}
__device__ __forceinline__ uint4 pack8(const float (&o)[8]) {
  return make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
}

// Walks the items (row, pixel, channel vector) of a [rows][W][cv] block in row-major order, `nt` items at a time,
// without a division per item.
struct ItemWalk {
  int r, w, cvi, dq, dc;
  __device__ __forceinline__ ItemWalk(int first, int nt, int W, int cv) {
    cvi = first % cv;
    const int t = first / cv;
    w = t % W;
    r = t / W;
    dq = nt / cv;
    dc = nt - dq * cv;
  }
  __device__ __forceinline__ void next(int W, int cv) {
    cvi += dc;
    w += dq;
    if (cvi >= cv) { cvi -= cv; ++w; }
    while (w >= W) { w -= W; ++r; }
  }
};

// ---------------- forward ----------------
// grid = B * ceil(OH / RO); one CTA produces RO pooled rows from the (RO-1)*stride + K input rows under them.
// The input is read from global memory (one 16-byte and two 8-byte loads per 8 outputs), normalised once per
// element into shared memory ([n_in][W][C] bf16), and pooled from there.
// K3S2: 3 x 3 windows with stride 2 (window size and stride are then constants of the pooling loops)
template <int HALF, bool K3S2>
__global__ void __launch_bounds__(512)
lrn_maxpool_forward_kernel(const bf16* __restrict__ x, bf16* __restrict__ p, uint8_t* __restrict__ argmax,
                           const GeepsPoolGeom g, const LrnCoef cf, int RO) {
  extern __shared__ __align__(16) uint8_t lp_smem[];
  const int C = g.C, cv = C >> 3, W = g.W;
  const int PK = K3S2 ? 3 : g.K, PS = K3S2 ? 2 : g.stride;
  const int row_elems = W * C;
  bf16* ys = reinterpret_cast<bf16*>(lp_smem);
  const int oh_blocks = (g.OH + RO - 1) / RO;
  const int b = blockIdx.x / oh_blocks, oh0 = (blockIdx.x - b * oh_blocks) * RO;
  const int n_out = min(RO, g.OH - oh0);
  const int ih_base = oh0 * PS - g.pad;                    // input row of shared-memory row 0 (may be < 0)
  const int r_lo = max(0, -ih_base);
  const int r_hi = min((n_out - 1) * PS + PK, g.H - ih_base);   // rows [r_lo, r_hi) exist
  const int tid = threadIdx.x, nt = blockDim.x;
  {
    const bf16* xbase = x + ((long long)b * g.H + ih_base + r_lo) * row_elems;
    bf16* ybase = ys + (size_t)r_lo * row_elems;
    const int nrows = r_hi - r_lo;
    for (ItemWalk it(tid, nt, W, cv); it.r < nrows; it.next(W, cv)) {
      const int c = it.cvi * 8;
      const int pix = it.r * row_elems + it.w * C;          // offsets inside a block of a few rows: 32 bits
      float v[16], t[16], ws[8], o[8];
      load16(xbase + pix, c, C, v);
#pragma unroll
      for (int j = 0; j < 16; ++j) t[j] = v[j] * v[j];
      window8<HALF>(t, ws);
      if (max8(ws) <= cf.w_max) {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = v[4 + e] * fmaf(ws[e], fmaf(ws[e], fmaf(ws[e], cf.p3, cf.p2), cf.p1), cf.p0);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = v[4 + e] * __powf(cf.k * fmaf(cf.es, ws[e], 1.f), -cf.beta);
      }
      *reinterpret_cast<uint4*>(ybase + pix + c) = pack8(o);
    }
  }
  __syncthreads();
  for (ItemWalk it(tid, nt, g.OW, cv); it.r < n_out; it.next(g.OW, cv)) {
    const int oh = oh0 + it.r, ow = it.w, c = it.cvi * 8;
    const int ih0 = oh * PS - g.pad;
    const int kh_lo = max(0, -ih0), kh_hi = min(PK, g.H - ih0);
    const int iw0 = ow * PS - g.pad;
    const int kw_lo = max(0, -iw0), kw_hi = min(PK, W - iw0);
    // packed: best value and window code per 16-bit lane; strict > keeps the first maximum
    const uint32_t neg = 0xff7fff7fu;                 // two bf16 lowest finite values
    __nv_bfloat162 best[4];
    uint32_t arg[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) { best[j] = *reinterpret_cast<const __nv_bfloat162*>(&neg); arg[j] = 0x00ff00ffu; }
    for (int kh = kh_lo; kh < kh_hi; ++kh) {
      const bf16* yr = ys + (ih0 + kh - ih_base) * row_elems + c;
      for (int kw = kw_lo; kw < kw_hi; ++kw) {
        const uint4 v = *reinterpret_cast<const uint4*>(yr + (iw0 + kw) * C);
        const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
        const uint32_t code1 = (uint32_t)(kh * PK + kw);
        const uint32_t code = code1 | (code1 << 16);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat162 x2 = *reinterpret_cast<const __nv_bfloat162*>(&vv[j]);
          const uint32_t gt = __hgt2_mask(x2, best[j]);
          best[j] = __hmax2(best[j], x2);
          arg[j] = (arg[j] & ~gt) | (code & gt);
        }
      }
    }
    const long long opix = ((long long)b * g.OH + oh) * g.OW + ow;
    *reinterpret_cast<uint4*>(p + opix * g.ldy + c) =
        make_uint4(*reinterpret_cast<const uint32_t*>(&best[0]), *reinterpret_cast<const uint32_t*>(&best[1]),
                   *reinterpret_cast<const uint32_t*>(&best[2]), *reinterpret_cast<const uint32_t*>(&best[3]));
    uint2 pk;      // 16-bit lanes -> bytes
    pk.x = __byte_perm(arg[0], arg[1], 0x6420);
    pk.y = __byte_perm(arg[2], arg[3], 0x6420);
    *reinterpret_cast<uint2*>(argmax + opix * C + c) = pk;
  }
}

// ---------------- backward ----------------
// Persistent: CTA i handles row blocks i, i + gridDim, ... (a row block = R input rows of one image).
// Shared memory: as, rs [R][W][C] bf16, dps [max_oh][OW][C] bf16, args [max_oh][OW][C] u8, cs [C] float.
//   as = dy * scale^-beta          rs = dy * x * scale^-(beta+1)       (dy = pooling gradient at the element)
//   dx = as - 2 alpha beta / n * x * (window sum of rs)
// The host picks blockDim as a multiple of C/8, so a thread keeps its channel vector for every item it visits and
// sums the bias gradient in registers.
// K3S2: the pooling window is 3 x 3 with stride 2 (AlexNet): window size and stride become constants, so the four
// divisions per pixel vector that find the windows covering it are shifts.
template <int HALF, bool K3S2>
__global__ void __launch_bounds__(512, 2)
lrn_maxpool_backward_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dp, const uint8_t* __restrict__ argmax,
                            bf16* __restrict__ dx, const GeepsPoolGeom g, int R, int max_oh, const LrnCoef cf, float coef,
                            int relu_mask, float* __restrict__ colsum) {
  extern __shared__ __align__(16) uint8_t lp_smem[];
  const int C = g.C, cv = C >> 3, W = g.W, OW = g.OW;
  const int PK = K3S2 ? 3 : g.K, PS = K3S2 ? 2 : g.stride;
  const int row_elems = W * C, orow_elems = OW * C;
  bf16* as = reinterpret_cast<bf16*>(lp_smem);
  bf16* rs = as + (size_t)R * row_elems;
  bf16* dps = rs + (size_t)R * row_elems;
  uint8_t* args = reinterpret_cast<uint8_t*>(dps + (size_t)max_oh * orow_elems);
  float* cs_sh = reinterpret_cast<float*>(args + (((size_t)max_oh * orow_elems + 15) & ~(size_t)15));
  const int tid = threadIdx.x, nt = blockDim.x;
  const int row_blocks = (g.H + R - 1) / R;
  const int total_blocks = g.B * row_blocks;
  const bool fixed_channel = nt % cv == 0;
  float cs[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) cs[e] = 0.f;
  if (colsum != nullptr) for (int j = tid; j < C; j += nt) cs_sh[j] = 0.f;

  for (int blk = blockIdx.x; blk < total_blocks; blk += gridDim.x) {
    const int b = blk / row_blocks, h0 = (blk - b * row_blocks) * R;
    const int nr = min(R, g.H - h0);
    const int oh_lo = max(0, (h0 + g.pad - PK + PS) / PS);
    const int oh_hi = min(g.OH - 1, (h0 + nr - 1 + g.pad) / PS);
    __syncthreads();                                   // the previous block's readers are done with the buffers
    {
      const long long opix0 = ((long long)b * g.OH + oh_lo) * OW;
      uint4* dd = reinterpret_cast<uint4*>(dps);
      uint2* da = reinterpret_cast<uint2*>(args);
      int i = tid;
      for (ItemWalk it(tid, nt, OW, cv); it.r <= oh_hi - oh_lo; it.next(OW, cv), i += nt) {
        const long long opix = opix0 + (long long)it.r * OW + it.w;
        dd[i] = *reinterpret_cast<const uint4*>(dp + opix * g.ldy + it.cvi * 8);
        da[i] = *reinterpret_cast<const uint2*>(argmax + opix * C + it.cvi * 8);
      }
    }
    __syncthreads();
    const bf16* xblk = x + ((long long)b * g.H + h0) * row_elems;
    // phase 2: pooling gradient; where it is non-zero, the two powers of the scale
    for (ItemWalk it(tid, nt, W, cv); it.r < nr; it.next(W, cv)) {
      const int c = it.cvi * 8;
      const int th = h0 + it.r + g.pad, tw = it.w + g.pad;
      const int roh_lo = max(oh_lo, (th - PK + PS) / PS), roh_hi = min(oh_hi, th / PS);
      const int ow_lo = max(0, (tw - PK + PS) / PS), ow_hi = min(OW - 1, tw / PS);
      float dy[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) dy[e] = 0.f;
      bool any = false;
      for (int oh = roh_lo; oh <= roh_hi; ++oh) {
        const uint32_t code_h = (uint32_t)((th - oh * PS) * PK + tw);
        for (int ow = ow_lo; ow <= ow_hi; ++ow) {
          const uint32_t code = code_h - (uint32_t)(ow * PS);
          const int o = (oh - oh_lo) * orow_elems + ow * C + c;
          const uint2 pk = *reinterpret_cast<const uint2*>(args + o);
          const uint32_t c4 = code * 0x01010101u;
          const uint32_t m0 = __vcmpeq4(pk.x, c4), m1 = __vcmpeq4(pk.y, c4);      // 0xff per matching channel
          if ((m0 | m1) == 0) continue;
          any = true;
          const uint4 d = *reinterpret_cast<const uint4*>(dps + o);
          // keep the gradients of the matching channels: byte mask -> 16-bit lane mask
          const uint32_t k0 = d.x & __byte_perm(m0, 0, 0x1100), k1 = d.y & __byte_perm(m0, 0, 0x3322);
          const uint32_t k2 = d.z & __byte_perm(m1, 0, 0x1100), k3 = d.w & __byte_perm(m1, 0, 0x3322);
          dy[0] += bf_lo(k0); dy[1] += bf_hi(k0); dy[2] += bf_lo(k1); dy[3] += bf_hi(k1);
          dy[4] += bf_lo(k2); dy[5] += bf_hi(k2); dy[6] += bf_lo(k3); dy[7] += bf_hi(k3);
        }
      }
      const int pix = it.r * row_elems + it.w * C;          // offsets inside a block of a few rows: 32 bits
      uint4 oa = make_uint4(0u, 0u, 0u, 0u), orat = make_uint4(0u, 0u, 0u, 0u);
      if (any) {
        float v[16], t[16], ws[8], a[8], rt[8];
        load16(xblk + pix, c, C, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) t[j] = v[j] * v[j];
        window8<HALF>(t, ws);
        if (max8(ws) <= cf.w_max) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            a[e] = dy[e] * fmaf(ws[e], fmaf(ws[e], fmaf(ws[e], cf.p3, cf.p2), cf.p1), cf.p0);
            rt[e] = dy[e] * v[4 + e] * fmaf(ws[e], fmaf(ws[e], fmaf(ws[e], cf.q3, cf.q2), cf.q1), cf.q0);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float sc = cf.k * fmaf(cf.es, ws[e], 1.f);
            a[e] = dy[e] * __powf(sc, -cf.beta);
            rt[e] = a[e] * v[4 + e] * __frcp_rn(sc);
          }
        }
        oa = pack8(a);
        orat = pack8(rt);
      }
      *reinterpret_cast<uint4*>(as + pix + c) = oa;
      *reinterpret_cast<uint4*>(rs + pix + c) = orat;
    }
    __syncthreads();
    // phase 3: dx = a - coef * x * (window sum of ratio), ReLU mask, per-channel sums
    bf16* dblk = dx + ((long long)b * g.H + h0) * row_elems;
    for (ItemWalk it(tid, nt, W, cv); it.r < nr; it.next(W, cv)) {
      const int c = it.cvi * 8;
      const int pix = it.r * row_elems + it.w * C;          // offsets inside a block of a few rows: 32 bits
      float rt[16], ws[8], o[8];
      load16(rs + pix, c, C, rt);
      window8<HALF>(rt, ws);
      const uint4 xv = *reinterpret_cast<const uint4*>(xblk + pix + c);
      const uint4 av = *reinterpret_cast<const uint4*>(as + pix + c);
      const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, aw[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float x0 = bf_lo(xw[j]), x1 = bf_hi(xw[j]);
        const float d0 = fmaf(-coef * x0, ws[2 * j], bf_lo(aw[j])), d1 = fmaf(-coef * x1, ws[2 * j + 1], bf_hi(aw[j]));
        o[2 * j] = (relu_mask && x0 <= 0.f) ? 0.f : d0;
        o[2 * j + 1] = (relu_mask && x1 <= 0.f) ? 0.f : d1;
      }
      *reinterpret_cast<uint4*>(dblk + pix + c) = pack8(o);
      if (colsum != nullptr) {
        if (fixed_channel) {
#pragma unroll
          for (int e = 0; e < 8; ++e) cs[e] += o[e];
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) atomicAdd(&cs_sh[c + e], o[e]);
        }
      }
    }
  }
  if (colsum != nullptr) {
    __syncthreads();
    if (fixed_channel) {
      const int c = (tid % cv) * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) atomicAdd(&cs_sh[c + e], cs[e]);
    }
    __syncthreads();
    for (int j = tid; j < C; j += nt) atomicAdd(colsum + j, cs_sh[j]);
  }
}

LrnCoef make_coef(int size, float alpha, float beta, float k) {
  LrnCoef cf;
  cf.beta = beta; cf.k = k;
  const double es = (double)alpha / ((double)size * k);
  cf.es = (float)es;
  cf.w_max = (float)(kPolyEps / es);
  const double b0 = beta, b1 = beta + 1.0;
  const double p0 = pow((double)k, -b0), q0 = pow((double)k, -b1);
  cf.p0 = (float)p0;
  cf.p1 = (float)(p0 * -b0 * es);
  cf.p2 = (float)(p0 * b0 * (b0 + 1) / 2 * es * es);
  cf.p3 = (float)(p0 * -b0 * (b0 + 1) * (b0 + 2) / 6 * es * es * es);
  cf.q0 = (float)q0;
  cf.q1 = (float)(q0 * -b1 * es);
  cf.q2 = (float)(q0 * b1 * (b1 + 1) / 2 * es * es);
  cf.q3 = (float)(q0 * -b1 * (b1 + 1) * (b1 + 2) / 6 * es * es * es);
  return cf;
}

// 1-D blocks whose size is a multiple of the channel-vector count where that is possible
int lp_threads(int cv, int max_threads) {
  if (cv >= max_threads) return max_threads;
  return max_threads / cv * cv;
}


bool lp_shape_ok(const GeepsPoolGeom* g, int size) {
  return g->C % 8 == 0 && g->ldx == g->C && g->ldy % 8 == 0 && g->K * g->K <= 255 && g->K >= 1 && g->stride >= 1 &&
         (size == 3 || size == 5 || size == 7);
}
// pooled rows per forward CTA: as many as fit three CTAs per SM (74 KB each), at most 4
constexpr size_t kLpMaxSmem = 200 * 1024;
constexpr size_t kLpTwoPerSm = 112 * 1024;    // two CTAs of this size share one SM's shared memory

int lp_env(const char* name, int dflt) {
  const char* e = getenv(name);
  return e ? atoi(e) : dflt;
}
int lp_fwd_rows(const GeepsPoolGeom* g) {
  static const int forced = lp_env("GEEPS_LP_FWD_RO", 0);
  if (forced > 0) return forced;
  int ro = 3;     // measured: 3 rows with 512 threads (two CTAs per SM) is the fastest of rows 2..4 x threads 256 / 512
  while (ro > 1 && (size_t)((ro - 1) * g->stride + g->K) * g->W * g->C * 2 > kLpTwoPerSm) --ro;
  return ro;
}
size_t lp_fwd_smem(const GeepsPoolGeom* g) { return (size_t)((lp_fwd_rows(g) - 1) * g->stride + g->K) * g->W * g->C * 2; }
int lp_bwd_rows(const GeepsPoolGeom* g) { return g->stride > 1 ? 2 * g->stride : 2; }
int lp_bwd_max_oh(const GeepsPoolGeom* g, int R) { return (R + g->K - 2) / g->stride + 1; }
size_t lp_bwd_smem(const GeepsPoolGeom* g, int R, int max_oh) {
  const size_t out = (size_t)max_oh * g->OW * g->C;
  return (size_t)2 * R * g->W * g->C * 2 + out * 2 + ((out + 15) & ~(size_t)15) + (size_t)g->C * 4;
}

}  // namespace

extern "C" {

int geeps_lrn_maxpool_supported(const GeepsPoolGeom* g, int size) {
  if (!lp_shape_ok(g, size)) return 0;
  int R = lp_bwd_rows(g);
  if (lp_fwd_smem(g) > kLpMaxSmem) return 0;
  while (R > 1 && lp_bwd_smem(g, R, lp_bwd_max_oh(g, R)) > kLpTwoPerSm) R >>= 1;
  return lp_bwd_smem(g, R, lp_bwd_max_oh(g, R)) <= kLpMaxSmem ? 1 : 0;
}

int geeps_lrn_maxpool_forward(const void* x, void* p, void* argmax, const GeepsPoolGeom* g, int size, float alpha,
                              float beta, float k, void* stream) {
  if (!geeps_lrn_maxpool_supported(g, size)) return (int)cudaErrorInvalidValue;
  const size_t smem = lp_fwd_smem(g);
  static const int fwd_threads = lp_env("GEEPS_LP_FWD_THREADS", 512);
  const int block = lp_threads(g->C / 8, fwd_threads);
  const LrnCoef cf = make_coef(size, alpha, beta, k);
  const int RO = lp_fwd_rows(g);
  const int grid = g->B * ((g->OH + RO - 1) / RO);
  cudaStream_t st = (cudaStream_t)stream;
#define LP_FWD(HALF, K3S2)                                                                                         \
  do {                                                                                                             \
    static bool attr_set = false;                                                                                  \
    if (!attr_set) {                                                                                               \
      cudaError_t e = cudaFuncSetAttribute(lrn_maxpool_forward_kernel<HALF, K3S2>,                                 \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLpMaxSmem);          \
      if (e != cudaSuccess) return (int)e;                                                                         \
      attr_set = true;                                                                                             \
    }                                                                                                              \
    lrn_maxpool_forward_kernel<HALF, K3S2><<<grid, block, smem, st>>>((const bf16*)x, (bf16*)p, (uint8_t*)argmax,   \
                                                                       *g, cf, RO);                                \
  } while (0)
  const bool k3s2 = g->K == 3 && g->stride == 2;
  if (size == 3) { if (k3s2) LP_FWD(1, true); else LP_FWD(1, false); }
  else if (size == 5) { if (k3s2) LP_FWD(2, true); else LP_FWD(2, false); }
  else { if (k3s2) LP_FWD(3, true); else LP_FWD(3, false); }
#undef LP_FWD
  return (int)cudaGetLastError();
}

int geeps_lrn_maxpool_backward(const void* x, const void* dp, const void* argmax, void* dx, const GeepsPoolGeom* g,
                               int size, float alpha, float beta, float k, int relu_mask, float* colsum, void* stream) {
  if (!geeps_lrn_maxpool_supported(g, size)) return (int)cudaErrorInvalidValue;
  int R = lp_bwd_rows(g);
  while (R > 1 && lp_bwd_smem(g, R, lp_bwd_max_oh(g, R)) > kLpTwoPerSm) R >>= 1;   // two CTAs per SM where possible
  const int max_oh = lp_bwd_max_oh(g, R);
  const size_t smem = lp_bwd_smem(g, R, max_oh);
  const int block = lp_threads(g->C / 8, 512);
  const LrnCoef cf = make_coef(size, alpha, beta, k);
  const float coef = 2.f * alpha * beta / (float)size;
  cudaStream_t st = (cudaStream_t)stream;
  const int row_blocks = (g->H + R - 1) / R;
  const long long total = (long long)g->B * row_blocks;
  const int per_sm = smem <= kLpTwoPerSm ? 2 : 1;
  int grid = geeps_sm_count() * per_sm;
  if (grid > total) grid = (int)total;
  if (colsum != nullptr) cudaMemsetAsync(colsum, 0, sizeof(float) * g->C, st);
#define LP_BWD(HALF, K3S2)                                                                                         \
  do {                                                                                                             \
    static bool attr_set = false;                                                                                  \
    if (!attr_set) {                                                                                               \
      cudaError_t e = cudaFuncSetAttribute(lrn_maxpool_backward_kernel<HALF, K3S2>,                                \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLpMaxSmem);          \
      if (e != cudaSuccess) return (int)e;                                                                         \
      attr_set = true;                                                                                             \
    }                                                                                                              \
    lrn_maxpool_backward_kernel<HALF, K3S2><<<grid, block, smem, st>>>((const bf16*)x, (const bf16*)dp,             \
                                                                 (const uint8_t*)argmax, (bf16*)dx, *g, R, max_oh,  \
                                                                 cf, coef, relu_mask, colsum);                     \
  } while (0)
  const bool k3s2 = g->K == 3 && g->stride == 2;
  if (size == 3) { if (k3s2) LP_BWD(1, true); else LP_BWD(1, false); }
  else if (size == 5) { if (k3s2) LP_BWD(2, true); else LP_BWD(2, false); }
  else { if (k3s2) LP_BWD(3, true); else LP_BWD(3, false); }
#undef LP_BWD
  return (int)cudaGetLastError();
}

}  // extern "C"
