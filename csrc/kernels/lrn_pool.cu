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
#include "common.cuh"
#include "nn_ops.h"

namespace {

typedef __nv_bfloat16 bf16;
__device__ __forceinline__ float bf(const bf16 v) { return __bfloat162float(v); }
struct alignas(16) Bf8 { bf16 v[8]; };
__device__ __forceinline__ Bf8 ld8(const bf16* p) { Bf8 r; *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p); return r; }
__device__ __forceinline__ void st8(bf16* p, const Bf8& r) { *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r); }

// scale of the 8 channels [c, c+8) of the pixel whose channel vector starts at px (shared memory), window
// half-width HALF <= 8: s[e] = k + a_n * sum_{|j| <= HALF} x[c+e+j]^2; xv receives x[c .. c+8)
template <int HALF>
__device__ __forceinline__ void lrn_scale8(const bf16* px, int c, int C, float a_n, float k, float (&s)[8], float (&xv)[8]) {
  float sq[24];
#pragma unroll
  for (int v = 0; v < 3; ++v) {
    const int cc = c + (v - 1) * 8;
    if (cc >= 0 && cc < C) {
      const Bf8 t = ld8(px + cc);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float f = bf(t.v[e]);
        if (v == 1) xv[e] = f;
        sq[v * 8 + e] = f * f;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) sq[v * 8 + e] = 0.f;
    }
  }
  float w = 0.f;
#pragma unroll
  for (int j = 8 - HALF; j <= 8 + HALF; ++j) w += sq[j];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    s[e] = k + a_n * w;
    if (e < 7) w += sq[8 + e + HALF + 1] - sq[8 + e - HALF];
  }
}

// ---------------- forward ----------------
// grid = B * OH; block = (channel vectors) x (pixels); dynamic shared memory = 2 * K * W * C bf16
template <int HALF>
__global__ void __launch_bounds__(256)
lrn_maxpool_forward_kernel(const bf16* __restrict__ x, bf16* __restrict__ p, uint8_t* __restrict__ argmax,
                           const GeepsPoolGeom g, float a_n, float beta, float k) {
  extern __shared__ __align__(16) uint8_t lp_smem[];
  const int C = g.C, cv = C >> 3, W = g.W;
  const int row_elems = W * C;
  bf16* xs = reinterpret_cast<bf16*>(lp_smem);       // [K][W][C] input rows
  bf16* ys = xs + (size_t)g.K * row_elems;           // [K][W][C] normalised rows
  const int oh = blockIdx.x % g.OH, b = blockIdx.x / g.OH;
  const int ih0 = oh * g.stride - g.pad;
  const int kh_lo = max(0, -ih0), kh_hi = min(g.K, g.H - ih0);
  const int tid = threadIdx.y * blockDim.x + threadIdx.x, nt = blockDim.x * blockDim.y;
  const int vec_per_row = row_elems >> 3;
  for (int kh = kh_lo; kh < kh_hi; ++kh) {
    const uint4* src = reinterpret_cast<const uint4*>(x + ((long long)b * g.H + ih0 + kh) * row_elems);
    uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)kh * row_elems);
    for (int i = tid; i < vec_per_row; i += nt) dst[i] = src[i];
  }
  __syncthreads();
  for (int kh = kh_lo; kh < kh_hi; ++kh) {
    for (int w = threadIdx.y; w < W; w += blockDim.y) {
      const bf16* px = xs + (size_t)kh * row_elems + (size_t)w * C;
      bf16* py = ys + (size_t)kh * row_elems + (size_t)w * C;
      for (int cvi = threadIdx.x; cvi < cv; cvi += blockDim.x) {
        const int c = cvi * 8;
        float s[8], xv[8];
        lrn_scale8<HALF>(px, c, C, a_n, k, s, xv);
        Bf8 o;
#pragma unroll
        for (int e = 0; e < 8; ++e) o.v[e] = __float2bfloat16(xv[e] * __powf(s[e], -beta));
        st8(py + c, o);
      }
    }
  }
  __syncthreads();
  const long long orow = ((long long)b * g.OH + oh) * g.OW;
  for (int ow = threadIdx.y; ow < g.OW; ow += blockDim.y) {
    const int iw0 = ow * g.stride - g.pad;
    const int kw_lo = max(0, -iw0), kw_hi = min(g.K, W - iw0);
    for (int cvi = threadIdx.x; cvi < cv; cvi += blockDim.x) {
      const int c = cvi * 8;
      // packed: best value and window code per 16-bit lane; strict > keeps the first maximum
      const uint32_t neg = 0xff7fff7fu;                 // two bf16 lowest finite values
      __nv_bfloat162 best[4];
      uint32_t arg[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) { best[j] = *reinterpret_cast<const __nv_bfloat162*>(&neg); arg[j] = 0x00ff00ffu; }
      for (int kh = kh_lo; kh < kh_hi; ++kh) {
        const bf16* yr = ys + (size_t)kh * row_elems + c;
        for (int kw = kw_lo; kw < kw_hi; ++kw) {
          const uint4 v = *reinterpret_cast<const uint4*>(yr + (size_t)(iw0 + kw) * C);
          const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
          const uint32_t code1 = (uint32_t)(kh * g.K + kw);
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
      const long long opix = orow + ow;
      *reinterpret_cast<uint4*>(p + opix * g.ldy + c) =
          make_uint4(*reinterpret_cast<const uint32_t*>(&best[0]), *reinterpret_cast<const uint32_t*>(&best[1]),
                     *reinterpret_cast<const uint32_t*>(&best[2]), *reinterpret_cast<const uint32_t*>(&best[3]));
      uint2 pk;      // 16-bit lanes -> bytes
      pk.x = __byte_perm(arg[0], arg[1], 0x6420);
      pk.y = __byte_perm(arg[2], arg[3], 0x6420);
      *reinterpret_cast<uint2*>(argmax + opix * C + c) = pk;
    }
  }
}

// ---------------- backward ----------------
// Persistent: CTA i handles row blocks i, i + gridDim, ... (a row block = R input rows of one image).
// Shared memory: xs, as, rs [R][W][C] bf16, dps [max_oh][OW][C] bf16, args [max_oh][OW][C] u8, cs [C] float.
template <int HALF>
__global__ void __launch_bounds__(512)
lrn_maxpool_backward_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dp, const uint8_t* __restrict__ argmax,
                            bf16* __restrict__ dx, const GeepsPoolGeom g, int R, int max_oh, float a_n, float coef,
                            float beta, float k, int relu_mask, float* __restrict__ colsum) {
  extern __shared__ __align__(16) uint8_t lp_smem[];
  const int C = g.C, cv = C >> 3, W = g.W, OW = g.OW;
  const int row_elems = W * C, orow_elems = OW * C;
  bf16* xs = reinterpret_cast<bf16*>(lp_smem);
  bf16* as = xs + (size_t)R * row_elems;             // dy * scale^-beta
  bf16* rs = as + (size_t)R * row_elems;             // dy * x * scale^(-beta-1)
  bf16* dps = rs + (size_t)R * row_elems;
  uint8_t* args = reinterpret_cast<uint8_t*>(dps + (size_t)max_oh * orow_elems);
  float* cs_sh = reinterpret_cast<float*>(args + (((size_t)max_oh * orow_elems + 15) & ~(size_t)15));
  const int tid = threadIdx.y * blockDim.x + threadIdx.x, nt = blockDim.x * blockDim.y;
  const int row_blocks = (g.H + R - 1) / R;
  const int total_blocks = g.B * row_blocks;
  const bool fixed_channel = cv <= (int)blockDim.x;   // every thread then keeps one channel vector: sums in registers
  float cs[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) cs[e] = 0.f;
  if (colsum != nullptr) for (int j = tid; j < C; j += nt) cs_sh[j] = 0.f;

  for (int blk = blockIdx.x; blk < total_blocks; blk += gridDim.x) {
    const int b = blk / row_blocks, h0 = (blk - b * row_blocks) * R;
    const int nr = min(R, g.H - h0);
    const int oh_lo = max(0, (h0 + g.pad - g.K + g.stride) / g.stride);
    const int oh_hi = min(g.OH - 1, (h0 + nr - 1 + g.pad) / g.stride);
    __syncthreads();                                   // the previous block's readers are done with the buffers
    {
      const uint4* src = reinterpret_cast<const uint4*>(x + ((long long)b * g.H + h0) * row_elems);
      uint4* dst = reinterpret_cast<uint4*>(xs);
      for (int i = tid; i < (nr * row_elems) >> 3; i += nt) dst[i] = src[i];
      for (int oh = oh_lo; oh <= oh_hi; ++oh) {
        const long long opix0 = ((long long)b * g.OH + oh) * OW;
        uint4* dd = reinterpret_cast<uint4*>(dps + (size_t)(oh - oh_lo) * orow_elems);
        uint2* da = reinterpret_cast<uint2*>(args + (size_t)(oh - oh_lo) * orow_elems);
        for (int i = tid; i < OW * cv; i += nt) {
          const int ow = i / cv, cvi = i - ow * cv;
          dd[i] = *reinterpret_cast<const uint4*>(dp + (opix0 + ow) * g.ldy + cvi * 8);
          da[i] = *reinterpret_cast<const uint2*>(argmax + (opix0 + ow) * C + cvi * 8);
        }
      }
    }
    __syncthreads();
    // phase 2: pooling gradient, scale, a = dy * s^-beta, ratio = a * x / s
    for (int r = 0; r < nr; ++r) {
      const int th = h0 + r + g.pad;
      const int roh_lo = max(oh_lo, (th - g.K + g.stride) / g.stride), roh_hi = min(oh_hi, th / g.stride);
      for (int w = threadIdx.y; w < W; w += blockDim.y) {
        const int tw = w + g.pad;
        const int ow_lo = max(0, (tw - g.K + g.stride) / g.stride), ow_hi = min(OW - 1, tw / g.stride);
        const bf16* px = xs + (size_t)r * row_elems + (size_t)w * C;
        for (int cvi = threadIdx.x; cvi < cv; cvi += blockDim.x) {
          const int c = cvi * 8;
          float dy[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) dy[e] = 0.f;
          bool any = false;
          for (int oh = roh_lo; oh <= roh_hi; ++oh) {
            const int kh = th - oh * g.stride;
            for (int ow = ow_lo; ow <= ow_hi; ++ow) {
              const uint32_t code = (uint32_t)(kh * g.K + (tw - ow * g.stride));
              const size_t o = (size_t)(oh - oh_lo) * orow_elems + (size_t)ow * C + c;
              const uint2 pk = *reinterpret_cast<const uint2*>(args + o);
              const uint32_t c4 = code * 0x01010101u;
              const uint32_t m0 = __vcmpeq4(pk.x, c4), m1 = __vcmpeq4(pk.y, c4);
              if ((m0 | m1) == 0) continue;
              any = true;
              const Bf8 d = ld8(dps + o);
#pragma unroll
              for (int e = 0; e < 8; ++e)
                if (((e < 4 ? m0 : m1) >> (8 * (e & 3))) & 1u) dy[e] += bf(d.v[e]);
            }
          }
          Bf8 oa, orat;
          if (any) {
            float s[8], xv[8];
            lrn_scale8<HALF>(px, c, C, a_n, k, s, xv);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float a = dy[e] * __powf(s[e], -beta);
              oa.v[e] = __float2bfloat16(a);
              orat.v[e] = __float2bfloat16(a * xv[e] * __frcp_rn(s[e]));
            }
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) { oa.v[e] = __float2bfloat16(0.f); orat.v[e] = __float2bfloat16(0.f); }
          }
          st8(as + (size_t)r * row_elems + (size_t)w * C + c, oa);
          st8(rs + (size_t)r * row_elems + (size_t)w * C + c, orat);
        }
      }
    }
    __syncthreads();
    // phase 3: dx = a - coef * x * (window sum of ratio), ReLU mask, per-channel sums
    for (int r = 0; r < nr; ++r) {
      bf16* drow = dx + ((long long)b * g.H + h0 + r) * row_elems;
      for (int w = threadIdx.y; w < W; w += blockDim.y) {
        const size_t pix = (size_t)r * row_elems + (size_t)w * C;
        for (int cvi = threadIdx.x; cvi < cv; cvi += blockDim.x) {
          const int c = cvi * 8;
          float ratio[24];
#pragma unroll
          for (int v = 0; v < 3; ++v) {
            const int cc = c + (v - 1) * 8;
            if (cc >= 0 && cc < C) {
              const Bf8 t = ld8(rs + pix + cc);
#pragma unroll
              for (int e = 0; e < 8; ++e) ratio[v * 8 + e] = bf(t.v[e]);
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) ratio[v * 8 + e] = 0.f;
            }
          }
          const Bf8 xv = ld8(xs + pix + c), av = ld8(as + pix + c);
          float acc = 0.f;
#pragma unroll
          for (int j = 8 - HALF; j <= 8 + HALF; ++j) acc += ratio[j];
          Bf8 o;
          float part[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float xe = bf(xv.v[e]);
            o.v[e] = __float2bfloat16((relu_mask && xe <= 0.f) ? 0.f : bf(av.v[e]) - coef * xe * acc);
            part[e] = bf(o.v[e]);
            if (e < 7) acc += ratio[8 + e + HALF + 1] - ratio[8 + e - HALF];
          }
          st8(drow + (size_t)w * C + c, o);
          if (colsum != nullptr) {
            if (fixed_channel) {
#pragma unroll
              for (int e = 0; e < 8; ++e) cs[e] += part[e];
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) atomicAdd(&cs_sh[c + e], part[e]);
            }
          }
        }
      }
    }
  }
  if (colsum != nullptr) {
    __syncthreads();
    if (fixed_channel && (int)threadIdx.x < cv) {
#pragma unroll
      for (int e = 0; e < 8; ++e) atomicAdd(&cs_sh[threadIdx.x * 8 + e], cs[e]);
    }
    __syncthreads();
    for (int j = tid; j < C; j += nt) atomicAdd(colsum + j, cs_sh[j]);
  }
}

inline dim3 lp_block(int cv, int threads) {
  int bx = cv < 1 ? 1 : (cv > threads ? threads : cv);
  int by = threads / bx;
  return dim3(bx, by < 1 ? 1 : by, 1);
}

constexpr size_t kLpMaxSmem = 200 * 1024;
constexpr size_t kLpTwoPerSm = 112 * 1024;    // two CTAs of this size share one SM's shared memory

bool lp_shape_ok(const GeepsPoolGeom* g, int size) {
  return g->C % 8 == 0 && g->ldx == g->C && g->ldy % 8 == 0 && g->K * g->K <= 255 && g->K >= 1 && g->stride >= 1 &&
         (size == 3 || size == 5 || size == 7);
}
size_t lp_fwd_smem(const GeepsPoolGeom* g) { return (size_t)2 * g->K * g->W * g->C * 2; }
int lp_bwd_rows(const GeepsPoolGeom* g) { return g->stride > 1 ? 2 * g->stride : 2; }
int lp_bwd_max_oh(const GeepsPoolGeom* g, int R) { return (R + g->K - 2) / g->stride + 1; }
size_t lp_bwd_smem(const GeepsPoolGeom* g, int R, int max_oh) {
  const size_t out = (size_t)max_oh * g->OW * g->C;
  return (size_t)3 * R * g->W * g->C * 2 + out * 2 + ((out + 15) & ~(size_t)15) + (size_t)g->C * 4;
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
  const dim3 block = lp_block(g->C / 8, 256);
  const float a_n = alpha / (float)size;
  cudaStream_t st = (cudaStream_t)stream;
#define LP_FWD(HALF)                                                                                               \
  do {                                                                                                             \
    static bool attr_set = false;                                                                                  \
    if (!attr_set) {                                                                                               \
      cudaError_t e = cudaFuncSetAttribute(lrn_maxpool_forward_kernel<HALF>,                                       \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLpMaxSmem);          \
      if (e != cudaSuccess) return (int)e;                                                                         \
      attr_set = true;                                                                                             \
    }                                                                                                              \
    lrn_maxpool_forward_kernel<HALF><<<g->B * g->OH, block, smem, st>>>((const bf16*)x, (bf16*)p, (uint8_t*)argmax, \
                                                                         *g, a_n, beta, k);                        \
  } while (0)
  if (size == 3) LP_FWD(1); else if (size == 5) LP_FWD(2); else LP_FWD(3);
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
  const dim3 block = lp_block(g->C / 8, 512);
  const float a_n = alpha / (float)size, coef = 2.f * alpha * beta / (float)size;
  cudaStream_t st = (cudaStream_t)stream;
  const int row_blocks = (g->H + R - 1) / R;
  const long long total = (long long)g->B * row_blocks;
  const int per_sm = smem <= kLpTwoPerSm ? 2 : 1;
  int grid = geeps_sm_count() * per_sm;
  if (grid > total) grid = (int)total;
  if (colsum != nullptr) cudaMemsetAsync(colsum, 0, sizeof(float) * g->C, st);
#define LP_BWD(HALF)                                                                                               \
  do {                                                                                                             \
    static bool attr_set = false;                                                                                  \
    if (!attr_set) {                                                                                               \
      cudaError_t e = cudaFuncSetAttribute(lrn_maxpool_backward_kernel<HALF>,                                      \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLpMaxSmem);          \
      if (e != cudaSuccess) return (int)e;                                                                         \
      attr_set = true;                                                                                             \
    }                                                                                                              \
    lrn_maxpool_backward_kernel<HALF><<<grid, block, smem, st>>>((const bf16*)x, (const bf16*)dp,                   \
                                                                 (const uint8_t*)argmax, (bf16*)dx, *g, R, max_oh,  \
                                                                 a_n, coef, beta, k, relu_mask, colsum);           \
  } while (0)
  if (size == 3) LP_BWD(1); else if (size == 5) LP_BWD(2); else LP_BWD(3);
#undef LP_BWD
  return (int)cudaGetLastError();
}

}  // extern "C"
