// Training ops around the tensor-core GEMM, all on NHWC bf16 activations with fp32
// arithmetic: layout conversion, im2col / col2im (conv forward, data- and weight-gradient
// run as GEMMs on the patch matrix), BatchNorm, ReLU, LRN, max / average pooling,
// softmax cross-entropy, column sums (bias gradients) and dropout.
//
// The reference ships none of these (its Caffe application is an un-fetched submodule,
// .gitmodules:1-4 of the reference); layer maths follows the usual Caffe definitions so that
// the AlexNet / Inception-BN configurations behave as the originals did.
#include "common.cuh"
#include "nn_ops.h"

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float bf(const bf16 v) { return __bfloat162float(v); }

struct alignas(16) Bf8 { bf16 v[8]; };
__device__ __forceinline__ Bf8 ld8(const bf16* p) { Bf8 r; *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p); return r; }
__device__ __forceinline__ void st8(bf16* p, const Bf8& r) { *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r); }

// t = q * stride exactly?  Strides 1 and 2 (every layer of the supported nets but conv1) avoid the divider.
__device__ __forceinline__ bool div_exact(int t, int stride, int& q) {
  if (stride == 1) { q = t; return true; }
  if (stride == 2) { q = t >> 1; return (t & 1) == 0; }
  q = t / stride;
  return q * stride == t;
}

// 256 threads as (8-channel vectors of a pixel) x (pixels of a row)
inline dim3 pool_block(int cv) {
  int bx = cv < 1 ? 1 : (cv > 256 ? 256 : cv);
  int by = 256 / bx;
  return dim3(bx, by < 1 ? 1 : by, 1);
}

inline int grid_1d(long long n, int block = 256, int cap = 0) {
  if (cap <= 0) cap = geeps_sm_count() * 16;
  long long b = (n + block - 1) / block;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

// ---------------- layout conversion ----------------
// The NCHW input batch is fp32 or bf16 (a host pipeline that ships bf16 halves the host-to-device bytes).
__device__ __forceinline__ float in_val(const float* p) { return __ldg(p); }
__device__ __forceinline__ float in_val(const bf16* p) { return __bfloat162float(*p); }

template <typename T>
__global__ void __launch_bounds__(256)
nchw_f32_to_nhwc_bf16_kernel(const T* __restrict__ x, bf16* __restrict__ y, int B, int C, int H, int W, int Cpad) {
  const long long total = (long long)B * H * W * Cpad;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % Cpad);
    long long p = i / Cpad;
    const int w = (int)(p % W); p /= W;
    const int h = (int)(p % H);
    const int b = (int)(p / H);
    y[i] = __float2bfloat16(c < C ? in_val(x + (((long long)b * C + c) * H + h) * W + w) : 0.f);
  }
}

// ---------------- im2col / col2im (NHWC, one channel group) ----------------
// col[(b,oh,ow)][(kh,kw,c)] = x[b][oh*s-p+kh][ow*s-p+kw][c0+c]; row pitch ldcol >= KH*KW*Cg.
// One warp builds one row of the patch matrix at a time: the pixel coordinates are decoded once per row
// and the lanes sweep the row's vectors, so the address arithmetic is two 32-bit divisions per vector.
template <int VEC>
__global__ void __launch_bounds__(256)
im2col_kernel(const bf16* __restrict__ x, bf16* __restrict__ col, const GeepsConvGeom g) {
  const int cv = g.Cg / VEC;
  const int per_kh = g.KW * cv;
  const int per_row = g.KH * per_kh;
  const long long rows = (long long)g.B * g.OH * g.OW;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long row = warp0; row < rows; row += nwarps) {
    const int ow = (int)(row % g.OW);
    const long long t = row / g.OW;
    const int oh = (int)(t % g.OH);
    const int b = (int)(t / g.OH);
    const int ih0 = oh * g.stride - g.pad, iw0 = ow * g.stride - g.pad;
    bf16* drow = col + row * g.ldcol;
    const bf16* xb = x + (long long)b * g.H * g.W * g.C + g.c0;
    for (int v = lane; v < per_row; v += 32) {
      const int kh = v / per_kh;
      const int rem = v - kh * per_kh;
      const int kw = rem / cv;
      const int c = (rem - kw * cv) * VEC;
      const int ih = ih0 + kh, iw = iw0 + kw;
      const bool in = ih >= 0 && ih < g.H && iw >= 0 && iw < g.W;
      bf16* dst = drow + (kh * g.KW + kw) * g.Cg + c;
      const bf16* src = xb + ((long long)ih * g.W + iw) * g.C + c;
      if (VEC == 8) {
        *reinterpret_cast<uint4*>(dst) = in ? *reinterpret_cast<const uint4*>(src) : make_uint4(0, 0, 0, 0);
      } else if (VEC == 4) {
        *reinterpret_cast<uint2*>(dst) = in ? *reinterpret_cast<const uint2*>(src) : make_uint2(0, 0);
      } else {
        *dst = in ? *src : __float2bfloat16(0.f);
      }
    }
  }
}

// Zero the pad columns [Kd, ldcol) of the patch matrix once (TMA reads them as K).
__global__ void zero_col_pad_kernel(bf16* col, long long rows, int kd, int ldcol) {
  const int padw = ldcol - kd;
  const long long total = rows * padw;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
    col[(i / padw) * ldcol + kd + (i % padw)] = __float2bfloat16(0.f);
}

// dx[b][ih][iw][c0+c] (+)= sum over (kh,kw) windows covering (ih,iw) of dcol[(b,oh,ow)][(kh,kw,c)]
// Gather form: no atomics, deterministic.
template <int VEC>
__global__ void __launch_bounds__(256)
col2im_kernel(const bf16* __restrict__ dcol, bf16* __restrict__ dx, const GeepsConvGeom g, int accumulate) {
  const int cv = g.Cg / VEC;
  const long long total = (long long)g.B * g.H * g.W * cv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % cv) * VEC;
    long long p = i / cv;
    const int iw = (int)(p % g.W); p /= g.W;
    const int ih = (int)(p % g.H);
    const int b = (int)(p / g.H);
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
    for (int kh = 0; kh < g.KH; ++kh) {
      const int th = ih + g.pad - kh;
      int oh, ow;
      if (th < 0 || !div_exact(th, g.stride, oh) || oh >= g.OH) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        const int tw = iw + g.pad - kw;
        if (tw < 0 || !div_exact(tw, g.stride, ow) || ow >= g.OW) continue;
        const bf16* src = dcol + (((long long)b * g.OH + oh) * g.OW + ow) * g.ldcol +
                          (long long)(kh * g.KW + kw) * g.Cg + c;
        if (VEC == 8) {
          Bf8 v = ld8(src);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += bf(v.v[e]);
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) acc[e] += bf(src[e]);
        }
      }
    }
    bf16* dst = dx + (((long long)b * g.H + ih) * g.W + iw) * g.C + g.c0 + c;
    if (VEC == 8) {
      Bf8 o;
      if (accumulate) { Bf8 old = ld8(dst);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += bf(old.v[e]); }
#pragma unroll
      for (int e = 0; e < 8; ++e) o.v[e] = __float2bfloat16(acc[e]);
      st8(dst, o);
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) dst[e] = __float2bfloat16(acc[e] + (accumulate ? bf(dst[e]) : 0.f));
    }
  }
}

// ---------------- per-channel reductions over a [P][C] (pitch ld) bf16 matrix ----------------
// MODE 0: out[c] += sum x, out[C+c] += sum x^2                  (BN forward statistics)
// MODE 1: out[c] += sum dy', out[C+c] += sum dy' * xhat          (BN backward; dy' = dy masked by y>0 if relu)
// MODE 2: out[c] += scale * sum x                                (bias gradient)
template <int MODE>
__device__ __forceinline__ void channel_reduce_body(const bf16* __restrict__ x, const bf16* __restrict__ dy,
                                                    const bf16* __restrict__ y, const float* __restrict__ mean_rstd,
                                                    float* __restrict__ out, long long P, int C, long long ldx,
                                                    long long lddy, int relu, float scale) {
  extern __shared__ float sacc[];  // [2*C]
  for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) sacc[i] = 0.f;
  __syncthreads();
  const int cv = C >> 3;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long groups = nthreads / cv;  // pixel lanes: each owns one 8-channel slot
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid < groups * cv) {
    const int c = (int)(tid % cv) * 8;
    float a0[8], a1[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { a0[e] = 0.f; a1[e] = 0.f; }
    float mu[8], rs[8];
    if (MODE == 1) {
#pragma unroll
      for (int e = 0; e < 8; ++e) { mu[e] = mean_rstd[c + e]; rs[e] = mean_rstd[C + c + e]; }
    }
    for (long long p = tid / cv; p < P; p += groups) {
      if (MODE == 0 || MODE == 2) {
        Bf8 v = ld8(x + p * ldx + c);
#pragma unroll
        for (int e = 0; e < 8; ++e) { float f = bf(v.v[e]); a0[e] += f; if (MODE == 0) a1[e] += f * f; }
      } else {
        Bf8 xv = ld8(x + p * ldx + c), dv = ld8(dy + p * lddy + c), yv;
        if (relu) yv = ld8(y + p * lddy + c);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float d = bf(dv.v[e]);
          if (relu && !(bf(yv.v[e]) > 0.f)) d = 0.f;
          a0[e] += d;
          a1[e] += d * (bf(xv.v[e]) - mu[e]) * rs[e];
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      atomicAdd(&sacc[c + e], a0[e]);
      if (MODE != 2) atomicAdd(&sacc[C + c + e], a1[e]);
    }
  }
  __syncthreads();
  const int nout = MODE == 2 ? C : 2 * C;
  for (int i = threadIdx.x; i < nout; i += blockDim.x) {
    const float v = sacc[i];
    if (v != 0.f) atomicAdd(out + i, MODE == 2 ? v * scale : v);
  }
}
template <int MODE>
__global__ void __launch_bounds__(256)
channel_reduce_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy, const bf16* __restrict__ y,
                      const float* __restrict__ mean_rstd, float* __restrict__ out, long long P, int C,
                      long long ldx, long long lddy, int relu, float scale) {
  channel_reduce_body<MODE>(x, dy, y, mean_rstd, out, P, C, ldx, lddy, relu, scale);
}

// any C, any pitch: one thread per column (small P: FC bias gradients with odd widths)
__global__ void colsum_simple_kernel(const bf16* __restrict__ x, float* __restrict__ out, long long P, int C,
                                     long long ldx, float scale, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float a = 0.f;
  for (long long p = 0; p < P; ++p) a += bf(x[p * ldx + c]);
  out[c] = a * scale + (accumulate ? out[c] : 0.f);
}

// sums -> mean / rstd (+ running statistics with Caffe-style moving average)
__global__ void bn_finalize_kernel(const float* __restrict__ sums, float* __restrict__ mean_rstd,
                                   float* running_mean, float* running_var, int C, float inv_count, float eps,
                                   float momentum) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float m = sums[c] * inv_count;
  float var = sums[C + c] * inv_count - m * m;
  var = fmaxf(var, 0.f);
  mean_rstd[c] = m;
  mean_rstd[C + c] = rsqrtf(var + eps);
  if (running_mean) {
    running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * m;
    running_var[c] = (1.f - momentum) * running_var[c] + momentum * var;
  }
}

__global__ void __launch_bounds__(256)
bn_apply_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, const float* __restrict__ mean_rstd,
                const float* __restrict__ gamma, const float* __restrict__ beta, long long P, int C,
                long long ldx, long long ldy, int relu) {
  const int cv = C >> 3;
  const long long total = P * cv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % cv) * 8;
    const long long p = i / cv;
    Bf8 v = ld8(x + p * ldx + c), o;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float f = (bf(v.v[e]) - mean_rstd[c + e]) * mean_rstd[C + c + e] * gamma[c + e] + beta[c + e];
      if (relu) f = fmaxf(f, 0.f);
      o.v[e] = __float2bfloat16(f);
    }
    st8(y + p * ldy + c, o);
  }
}

// Normalisation with the statistics finalised inside: every thread derives mean and 1/std of its eight channels from
// the channel sums (no separate finalisation launch); the threads of the first pixel also store mean / rstd for the
// backward pass, update the running statistics and zero `zero_after` (2 C floats: the scratch of the NEXT reduction
// of this layer, e.g. the backward one, so that no memset node sits in front of it).
__device__ __forceinline__ void bn_apply_fused_body(const bf16* __restrict__ x, bf16* __restrict__ y,
                                                    const float* sums, float* mean_rstd,
                                                    float* running_mean, float* running_var,
                                                    const float* __restrict__ gamma, const float* __restrict__ beta,
                                                    float* zero_after, long long P, int C, long long ldx, long long ldy,
                                                    int relu, float inv_count, float eps, float momentum) {
  const int cv = C >> 3;
  const long long total = P * cv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % cv) * 8;
    const long long p = i / cv;
    float m[8], r[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      m[e] = sums[c + e] * inv_count;
      const float var = fmaxf(sums[C + c + e] * inv_count - m[e] * m[e], 0.f);
      r[e] = rsqrtf(var + eps);
      if (p == 0) {
        mean_rstd[c + e] = m[e];
        mean_rstd[C + c + e] = r[e];
        if (running_mean) {
          running_mean[c + e] = (1.f - momentum) * running_mean[c + e] + momentum * m[e];
          running_var[c + e] = (1.f - momentum) * running_var[c + e] + momentum * var;
        }
        if (zero_after) { zero_after[c + e] = 0.f; zero_after[C + c + e] = 0.f; }
      }
    }
    Bf8 v = ld8(x + p * ldx + c), o;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float f = (bf(v.v[e]) - m[e]) * r[e] * gamma[c + e] + beta[c + e];
      if (relu) f = fmaxf(f, 0.f);
      o.v[e] = __float2bfloat16(f);
    }
    st8(y + p * ldy + c, o);
  }
}
__global__ void __launch_bounds__(256)
bn_apply_fused_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, const float* __restrict__ sums,
                      float* __restrict__ mean_rstd, float* running_mean, float* running_var,
                      const float* __restrict__ gamma, const float* __restrict__ beta, float* zero_after, long long P,
                      int C, long long ldx, long long ldy, int relu, float inv_count, float eps, float momentum) {
  bn_apply_fused_body(x, y, sums, mean_rstd, running_mean, running_var, gamma, beta, zero_after, P, C, ldx, ldy, relu,
                      inv_count, eps, momentum);
}

// dx = gamma * rstd * (dy' - sum_dy/P - xhat * sum_dy_xhat/P); also emits dgamma, dbeta (scaled).
__device__ __forceinline__ void bn_backward_body(const bf16* __restrict__ x, const bf16* __restrict__ dy,
                                                 const bf16* __restrict__ y, bf16* __restrict__ dx,
                                                 const float* mean_rstd, const float* __restrict__ gamma,
                                                 const float* sums, float* dgamma, float* dbeta, long long P, int C,
                                                 long long ldx, long long lddy, long long lddx, int relu,
                                                 float grad_scale, float* zero_after) {
  const int cv = C >> 3;
  const long long total = P * cv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float invP = 1.f / (float)P;
  const long long tid0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid0 < C) {
    if (dbeta) dbeta[tid0] = sums[tid0] * grad_scale;
    if (dgamma) dgamma[tid0] = sums[C + tid0] * grad_scale;
    // the scratch of this layer's next forward reduction (nobody reads it during the backward pass)
    if (zero_after) { zero_after[tid0] = 0.f; zero_after[C + tid0] = 0.f; }
  }
  for (long long i = tid0; i < total; i += stride) {
    const int c = (int)(i % cv) * 8;
    const long long p = i / cv;
    Bf8 xv = ld8(x + p * ldx + c), dv = ld8(dy + p * lddy + c), yv, o;
    if (relu) yv = ld8(y + p * lddy + c);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float d = bf(dv.v[e]);
      if (relu && !(bf(yv.v[e]) > 0.f)) d = 0.f;
      const float rs = mean_rstd[C + c + e];
      const float xhat = (bf(xv.v[e]) - mean_rstd[c + e]) * rs;
      o.v[e] = __float2bfloat16(gamma[c + e] * rs * (d - sums[c + e] * invP - xhat * sums[C + c + e] * invP));
    }
    st8(dx + p * lddx + c, o);
  }
}
__global__ void __launch_bounds__(256)
bn_backward_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy, const bf16* __restrict__ y,
                   bf16* __restrict__ dx, const float* __restrict__ mean_rstd, const float* __restrict__ gamma,
                   const float* __restrict__ sums, float* dgamma, float* dbeta, long long P, int C,
                   long long ldx, long long lddy, long long lddx, int relu, float grad_scale, float* zero_after) {
  bn_backward_body(x, dy, y, dx, mean_rstd, gamma, sums, dgamma, dbeta, P, C, ldx, lddy, lddx, relu, grad_scale,
                   zero_after);
}

// ---- one launch per direction: reduction, grid barrier, normalisation (cooperative launch: all blocks resident) ----
// bar[0] counts arrivals, bar[1] counts blocks that are done (the last one resets both for the next launch), bar[2]
// is set when a block gave up waiting (it then skips the second phase: the output stays stale and mean_rstd[0] is
// made NaN so that the failure shows in the loss).
__device__ __forceinline__ bool bn_grid_barrier(int* bar, int nblocks) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(bar, 1);
    s_ok = geeps_wait_ge(bar, nblocks, 1000000000ull, nullptr) ? 1 : 0;
    __threadfence();
  }
  __syncthreads();
  return s_ok != 0;
}
__device__ __forceinline__ void bn_grid_done(int* bar, int nblocks) {
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(bar + 1, 1) == nblocks - 1) {
    bar[0] = 0; bar[1] = 0;
    __threadfence();
  }
}
__global__ void __launch_bounds__(256)
bn_forward_coop_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, float* sums, float* mean_rstd,
                       float* running_mean, float* running_var, const float* __restrict__ gamma,
                       const float* __restrict__ beta, float* zero_after, int* bar, long long P, int C, long long ldx,
                       long long ldy, int relu, float inv_count, float eps, float momentum) {
  channel_reduce_body<0>(x, nullptr, nullptr, nullptr, sums, P, C, ldx, 0, 0, 1.f);
  if (bn_grid_barrier(bar, (int)gridDim.x))
    bn_apply_fused_body(x, y, sums, mean_rstd, running_mean, running_var, gamma, beta, zero_after, P, C, ldx, ldy, relu,
                        inv_count, eps, momentum);
  else if (threadIdx.x == 0) { bar[2] = 1; mean_rstd[0] = __int_as_float(0x7fc00000); }
  bn_grid_done(bar, (int)gridDim.x);
}
__global__ void __launch_bounds__(256)
bn_backward_coop_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy, const bf16* __restrict__ y,
                        bf16* __restrict__ dx, float* mean_rstd, const float* __restrict__ gamma, float* sums,
                        float* dgamma, float* dbeta, float* zero_after, int* bar, long long P, int C, long long ldx,
                        long long lddy, long long lddx, int relu, float grad_scale) {
  channel_reduce_body<1>(x, dy, y, mean_rstd, sums, P, C, ldx, lddy, relu, 1.f);
  if (bn_grid_barrier(bar, (int)gridDim.x))
    bn_backward_body(x, dy, y, dx, mean_rstd, gamma, sums, dgamma, dbeta, P, C, ldx, lddy, lddx, relu, grad_scale,
                     zero_after);
  else if (threadIdx.x == 0) { bar[2] = 1; mean_rstd[0] = __int_as_float(0x7fc00000); }
  bn_grid_done(bar, (int)gridDim.x);
}

// ---------------- ReLU backward / dropout ----------------
__global__ void __launch_bounds__(256)
relu_backward_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ y, bf16* __restrict__ dx, long long n8) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
    Bf8 d = ld8(dy + i * 8), v = ld8(y + i * 8), o;
#pragma unroll
    for (int e = 0; e < 8; ++e) o.v[e] = bf(v.v[e]) > 0.f ? d.v[e] : __float2bfloat16(0.f);
    st8(dx + i * 8, o);
  }
}

// 2-D variant with row pitches (channel slices of concat tensors)
__global__ void __launch_bounds__(256)
relu_backward_2d_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ y, bf16* __restrict__ dx, long long P,
                        int C, long long lddy, long long ldy, long long lddx) {
  const int cv = C >> 3;
  const long long total = P * cv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % cv) * 8;
    const long long p = i / cv;
    Bf8 d = ld8(dy + p * lddy + c), v = ld8(y + p * ldy + c), o;
#pragma unroll
    for (int e = 0; e < 8; ++e) o.v[e] = bf(v.v[e]) > 0.f ? d.v[e] : __float2bfloat16(0.f);
    st8(dx + p * lddx + c, o);
  }
}
// dst = bf16(relu ? max(src, 0) : src) over a [P][C] fp32 matrix with row pitches: the finishing pass of a split-K
// GEMM whose partial sums were reduce-added in fp32
__global__ void __launch_bounds__(256)
f32_to_bf16_2d_kernel(const float* __restrict__ src, bf16* __restrict__ dst, long long P, int C, long long lds,
                      long long ldd, int relu) {
  const int cv = C >> 3;
  const long long total = P * cv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float lo = relu ? 0.f : -INFINITY;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % cv) * 8;
    const long long p = i / cv;
    const float4 a = *reinterpret_cast<const float4*>(src + p * lds + c);
    const float4 b = *reinterpret_cast<const float4*>(src + p * lds + c + 4);
    *reinterpret_cast<uint4*>(dst + p * ldd + c) =
        make_uint4(pack_bf16x2(fmaxf(a.x, lo), fmaxf(a.y, lo)), pack_bf16x2(fmaxf(a.z, lo), fmaxf(a.w, lo)),
                   pack_bf16x2(fmaxf(b.x, lo), fmaxf(b.y, lo)), pack_bf16x2(fmaxf(b.z, lo), fmaxf(b.w, lo)));
  }
}
// ReLU backward fused with the per-channel sums of its result (the bias gradient of the layer whose output y is):
// dx = y > 0 ? dy : 0, out[c] += sum over pixels of dx.  Every thread keeps one 8-channel slot and strides over
// the pixels, as in channel_reduce_kernel.
__global__ void __launch_bounds__(256)
relu_backward_colsum_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ y, bf16* __restrict__ dx,
                            float* __restrict__ out, long long P, int C, long long lddy, long long ldy, long long lddx) {
  extern __shared__ float sacc[];  // [C]
  for (int i = threadIdx.x; i < C; i += blockDim.x) sacc[i] = 0.f;
  __syncthreads();
  const int cv = C >> 3;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long groups = nthreads / cv;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid < groups * cv) {
    const int c = (int)(tid % cv) * 8;
    float a[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = 0.f;
    for (long long p = tid / cv; p < P; p += groups) {
      const Bf8 d = ld8(dy + p * lddy + c), v = ld8(y + p * ldy + c);
      Bf8 o;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const bool on = bf(v.v[e]) > 0.f;
        o.v[e] = on ? d.v[e] : __float2bfloat16(0.f);
        a[e] += on ? bf(d.v[e]) : 0.f;
      }
      st8(dx + p * lddx + c, o);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) atomicAdd(&sacc[c + e], a[e]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < C; i += blockDim.x) atomicAdd(out + i, sacc[i]);
}
// dst += src over 2-D views (sum of branch gradients)
__global__ void __launch_bounds__(256)
add_2d_kernel(bf16* __restrict__ dst, const bf16* __restrict__ src, long long P, int C, long long ldd, long long lds) {
  const int cv = C >> 3;
  const long long total = P * cv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % cv) * 8;
    const long long p = i / cv;
    Bf8 a = ld8(dst + p * ldd + c), b = ld8(src + p * lds + c), o;
#pragma unroll
    for (int e = 0; e < 8; ++e) o.v[e] = __float2bfloat16(bf(a.v[e]) + bf(b.v[e]));
    st8(dst + p * ldd + c, o);
  }
}

__device__ __forceinline__ uint32_t mix32(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return (uint32_t)((z ^ (z >> 31)) >> 32);
}
// y = x * keep(seed, idx) / (1 - p); the same call with dy as input gives dx.
__global__ void __launch_bounds__(256)
dropout_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long n, float p, unsigned long long seed,
               const int* __restrict__ step_ref) {
  if (step_ref != nullptr) seed += (unsigned long long)(long long)*step_ref;
  const float inv = 1.f / (1.f - p);
  const uint32_t thresh = (uint32_t)(p * 4294967296.0);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = mix32(seed * 0x100000001B3ull + (uint64_t)i) >= thresh ? __float2bfloat16(bf(x[i]) * inv) : __float2bfloat16(0.f);
}

// ---------------- LRN across channels ----------------
// Forward keeps r = 1 / scale per element in bf16 for the backward pass (scale = k + alpha/n * window sum of x^2):
// half the bytes of an fp32 scale buffer in both directions, and the backward needs 1/scale (for dy*y/scale) and
// scale^-beta = r^beta only.
__global__ void __launch_bounds__(256)
lrn_forward_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, bf16* __restrict__ scale, long long P, int C,
                   int size, float alpha, float beta, float k) {
  const long long total = P * C;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const int half = size / 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % C);
    const bf16* row = x + (i - c);
    float s = 0.f;
    const int lo = max(0, c - half), hi = min(C - 1, c + half);
    for (int j = lo; j <= hi; ++j) { float f = bf(row[j]); s += f * f; }
    const float sc = k + alpha / (float)size * s;
    scale[i] = __float2bfloat16(__frcp_rn(sc));
    y[i] = __float2bfloat16(bf(row[c]) * __powf(sc, -beta));
  }
}
__global__ void __launch_bounds__(256)
lrn_backward_kernel(const bf16* __restrict__ x, const bf16* __restrict__ y, const bf16* __restrict__ scale,
                    const bf16* __restrict__ dy, bf16* __restrict__ dx, long long P, int C, int size, float alpha,
                    float beta, int relu_mask) {
  const long long total = P * C;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const int half = size / 2;
  const float coef = 2.f * alpha * beta / (float)size;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % C);
    const long long base = i - c;
    float acc = 0.f;
    const int lo = max(0, c - half), hi = min(C - 1, c + half);
    for (int j = lo; j <= hi; ++j) acc += bf(dy[base + j]) * bf(y[base + j]) * bf(scale[base + j]);
    const float xi = bf(x[i]);
    const float d = bf(dy[i]) * __powf(bf(scale[i]), beta) - coef * xi * acc;
    dx[i] = __float2bfloat16((relu_mask && xi <= 0.f) ? 0.f : d);
  }
}

// Vector forms: one thread owns 8 consecutive channels of a pixel and slides the window over the
// 24 channels around them (window half-width <= 8); each squared value / ratio is computed once.
template <int HALF>
__global__ void __launch_bounds__(256)
lrn_forward_v8_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, bf16* __restrict__ scale, long long P, int C,
                      int size, float alpha, float beta, float k) {
  const int cv = C >> 3;
  const long long total = P * cv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float a_n = alpha / (float)size;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % cv) * 8;
    const long long base = (i / cv) * C;
    float sq[24];
#pragma unroll
    for (int v = 0; v < 3; ++v) {
      const int cc = c + (v - 1) * 8;
      if (cc >= 0 && cc < C) {
        Bf8 t = ld8(x + base + cc);
#pragma unroll
        for (int e = 0; e < 8; ++e) { float f = bf(t.v[e]); sq[v * 8 + e] = v == 1 ? f : f * f; }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) sq[v * 8 + e] = 0.f;
      }
    }
    float xv[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { xv[e] = sq[8 + e]; sq[8 + e] = xv[e] * xv[e]; }
    Bf8 o, r;
    float s = 0.f;       // sliding window over the 2*HALF+1 channels around output e
#pragma unroll
    for (int j = 8 - HALF; j <= 8 + HALF; ++j) s += sq[j];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sc = k + a_n * s;
      o.v[e] = __float2bfloat16(xv[e] * __powf(sc, -beta));
      r.v[e] = __float2bfloat16(__frcp_rn(sc));
      if (e < 7) s += sq[8 + e + HALF + 1] - sq[8 + e - HALF];
    }
    st8(y + base + c, o);
    st8(scale + base + c, r);
  }
}
template <int HALF>
__global__ void __launch_bounds__(256)
lrn_backward_v8_kernel(const bf16* __restrict__ x, const bf16* __restrict__ y, const bf16* __restrict__ scale,
                       const bf16* __restrict__ dy, bf16* __restrict__ dx, long long P, int C, int size, float alpha,
                       float beta, int relu_mask, float* __restrict__ colsum) {
  // colsum (optional): per-channel sums of dx over all pixels - the bias gradient of the convolution whose
  // ReLU is folded in here.  The host sizes the grid so that gridDim * blockDim is a multiple of C/8: every
  // thread then keeps one channel group for all its pixels and sums in registers.
  extern __shared__ float lrn_cs[];
  const int cv = C >> 3;
  const long long total = P * cv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float coef = 2.f * alpha * beta / (float)size;
  float cs[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) cs[e] = 0.f;
  if (colsum != nullptr) {
    for (int j = threadIdx.x; j < C; j += blockDim.x) lrn_cs[j] = 0.f;
    __syncthreads();
  }
  const int c_fixed = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) % cv) * 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % cv) * 8;
    const long long base = (i / cv) * C;
    float ratio[24], dyc[8], scc[8];
#pragma unroll
    for (int v = 0; v < 3; ++v) {
      const int cc = c + (v - 1) * 8;
      if (cc >= 0 && cc < C) {
        Bf8 d = ld8(dy + base + cc), yy = ld8(y + base + cc), rr = ld8(scale + base + cc);   // rr = 1 / scale
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          ratio[v * 8 + e] = bf(d.v[e]) * bf(yy.v[e]) * bf(rr.v[e]);
          if (v == 1) { dyc[e] = bf(d.v[e]); scc[e] = bf(rr.v[e]); }
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) ratio[v * 8 + e] = 0.f;
      }
    }
    Bf8 xv = ld8(x + base + c), o;
    float acc = 0.f;
#pragma unroll
    for (int j = 8 - HALF; j <= 8 + HALF; ++j) acc += ratio[j];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float xe = bf(xv.v[e]);
      // relu_mask: x is the output of a ReLU whose backward is folded in here (no gradient where it clipped)
      o.v[e] = __float2bfloat16((relu_mask && xe <= 0.f) ? 0.f : dyc[e] * __powf(scc[e], beta) - coef * xe * acc);
      cs[e] += bf(o.v[e]);
      if (e < 7) acc += ratio[8 + e + HALF + 1] - ratio[8 + e - HALF];
    }
    st8(dx + base + c, o);
  }
  if (colsum != nullptr) {
#pragma unroll
    for (int e = 0; e < 8; ++e) atomicAdd(&lrn_cs[c_fixed + e], cs[e]);
    __syncthreads();
    for (int j = threadIdx.x; j < C; j += blockDim.x) atomicAdd(colsum + j, lrn_cs[j]);
  }
}

// NCHW fp32 -> NHWC bf16, one thread per pixel: reads are coalesced along W in every channel plane
template <typename T>
__global__ void __launch_bounds__(256)
nchw_to_nhwc_pix_kernel(const T* __restrict__ x, bf16* __restrict__ y, int B, int C, int HW, int Cpad) {
  const long long total = (long long)B * HW;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long b = i / HW, p = i % HW;
    const T* src = x + b * C * HW + p;
    bf16* dst = y + i * Cpad;
    for (int c0 = 0; c0 < Cpad; c0 += 4) {
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = (c0 + e < C) ? in_val(src + (long long)(c0 + e) * HW) : 0.f;
      *reinterpret_cast<uint2*>(dst + c0) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
    }
  }
}

// NCHW fp32 -> space-to-depth NHWC bf16: y[b][hs][ws][(dy*S + dx)*C + c] = x[b][c][hs*S + dy][ws*S + dx]
// (zero past the image edge and in the channel padding).  A stride-S convolution over x is then a
// stride-1 convolution with ceil(k/S) taps per dimension over y.  One thread per output pixel; the
// 4 x 3-channel case keeps the pixel's 48 values in registers and reads 16 contiguous bytes per (c, dy).
template <int S, int C, typename T>
__global__ void __launch_bounds__(256)
nchw_to_s2d_kernel(const T* __restrict__ x, bf16* __restrict__ y, int B, int H, int W, int Hs, int Ws, int Cpad) {
  constexpr int N = S * S * C;
  const long long total = (long long)B * Hs * Ws;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int ws = (int)(i % Ws);
    const long long t = i / Ws;
    const int hs = (int)(t % Hs);
    const long long b = t / Hs;
    float v[N];
#pragma unroll
    for (int c = 0; c < C; ++c) {
#pragma unroll
      for (int dy = 0; dy < S; ++dy) {
        const int h = hs * S + dy;
        const T* row = x + ((b * C + c) * H + h) * (long long)W;
#pragma unroll
        for (int dx = 0; dx < S; ++dx) {
          const int w = ws * S + dx;
          v[(dy * S + dx) * C + c] = (h < H && w < W) ? in_val(row + w) : 0.f;
        }
      }
    }
    bf16* dst = y + i * Cpad;
#pragma unroll
    for (int j = 0; j + 8 <= N; j += 8)
      *reinterpret_cast<uint4*>(dst + j) = make_uint4(pack_bf16x2(v[j], v[j + 1]), pack_bf16x2(v[j + 2], v[j + 3]),
                                                      pack_bf16x2(v[j + 4], v[j + 5]), pack_bf16x2(v[j + 6], v[j + 7]));
    int j = N & ~7;
    if ((N & 7) == 0)
      for (; j + 8 <= Cpad; j += 8) *reinterpret_cast<uint4*>(dst + j) = make_uint4(0, 0, 0, 0);
    for (; j < Cpad; ++j) dst[j] = __float2bfloat16(j < N ? v[j] : 0.f);
  }
}

// The same layout for S = 4, C = 3 with coalesced traffic on both sides: a block of four warps converts 32
// consecutive output pixels of one output row.  Warp dy reads, for each colour, the 128 consecutive input elements of
// image row 4 hs + dy that those pixels cover (32 consecutive elements per load), the values meet in a [32 pixels][Cpad]
// tile in shared memory, and the tile leaves as one contiguous run of 32 * Cpad * 2 bytes in 16-byte stores.
template <typename T>
__global__ void __launch_bounds__(128)
nchw_to_s2d43_tile_kernel(const T* __restrict__ x, bf16* __restrict__ y, int B, int H, int W, int Hs, int Ws, int Cpad,
                          int segs) {
  constexpr int S = 4, C = 3, PIX = 32, PITCH = 72;      // tile row pitch in elements: 144 bytes staggers the banks
  __shared__ __align__(16) bf16 tile[PIX * PITCH];
  const int lane = threadIdx.x & 31, dy = threadIdx.x >> 5;
  long long blk = blockIdx.x;
  const int seg = (int)(blk % segs); blk /= segs;
  const int hs = (int)(blk % Hs);
  const long long b = blk / Hs;
  const int ws0 = seg * PIX;
  // channels past S * S * C are zero (this warp's share of them: pixel `lane`, slots 48 + 4 dy .. + 4, when they exist)
  for (int j = S * S * C + dy * 4; j < Cpad && j < S * S * C + dy * 4 + 4; ++j) tile[lane * PITCH + j] = __float2bfloat16(0.f);
  const int h = hs * S + dy;
  // the 128 consecutive input elements of this image row that the 32 pixels cover, 32 at a time: every load
  // instruction of the warp is one contiguous run (also when x is pinned host memory read over PCIe)
  const int wbase = ws0 * S;
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const T* row = x + ((b * C + c) * H + h) * (long long)W;
#pragma unroll
    for (int i = 0; i < S; ++i) {
      const int e = i * 32 + lane;                      // element of the run: pixel e / 4, column offset e % 4
      const int w = wbase + e;
      const float v = (h < H && w < W) ? in_val(row + w) : 0.f;
      tile[(e >> 2) * PITCH + (dy * S + (e & 3)) * C + c] = __float2bfloat16(v);
    }
  }
  __syncthreads();
  const int per_pix = Cpad >> 3;                          // 16-byte pieces per pixel
  const int npix = min(PIX, Ws - ws0);
  bf16* dst = y + ((b * Hs + hs) * (long long)Ws + ws0) * Cpad;
  for (int i = threadIdx.x; i < npix * per_pix; i += blockDim.x) {
    const int px = i / per_pix, piece = i - px * per_pix;
    *reinterpret_cast<uint4*>(dst + (long long)i * 8) = *reinterpret_cast<const uint4*>(tile + px * PITCH + piece * 8);
  }
}

// any S, C: one thread per output element
template <typename T>
__global__ void __launch_bounds__(256)
nchw_to_s2d_generic_kernel(const T* __restrict__ x, bf16* __restrict__ y, int B, int C, int H, int W, int S,
                           int Hs, int Ws, int Cpad) {
  const long long total = (long long)B * Hs * Ws * Cpad;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int j = (int)(i % Cpad);
    long long t = i / Cpad;
    const int ws = (int)(t % Ws); t /= Ws;
    const int hs = (int)(t % Hs);
    const long long b = t / Hs;
    float v = 0.f;
    if (j < S * S * C) {
      const int c = j % C, q = j / C, dx = q % S, dy = q / S;
      const int h = hs * S + dy, w = ws * S + dx;
      if (h < H && w < W) v = in_val(x + ((b * C + c) * H + h) * (long long)W + w);
    }
    y[i] = __float2bfloat16(v);
  }
}

// ---- data transformer: uint8 NCHW source images -> cropped / mirrored / mean-subtracted / scaled bf16 activations ----
// The work of Caffe's DataTransformer (crop_size, mirror, mean_value, scale), done on the device so that the host ships
// one byte per value.  aug (NULL: centre crop, no mirror) holds {h_off, w_off, mirror} per image.
struct XformDev {
  const uint8_t* x;
  const int* aug;
  int Hin, Win;          // source image
  int H, W;              // cropped image (what the network sees)
  int h_off, w_off;      // centre crop, used when aug == NULL
  float mean[4], scale;
};

__device__ __forceinline__ void xform_image(const XformDev& t, long long b, int& h_off, int& w_off, int& mirror) {
  if (t.aug != nullptr) {
    // out-of-range offsets are clamped: a bad entry reads a valid window instead of another image
    h_off = min(max(t.aug[b * 3 + 0], 0), t.Hin - t.H);
    w_off = min(max(t.aug[b * 3 + 1], 0), t.Win - t.W);
    mirror = t.aug[b * 3 + 2] != 0;
  } else {
    h_off = t.h_off; w_off = t.w_off; mirror = 0;
  }
}

// S = 4, C = 3 with the tile scheme of nchw_to_s2d43_tile_kernel: warp dy reads, for each colour, the 128 consecutive
// source bytes that 32 output pixels cover (reversed when the image is mirrored, still one contiguous run per load)
__global__ void __launch_bounds__(128)
u8_xform_s2d43_tile_kernel(XformDev t, bf16* __restrict__ y, int Hs, int Ws, int Cpad, int segs) {
  constexpr int S = 4, C = 3, PIX = 32, PITCH = 72;
  __shared__ __align__(16) bf16 tile[PIX * PITCH];
  const int lane = threadIdx.x & 31, dy = threadIdx.x >> 5;
  long long blk = blockIdx.x;
  const int seg = (int)(blk % segs); blk /= segs;
  const int hs = (int)(blk % Hs);
  const long long b = blk / Hs;
  const int ws0 = seg * PIX;
  int h_off, w_off, mirror;
  xform_image(t, b, h_off, w_off, mirror);
  for (int j = S * S * C + dy * 4; j < Cpad && j < S * S * C + dy * 4 + 4; ++j) tile[lane * PITCH + j] = __float2bfloat16(0.f);
  const int h = hs * S + dy;
  const int wbase = ws0 * S;
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const uint8_t* row = t.x + ((b * C + c) * t.Hin + (h + h_off)) * (long long)t.Win + w_off;
#pragma unroll
    for (int i = 0; i < S; ++i) {
      const int e = i * 32 + lane;
      const int w = wbase + e;
      float v = 0.f;
      if (h < t.H && w < t.W) v = ((float)__ldg(row + (mirror ? t.W - 1 - w : w)) - t.mean[c]) * t.scale;
      tile[(e >> 2) * PITCH + (dy * S + (e & 3)) * C + c] = __float2bfloat16(v);
    }
  }
  __syncthreads();
  const int per_pix = Cpad >> 3;
  const int npix = min(PIX, Ws - ws0);
  bf16* dst = y + ((b * Hs + hs) * (long long)Ws + ws0) * Cpad;
  for (int i = threadIdx.x; i < npix * per_pix; i += blockDim.x) {
    const int px = i / per_pix, piece = i - px * per_pix;
    *reinterpret_cast<uint4*>(dst + (long long)i * 8) = *reinterpret_cast<const uint4*>(tile + px * PITCH + piece * 8);
  }
}

// any S >= 1 (S = 1: plain NHWC) and C <= 4: one thread per output element
__global__ void __launch_bounds__(256)
u8_xform_generic_kernel(XformDev t, bf16* __restrict__ y, int B, int C, int S, int Hs, int Ws, int Cpad) {
  const long long total = (long long)B * Hs * Ws * Cpad;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int j = (int)(i % Cpad);
    long long r = i / Cpad;
    const int ws = (int)(r % Ws); r /= Ws;
    const int hs = (int)(r % Hs);
    const long long b = r / Hs;
    float v = 0.f;
    if (j < S * S * C) {
      const int c = j % C, q = j / C, dx = q % S, dy = q / S;
      const int h = hs * S + dy, w = ws * S + dx;
      if (h < t.H && w < t.W) {
        int h_off, w_off, mirror;
        xform_image(t, b, h_off, w_off, mirror);
        const uint8_t* row = t.x + ((b * C + c) * t.Hin + (h + h_off)) * (long long)t.Win + w_off;
        v = ((float)__ldg(row + (mirror ? t.W - 1 - w : w)) - t.mean[c]) * t.scale;
      }
    }
    y[i] = __float2bfloat16(v);
  }
}

// g[r][c] = 0 where mask[c] == 0
__global__ void __launch_bounds__(256)
col_mask_kernel(float* __restrict__ g, const uint8_t* __restrict__ mask, long long rows, int cols, long long ld) {
  const long long total = rows * cols;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % cols);
    if (!mask[c]) g[(i / cols) * ld + c] = 0.f;
  }
}

// ---------------- pooling (NHWC, 8 channels per thread) ----------------
// Output may be a channel slice of a wider tensor (pitch ldy, offset applied by the caller).
// ---- packed helpers for max pooling: 8 channels at a time, two per 32-bit register ----
// Window code per 16-bit lane.
__device__ __forceinline__ uint32_t dup16(uint32_t code) { return code | (code << 16); }
// acc (4 x bf16x2) += d where argmax byte == code.  `pk` holds the 8 argmax bytes, `d` the 8 gradients.
__device__ __forceinline__ void pool_bwd_accum(__nv_bfloat162 (&acc)[4], const uint2 pk, const uint4 d, uint32_t code) {
  const uint32_t c4 = code * 0x01010101u;
  const uint32_t m0 = __vcmpeq4(pk.x, c4), m1 = __vcmpeq4(pk.y, c4);     // 0xff per matching channel
  if ((m0 | m1) == 0) return;
  const uint32_t dv[4] = {d.x, d.y, d.z, d.w};
  const uint32_t mk[4] = {__byte_perm(m0, 0, 0x1100), __byte_perm(m0, 0, 0x3322), __byte_perm(m1, 0, 0x1100),
                          __byte_perm(m1, 0, 0x3322)};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t sel = dv[j] & mk[j];
    acc[j] = __hadd2(acc[j], *reinterpret_cast<const __nv_bfloat162*>(&sel));
  }
}
__device__ __forceinline__ uint4 pool_bwd_pack(const __nv_bfloat162 (&acc)[4]) {
  return make_uint4(*reinterpret_cast<const uint32_t*>(&acc[0]), *reinterpret_cast<const uint32_t*>(&acc[1]),
                    *reinterpret_cast<const uint32_t*>(&acc[2]), *reinterpret_cast<const uint32_t*>(&acc[3]));
}

// One block per output row (b, oh): threadIdx.x walks the 8-channel vectors of a pixel, threadIdx.y the
// pixels of the row, so no thread ever divides to find its coordinates and a warp reads contiguous pixels.
__global__ void __launch_bounds__(256)
maxpool_forward_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, uint8_t* __restrict__ argmax,
                       const GeepsPoolGeom g) {
  const int cv = g.C >> 3;
  const int oh = blockIdx.x % g.OH, b = blockIdx.x / g.OH;
  const int ih0 = oh * g.stride - g.pad;
  const int kh_lo = max(0, -ih0), kh_hi = min(g.K, g.H - ih0);
  const bf16* xb = x + (long long)b * g.H * g.W * g.ldx;
  const long long orow = ((long long)b * g.OH + oh) * g.OW;
  for (int ow = threadIdx.y; ow < g.OW; ow += blockDim.y) {
    const int iw0 = ow * g.stride - g.pad;
    const int kw_lo = max(0, -iw0), kw_hi = min(g.K, g.W - iw0);
    for (int cvi = threadIdx.x; cvi < cv; cvi += blockDim.x) {
      const int c = cvi * 8;
      // packed: best value and window code per 16-bit lane; strict > keeps the first maximum
      const uint32_t neg = 0xff7fff7fu;                 // two bf16 lowest finite values
      __nv_bfloat162 best[4];
      uint32_t arg[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) { best[j] = *reinterpret_cast<const __nv_bfloat162*>(&neg); arg[j] = 0x00ff00ffu; }
      for (int kh = kh_lo; kh < kh_hi; ++kh) {
        const bf16* xr = xb + ((long long)(ih0 + kh) * g.W + iw0) * g.ldx + c;
        for (int kw = kw_lo; kw < kw_hi; ++kw) {
          const uint4 v = *reinterpret_cast<const uint4*>(xr + (long long)kw * g.ldx);
          const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
          const uint32_t code = dup16((uint32_t)(kh * g.K + kw));
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
      *reinterpret_cast<uint4*>(y + opix * g.ldy + c) = pool_bwd_pack(best);
      uint2 pk;      // 16-bit lanes -> bytes
      pk.x = __byte_perm(arg[0], arg[1], 0x6420);
      pk.y = __byte_perm(arg[2], arg[3], 0x6420);
      *reinterpret_cast<uint2*>(argmax + opix * g.C + c) = pk;
    }
  }
}
// One block per input row (b, ih).  The output rows whose window covers ih are the same for the whole
// block, the output columns covering iw are a short range: only those windows are visited.
__global__ void __launch_bounds__(256)
maxpool_backward_kernel(const bf16* __restrict__ dy, const uint8_t* __restrict__ argmax, bf16* __restrict__ dx,
                        const GeepsPoolGeom g, int accumulate) {
  const int cv = g.C >> 3;
  const int ih = blockIdx.x % g.H, b = blockIdx.x / g.H;
  const int th = ih + g.pad;
  // oh * stride <= th <= oh * stride + K - 1
  const int oh_lo = max(0, (th - g.K + g.stride) / g.stride), oh_hi = min(g.OH - 1, th / g.stride);
  const long long obase = (long long)b * g.OH * g.OW;
  bf16* drow = dx + ((long long)b * g.H + ih) * g.W * g.ldx;
  for (int iw = threadIdx.y; iw < g.W; iw += blockDim.y) {
    const int tw = iw + g.pad;
    const int ow_lo = max(0, (tw - g.K + g.stride) / g.stride), ow_hi = min(g.OW - 1, tw / g.stride);
    for (int cvi = threadIdx.x; cvi < cv; cvi += blockDim.x) {
      const int c = cvi * 8;
      __nv_bfloat162 acc[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] = __floats2bfloat162_rn(0.f, 0.f);
      for (int oh = oh_lo; oh <= oh_hi; ++oh) {
        const int kh = th - oh * g.stride;
        for (int ow = ow_lo; ow <= ow_hi; ++ow) {
          const int code = kh * g.K + (tw - ow * g.stride);
          const long long opix = obase + (long long)oh * g.OW + ow;
          const uint2 pk = *reinterpret_cast<const uint2*>(argmax + opix * g.C + c);
          const uint4 d = *reinterpret_cast<const uint4*>(dy + opix * g.ldy + c);
          pool_bwd_accum(acc, pk, d, (uint32_t)code);
        }
      }
      bf16* dst = drow + (long long)iw * g.ldx + c;
      if (accumulate) {
        const uint4 old = *reinterpret_cast<const uint4*>(dst);
        const uint32_t ov[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] = __hadd2(acc[j], *reinterpret_cast<const __nv_bfloat162*>(&ov[j]));
      }
      *reinterpret_cast<uint4*>(dst) = pool_bwd_pack(acc);
    }
  }
}

// Same product, staged through shared memory: a block owns `stride` consecutive input rows of one image; the few
// output rows whose windows cover them (dy and argmax) are copied into shared memory once and every input
// pixel then gathers from there.  The direct kernel re-reads each dy / argmax element from L2 for every input
// pixel of its window (K*K times); here it crosses L2 -> SM once per block.
__global__ void __launch_bounds__(256)
maxpool_backward_smem_kernel(const bf16* __restrict__ dy, const uint8_t* __restrict__ argmax, bf16* __restrict__ dx,
                             const GeepsPoolGeom g, int accumulate, int rows_per_block, int max_oh) {
  extern __shared__ __align__(16) uint8_t pool_smem[];
  const int cv = g.C >> 3;
  const int row_blocks = (g.H + rows_per_block - 1) / rows_per_block;
  const int rb = blockIdx.x % row_blocks, b = blockIdx.x / row_blocks;
  const int ih_lo = rb * rows_per_block, ih_hi = min(g.H, ih_lo + rows_per_block);      // [lo, hi)
  const int oh_lo = max(0, (ih_lo + g.pad - g.K + g.stride) / g.stride);
  const int oh_hi = min(g.OH - 1, (ih_hi - 1 + g.pad) / g.stride);
  const int n_oh = oh_hi - oh_lo + 1;
  bf16* s_dy = reinterpret_cast<bf16*>(pool_smem);                                        // [max_oh][OW][C]
  uint8_t* s_arg = pool_smem + (size_t)max_oh * g.OW * g.C * sizeof(bf16);                // [max_oh][OW][C]
  const int tid = threadIdx.y * blockDim.x + threadIdx.x, nthreads = blockDim.x * blockDim.y;
  if (n_oh > 0) {
    const long long obase = ((long long)b * g.OH + oh_lo) * g.OW;
    const int vecs = n_oh * g.OW * cv;
    for (int v = tid; v < vecs; v += nthreads) {
      const int pix = v / cv, c = (v - pix * cv) * 8;
      *reinterpret_cast<uint4*>(s_dy + (size_t)pix * g.C + c) =
          *reinterpret_cast<const uint4*>(dy + (obase + pix) * g.ldy + c);
      *reinterpret_cast<uint2*>(s_arg + (size_t)pix * g.C + c) =
          *reinterpret_cast<const uint2*>(argmax + (obase + pix) * g.C + c);
    }
  }
  __syncthreads();
  for (int ih = ih_lo; ih < ih_hi; ++ih) {
    const int th = ih + g.pad;
    const int r_lo = max(oh_lo, (th - g.K + g.stride) / g.stride), r_hi = min(oh_hi, th / g.stride);
    bf16* drow = dx + ((long long)b * g.H + ih) * g.W * g.ldx;
    for (int iw = threadIdx.y; iw < g.W; iw += blockDim.y) {
      const int tw = iw + g.pad;
      const int ow_lo = max(0, (tw - g.K + g.stride) / g.stride), ow_hi = min(g.OW - 1, tw / g.stride);
      for (int cvi = threadIdx.x; cvi < cv; cvi += blockDim.x) {
        const int c = cvi * 8;
        __nv_bfloat162 acc[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] = __floats2bfloat162_rn(0.f, 0.f);
        for (int oh = r_lo; oh <= r_hi; ++oh) {
          const int kh = th - oh * g.stride;
          for (int ow = ow_lo; ow <= ow_hi; ++ow) {
            const int code = kh * g.K + (tw - ow * g.stride);
            const size_t sp = ((size_t)(oh - oh_lo) * g.OW + ow) * g.C + c;
            pool_bwd_accum(acc, *reinterpret_cast<const uint2*>(s_arg + sp), *reinterpret_cast<const uint4*>(s_dy + sp),
                           (uint32_t)code);
          }
        }
        bf16* dst = drow + (long long)iw * g.ldx + c;
        if (accumulate) {
          const uint4 old = *reinterpret_cast<const uint4*>(dst);
          const uint32_t ov[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[j] = __hadd2(acc[j], *reinterpret_cast<const __nv_bfloat162*>(&ov[j]));
        }
        *reinterpret_cast<uint4*>(dst) = pool_bwd_pack(acc);
      }
    }
  }
}

// Caffe average pooling: divisor is the window area clipped to the padded extent.
__device__ __forceinline__ int avg_area(int o, int stride, int pad, int K, int size) {
  const int s = o * stride - pad;
  const int e = min(s + K, size + pad);
  return e - s;
}
__global__ void __launch_bounds__(256)
avgpool_forward_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, const GeepsPoolGeom g) {
  const int cv = g.C >> 3;
  const long long total = (long long)g.B * g.OH * g.OW * cv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % cv) * 8;
    long long p = i / cv;
    const int ow = (int)(p % g.OW); p /= g.OW;
    const int oh = (int)(p % g.OH);
    const int b = (int)(p / g.OH);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int kh = 0; kh < g.K; ++kh) {
      const int ih = oh * g.stride - g.pad + kh;
      if (ih < 0 || ih >= g.H) continue;
      for (int kw = 0; kw < g.K; ++kw) {
        const int iw = ow * g.stride - g.pad + kw;
        if (iw < 0 || iw >= g.W) continue;
        Bf8 v = ld8(x + (((long long)b * g.H + ih) * g.W + iw) * g.ldx + c);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += bf(v.v[e]);
      }
    }
    const float inv = 1.f / (float)(avg_area(oh, g.stride, g.pad, g.K, g.H) * avg_area(ow, g.stride, g.pad, g.K, g.W));
    Bf8 o;
#pragma unroll
    for (int e = 0; e < 8; ++e) o.v[e] = __float2bfloat16(acc[e] * inv);
    st8(y + (((long long)b * g.OH + oh) * g.OW + ow) * g.ldy + c, o);
  }
}
__global__ void __launch_bounds__(256)
avgpool_backward_kernel(const bf16* __restrict__ dy, bf16* __restrict__ dx, const GeepsPoolGeom g, int accumulate) {
  const int cv = g.C >> 3;
  const long long total = (long long)g.B * g.H * g.W * cv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % cv) * 8;
    long long p = i / cv;
    const int iw = (int)(p % g.W); p /= g.W;
    const int ih = (int)(p % g.H);
    const int b = (int)(p / g.H);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int kh = 0; kh < g.K; ++kh) {
      const int th = ih + g.pad - kh;
      int oh, ow;
      if (th < 0 || !div_exact(th, g.stride, oh) || oh >= g.OH) continue;
      for (int kw = 0; kw < g.K; ++kw) {
        const int tw = iw + g.pad - kw;
        if (tw < 0 || !div_exact(tw, g.stride, ow) || ow >= g.OW) continue;
        const float inv = 1.f / (float)(avg_area(oh, g.stride, g.pad, g.K, g.H) * avg_area(ow, g.stride, g.pad, g.K, g.W));
        Bf8 d = ld8(dy + (((long long)b * g.OH + oh) * g.OW + ow) * g.ldy + c);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += bf(d.v[e]) * inv;
      }
    }
    bf16* dst = dx + (((long long)b * g.H + ih) * g.W + iw) * g.ldx + c;
    Bf8 o;
    if (accumulate) { Bf8 old = ld8(dst);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += bf(old.v[e]); }
#pragma unroll
    for (int e = 0; e < 8; ++e) o.v[e] = __float2bfloat16(acc[e]);
    st8(dst, o);
  }
}

// ---------------- softmax cross-entropy (one CTA per sample) ----------------
__device__ __forceinline__ float block_reduce(float v, bool is_max, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, t) : v + t;
  }
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  if (w == 0) {
    v = lane < (int)(blockDim.x >> 5) ? sh[lane] : (is_max ? -3.0e38f : 0.f);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float t = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? fmaxf(v, t) : v + t;
    }
    if (lane == 0) sh[0] = v;
  }
  __syncthreads();
  return sh[0];
}
// loss_sum += -log softmax(logits[b])[label[b]] * loss_scale;  dlogits = (softmax - onehot) * grad_scale
__global__ void __launch_bounds__(256)
softmax_ce_kernel(const float* __restrict__ logits, const long long* __restrict__ labels, float* loss_sum,
                  float* __restrict__ per_sample, bf16* __restrict__ dlogits, int C, long long ldl, long long ldd,
                  float loss_scale, float grad_scale, int* status) {
  __shared__ float sh[32];
  const int b = blockIdx.x;
  const float* row = logits + (long long)b * ldl;
  float mx = -3.0e38f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) mx = fmaxf(mx, row[c]);
  mx = block_reduce(mx, true, sh);
  float s = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) s += __expf(row[c] - mx);
  s = block_reduce(s, false, sh);
  long long lab = labels[b];
  if (lab < 0 || lab >= C) {
    if (threadIdx.x == 0) geeps_report(status, GEEPS_ERR_BOUNDS, 30, b, (int)lab);
    lab = 0;
  }
  const float inv = 1.f / s;
  if (dlogits != nullptr) {
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float pr = __expf(row[c] - mx) * inv;
      dlogits[(long long)b * ldd + c] = __float2bfloat16((pr - (c == lab ? 1.f : 0.f)) * grad_scale);
    }
  }
  if (threadIdx.x == 0) {
    const float l = -(row[lab] - mx - __logf(s));
    if (per_sample) per_sample[b] = l;
    if (loss_sum) atomicAdd(loss_sum, l * loss_scale);
  }
}

}  // namespace

#define CK() ((int)cudaGetLastError())

template <typename T>
static int nchw_to_nhwc_launch(const T* x, void* y, int B, int C, int H, int W, int Cpad, cudaStream_t st) {
  const long long n = (long long)B * H * W * Cpad;
  if (Cpad % 4 == 0)
    nchw_to_nhwc_pix_kernel<T><<<grid_1d((long long)B * H * W), 256, 0, st>>>(x, (bf16*)y, B, C, H * W, Cpad);
  else
    nchw_f32_to_nhwc_bf16_kernel<T><<<grid_1d(n), 256, 0, st>>>(x, (bf16*)y, B, C, H, W, Cpad);
  return CK();
}

template <typename T>
static int nchw_to_s2d_launch(const T* x, void* y, int B, int C, int H, int W, int S, int Hs, int Ws, int Cpad,
                              cudaStream_t st) {
  if (S == 4 && C == 3 && Cpad % 8 == 0 && Cpad >= 48 && Cpad <= 64 && (((uintptr_t)y) & 15) == 0) {
    const int segs = (Ws + 31) / 32;
    nchw_to_s2d43_tile_kernel<T><<<(unsigned)((long long)B * Hs * segs), 128, 0, st>>>(x, (bf16*)y, B, H, W, Hs, Ws, Cpad,
                                                                                      segs);
  } else if (S == 4 && C == 3)
    nchw_to_s2d_kernel<4, 3, T><<<grid_1d((long long)B * Hs * Ws), 256, 0, st>>>(x, (bf16*)y, B, H, W, Hs, Ws, Cpad);
  else
    nchw_to_s2d_generic_kernel<T><<<grid_1d((long long)B * Hs * Ws * Cpad), 256, 0, st>>>(x, (bf16*)y, B, C, H, W, S,
                                                                                         Hs, Ws, Cpad);
  return CK();
}

extern "C" {

int geeps_nchw_to_nhwc_bf16(const void* x, int x_is_bf16, void* y, int B, int C, int H, int W, int Cpad, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  return x_is_bf16 ? nchw_to_nhwc_launch((const bf16*)x, y, B, C, H, W, Cpad, st)
                   : nchw_to_nhwc_launch((const float*)x, y, B, C, H, W, Cpad, st);
}
int geeps_nchw_f32_to_nhwc_bf16(const float* x, void* y, int B, int C, int H, int W, int Cpad, void* stream) {
  return geeps_nchw_to_nhwc_bf16(x, 0, y, B, C, H, W, Cpad, stream);
}

int geeps_nchw_to_s2d_bf16(const void* x, int x_is_bf16, void* y, int B, int C, int H, int W, int S, int Hs, int Ws,
                           int Cpad, void* stream) {
  if (S <= 0 || Cpad < S * S * C || (Cpad & 7)) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  return x_is_bf16 ? nchw_to_s2d_launch((const bf16*)x, y, B, C, H, W, S, Hs, Ws, Cpad, st)
                   : nchw_to_s2d_launch((const float*)x, y, B, C, H, W, S, Hs, Ws, Cpad, st);
}

int geeps_u8_transform_bf16(const GeepsU8Transform* p, void* stream) {
  if (p == nullptr || p->x == nullptr || p->y == nullptr) return (int)cudaErrorInvalidValue;
  const int S = p->S < 1 ? 1 : p->S;
  if (p->C < 1 || p->C > 4 || p->B < 1 || p->H < 1 || p->W < 1 || p->Hin < p->H || p->Win < p->W ||
      p->Cpad < S * S * p->C || p->Hs < 1 || p->Ws < 1)
    return (int)cudaErrorInvalidValue;
  // every source element an output position can name lies inside the cropped image
  if ((long long)(p->Hs - 1) * S >= p->H || (long long)(p->Ws - 1) * S >= p->W) return (int)cudaErrorInvalidValue;
  XformDev t;
  t.x = p->x; t.aug = p->aug;
  t.Hin = p->Hin; t.Win = p->Win; t.H = p->H; t.W = p->W;
  t.h_off = (p->Hin - p->H) / 2; t.w_off = (p->Win - p->W) / 2;
  for (int c = 0; c < 4; ++c) t.mean[c] = p->mean[c];
  t.scale = p->scale;
  cudaStream_t st = (cudaStream_t)stream;
  if (S == 4 && p->C == 3 && p->Cpad % 8 == 0 && p->Cpad >= 48 && p->Cpad <= 64 && (((uintptr_t)p->y) & 15) == 0) {
    const int segs = (p->Ws + 31) / 32;
    u8_xform_s2d43_tile_kernel<<<(unsigned)((long long)p->B * p->Hs * segs), 128, 0, st>>>(t, (bf16*)p->y, p->Hs, p->Ws,
                                                                                          p->Cpad, segs);
  } else {
    u8_xform_generic_kernel<<<grid_1d((long long)p->B * p->Hs * p->Ws * p->Cpad), 256, 0, st>>>(t, (bf16*)p->y, p->B, p->C,
                                                                                              S, p->Hs, p->Ws, p->Cpad);
  }
  return CK();
}

int geeps_col_mask_f32(float* g, const unsigned char* mask, long long rows, int cols, long long ld, void* stream) {
  col_mask_kernel<<<grid_1d(rows * cols), 256, 0, (cudaStream_t)stream>>>(g, mask, rows, cols, ld);
  return CK();
}

int geeps_im2col(const void* x, void* col, const GeepsConvGeom* g, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const long long rows = (long long)g->B * g->OH * g->OW;
  const int kd = g->KH * g->KW * g->Cg;
  if (g->ldcol > kd)
    zero_col_pad_kernel<<<grid_1d(rows * (g->ldcol - kd)), 256, 0, st>>>((bf16*)col, rows, kd, g->ldcol);
  const bool a8 = (g->Cg % 8 == 0) && (g->C % 8 == 0) && (g->c0 % 8 == 0) && (g->ldcol % 8 == 0);
  const bool a4 = (g->Cg % 4 == 0) && (g->C % 4 == 0) && (g->c0 % 4 == 0) && (g->ldcol % 4 == 0);
  const int wgrid = grid_1d(rows * 32);   // one warp per patch-matrix row
  if (a8) im2col_kernel<8><<<wgrid, 256, 0, st>>>((const bf16*)x, (bf16*)col, *g);
  else if (a4) im2col_kernel<4><<<wgrid, 256, 0, st>>>((const bf16*)x, (bf16*)col, *g);
  else im2col_kernel<1><<<wgrid, 256, 0, st>>>((const bf16*)x, (bf16*)col, *g);
  return CK();
}

int geeps_col2im(const void* dcol, void* dx, const GeepsConvGeom* g, int accumulate, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const long long pix = (long long)g->B * g->H * g->W;
  const bool a8 = (g->Cg % 8 == 0) && (g->C % 8 == 0) && (g->c0 % 8 == 0) && (g->ldcol % 8 == 0);
  if (a8) col2im_kernel<8><<<grid_1d(pix * (g->Cg / 8)), 256, 0, st>>>((const bf16*)dcol, (bf16*)dx, *g, accumulate);
  else col2im_kernel<1><<<grid_1d(pix * g->Cg), 256, 0, st>>>((const bf16*)dcol, (bf16*)dx, *g, accumulate);
  return CK();
}

static int reduce_grid(long long P, int C) {
  long long want = (P * (C / 8) + 255) / 256;
  if (want > geeps_sm_count() * 4) want = geeps_sm_count() * 4;
  long long min_blocks = ((long long)(C / 8) + 255) / 256;
  if (want < min_blocks) want = min_blocks;
  return (int)(want < 1 ? 1 : want);
}

int geeps_bn_forward(const void* x, void* y, const float* gamma, const float* beta, float* sums,
                     float* mean_rstd, float* running_mean, float* running_var, long long P, int C,
                     long long ldx, long long ldy, float eps, float momentum, int relu, void* stream) {
  if (C % 8) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  cudaMemsetAsync(sums, 0, sizeof(float) * 2 * C, st);
  channel_reduce_kernel<0><<<reduce_grid(P, C), 256, 2 * C * sizeof(float), st>>>(
      (const bf16*)x, nullptr, nullptr, nullptr, sums, P, C, ldx, 0, 0, 1.f);
  bn_finalize_kernel<<<(C + 127) / 128, 128, 0, st>>>(sums, mean_rstd, running_mean, running_var, C,
                                                      1.f / (float)P, eps, momentum);
  bn_apply_kernel<<<grid_1d(P * (C / 8)), 256, 0, st>>>((const bf16*)x, (bf16*)y, mean_rstd, gamma, beta, P, C, ldx,
                                                        ldy, relu);
  return CK();
}

int geeps_bn_backward(const void* x, const void* dy, const void* y, void* dx, const float* mean_rstd,
                      const float* gamma, float* sums, float* dgamma, float* dbeta, long long P, int C,
                      long long ldx, long long lddy, long long lddx, int relu, float grad_scale, void* stream) {
  if (C % 8) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  cudaMemsetAsync(sums, 0, sizeof(float) * 2 * C, st);
  channel_reduce_kernel<1><<<reduce_grid(P, C), 256, 2 * C * sizeof(float), st>>>(
      (const bf16*)x, (const bf16*)dy, (const bf16*)y, mean_rstd, sums, P, C, ldx, lddy, relu, 1.f);
  bn_backward_kernel<<<grid_1d(P * (C / 8)), 256, 0, st>>>((const bf16*)x, (const bf16*)dy, (const bf16*)y,
                                                           (bf16*)dx, mean_rstd, gamma, sums, dgamma, dbeta, P, C,
                                                           ldx, lddy, lddx, relu, grad_scale, nullptr);
  return CK();
}

// The training-loop forms: `sums` must be zero on entry (2 C floats) and `zero_after` (or NULL) is zeroed for the
// layer's next reduction, so a BatchNorm layer that alternates forward and backward needs no memset and no separate
// finalisation launch: 2 launches per direction instead of 4 and 3.
// grid of a single-launch BatchNorm kernel: enough blocks for the reduction, never more than can be resident at
// once beside other kernels (the blocks wait for one another at the grid barrier)
static int bn_coop_grid(long long P, int C) {
  int g = reduce_grid(P, C);
  const int cap = geeps_sm_count();
  return g > cap ? cap : g;
}
static bool bn_coop_enabled() {
  static int v = -1;
  // off by default: with at most one block per SM and a grid barrier the single launch is slower than two full-width
  // launches (Inception-BN-22K 5.84 against 5.65 ms per step, small net 1.96 against 1.95 ms)
  if (v < 0) { const char* e = getenv("GEEPS_BN_COOP"); v = e ? atoi(e) : 0; }
  return v != 0;
}

int geeps_bn_forward_fused(const void* x, void* y, const float* gamma, const float* beta, float* sums,
                           float* mean_rstd, float* running_mean, float* running_var, float* zero_after, int* barrier,
                           long long P, int C, long long ldx, long long ldy, float eps, float momentum, int relu,
                           void* stream) {
  if (C % 8) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  if (barrier != nullptr && bn_coop_enabled()) {
    const bf16* xx = (const bf16*)x; bf16* yy = (bf16*)y;
    float inv_count = 1.f / (float)P;
    void* args[] = {&xx, &yy, &sums, &mean_rstd, &running_mean, &running_var, &gamma, &beta, &zero_after, &barrier,
                    &P, &C, &ldx, &ldy, &relu, &inv_count, &eps, &momentum};
    cudaError_t e = cudaLaunchCooperativeKernel((void*)bn_forward_coop_kernel, dim3(bn_coop_grid(P, C)), dim3(256), args,
                                                2 * C * sizeof(float), st);
    return e == cudaSuccess ? CK() : (int)e;
  }
  channel_reduce_kernel<0><<<reduce_grid(P, C), 256, 2 * C * sizeof(float), st>>>(
      (const bf16*)x, nullptr, nullptr, nullptr, sums, P, C, ldx, 0, 0, 1.f);
  bn_apply_fused_kernel<<<grid_1d(P * (C / 8)), 256, 0, st>>>((const bf16*)x, (bf16*)y, sums, mean_rstd, running_mean,
                                                              running_var, gamma, beta, zero_after, P, C, ldx, ldy, relu,
                                                              1.f / (float)P, eps, momentum);
  return CK();
}
int geeps_bn_backward_fused(const void* x, const void* dy, const void* y, void* dx, float* mean_rstd,
                            const float* gamma, float* sums, float* dgamma, float* dbeta, float* zero_after,
                            int* barrier, long long P, int C, long long ldx, long long lddy, long long lddx, int relu,
                            float grad_scale, void* stream) {
  if (C % 8) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  if (barrier != nullptr && bn_coop_enabled()) {
    const bf16* xx = (const bf16*)x; const bf16* dd = (const bf16*)dy; const bf16* yy = (const bf16*)y;
    bf16* dxx = (bf16*)dx;
    void* args[] = {&xx, &dd, &yy, &dxx, &mean_rstd, &gamma, &sums, &dgamma, &dbeta, &zero_after, &barrier,
                    &P, &C, &ldx, &lddy, &lddx, &relu, &grad_scale};
    cudaError_t e = cudaLaunchCooperativeKernel((void*)bn_backward_coop_kernel, dim3(bn_coop_grid(P, C)), dim3(256),
                                                args, 2 * C * sizeof(float), st);
    return e == cudaSuccess ? CK() : (int)e;
  }
  channel_reduce_kernel<1><<<reduce_grid(P, C), 256, 2 * C * sizeof(float), st>>>(
      (const bf16*)x, (const bf16*)dy, (const bf16*)y, mean_rstd, sums, P, C, ldx, lddy, relu, 1.f);
  bn_backward_kernel<<<grid_1d(P * (C / 8)), 256, 0, st>>>((const bf16*)x, (const bf16*)dy, (const bf16*)y,
                                                           (bf16*)dx, mean_rstd, gamma, sums, dgamma, dbeta, P, C,
                                                           ldx, lddy, lddx, relu, grad_scale, zero_after);
  return CK();
}

int geeps_colsum(const void* x, float* out, long long P, int C, long long ldx, float scale, int zero_first,
                 void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if ((C % 8) || (ldx % 8) || C > 4096) {
    colsum_simple_kernel<<<(C + 127) / 128, 128, 0, st>>>((const bf16*)x, out, P, C, ldx, scale, !zero_first);
    return CK();
  }
  if (zero_first) cudaMemsetAsync(out, 0, sizeof(float) * C, st);
  channel_reduce_kernel<2><<<reduce_grid(P, C), 256, 2 * C * sizeof(float), st>>>(
      (const bf16*)x, nullptr, nullptr, nullptr, out, P, C, ldx, 0, 0, scale);
  return CK();
}

int geeps_copy_f32(float* dst, const float* src, long long n, void* stream) {
  return (int)cudaMemcpyAsync(dst, src, sizeof(float) * (size_t)n, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
}

int geeps_relu_backward(const void* dy, const void* y, void* dx, long long n, void* stream) {
  if (n % 8) return (int)cudaErrorInvalidValue;
  relu_backward_kernel<<<grid_1d(n / 8), 256, 0, (cudaStream_t)stream>>>((const bf16*)dy, (const bf16*)y, (bf16*)dx, n / 8);
  return CK();
}

int geeps_relu_backward_2d(const void* dy, const void* y, void* dx, long long P, int C, long long lddy, long long ldy,
                           long long lddx, void* stream) {
  if (C % 8 || lddy % 8 || ldy % 8 || lddx % 8) return (int)cudaErrorInvalidValue;
  relu_backward_2d_kernel<<<grid_1d(P * (C / 8)), 256, 0, (cudaStream_t)stream>>>((const bf16*)dy, (const bf16*)y,
                                                                                 (bf16*)dx, P, C, lddy, ldy, lddx);
  return CK();
}
int geeps_relu_backward_colsum(const void* dy, const void* y, void* dx, float* colsum, long long P, int C,
                               long long lddy, long long ldy, long long lddx, void* stream) {
  if (C % 8 || lddy % 8 || ldy % 8 || lddx % 8 || C > 8192) return (int)cudaErrorInvalidValue;
  cudaStream_t st = (cudaStream_t)stream;
  cudaMemsetAsync(colsum, 0, sizeof(float) * C, st);
  // enough CTAs that every pixel lane has work, a whole number of channel slots per grid
  long long want = (P * (C / 8) + 255) / 256;
  if (want > geeps_sm_count() * 8) want = geeps_sm_count() * 8;
  const long long min_blocks = ((long long)(C / 8) + 255) / 256;
  if (want < min_blocks) want = min_blocks;
  relu_backward_colsum_kernel<<<(int)(want < 1 ? 1 : want), 256, C * sizeof(float), st>>>(
      (const bf16*)dy, (const bf16*)y, (bf16*)dx, colsum, P, C, lddy, ldy, lddx);
  return CK();
}
int geeps_f32_to_bf16_2d(const float* src, void* dst, long long P, int C, long long lds, long long ldd, int relu,
                         void* stream) {
  if (C % 8 || lds % 4 || ldd % 8 || ((uintptr_t)src & 15) || ((uintptr_t)dst & 15)) return (int)cudaErrorInvalidValue;
  f32_to_bf16_2d_kernel<<<grid_1d(P * (C / 8)), 256, 0, (cudaStream_t)stream>>>(src, (bf16*)dst, P, C, lds, ldd, relu);
  return CK();
}
int geeps_add_bf16_2d(void* dst, const void* src, long long P, int C, long long ldd, long long lds, void* stream) {
  if (C % 8 || ldd % 8 || lds % 8) return (int)cudaErrorInvalidValue;
  add_2d_kernel<<<grid_1d(P * (C / 8)), 256, 0, (cudaStream_t)stream>>>((bf16*)dst, (const bf16*)src, P, C, ldd, lds);
  return CK();
}

int geeps_dropout(const void* x, void* y, long long n, float p, unsigned long long seed, void* stream) {
  dropout_kernel<<<grid_1d(n), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, n, p, seed, nullptr);
  return CK();
}
int geeps_dropout_ref(const void* x, void* y, long long n, float p, unsigned long long seed, const int* step_ref,
                      void* stream) {
  dropout_kernel<<<grid_1d(n), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, n, p, seed, step_ref);
  return CK();
}

int geeps_lrn_forward(const void* x, void* y, void* rscale, long long P, int C, int size, float alpha, float beta,
                      float k, void* stream) {
  const int g8 = grid_1d(P * (C / 8));
  cudaStream_t st8 = (cudaStream_t)stream;
  if (C % 8 == 0 && size == 5)
    lrn_forward_v8_kernel<2><<<g8, 256, 0, st8>>>((const bf16*)x, (bf16*)y, (bf16*)rscale, P, C, size, alpha, beta, k);
  else if (C % 8 == 0 && size == 3)
    lrn_forward_v8_kernel<1><<<g8, 256, 0, st8>>>((const bf16*)x, (bf16*)y, (bf16*)rscale, P, C, size, alpha, beta, k);
  else if (C % 8 == 0 && size == 7)
    lrn_forward_v8_kernel<3><<<g8, 256, 0, st8>>>((const bf16*)x, (bf16*)y, (bf16*)rscale, P, C, size, alpha, beta, k);
  else
    lrn_forward_kernel<<<grid_1d(P * C), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, (bf16*)rscale, P, C, size,
                                                                        alpha, beta, k);
  return CK();
}
int geeps_lrn_backward(const void* x, const void* y, const void* rscale, const void* dy, void* dx, long long P,
                       int C, int size, float alpha, float beta, int relu_mask, float* colsum, void* stream) {
  int g8 = grid_1d(P * (C / 8));
  cudaStream_t st8 = (cudaStream_t)stream;
  size_t cs_smem = 0;
  if (colsum != nullptr) {
    if (C % 8 || (size != 3 && size != 5 && size != 7) || C > 8192) return (int)cudaErrorInvalidValue;
    // gridDim * 256 must be a multiple of C/8 (one channel group per thread): round the grid down to a multiple of m
    int cv = C / 8, a = cv, b = 256;
    while (b) { int t = a % b; a = b; b = t; }
    const int m = cv / a;
    g8 = g8 >= m ? g8 / m * m : m;
    cs_smem = sizeof(float) * C;
    cudaMemsetAsync(colsum, 0, sizeof(float) * C, st8);
  }
  if (C % 8 == 0 && size == 5)
    lrn_backward_v8_kernel<2><<<g8, 256, cs_smem, st8>>>((const bf16*)x, (const bf16*)y, (const bf16*)rscale, (const bf16*)dy, (bf16*)dx, P, C, size, alpha, beta, relu_mask, colsum);
  else if (C % 8 == 0 && size == 3)
    lrn_backward_v8_kernel<1><<<g8, 256, cs_smem, st8>>>((const bf16*)x, (const bf16*)y, (const bf16*)rscale, (const bf16*)dy, (bf16*)dx, P, C, size, alpha, beta, relu_mask, colsum);
  else if (C % 8 == 0 && size == 7)
    lrn_backward_v8_kernel<3><<<g8, 256, cs_smem, st8>>>((const bf16*)x, (const bf16*)y, (const bf16*)rscale, (const bf16*)dy, (bf16*)dx, P, C, size, alpha, beta, relu_mask, colsum);
  else
    lrn_backward_kernel<<<grid_1d(P * C), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (const bf16*)y, (const bf16*)rscale,
                                                                         (const bf16*)dy, (bf16*)dx, P, C, size, alpha,
                                                                         beta, relu_mask);
  return CK();
}

int geeps_maxpool_forward(const void* x, void* y, void* argmax, const GeepsPoolGeom* g, void* stream) {
  if (g->C % 8 || g->ldx % 8 || g->ldy % 8 || g->K * g->K > 255) return (int)cudaErrorInvalidValue;
  maxpool_forward_kernel<<<g->B * g->OH, pool_block(g->C / 8), 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y,
                                                                                        (uint8_t*)argmax, *g);
  return CK();
}
int geeps_maxpool_backward(const void* dy, const void* argmax, void* dx, const GeepsPoolGeom* g, int accumulate,
                           void* stream) {
  if (g->C % 8 || g->ldx % 8 || g->ldy % 8) return (int)cudaErrorInvalidValue;
  // overlapping windows: stage the covering output rows in shared memory when they fit
  const int rows_per_block = g->stride > 1 ? 2 * g->stride : 2;
  const int max_oh = (rows_per_block + g->K - 2) / g->stride + 1;
  const size_t smem = (size_t)max_oh * g->OW * g->C * 3;
  if (g->K > g->stride && smem <= 96 * 1024) {
    static bool attr_set = false;
    if (!attr_set) {
      cudaFuncSetAttribute(maxpool_backward_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      attr_set = true;
    }
    const int row_blocks = (g->H + rows_per_block - 1) / rows_per_block;
    maxpool_backward_smem_kernel<<<g->B * row_blocks, pool_block(g->C / 8), smem, (cudaStream_t)stream>>>(
        (const bf16*)dy, (const uint8_t*)argmax, (bf16*)dx, *g, accumulate, rows_per_block, max_oh);
    return CK();
  }
  maxpool_backward_kernel<<<g->B * g->H, pool_block(g->C / 8), 0, (cudaStream_t)stream>>>(
      (const bf16*)dy, (const uint8_t*)argmax, (bf16*)dx, *g, accumulate);
  return CK();
}
int geeps_avgpool_forward(const void* x, void* y, const GeepsPoolGeom* g, void* stream) {
  if (g->C % 8 || g->ldx % 8 || g->ldy % 8) return (int)cudaErrorInvalidValue;
  const long long n = (long long)g->B * g->OH * g->OW * (g->C / 8);
  avgpool_forward_kernel<<<grid_1d(n), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, *g);
  return CK();
}
int geeps_avgpool_backward(const void* dy, void* dx, const GeepsPoolGeom* g, int accumulate, void* stream) {
  if (g->C % 8 || g->ldx % 8 || g->ldy % 8) return (int)cudaErrorInvalidValue;
  const long long n = (long long)g->B * g->H * g->W * (g->C / 8);
  avgpool_backward_kernel<<<grid_1d(n), 256, 0, (cudaStream_t)stream>>>((const bf16*)dy, (bf16*)dx, *g, accumulate);
  return CK();
}

int geeps_softmax_ce(const float* logits, const long long* labels, float* loss_sum, float* per_sample,
                     void* dlogits, int B, int C, long long ldl, long long ldd, float loss_scale, float grad_scale,
                     int zero_loss, int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (zero_loss && loss_sum) cudaMemsetAsync(loss_sum, 0, sizeof(float), st);
  softmax_ce_kernel<<<B, 256, 0, st>>>(logits, labels, loss_sum, per_sample, (bf16*)dlogits, C, ldl, ldd, loss_scale,
                                       grad_scale, status);
  return CK();
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// BatchNorm forward for callers that must not allocate device memory.
//
// geeps_bn_forward needs 2*C floats of scratch for the per-channel sums and leaves it to the
// caller to provide them.  Two kinds of callers of this library cannot do that: code running
// under the parameter server's memory plan, where every byte of the GPU budget has been handed
// out before the first clock and no allocator exists in steady state, and plain C/C++ hosts that
// link the library without any device allocator of their own and must not pay cudaMalloc's
// device-wide synchronisation inside their step loop.  For them the scratch lives in the
// library image itself: a fixed array in device memory, sized for GEEPS_BN_NOALLOC_MAX_CHANNELS
// channels (32 KB), that every GPU loading the library holds until the process exits.
//
// The array is shared by all calls and keeps whatever the previous call left in it, so the
// entry point clears the part it uses on the caller's stream before the reduction.  Two calls
// whose kernels can overlap on the GPU (different streams, no ordering between them) race on it.
// ---------------------------------------------------------------------------------------------
#include <stdio.h>
#include <mutex>

#define GEEPS_BN_NOALLOC_MAX_CHANNELS_IMPL 4096
static __device__ __align__(256) float g_bn_noalloc_scratch[2 * GEEPS_BN_NOALLOC_MAX_CHANNELS_IMPL];

namespace {
constexpr int kNoallocMaxDevices = 64;
float* g_bn_noalloc_ptr[kNoallocMaxDevices] = {};
std::mutex g_bn_noalloc_mu;

// Device address of the scratch array on the current device.  In host code the array's name is
// only a handle for the runtime; the address a kernel can use comes from cudaGetSymbolAddress,
// looked up once per device with that device current.
int bn_noalloc_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kNoallocMaxDevices) return (int)cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lk(g_bn_noalloc_mu);
  if (g_bn_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_bn_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_bn_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_bn_noalloc_ptr[dev];
  return 0;
}
}  // namespace

extern "C" {

int geeps_bn_noalloc_max_channels() { return GEEPS_BN_NOALLOC_MAX_CHANNELS_IMPL; }

int geeps_bn_forward_noalloc(const void* x, void* y, const float* gamma, const float* beta, float* mean_rstd,
                             float* running_mean, float* running_var, long long P, int C, long long ldx,
                             long long ldy, float eps, float momentum, int relu, void* stream) {
  if (C <= 0 || C % 8) return (int)cudaErrorInvalidValue;
  if (C > GEEPS_BN_NOALLOC_MAX_CHANNELS_IMPL) {
    fprintf(stderr, "geeps_bn_forward_noalloc: %d channels exceed the built-in scratch of %d channels; "
                    "use geeps_bn_forward with caller-provided scratch\n", C, GEEPS_BN_NOALLOC_MAX_CHANNELS_IMPL);
    return GEEPS_ERR_NOALLOC_TOO_LARGE;
  }
  float* sums = nullptr;
  const int rc = bn_noalloc_scratch(&sums);   // first call on a device resolves the address
  if (rc != 0) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(sums, 0, sizeof(float) * 2 * C, st);   // the array keeps the last call's sums
  if (e != cudaSuccess) return (int)e;
  channel_reduce_kernel<0><<<reduce_grid(P, C), 256, 2 * C * sizeof(float), st>>>(
      (const bf16*)x, nullptr, nullptr, nullptr, sums, P, C, ldx, 0, 0, 1.f);
  bn_finalize_kernel<<<(C + 127) / 128, 128, 0, st>>>(sums, mean_rstd, running_mean, running_var, C,
                                                      1.f / (float)P, eps, momentum);
  bn_apply_kernel<<<grid_1d(P * (C / 8)), 256, 0, st>>>((const bf16*)x, (bf16*)y, mean_rstd, gamma, beta, P, C, ldx,
                                                        ldy, relu);
  return CK();
}

}  // extern "C"
