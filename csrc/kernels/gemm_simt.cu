// Plain SIMT bf16 GEMM with the same contract as geeps_gemm_bf16.  It exists for shapes the
// TMA path cannot take (leading dimensions that are not multiples of 16 bytes) and as an
// independent on-device cross-check of the tcgen05 kernel in the tests.  64x64 tile,
// 16-deep k slab, 256 threads x 4x4 outputs, fp32 accumulate.
#include "common.cuh"
#include "kernels.h"

namespace {

__global__ void __launch_bounds__(256)
gemm_simt_kernel(const GeepsGemmParams p) {
  __shared__ float As[16][64 + 1];
  __shared__ float Bs[16][64 + 1];
  const __nv_bfloat16* A = (const __nv_bfloat16*)p.A;
  const __nv_bfloat16* B = (const __nv_bfloat16*)p.B;
  const long long m0 = (long long)blockIdx.x * 64, n0 = (long long)blockIdx.y * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  // element (row, k) of an operand: K-major -> base[row*ld + k]; MN-major -> base[k*ld + row]
  const long long sa_r = p.a_mn_major ? 1 : p.lda, sa_k = p.a_mn_major ? p.lda : 1;
  const long long sb_r = p.b_mn_major ? 1 : p.ldb, sb_k = p.b_mn_major ? p.ldb : 1;
  float acc[4][4] = {};
  for (long long k0 = 0; k0 < p.K; k0 += 16) {
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
      int r, k;
      if (p.a_mn_major) { r = e & 63; k = e >> 6; } else { k = e & 15; r = e >> 4; }
      As[k][r] = (m0 + r < p.M && k0 + k < p.K) ? __bfloat162float(A[(m0 + r) * sa_r + (k0 + k) * sa_k]) : 0.f;
      if (p.b_mn_major) { r = e & 63; k = e >> 6; } else { k = e & 15; r = e >> 4; }
      Bs[k][r] = (n0 + r < p.N && k0 + k < p.K) ? __bfloat162float(B[(n0 + r) * sb_r + (k0 + k) * sb_k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[k][ty * 4 + i]; b[i] = Bs[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; ++i) {
    const long long m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
    for (int j = 0; j < 4; ++j) {
      const long long n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      float v = p.alpha * acc[i][j];
      if (p.bias != nullptr) {
        if (p.bias_mode == 1) v += p.bias[n]; else if (p.bias_mode == 2) v += p.bias[m];
      }
      if (p.out_fp32) {
        float* c = (float*)p.C + m * p.ldc + n;
        if (p.beta != 0.f) v += p.beta * *c;
        if (p.relu) v = fmaxf(v, 0.f);
        *c = v;
      } else {
        __nv_bfloat16* c = (__nv_bfloat16*)p.C + m * p.ldc + n;
        if (p.beta != 0.f) v += p.beta * __bfloat162float(*c);
        if (p.relu) v = fmaxf(v, 0.f);
        *c = __float2bfloat16(v);
      }
    }
  }
}

__global__ void scale_matrix_kernel(float* c, long long M, long long N, long long ldc, float beta) {
  const long long total = M * N;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    float* e = c + (i / N) * ldc + (i % N);
    *e = beta == 0.f ? 0.f : beta * *e;
  }
}

}  // namespace

extern "C" {

int geeps_gemm_bf16_simt(const GeepsGemmParams* p, void* stream) {
  if (p->M <= 0 || p->N <= 0 || p->K <= 0) return (int)cudaErrorInvalidValue;
  dim3 grid((unsigned)((p->M + 63) / 64), (unsigned)((p->N + 63) / 64));
  gemm_simt_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(*p);
  return (int)cudaGetLastError();
}

int geeps_scale_matrix_f32(float* c, long long M, long long N, long long ldc, float beta, void* stream) {
  long long total = M * N;
  if (total <= 0) return 0;
  long long blocks = (total + 255) / 256;
  if (blocks > geeps_sm_count() * 8) blocks = geeps_sm_count() * 8;
  scale_matrix_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(c, M, N, ldc, beta);
  return (int)cudaGetLastError();
}

}  // extern "C"
