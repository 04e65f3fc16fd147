// bf16 GEMM on the 5th-generation tensor cores: TMA -> swizzled SMEM ring ->
// tcgen05.mma (one issuing thread) -> fp32 accumulators in TMEM -> tcgen05.ld epilogue.
//
//   C[M,N] = alpha * A[M,K] * B[N,K]^T + beta * C + bias, optional ReLU, bf16 or fp32 out.
//
// Both operands may be K-major (row-major [rows][K]) or MN-major (stored [K][rows]), so
// forward (X W^T), data-gradient (dY W) and weight-gradient (dY^T X) products of FC and
// im2col-conv layers all run here without materialising a transpose.
//
// CTA = 6 warps: warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-5 epilogue
// (one TMEM lane quarter each).  Tile 128 x BN x 64, BN in {64,128,256}; partial tiles are
// handled by TMA zero fill on loads and bounds checks on stores, so any M, N, K work as
// long as the leading dimensions are multiples of 8 elements (16 bytes).
// Every mbarrier wait is bounded; on expiry the CTA records TIMEOUT in `status`, stops
// issuing work, frees its TMEM and returns.
//
// The reference has no GEMM kernel of its own: it only carries cuBLAS wrappers
// (src/common/gpu-util/math_functions_cuda.cu:14-60) that the parameter server never calls.
#include <cuda.h>
#include <mutex>
#include <stdio.h>

#include "kernels.h"
#include "tc05.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;              // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KB
constexpr int MAX_STAGES = 8;
constexpr uint64_t WAIT_BUDGET_NS = 2000000000ull;  // 2 s

struct GemmDev {
  void* C; const float* bias; int* status;
  long long M, N, K, ldc;
  float alpha, beta;
  int out_fp32, bias_mode, relu, split_k, kt_total, stages;
};

struct SmemCtl {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full;
  uint32_t tmem_base;
  int abort_flag;
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const GemmDev d) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int B_STAGE_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  SmemCtl* ctl = (SmemCtl*)(tiles + (size_t)d.stages * STAGE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM;
  const int n0 = blockIdx.y * BN;
  // split-K: this CTA covers k-tiles [kt_begin, kt_end)
  const int kt_per = (d.kt_total + d.split_k - 1) / d.split_k;
  const int kt_begin = blockIdx.z * kt_per;
  const int kt_end = min(d.kt_total, kt_begin + kt_per);
  const int nkt = kt_end - kt_begin;
  const int S = d.stages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { tc05::mbar_init(&ctl->full[s], 1); tc05::mbar_init(&ctl->empty[s], 1); }
    tc05::mbar_init(&ctl->tmem_full, 1);
    ctl->abort_flag = 0;
    tc05::mbar_fence_init();
  }
  if (warp == 1) {
    tc05::tmem_alloc(&ctl->tmem_base, BN);
    tc05::tmem_relinquish();
  }
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;

  if (nkt > 0) {
    if (warp == 0) {
      // ---------------- TMA producer ----------------
      if (lane == 0) {
        tc05::tma_prefetch_desc(&tmA);
        tc05::tma_prefetch_desc(&tmB);
        for (int i = 0; i < nkt; ++i) {
          const int s = i % S;
          const uint32_t ph = (uint32_t)(i / S) & 1u;
          if (!tc05::mbar_wait(&ctl->empty[s], ph ^ 1u, abort_flag, WAIT_BUDGET_NS)) break;
          uint8_t* sa = tiles + (size_t)s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          const int k0 = (kt_begin + i) * BK;
          tc05::mbar_expect_tx(&ctl->full[s], STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int h = 0; h < BM / 64; ++h)
              tc05::tma_load_2d(sa + h * (64 * BK * 2), &tmA, &ctl->full[s], m0 + 64 * h, k0);
          } else {
            tc05::tma_load_2d(sa, &tmA, &ctl->full[s], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int h = 0; h < BN / 64; ++h)
              tc05::tma_load_2d(sb + h * (64 * BK * 2), &tmB, &ctl->full[s], n0 + 64 * h, k0);
          } else {
            tc05::tma_load_2d(sb, &tmB, &ctl->full[s], k0, n0);
          }
        }
      }
    } else if (warp == 1) {
      // ---------------- MMA issuer ----------------
      if (lane == 0) {
        constexpr uint32_t idesc = tc05::make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
        bool ok = true;
        for (int i = 0; i < nkt && ok; ++i) {
          const int s = i % S;
          const uint32_t ph = (uint32_t)(i / S) & 1u;
          if (!tc05::mbar_wait(&ctl->full[s], ph, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
          tc05::fence_after_sync();
          const uint32_t sa = tc05::smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: 16 k-elements = 32 bytes inside the 128-byte swizzle row.
            // MN-major: 16 k-rows of 128 bytes = two 8-row groups of 1024 bytes.
            const uint64_t da = A_MN ? tc05::make_smem_desc(sa + k * 2048, 64 * BK * 2, 1024)
                                     : tc05::make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? tc05::make_smem_desc(sb + k * 2048, 64 * BK * 2, 1024)
                                     : tc05::make_smem_desc(sb + k * 32, 16, 1024);
            tc05::mma_bf16_ss(tmem, da, db, idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
          tc05::mma_commit(&ctl->empty[s]);  // frees the stage when these MMAs have read it
        }
        if (ok) tc05::mma_commit(&ctl->tmem_full);
      }
    } else {
      // ---------------- epilogue: TMEM -> registers -> global ----------------
      const int q = warp & 3;  // TMEM lane quarter this warp may access
      const bool ok = tc05::mbar_wait(&ctl->tmem_full, 0, abort_flag, WAIT_BUDGET_NS);
      tc05::fence_after_sync();
      if (ok) {
        const long long row = (long long)m0 + q * 32 + lane;
        const float bias_m = (d.bias_mode == 2 && row < d.M) ? d.bias[row] : 0.f;
        const bool add_bias = (d.split_k == 1) || (blockIdx.z == 0);
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tc05::tmem_ld_32x32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)c, r);
          tc05::tmem_ld_wait();
          const long long col0 = (long long)n0 + c;
          if (row < d.M && col0 < d.N) {
            const int ncols = (int)min((long long)32, d.N - col0);
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float x = d.alpha * __uint_as_float(r[j]);
              if (add_bias) {
                if (d.bias_mode == 1 && j < ncols) x += d.bias[col0 + j];
                else if (d.bias_mode == 2) x += bias_m;
              }
              v[j] = x;
            }
            if (d.split_k > 1) {
              float* out = (float*)d.C + row * d.ldc + col0;
              for (int j = 0; j < ncols; ++j) atomicAdd(out + j, v[j]);
            } else if (d.out_fp32) {
              float* out = (float*)d.C + row * d.ldc + col0;
              const bool vec = (ncols == 32) && ((((uintptr_t)out) & 15) == 0);
              if (vec) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                  if (d.beta != 0.f) {
                    float4 old = ld_f4(out + j);
                    o.x += d.beta * old.x; o.y += d.beta * old.y; o.z += d.beta * old.z; o.w += d.beta * old.w;
                  }
                  if (d.relu) { o.x = fmaxf(o.x, 0.f); o.y = fmaxf(o.y, 0.f); o.z = fmaxf(o.z, 0.f); o.w = fmaxf(o.w, 0.f); }
                  st_f4(out + j, o);
                }
              } else {
                for (int j = 0; j < ncols; ++j) {
                  float o = v[j];
                  if (d.beta != 0.f) o += d.beta * out[j];
                  if (d.relu) o = fmaxf(o, 0.f);
                  out[j] = o;
                }
              }
            } else {
              __nv_bfloat16* out = (__nv_bfloat16*)d.C + row * d.ldc + col0;
              const bool vec = (ncols == 32) && ((((uintptr_t)out) & 15) == 0);
              if (vec) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  float o[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e) o[e] = v[j + e];
                  if (d.beta != 0.f) {
                    uint4 oldv = *reinterpret_cast<const uint4*>(out + j);
                    const __nv_bfloat16* ob = reinterpret_cast<const __nv_bfloat16*>(&oldv);
#pragma unroll
                    for (int e = 0; e < 8; ++e) o[e] += d.beta * __bfloat162float(ob[e]);
                  }
                  if (d.relu) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) o[e] = fmaxf(o[e], 0.f);
                  }
                  uint4 pk = make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]),
                                        pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
                  *reinterpret_cast<uint4*>(out + j) = pk;
                }
              } else {
                for (int j = 0; j < ncols; ++j) {
                  float o = v[j];
                  if (d.beta != 0.f) o += d.beta * __bfloat162float(out[j]);
                  if (d.relu) o = fmaxf(o, 0.f);
                  out[j] = __float2bfloat16(o);
                }
              }
            }
          }
        }
      }
    }
  }

  tc05::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && ctl->abort_flag)
    geeps_report(d.status, GEEPS_ERR_TIMEOUT, KID_GEMM_TC, (int)(blockIdx.y * gridDim.x + blockIdx.x), 0);
  if (warp == 1) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc(tmem, BN);
  }
}

// ---------------- host side ----------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
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

// 2-D bf16 tensor map: `inner` contiguous elements per line, `outer` lines of `ld` elements.
bool make_map(CUtensorMap* map, const void* base, long long inner, long long outer, long long ld,
              int box_inner, int box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int BN, bool A_MN, bool B_MN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmDev& d, dim3 grid, cudaStream_t st) {
  const int stage_bytes = A_STAGE_BYTES + BN * BK * 2;
  const size_t smem = (size_t)d.stages * stage_bytes + sizeof(SmemCtl) + 1024;
  static bool attr_set = false;  // per instantiation
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, A_MN, B_MN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  gemm_tc_kernel<BN, A_MN, B_MN><<<grid, 192, smem, st>>>(ta, tb, d);
  return (int)cudaGetLastError();
}

template <int BN>
int launch_bn(int a_mn, int b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmDev& d, dim3 grid,
              cudaStream_t st) {
  if (!a_mn && !b_mn) return launch<BN, false, false>(ta, tb, d, grid, st);
  if (a_mn && !b_mn) return launch<BN, true, false>(ta, tb, d, grid, st);
  if (!a_mn && b_mn) return launch<BN, false, true>(ta, tb, d, grid, st);
  return launch<BN, true, true>(ta, tb, d, grid, st);
}

}  // namespace

extern "C" {

int geeps_gemm_tc_supported(const GeepsGemmParams* p) {
  if (p->M <= 0 || p->N <= 0 || p->K <= 0) return 0;
  if (((uintptr_t)p->A & 15) || ((uintptr_t)p->B & 15)) return 0;
  if ((p->lda & 7) || (p->ldb & 7)) return 0;
  if (p->split_k > 1 && (!p->out_fp32 || p->relu)) return 0;
  if (p->M > 0x7fffffffLL || p->N > 0x7fffffffLL || p->K > 0x7fffffffLL) return 0;
  return 1;
}

int geeps_gemm_bf16(const GeepsGemmParams* p, void* stream) {
  if (!geeps_gemm_tc_supported(p)) return (int)cudaErrorInvalidValue;
  const int m_tiles = (int)((p->M + BM - 1) / BM);
  int bn = p->block_n;
  if (bn != 64 && bn != 128 && bn != 256) {
    if (p->N <= 64) bn = 64;
    else if ((long long)m_tiles * ((p->N + 255) / 256) >= 2 * 148) bn = 256;
    else if ((long long)m_tiles * ((p->N + 127) / 128) >= 148 || p->N <= 128) bn = 128;
    else bn = 64;
  }
  CUtensorMap ta, tb;
  bool ok = p->a_mn_major ? make_map(&ta, p->A, p->M, p->K, p->lda, 64, BK)
                          : make_map(&ta, p->A, p->K, p->M, p->lda, BK, BM);
  ok = ok && (p->b_mn_major ? make_map(&tb, p->B, p->N, p->K, p->ldb, 64, BK)
                            : make_map(&tb, p->B, p->K, p->N, p->ldb, BK, bn));
  if (!ok) return (int)cudaErrorInvalidValue;
  GemmDev d;
  d.C = p->C; d.bias = p->bias; d.status = p->status;
  d.M = p->M; d.N = p->N; d.K = p->K; d.ldc = p->ldc;
  d.alpha = p->alpha; d.beta = p->beta;
  d.out_fp32 = p->out_fp32; d.bias_mode = p->bias ? p->bias_mode : 0; d.relu = p->relu;
  d.kt_total = (int)((p->K + BK - 1) / BK);
  const long long n_tiles = (p->N + bn - 1) / bn;
  int split = p->split_k;
  if (split == 0) {  // auto: fill the 148 SMs twice over when the output has few tiles
    split = 1;
    const long long tiles = (long long)m_tiles * n_tiles;
    if (p->out_fp32 && !p->relu && tiles < 148 && d.kt_total >= 8) {
      long long want = (2 * 148 + tiles - 1) / tiles;
      long long cap = d.kt_total / 4;
      split = (int)(want < cap ? want : cap);
      if (split < 1) split = 1;
    }
  }
  d.split_k = split < 1 ? 1 : (split > d.kt_total ? d.kt_total : split);
  if (d.split_k > 1) {
    // partial sums are accumulated with atomics: bring C to beta*C (or zero) first
    int e = geeps_scale_matrix_f32((float*)p->C, p->M, p->N, p->ldc, p->beta, stream);
    if (e) return e;
    d.beta = 0.f;
  }
  // two CTAs per SM for BN <= 128 (epilogue of one overlaps the main loop of the other)
  d.stages = bn == 256 ? 4 : (bn == 128 ? 3 : 4);
  if (d.stages > d.kt_total + 1) d.stages = d.kt_total + 1 > 2 ? d.kt_total + 1 : 2;
  dim3 grid((unsigned)m_tiles, (unsigned)((p->N + bn - 1) / bn), (unsigned)d.split_k);
  cudaStream_t st = (cudaStream_t)stream;
  if (bn == 64) return launch_bn<64>(p->a_mn_major, p->b_mn_major, ta, tb, d, grid, st);
  if (bn == 128) return launch_bn<128>(p->a_mn_major, p->b_mn_major, ta, tb, d, grid, st);
  return launch_bn<256>(p->a_mn_major, p->b_mn_major, ta, tb, d, grid, st);
}

}  // extern "C"
