// bf16 GEMM on the 5th-generation tensor cores: TMA -> swizzled SMEM ring ->
// tcgen05.mma (one issuing thread) -> fp32 accumulators in TMEM -> tcgen05.ld epilogue.
//
//   C[M,N] = alpha * A[M,K] * B[N,K]^T + beta * C + bias, optional ReLU, bf16 or fp32 out.
//
// Both operands may be K-major (row-major [rows][K]) or MN-major (stored [K][rows]), so
// forward (X W^T), data-gradient (dY W) and weight-gradient (dY^T X) products of FC and
// im2col-conv layers all run here without materialising a transpose.
//
// Persistent CTAs (one per SM) of 6 warps: warp 0 TMA producer, warp 1 MMA issuer + TMEM owner,
// warps 2-5 epilogue (one TMEM lane quarter each).  Two accumulators live in TMEM, so the epilogue
// of a tile overlaps the main loop of the next one.  Tile 128 x BN x 64 with BN any multiple of 32
// up to 256 (chosen per problem so that narrow outputs do not pad the MMA); partial tiles are
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
constexpr int C_SLAB_BYTES = BM * 128;       // epilogue staging slab: 128 rows x 128 bytes, two of them

struct GemmDev {
  void* C; const float* bias; int* status;
  long long M, N, K, ldc;
  float alpha, beta;
  int out_fp32, bias_mode, relu, split_k, kt_total, stages;
  int bn;           // tile width: multiple of 32 (64 for an MN-major B), <= 256
  int tmem_cols;    // power of two >= 2 * bn: two accumulators, so the epilogue of a tile overlaps the next main loop
  int m_tiles, n_tiles;
  int tma_store;    // 1: epilogue stages 128-byte-wide slabs in swizzled smem and stores them with TMA
};

struct SmemCtl {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Persistent kernel: one CTA per SM walks the tile list t = blockIdx.x, blockIdx.x + gridDim.x, ...
// Consecutive CTAs take consecutive M tiles of the same N tile, so the B tile they share stays in L2.
template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const GemmDev d) {
  extern __shared__ uint8_t smem_raw[];
  const int BN = d.bn;
  const int B_STAGE_BYTES = BN * BK * 2;
  const int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* cslab = tiles + (size_t)d.stages * STAGE_BYTES;          // 2 x C_SLAB_BYTES, 1024-byte aligned
  SmemCtl* ctl = (SmemCtl*)(cslab + 2 * C_SLAB_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = d.stages;
  const int kt_per = (d.kt_total + d.split_k - 1) / d.split_k;
  const int tiles_mn = d.m_tiles * d.n_tiles;
  const int num_tiles = tiles_mn * d.split_k;
  const int acc_stride = d.tmem_cols >> 1;

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
      // ring slot and phase advance incrementally: a division per k-tile in this single thread would cost
      // more than issuing the loads
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int mn = t % tiles_mn, z = t / tiles_mn;
        const int m0 = (mn % d.m_tiles) * BM, n0 = (mn / d.m_tiles) * BN;
        const int kt_begin = z * kt_per, kt_end = min(d.kt_total, kt_begin + kt_per);
        for (int kt = kt_begin; kt < kt_end; ++kt) {
          if (!tc05::mbar_wait_warp(&ctl->empty[s], ph ^ 1u, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
          uint8_t* sa = tiles + (size_t)s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          const int k0 = kt * BK;
          if (leader) {
          tc05::mbar_expect_tx(&ctl->full[s], STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int h = 0; h < BM / 64; ++h)
              tc05::tma_load_2d(sa + h * (64 * BK * 2), &tmA, &ctl->full[s], m0 + 64 * h, k0);
          } else {
            tc05::tma_load_2d(sa, &tmA, &ctl->full[s], k0, m0);
          }
          if (B_MN) {
            for (int h = 0; h < BN / 64; ++h)
              tc05::tma_load_2d(sb + h * (64 * BK * 2), &tmB, &ctl->full[s], n0 + 64 * h, k0);
          } else {
            tc05::tma_load_2d(sb, &tmB, &ctl->full[s], k0, n0);
          }
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
        // the epilogue must have drained this accumulator (two tiles ago)
        if (!tc05::mbar_wait_warp(&ctl->tmem_empty[acc], acc_ph ^ 1u, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
        tc05::fence_after_sync();
        const uint32_t tacc = tmem + acc * (uint32_t)acc_stride;
        for (int kt = kt_begin; kt < kt_end; ++kt) {
          if (!tc05::mbar_wait_warp(&ctl->full[s], ph, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
          tc05::fence_after_sync();
          const uint32_t sa = tc05::smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
          if (leader) {
          // descriptors as 32-bit halves: per MMA this one thread spends an add per operand, not a rebuild.
          // K-major: 16 k-elements = 32 bytes inside the 128-byte swizzle row (2 units of 16 bytes);
          // MN-major: 16 k-rows of 128 bytes = two 8-row groups of 1024 bytes (128 units).
          const uint32_t a_lo = tc05::desc_lo(sa, A_MN ? 64 * BK * 2 : 16), b_lo = tc05::desc_lo(sb, B_MN ? 64 * BK * 2 : 16);
          constexpr uint32_t d_hi = tc05::desc_hi(1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc05::mma_bf16_ss_lohi(tacc, a_lo + (A_MN ? 128 : 2) * k, d_hi, b_lo + (B_MN ? 128 : 2) * k, d_hi, idesc,
                                   (kt > kt_begin || k > 0) ? 1u : 0u);
          tc05::mma_commit(&ctl->empty[s]);  // frees the stage when these MMAs have read it
          }
          if (++s == S) { s = 0; ph ^= 1u; }
        }
        if (ok && leader) tc05::mma_commit(&ctl->tmem_full[acc]);
      }
    }
  } else {
    // ---------------- epilogue: TMEM -> registers -> global ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint32_t tile_i = 0, slab_i = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++tile_i) {
      const int mn = t % tiles_mn, z = t / tiles_mn;
      const int m0 = (mn % d.m_tiles) * BM, n0 = (mn / d.m_tiles) * BN;
      const int kt_begin = z * kt_per, kt_end = min(d.kt_total, kt_begin + kt_per);
      const uint32_t acc = tile_i & 1u, acc_ph = (tile_i >> 1) & 1u;
      if (!tc05::mbar_wait(&ctl->tmem_full[acc], acc_ph, abort_flag, WAIT_BUDGET_NS)) break;
      tc05::fence_after_sync();
      const uint32_t tacc = tmem + acc * (uint32_t)acc_stride + ((uint32_t)(q * 32) << 16);
      const long long row = (long long)m0 + q * 32 + lane;
      const float bias_m = (d.bias_mode == 2 && row < d.M) ? d.bias[row] : 0.f;
      const bool add_bias = (d.split_k == 1) || (z == 0);
      const bool has_k = kt_end > kt_begin;
      if (d.tma_store) {
        // 128-byte-wide slabs (64 bf16 or 32 fp32 columns) go through swizzled smem and leave with one
        // TMA store (or reduce-add for split-K) each: coalesced, asynchronous, clipped at the matrix edge
        const int cols_per_slab = d.out_fp32 ? 32 : 64;
        const bool issuer = threadIdx.x == 64;
        const int rloc = q * 32 + lane;          // row inside the tile = TMEM lane
        const uint32_t row_off = (uint32_t)rloc * 128u, rsw = (uint32_t)(rloc & 7);
        // everything that does not depend on the column is hoisted out of the slab loop
        const int bmode = add_bias ? d.bias_mode : 0;
        const float alpha = has_k ? d.alpha : 0.f;
        const float bias_row = bmode == 2 ? bias_m : 0.f;
        const bool relu = d.relu != 0;
        const int n_lim = (int)d.N;
#pragma unroll 1
        for (int c = 0; c < BN; c += cols_per_slab) {
          if ((long long)n0 + c >= d.N) break;
          uint8_t* slab = cslab + (size_t)(slab_i & 1u) * C_SLAB_BYTES;
          if (issuer) tc05::bulk_wait_read<1>();   // the slab stored two slabs ago has been read out
          tc05::named_bar_sync(1, 128);
          for (int h = 0; h < cols_per_slab; h += 32) {
            uint32_t r[32];
            tc05::tmem_ld_32x32(tacc + (uint32_t)(c + h), r);
            tc05::tmem_ld_wait();
            const int col0 = n0 + c + h;
            float v[32];
            if (bmode == 1) {
              // per-column bias: the same 32 values for every row of the slab (broadcast loads)
              if (col0 + 32 <= n_lim) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = fmaf(alpha, __uint_as_float(r[j]), __ldg(d.bias + col0 + j));
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  v[j] = fmaf(alpha, __uint_as_float(r[j]), col0 + j < n_lim ? __ldg(d.bias + col0 + j) : 0.f);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = fmaf(alpha, __uint_as_float(r[j]), bias_row);
            }
            if (relu) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
            }
            if (d.out_fp32) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {   // 8 chunks of 4 floats
                const uint32_t off = row_off + (uint32_t)((j ^ rsw) << 4);
                *reinterpret_cast<float4*>(slab + off) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {   // 4 chunks of 8 bf16 per 32 columns
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
            if (d.split_k > 1) tc05::tma_reduce_add_2d(&tmC, slab, n0 + c, m0);
            else tc05::tma_store_2d(&tmC, slab, n0 + c, m0);
            tc05::bulk_commit();
          }
          ++slab_i;
        }
      } else {
  #pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tc05::tmem_ld_32x32(tacc + (uint32_t)c, r);
          tc05::tmem_ld_wait();
          const long long col0 = (long long)n0 + c;
          if (row < d.M && col0 < d.N && has_k) {
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
      // this warp is done reading the accumulator: hand it back to the MMA warp
      tc05::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive(&ctl->tmem_empty[acc]);
    }
  }

  if (d.tma_store && threadIdx.x == 64) tc05::bulk_wait<0>();   // all TMA stores of this CTA have landed
  tc05::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && ctl->abort_flag)
    geeps_report(d.status, GEEPS_ERR_TIMEOUT, KID_GEMM_TC, (int)blockIdx.x, 0);
  if (warp == 1) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc(tmem, (uint32_t)d.tmem_cols);
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
              int box_inner, int box_outer, bool fp32 = false) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * (fp32 ? 4 : 2)};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <bool A_MN, bool B_MN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmDev& d, int grid,
           cudaStream_t st) {
  const int stage_bytes = A_STAGE_BYTES + d.bn * BK * 2;
  const size_t smem = (size_t)d.stages * stage_bytes + 2 * C_SLAB_BYTES + sizeof(SmemCtl) + 1024;
  static bool attr_set = false;  // per instantiation
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         220 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  gemm_tc_kernel<A_MN, B_MN><<<grid, 192, smem, st>>>(ta, tb, tc, d);
  return (int)cudaGetLastError();
}

int round_up(long long v, int m) { return (int)((v + m - 1) / m * m); }

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
  const int kSMs = geeps_sm_count();
  // large K-major products go to CTA pairs (half the B traffic per SM) when 256-row tiles can fill the machine
  if (p->block_n == 0 && p->split_k <= 1 && geeps_gemm_pair_supported(p) &&
      ((p->M + 255) / 256) * ((p->N + 255) / 256) >= kSMs / 2)
    return geeps_gemm_bf16_pair(p, stream);
  const int m_tiles = (int)((p->M + BM - 1) / BM);
  const int unit = p->b_mn_major ? 64 : 32;
  const int kt_total = (int)((p->K + BK - 1) / BK);
  // tile width: as few N tiles as possible with little padding ...
  // TMA-store epilogue: C 16-byte aligned with a 16-byte-multiple pitch, no read-modify-write of C
  const int esz = p->out_fp32 ? 4 : 2;
  const bool tma_c = (((uintptr_t)p->C & 15) == 0) && ((p->ldc * esz) % 16 == 0) && p->beta == 0.f;
  int bn = p->block_n;
  if (bn <= 0 || bn > 256 || bn % unit) {
    const long long nt = (p->N + 255) / 256;
    bn = round_up((p->N + nt - 1) / nt, unit);
    // ... but enough tiles to occupy every SM when the problem allows it
    const bool can_split = p->split_k == 0 && p->out_fp32 && !p->relu && kt_total >= 16;
    while (!can_split && bn > 64 && (long long)m_tiles * ((p->N + bn - 1) / bn) < kSMs) {
      const int smaller = round_up(bn / 2, unit);
      if (smaller >= bn) break;
      bn = smaller;
    }
  }
  if (bn > 256) bn = 256;
  // a bf16 slab is 64 columns wide: with several N tiles the tile width must be a multiple of it
  if (tma_c && !p->out_fp32 && (bn % 64) && (p->N + bn - 1) / bn > 1) bn = round_up(bn, 64);
  const long long n_tiles = (p->N + bn - 1) / bn;
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
  d.kt_total = kt_total;
  d.bn = bn;
  d.m_tiles = m_tiles;
  d.n_tiles = (int)n_tiles;
  int tmem_cols = 32;
  while (tmem_cols < 2 * bn) tmem_cols <<= 1;
  d.tmem_cols = tmem_cols;
  int split = p->split_k;
  if (split == 0) {  // auto: occupy the SMs about twice over when the output has few tiles
    split = 1;
    const long long tiles = (long long)m_tiles * n_tiles;
    if (p->out_fp32 && !p->relu && tiles < kSMs && d.kt_total >= 8) {
      long long want = (2 * kSMs) / tiles;   // at most two full waves: one work item more would add a third round
      long long cap = d.kt_total / 4;
      split = (int)(want < cap ? want : cap);
      if (split < 1) split = 1;
    }
  }
  d.split_k = split < 1 ? 1 : (split > d.kt_total ? d.kt_total : split);
  if (d.split_k > 1) {
    // every k-slice must be non-empty, otherwise its tile would never be completed by an MMA commit
    const int per = (d.kt_total + d.split_k - 1) / d.split_k;
    d.split_k = (d.kt_total + per - 1) / per;
  }
  if (d.split_k > 1) {
    // partial sums are accumulated with atomics: bring C to beta*C (or zero) first
    int e = geeps_scale_matrix_f32((float*)p->C, p->M, p->N, p->ldc, p->beta, stream);
    if (e) return e;
    d.beta = 0.f;
  }
  d.tma_store = tma_c ? 1 : 0;
  CUtensorMap tc;
  if (tma_c) {
    if (!make_map(&tc, p->C, p->N, p->M, p->ldc, p->out_fp32 ? 32 : 64, BM, p->out_fp32 != 0)) d.tma_store = 0;
  }
  if (!d.tma_store) tc = ta;   // unused by the kernel
  const int stage_bytes = A_STAGE_BYTES + bn * BK * 2;
  d.stages = (200 * 1024 - 2 * C_SLAB_BYTES) / stage_bytes;
  if (d.stages > MAX_STAGES) d.stages = MAX_STAGES;
  if (d.stages < 2) d.stages = 2;
  const long long num_tiles = (long long)m_tiles * n_tiles * d.split_k;
  const int grid = (int)(num_tiles < kSMs ? num_tiles : kSMs);
  cudaStream_t st = (cudaStream_t)stream;
  if (!p->a_mn_major && !p->b_mn_major) return launch<false, false>(ta, tb, tc, d, grid, st);
  if (p->a_mn_major && !p->b_mn_major) return launch<true, false>(ta, tb, tc, d, grid, st);
  if (!p->a_mn_major && p->b_mn_major) return launch<false, true>(ta, tb, tc, d, grid, st);
  return launch<true, true>(ta, tb, tc, d, grid, st);
}

}  // extern "C"
