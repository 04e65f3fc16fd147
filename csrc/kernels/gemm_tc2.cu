// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): two SMs of a 2-CTA cluster compute one 256 x BN tile.
//
//   C[M,N] = alpha * A[M,K] * B[N,K]^T + bias, optional ReLU, bf16 or fp32 out   (A, B K-major)
//
// The single-CTA kernel in gemm_tc.cu is bound by operand traffic from L2 into shared memory: a 128 x 256
// tile needs 48 KB per 64-deep k-step.  Here each CTA of the pair loads its own 128 rows of A and only its
// own half of B's rows (32 KB per k-step per SM for the same FLOPs); the leader CTA issues one
// tcgen05.mma.cta_group::2 that reads both halves and writes each CTA's 128 accumulator rows into that CTA's
// own TMEM.  No load is multicast: each CTA fetches its own tiles with plain tiled TMA loads whose completion
// bytes are counted on the leader's mbarrier.
//
// Roles per CTA (192 threads): warp 0 TMA producer, warp 1 TMEM owner (+ MMA issuer in the leader),
// warps 2-5 epilogue.  Stage release (tcgen05.commit with cluster multicast) and accumulator hand-over reach
// both CTAs; the epilogue warps of both CTAs report to the leader when they drained an accumulator.
// Every mbarrier wait is bounded; the two cluster barriers (after setup, before TMEM release) are reached by
// every thread on every path.
//
// The reference has no GEMM kernel of its own (cuBLAS wrappers only,
// src/common/gpu-util/math_functions_cuda.cu:14-60).
#include <cuda.h>
#include <mutex>
#include <stdio.h>

#include "kernels.h"
#include "tc05.cuh"

namespace {

constexpr int BM = 128;             // rows per CTA; a pair covers 256
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int MAX_STAGES = 10;
constexpr uint64_t WAIT_BUDGET_NS = 2000000000ull;
constexpr int C_SLAB_BYTES = BM * 128;

struct PairDev {
  const float* bias; int* status;
  long long M, N, K;
  float alpha;
  int out_fp32, bias_mode, relu, kt_total, stages;
  int bn, tmem_cols, m_tiles, n_tiles;   // m_tiles counts 256-row tiles
};

struct SmemCtl {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const PairDev d) {
  extern __shared__ uint8_t smem_raw[];
  const int BN = d.bn;
  const int B_STAGE_BYTES = (BN / 2) * BK * 2;         // this CTA's half of the B tile
  const int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* cslab = tiles + (size_t)d.stages * STAGE_BYTES;
  SmemCtl* ctl = (SmemCtl*)(cslab + 2 * C_SLAB_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = tc05::cluster_ctarank();
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int S = d.stages;
  const int num_tiles = d.m_tiles * d.n_tiles;
  const int acc_stride = d.tmem_cols >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { tc05::mbar_init(&ctl->full[s], 1); tc05::mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { tc05::mbar_init(&ctl->tmem_full[a], 1); tc05::mbar_init(&ctl->tmem_empty[a], 8); }
    ctl->abort_flag = 0;
    tc05::mbar_fence_init();
  }
  if (warp == 1) {
    tc05::tmem_alloc_pair(&ctl->tmem_base, (uint32_t)d.tmem_cols);
    tc05::tmem_relinquish_pair();
  }
  tc05::fence_before_sync();
  __syncthreads();
  tc05::cluster_sync();            // the peer's barriers are initialised before anything signals them
  tc05::fence_after_sync();
  const uint32_t tmem = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs): own A rows, own half of B ----------------
    if (lane == 0) {
      tc05::tma_prefetch_desc(&tmA);
      tc05::tma_prefetch_desc(&tmB);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += npairs) {
        const int mi = t % d.m_tiles, ni = t / d.m_tiles;
        const int m0 = mi * (2 * BM) + (int)rank * BM;
        const int n0 = ni * BN + (int)rank * (BN / 2);
        for (int kt = 0; kt < d.kt_total; ++kt) {
          if (!tc05::mbar_wait(&ctl->empty[s], ph ^ 1u, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
          uint8_t* sa = tiles + (size_t)s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          // the leader's barrier counts the bytes of both CTAs
          if (rank == 0) tc05::mbar_expect_tx(&ctl->full[s], 2u * (uint32_t)STAGE_BYTES);
          const uint32_t bar = tc05::map_to_cta(tc05::smem_u32(&ctl->full[s]), 0);
          tc05::tma_load_2d_pair(sa, &tmA, bar, kt * BK, m0);
          tc05::tma_load_2d_pair(sb, &tmB, bar, kt * BK, n0);
          if (++s == S) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader only) ----------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = tc05::make_idesc_bf16(2 * BM, BN, 0, 0);
      uint32_t tile_i = 0, ph = 0;
      int s = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += npairs, ++tile_i) {
        const uint32_t acc = tile_i & 1u, acc_ph = (tile_i >> 1) & 1u;
        if (!tc05::mbar_wait(&ctl->tmem_empty[acc], acc_ph ^ 1u, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
        tc05::fence_after_sync();
        const uint32_t tacc = tmem + acc * (uint32_t)acc_stride;
        for (int kt = 0; kt < d.kt_total; ++kt) {
          if (!tc05::mbar_wait(&ctl->full[s], ph, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
          tc05::fence_after_sync();
          const uint32_t sa = tc05::smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = tc05::make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = tc05::make_smem_desc(sb + k * 32, 16, 1024);
            tc05::mma_bf16_ss_pair(tacc, da, db, idesc, (kt > 0 || k > 0) ? 1u : 0u);
          }
          tc05::mma_commit_pair(&ctl->empty[s], 3);      // frees the stage in both CTAs
          if (++s == S) { s = 0; ph ^= 1u; }
        }
        if (ok) tc05::mma_commit_pair(&ctl->tmem_full[acc], 3);
      }
    }
  } else {
    // ---------------- epilogue (both CTAs): own 128 rows ----------------
    const int q = warp & 3;
    uint32_t tile_i = 0, slab_i = 0;
    const int cols_per_slab = d.out_fp32 ? 32 : 64;
    const bool issuer = threadIdx.x == 64;
    const int rloc = q * 32 + lane;
    const uint32_t row_off = (uint32_t)rloc * 128u, rsw = (uint32_t)(rloc & 7);
    const bool relu = d.relu != 0;
    const int n_lim = (int)d.N;
    for (int t = pair; t < num_tiles; t += npairs, ++tile_i) {
      const int mi = t % d.m_tiles, ni = t / d.m_tiles;
      const int m0 = mi * (2 * BM) + (int)rank * BM, n0 = ni * BN;
      const uint32_t acc = tile_i & 1u, acc_ph = (tile_i >> 1) & 1u;
      if (!tc05::mbar_wait(&ctl->tmem_full[acc], acc_ph, abort_flag, WAIT_BUDGET_NS)) break;
      tc05::fence_after_sync();
      const uint32_t tacc = tmem + acc * (uint32_t)acc_stride + ((uint32_t)(q * 32) << 16);
      const long long row = (long long)m0 + rloc;
      const float bias_row = (d.bias_mode == 2 && row < d.M) ? d.bias[row] : 0.f;
#pragma unroll 1
      for (int c = 0; c < BN; c += cols_per_slab) {
        if (n0 + c >= n_lim) break;
        uint8_t* slab = cslab + (size_t)(slab_i & 1u) * C_SLAB_BYTES;
        if (issuer) tc05::bulk_wait_read<1>();
        tc05::named_bar_sync(1, 128);
        for (int h = 0; h < cols_per_slab; h += 32) {
          uint32_t r[32];
          tc05::tmem_ld_32x32(tacc + (uint32_t)(c + h), r);
          tc05::tmem_ld_wait();
          const int col0 = n0 + c + h;
          float v[32];
          if (d.bias_mode == 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = fmaf(d.alpha, __uint_as_float(r[j]), col0 + j < n_lim ? __ldg(d.bias + col0 + j) : 0.f);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaf(d.alpha, __uint_as_float(r[j]), bias_row);
          }
          if (relu) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
          }
          if (d.out_fp32) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t off = row_off + (uint32_t)((j ^ rsw) << 4);
              *reinterpret_cast<float4*>(slab + off) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            }
          } else {
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
          tc05::tma_store_2d(&tmC, slab, n0 + c, m0);
          tc05::bulk_commit();
        }
        ++slab_i;
      }
      // this warp has drained the accumulator: tell the leader's MMA thread (8 warps report per tile)
      tc05::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive_cluster(tc05::map_to_cta(tc05::smem_u32(&ctl->tmem_empty[acc]), 0));
    }
  }

  if (threadIdx.x == 64) tc05::bulk_wait<0>();
  tc05::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && ctl->abort_flag)
    geeps_report(d.status, GEEPS_ERR_TIMEOUT, KID_GEMM_TC, (int)blockIdx.x, 1);
  // neither CTA may release TMEM or exit while the peer can still signal its barriers or use the pair's TMEM
  tc05::cluster_sync();
  if (warp == 1) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc_pair(tmem, (uint32_t)d.tmem_cols);
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

bool make_map(CUtensorMap* map, const void* base, long long inner, long long outer, long long ld, int box_inner,
              int box_outer, bool fp32 = false) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * (fp32 ? 4 : 2)};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
            dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" {

int geeps_gemm_pair_supported(const GeepsGemmParams* p) {
  if (!geeps_gemm_tc_supported(p)) return 0;
  if (p->a_mn_major || p->b_mn_major || p->split_k > 1 || p->beta != 0.f) return 0;
  const int esz = p->out_fp32 ? 4 : 2;
  if (((uintptr_t)p->C & 15) || (p->ldc * esz) % 16) return 0;
  if (p->M < 256 || p->N < 64) return 0;
  return 1;
}

int geeps_gemm_bf16_pair(const GeepsGemmParams* p, void* stream) {
  if (!geeps_gemm_pair_supported(p)) return (int)cudaErrorInvalidValue;
  const int kPairs = 74;
  int bn = p->block_n;
  if (bn <= 0 || bn > 256 || bn % 64) {
    const long long nt = (p->N + 255) / 256;
    bn = (int)(((p->N + nt - 1) / nt + 63) / 64 * 64);
  }
  PairDev d;
  d.bias = p->bias; d.status = p->status;
  d.M = p->M; d.N = p->N; d.K = p->K;
  d.alpha = p->alpha;
  d.out_fp32 = p->out_fp32; d.bias_mode = p->bias ? p->bias_mode : 0; d.relu = p->relu;
  d.kt_total = (int)((p->K + BK - 1) / BK);
  d.bn = bn;
  d.m_tiles = (int)((p->M + 2 * BM - 1) / (2 * BM));
  d.n_tiles = (int)((p->N + bn - 1) / bn);
  int tmem_cols = 32;
  while (tmem_cols < 2 * bn) tmem_cols <<= 1;
  d.tmem_cols = tmem_cols;
  const int stage_bytes = A_STAGE_BYTES + (bn / 2) * BK * 2;
  d.stages = (200 * 1024 - 2 * C_SLAB_BYTES) / stage_bytes;
  if (d.stages > MAX_STAGES) d.stages = MAX_STAGES;
  if (d.stages < 2) d.stages = 2;
  CUtensorMap ta, tb, tc;
  if (!make_map(&ta, p->A, p->K, p->M, p->lda, BK, BM) || !make_map(&tb, p->B, p->K, p->N, p->ldb, BK, bn / 2) ||
      !make_map(&tc, p->C, p->N, p->M, p->ldc, p->out_fp32 ? 32 : 64, BM, p->out_fp32 != 0))
    return (int)cudaErrorInvalidValue;
  const long long num_tiles = (long long)d.m_tiles * d.n_tiles;
  const int pairs = (int)(num_tiles < kPairs ? num_tiles : kPairs);
  const size_t smem = (size_t)d.stages * stage_bytes + 2 * C_SLAB_BYTES + sizeof(SmemCtl) + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  gemm_pair_kernel<<<2 * pairs, 192, smem, (cudaStream_t)stream>>>(ta, tb, tc, d);
  return (int)cudaGetLastError();
}

}  // extern "C"
