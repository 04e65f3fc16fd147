// Parameter pull fused with the first GEMM that consumes the rows (all-gather -> GEMM in one kernel):
//
//   Y[M,N] = X[M,K] * W[N,K]^T + bias (+ReLU),   M <= 256 (one batch of an FC / classifier layer)
//
// W is NOT local: its rows are spread over the server shards (contiguous row ranges, bf16 compute copy
// of the fp32 master rows, written by the owning shard's apply kernel).  Each CTA owns one N tile; its
// four loader warps wait (bounded) for the owning shard's clock stamp, read the tile's weight rows
// straight out of the owner's HBM over NVLink with plain 16-byte system-scope loads, write them into the
// 128-byte-swizzled SMEM stage that tcgen05.mma reads, and - optionally - also store them into the local
// parameter cache so the backward pass finds them in local memory.  X tiles come from local memory by
// TMA (no multicast); both M tiles of a batch of 256 share the weight tile in SMEM, so every weight
// element crosses NVLink once per GPU.  Accumulators live in TMEM; the loader warps turn into the
// epilogue warps after the main loop.  No TMA and no multicast object ever touches peer memory.
//
// This is the device-side replacement of the reference's pull path - whole-shard broadcast by the server
// (src/server/tablet-server.cpp:147-163), pinned bounce + H2D install (src/client/clientlib-data.cpp:110-151)
// and the gather into the application's read buffer (src/common/row-op-util.cu:39-72) - for tables whose
// first consumer is a GEMM.  Every wait is bounded and reports TIMEOUT into `status`.
#include <cuda.h>
#include <mutex>

#include "kernels.h"
#include "tc05.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BM * BK * 2;
constexpr int MAX_A_STAGES = 8;
constexpr int MAX_B_STAGES = 24;
constexpr uint64_t WAIT_BUDGET_NS = 2000000000ull;

struct PullGemmDev {
  GeepsPullGemmParams p;
  int bn, stages_a, stages_b, m_tiles, tmem_cols, kt_total;
};

// X (local, TMA) and W (remote, SM loads) have rings of their own: X tiles are large and arrive fast,
// W tiles are small and arrive after an NVLink round trip, so the W ring is much deeper.
struct SmemCtl {
  uint64_t full_a[MAX_A_STAGES];
  uint64_t empty_a[MAX_A_STAGES];
  uint64_t full_b[MAX_B_STAGES];
  uint64_t empty_b[MAX_B_STAGES];
  uint64_t staged[MAX_B_STAGES];   // loaders -> committer: the W tile of the stage is in SMEM
  uint64_t tmem_full;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint4 ld_peer_16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(192, 1)
pull_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const PullGemmDev d) {
  extern __shared__ uint8_t smem_raw[];
  const GeepsPullGemmParams& p = d.p;
  const int BN = d.bn;
  const int A_STAGE = d.m_tiles * A_TILE_BYTES;
  const int B_STAGE = BN * BK * 2;
  uint8_t* tiles_a = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* tiles_b = tiles_a + (size_t)d.stages_a * A_STAGE;
  SmemCtl* ctl = (SmemCtl*)(tiles_b + (size_t)d.stages_b * B_STAGE);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int SA = d.stages_a, SB = d.stages_b;
  const int n0 = blockIdx.x * BN;
  const int KT = d.kt_total;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SA; ++s) { tc05::mbar_init(&ctl->full_a[s], 1); tc05::mbar_init(&ctl->empty_a[s], 1); }
    for (int s = 0; s < SB; ++s) {
      tc05::mbar_init(&ctl->full_b[s], 1);
      tc05::mbar_init(&ctl->empty_b[s], 1);
      tc05::mbar_init(&ctl->staged[s], 96);
    }
    tc05::mbar_init(&ctl->tmem_full, 1);
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
    // ---------------- X tiles: TMA from local memory ----------------
    if (lane == 0) {
      tc05::tma_prefetch_desc(&tmA);
      // ring slots and phases advance incrementally everywhere in this kernel: a division per k-tile in a
      // single-thread role costs more than the work it schedules
      int s = 0;
      uint32_t ph = 0;
      for (int kt = 0; kt < KT; ++kt) {
        if (!tc05::mbar_wait(&ctl->empty_a[s], ph ^ 1u, abort_flag, WAIT_BUDGET_NS)) break;
        uint8_t* sa = tiles_a + (size_t)s * A_STAGE;
        tc05::mbar_expect_tx(&ctl->full_a[s], (uint32_t)A_STAGE);
        for (int mt = 0; mt < d.m_tiles; ++mt)
          tc05::tma_load_2d(sa + mt * A_TILE_BYTES, &tmA, &ctl->full_a[s], kt * BK, mt * BM);
        if (++s == SA) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: both M tiles share the weight tile ----------------
    if (lane == 0) {
      const uint32_t idesc = tc05::make_idesc_bf16(BM, BN, 0, 0);
      bool ok = true;
      int s = 0, t = 0;
      uint32_t pha = 0, phb = 0;
      for (int kt = 0; kt < KT && ok; ++kt) {
        if (!tc05::mbar_wait(&ctl->full_a[s], pha, abort_flag, WAIT_BUDGET_NS) ||
            !tc05::mbar_wait(&ctl->full_b[t], phb, abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
        tc05::fence_after_sync();
        const uint32_t sa = tc05::smem_u32(tiles_a + (size_t)s * A_STAGE);
        const uint32_t sb = tc05::smem_u32(tiles_b + (size_t)t * B_STAGE);
        for (int mt = 0; mt < d.m_tiles; ++mt) {
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = tc05::make_smem_desc(sa + mt * A_TILE_BYTES + k * 32, 16, 1024);
            const uint64_t db = tc05::make_smem_desc(sb + k * 32, 16, 1024);
            tc05::mma_bf16_ss(tmem + (uint32_t)(mt * BN), da, db, idesc, (kt > 0 || k > 0) ? 1u : 0u);
          }
        }
        tc05::mma_commit(&ctl->empty_a[s]);
        tc05::mma_commit(&ctl->empty_b[t]);
        if (++s == SA) { s = 0; pha ^= 1u; }
        if (++t == SB) { t = 0; phb ^= 1u; }
      }
      if (ok) tc05::mma_commit(&ctl->tmem_full);
    }
  } else {
    // ---------------- W tiles: peer memory -> swizzled SMEM (+ local cache) ----------------
    // Warps 2-4 (96 threads) copy with cp.async (16-byte SM-issued global->shared copies, no TMA): the
    // copies need no registers, so each thread keeps as many k-tiles in flight as the W ring is deep and
    // the NVLink round trip is hidden.  Warp 5 waits for a tile to land, mirrors it into the local cache,
    // crosses into the async proxy and publishes the stage to the MMA warp.
    if (warp < 5) {
      const int ltid = threadIdx.x - 64;           // 0..95
      constexpr int NS = 11;                       // (row, chunk) slots per thread: 128 rows x 8 chunks / 96
      const __nv_bfloat16* src_row[NS];
      uint32_t soff[NS];
      const int chunks = BN * 8;                   // 16-byte chunks per stage
      bool ok = true;
      int nslots = 0;
      for (int i = 0; i < NS; ++i) {
        const int idx = ltid + i * 96;
        src_row[i] = nullptr; soff[i] = 0;
        if (idx >= chunks) continue;
        nslots = i + 1;
        const int row = idx >> 3, chunk = idx & 7;
        soff[i] = (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
        const long long n = (long long)n0 + row;
        if (n >= p.N) continue;                    // rows past the matrix edge are filled with zeros
        int sh = 0;
        while (sh + 1 < p.n_shards && n >= p.n_start[sh + 1]) ++sh;
        // bounded wait for the owner's stamp (its apply kernel has written these rows)
        if (p.ready[sh] != nullptr) {
          int seen = 0;
          if (!geeps_wait_ge(p.ready[sh], p.needed_stamp, p.wait_budget_ns, &seen)) {
            geeps_report(p.status, GEEPS_ERR_TIMEOUT, KID_PULL_GEMM, sh, seen);
            ok = false;
          }
        }
        src_row[i] = (const __nv_bfloat16*)p.w_shard[sh] + (n - p.n_start[sh]) * p.ldw + chunk * 8;
      }
      if (!ok) ctl->abort_flag = 1;
      const __nv_bfloat16* any_valid = (const __nv_bfloat16*)p.X;   // address for zero-size (zero-fill) copies
      // copy this thread's own chunks of k-tile `kt_old` from its SMEM stage into the local parameter cache;
      // the thread's later cp.async into the same SMEM addresses follows in program order
      auto mirror = [&](int kt_old, int slot) {
        const uint8_t* st = tiles_b + (size_t)slot * B_STAGE;
#pragma unroll
        for (int i = 0; i < NS; ++i) {
          if (i >= nslots || !src_row[i]) continue;
          const int idx = ltid + i * 96;
          const long long n = (long long)n0 + (idx >> 3);
          const uint4 v = *reinterpret_cast<const uint4*>(st + soff[i]);
          *reinterpret_cast<uint4*>((__nv_bfloat16*)p.w_local + n * p.ldw + (long long)kt_old * BK + (idx & 7) * 8) = v;
        }
      };
      int s = 0;
      uint32_t ph = 0;
      for (int kt = 0; kt < KT; ++kt) {
        if (!tc05::mbar_wait(&ctl->empty_b[s], ph ^ 1u, abort_flag, WAIT_BUDGET_NS)) break;
        const uint32_t sb = tc05::smem_u32(tiles_b + (size_t)s * B_STAGE);
        if (p.w_local != nullptr && kt >= SB) mirror(kt - SB, s);   // the tile this stage held has been consumed
#pragma unroll
        for (int i = 0; i < NS; ++i) {
          if (i >= nslots) continue;
          const void* src = src_row[i] ? (const void*)(src_row[i] + (long long)kt * BK) : (const void*)any_valid;
          const int bytes = src_row[i] ? 16 : 0;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sb + soff[i]), "l"(src), "r"(bytes) : "memory");
        }
        // arrives on `staged` once this thread's copies above have landed
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(tc05::smem_u32(&ctl->staged[s])) : "memory");
        if (++s == SB) { s = 0; ph ^= 1u; }
      }
      asm volatile("cp.async.wait_all;" ::: "memory");
      if (p.w_local != nullptr) {
        // the last SB tiles: wait until the MMAs have consumed everything, then mirror them
        if (tc05::mbar_wait(&ctl->tmem_full, 0, abort_flag, WAIT_BUDGET_NS))
          for (int kt = (KT > SB ? KT - SB : 0); kt < KT; ++kt) mirror(kt, kt % SB);
      }
    } else {
      // committer warp.  The cross-proxy fence is expensive while copies are in flight (it waits for
      // them), so one fence publishes a group of G landed tiles.
      const int G = SB >= 12 ? 4 : (SB >= 6 ? 2 : 1);
      if (lane == 0) {
        int s = 0;
        uint32_t ph = 0;
        for (int kt0 = 0; kt0 < KT; kt0 += G) {
          const int ng = min(G, KT - kt0);
          bool okc = true;
          int sw = s;
          uint32_t phw = ph;
          for (int g = 0; g < ng && okc; ++g) {
            okc = tc05::mbar_wait(&ctl->staged[sw], phw, abort_flag, WAIT_BUDGET_NS);
            if (++sw == SB) { sw = 0; phw ^= 1u; }
          }
          if (!okc) break;
          tc05::fence_proxy_async_smem();
          for (int g = 0; g < ng; ++g) {
            tc05::mbar_arrive(&ctl->full_b[s]);
            if (++s == SB) { s = 0; ph ^= 1u; }
          }
        }
      }
    }
    __syncwarp();
    // ---------------- epilogue (same warps): TMEM -> registers -> global ----------------
    const int q = warp & 3;
    const bool have = tc05::mbar_wait(&ctl->tmem_full, 0, abort_flag, WAIT_BUDGET_NS);
    tc05::fence_after_sync();
    if (have) {
      for (int mt = 0; mt < d.m_tiles; ++mt) {
        const long long row = (long long)mt * BM + q * 32 + lane;
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tc05::tmem_ld_32x32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(mt * BN + c), r);
          tc05::tmem_ld_wait();
          if (row >= p.M) continue;
          for (int j = 0; j < 32; ++j) {
            const long long col = (long long)n0 + c + j;
            if (col >= p.N) break;
            float x = __uint_as_float(r[j]);
            if (p.bias) x += p.bias[col];
            if (p.relu) x = fmaxf(x, 0.f);
            if (p.out_fp32) ((float*)p.Y)[row * p.ldy + col] = x;
            else ((__nv_bfloat16*)p.Y)[row * p.ldy + col] = __float2bfloat16(x);
          }
        }
      }
    }
  }
  tc05::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && ctl->abort_flag)
    geeps_report(p.status, GEEPS_ERR_TIMEOUT, KID_PULL_GEMM, (int)blockIdx.x, 0);
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
    void* q = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &q, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)q;
  });
  return fn;
}

}  // namespace

extern "C" {

int geeps_pull_gemm_bf16(const GeepsPullGemmParams* params, void* stream) {
  const GeepsPullGemmParams& p = *params;
  if (p.M <= 0 || p.M > 2 * BM || p.N <= 0 || p.K <= 0 || (p.K % BK) || (p.ldx % 8) || (p.ldw % 8) ||
      ((uintptr_t)p.X & 15) || p.n_shards < 1 || p.n_shards > GEEPS_MAX_RANKS)
    return (int)cudaErrorInvalidValue;
  EncodeTiledFn fn = encode_fn();
  if (!fn) return (int)cudaErrorInvalidValue;
  CUtensorMap ta;
  cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)p.M};
  cuuint64_t strides[1] = {(cuuint64_t)p.ldx * 2};
  cuuint32_t box[2] = {BK, BM};
  cuuint32_t estr[2] = {1, 1};
  if (fn(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(p.X), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return (int)cudaErrorInvalidValue;
  PullGemmDev d;
  d.p = p;
  d.m_tiles = (int)((p.M + BM - 1) / BM);
  // narrow tiles: the kernel is bound by the link, so what matters is many CTAs with loads in flight
  // wide tiles: every CTA streams all of X, so X traffic is (N / bn) * |X|; what hides the link latency is
  // the depth of the W ring, not the number of CTAs
  d.bn = p.block_n > 0 ? p.block_n : (p.N >= 64 * 64 ? 64 : 32);
  if (d.bn % 32 || d.bn > 128) return (int)cudaErrorInvalidValue;
  d.kt_total = (int)(p.K / BK);
  int tc = 32;
  while (tc < d.m_tiles * d.bn) tc <<= 1;
  d.tmem_cols = tc;
  const int a_stage = d.m_tiles * A_TILE_BYTES, b_stage = d.bn * BK * 2;
  // the X ring sets how many k-tiles are in flight between TMA issue and the MMA's commit: as deep as fits
  d.stages_a = d.m_tiles == 2 ? 5 : 8;
  d.stages_b = (212 * 1024 - d.stages_a * a_stage) / b_stage;
  if (d.stages_b > MAX_B_STAGES) d.stages_b = MAX_B_STAGES;
  if (d.stages_b < 2) d.stages_b = 2;
  const size_t smem = (size_t)d.stages_a * a_stage + (size_t)d.stages_b * b_stage + sizeof(SmemCtl) + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(pull_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int grid = (int)((p.N + d.bn - 1) / d.bn);
  pull_gemm_kernel<<<grid, 192, smem, (cudaStream_t)stream>>>(ta, d);
  return (int)cudaGetLastError();
}

}  // extern "C"
