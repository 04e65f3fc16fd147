// Parameter-server data-path kernels over peer-mapped memory (NVLink 5 / NVSwitch).
//
// One launch per table (or table bucket) per clock on the owning GPU's comm stream.
//
//   geeps_ps_push_apply : reduce-scatter of the workers' row updates fused with the
//                         shard's apply (additive, or momentum SGD with weight decay on
//                         fp32 master rows) and, optionally, with the publish of the new
//                         rows into every worker's parameter cache (fp32 and/or bf16
//                         compute copy) followed by the data_age stamp.
//   geeps_ps_pull       : all-gather of master rows into this worker's cache for the
//                         split push / pull mode (bounded wait on each shard's clock).
//   geeps_flag_*        : monotone clock-stamp flags with bounded waits.
//
// What this replaces in the reference: the per-clock ZeroMQ round trip
//   client push  src/client/clientlib-data.cpp:436-522  (D2H of the oplog, one message per server)
//   server apply src/server/tablet-server.cpp:81-134    (cpu_add(master, update) in host RAM)
//   server bcast src/server/tablet-server.cpp:147-212   (whole shard to every client per clock)
//   client recv  src/client/clientlib-data.cpp:51-151   (pinned bounce + H2D + saxpy replay)
// Here a shard's CTAs read the workers' update rows straight out of their HBM with plain
// system-scope loads in fixed rank order (bit-reproducible sums), keep master and momentum
// in registers for the apply, and store the result into the peers' caches.  The vector
// clock is a set of int flags in peer-mapped memory; every wait is bounded and reports
// into a status block instead of hanging.
#include "common.cuh"
#include "kernels.h"

namespace {

__device__ __forceinline__ float4 f4_add(float4 a, float4 b) {
  return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}

// Grid-wide "last CTA" rendezvous: returns true in exactly one CTA (thread 0 of it),
// after every CTA's prior global/peer stores are visible system-wide.
__device__ __forceinline__ bool last_cta_arrive(int* counter) {
  __syncthreads();
  bool last = false;
  if (threadIdx.x == 0) {
    __threadfence_system();
    int prev = atomicAdd(counter, 1);
    if (prev == (int)gridDim.x - 1) {
      __threadfence_system();
      *counter = 0;  // ready for the next launch on this stream
      last = true;
    }
  }
  return last;
}

// The workers' updates are complete before the push-ready flags this stream waited on, so plain weak loads
// (L1 bypassed) are enough; with `in_kernel_wait` the flags were acquired inside this kernel by other
// threads, and the loads have to be system-scope relaxed ones.
template <int NR>
__device__ __forceinline__ float4 reduce_fixed_order(const GeepsPushApplyParams& p, long long off, bool strong) {
  float4 v[NR];
#pragma unroll
  for (int w = 0; w < NR; ++w) v[w] = strong ? ld_f4_peer(p.upd[w] + off) : ld_f4_cg(p.upd[w] + off);
  float4 g = v[0];
#pragma unroll
  for (int w = 1; w < NR; ++w) g = f4_add(g, v[w]);
  return g;
}

__device__ __forceinline__ float4 reduce_dyn(const GeepsPushApplyParams& p, long long off, bool strong) {
  float4 g = strong ? ld_f4_peer(p.upd[0] + off) : ld_f4_cg(p.upd[0] + off);
  for (int w = 1; w < p.n_ranks; ++w) g = f4_add(g, strong ? ld_f4_peer(p.upd[w] + off) : ld_f4_cg(p.upd[w] + off));
  return g;
}

__device__ __forceinline__ float sgd1(float& m, float pv, float g, const GeepsPushApplyParams& p) {
  m = p.momentum_coef * m + p.lr * (g * p.grad_scale + p.weight_decay * pv);
  return pv - m;
}

template <int NR>
__global__ void __launch_bounds__(256)
push_apply_kernel(const GeepsPushApplyParams p) {
  __shared__ int s_ok;
  // ---- bounded wait: every worker's update for this clock is complete ----
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (p.push_ready != nullptr && (int)threadIdx.x < p.n_ranks) {
    int seen = 0;
    if (!geeps_wait_ge(p.push_ready + threadIdx.x, p.clock_stamp, p.wait_budget_ns, &seen)) {
      geeps_report(p.status, GEEPS_ERR_TIMEOUT, KID_PUSH_APPLY, (int)threadIdx.x, seen);
      s_ok = 0;
    }
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  const bool strong = p.push_ready != nullptr;   // flags were awaited inside this kernel

  if (ok) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long i = warp0; i < p.n_owned; i += nwarps) {
      const long long grow = p.row_start + i * p.row_stride;  // row id inside the table
      if (grow < 0 || grow >= p.total_rows) {
        if (lane == 0) geeps_report(p.status, GEEPS_ERR_BOUNDS, KID_PUSH_APPLY, (int)i, (int)grow);
        continue;
      }
      const long long goff = grow * GEEPS_ROW_FLOATS + lane * 4;  // offset in full-table buffers
      const long long loff = i * GEEPS_ROW_FLOATS + lane * 4;     // offset in shard-local buffers
      float4 g = (NR > 0) ? reduce_fixed_order<(NR > 0 ? NR : 1)>(p, goff, strong) : reduce_dyn(p, goff, strong);
      float4 w = ld_f4(p.master + loff);
      if (p.mode == GEEPS_TABLE_SGD_MOMENTUM) {
        float4 m = ld_f4(p.momentum + loff);
        w.x = sgd1(m.x, w.x, g.x, p); w.y = sgd1(m.y, w.y, g.y, p);
        w.z = sgd1(m.z, w.z, g.z, p); w.w = sgd1(m.w, w.w, g.w, p);
        st_f4(p.momentum + loff, m);
      } else {
        w = f4_add(w, g);
      }
      st_f4(p.master + loff, w);
      // ---- fused publish into every worker's parameter cache ----
      if (p.publish) {
        const uint2 h = make_uint2(pack_bf16x2(w.x, w.y), pack_bf16x2(w.z, w.w));
        const bool fp32_too = grow >= p.fp32_from_row;   // weights consumed in bf16 only skip two thirds of the bytes
        for (int q = 0; q < p.n_ranks; ++q) {
          if (fp32_too && p.cache[q] != nullptr) st_f4(p.cache[q] + goff, w);
          if (p.cache16[q] != nullptr) *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.cache16[q]) + goff) = h;
        }
      }
    }
  }
  // ---- stamp: rows (or at least the master) are globally visible ----
  if (last_cta_arrive(p.cta_counter)) {
    if (ok) {
      if (p.global_clock != nullptr) st_release_sys(p.global_clock, p.clock_stamp);
      if (p.publish)
        for (int q = 0; q < p.n_ranks; ++q)
          if (p.data_age[q] != nullptr) st_release_sys(p.data_age[q] + p.rank, p.clock_stamp);
    }
  }
}

// Worker-side pull: copy every shard's master rows into the local cache once the
// shard's global clock reached the needed age.
__global__ void __launch_bounds__(256)
pull_kernel(const GeepsPullParams p) {
  __shared__ int s_ok;
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  // shards are visited starting at our own rank so that every NVLink port is loaded evenly
  for (int k = 0; k < p.n_ranks; ++k) {
    const int s = (p.rank + k) % p.n_ranks;
    if (threadIdx.x == 0) {
      int seen = 0;
      s_ok = 1;
      if (p.global_clock[s] != nullptr &&
          !geeps_wait_ge(p.global_clock[s], p.needed_stamp, p.wait_budget_ns, &seen)) {
        geeps_report(p.status, GEEPS_ERR_TIMEOUT, KID_PULL, s, seen);
        s_ok = 0;
      }
    }
    __syncthreads();
    const bool ok = s_ok != 0;
    __syncthreads();
    if (!ok) continue;
    const long long n_owned = p.n_owned[s];
    const long long warp0 = (long long)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * warps_per_cta;
    for (long long i = warp0; i < n_owned; i += nwarps) {
      const long long grow = p.row_start[s] + i * p.row_stride[s];
      if (grow < 0 || grow >= p.total_rows) {
        if (lane == 0) geeps_report(p.status, GEEPS_ERR_BOUNDS, KID_PULL, (int)i, (int)grow);
        continue;
      }
      float4 w = ld_f4_peer(p.master[s] + i * GEEPS_ROW_FLOATS + lane * 4);
      const long long goff = grow * GEEPS_ROW_FLOATS + lane * 4;
      if (p.cache != nullptr) st_f4(p.cache + goff, w);
      if (p.cache16 != nullptr)
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.cache16) + goff) =
            make_uint2(pack_bf16x2(w.x, w.y), pack_bf16x2(w.z, w.w));
    }
  }
  if (last_cta_arrive(p.cta_counter)) {
    if (p.data_age_local != nullptr)
      for (int s = 0; s < p.n_ranks; ++s) st_release_sys(p.data_age_local + s, p.needed_stamp);
  }
}

// Write `stamp` into slot `index` of each listed flag array (peer pointers).
__global__ void flag_signal_kernel(GeepsFlagList list, int index, int stamp) {
  if (threadIdx.x < list.n && list.ptr[threadIdx.x] != nullptr) {
    __threadfence_system();
    st_release_sys(list.ptr[threadIdx.x] + index, stamp);
  }
}

// Wait until flags[i] >= stamp for all i < n; record TIMEOUT in status otherwise.
__global__ void flag_wait_kernel(const int* flags, int n, int stamp, unsigned long long budget_ns,
                                 int* status) {
  if ((int)threadIdx.x < n) {
    int seen = 0;
    if (!geeps_wait_ge(flags + threadIdx.x, stamp, budget_ns, &seen))
      geeps_report(status, GEEPS_ERR_TIMEOUT, KID_FLAG_WAIT, (int)threadIdx.x, seen);
  }
}

// fp32 rows -> bf16 compute copy (local refresh of the compute cache)
__global__ void __launch_bounds__(256)
f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  const long long n4 = n >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 v = ld_f4(src + i * 4);
    *reinterpret_cast<uint2*>(dst + i * 4) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    long long i = (n4 << 2) + threadIdx.x;
    dst[i] = __float2bfloat16(src[i]);
  }
}

int pick_grid(long long rows, int max_ctas) {
  long long blocks = (rows + 7) / 8;
  if (max_ctas <= 0) max_ctas = 148 * 4;
  if (blocks > max_ctas) blocks = max_ctas;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace

extern "C" {

int geeps_ps_push_apply(const GeepsPushApplyParams* params, int max_ctas, void* stream) {
  const GeepsPushApplyParams& p = *params;
  if (p.n_ranks < 1 || p.n_ranks > GEEPS_MAX_RANKS) return (int)cudaErrorInvalidValue;
  const int grid = pick_grid(p.n_owned, max_ctas);
  cudaStream_t st = (cudaStream_t)stream;
  switch (p.n_ranks) {
    case 1: push_apply_kernel<1><<<grid, 256, 0, st>>>(p); break;
    case 2: push_apply_kernel<2><<<grid, 256, 0, st>>>(p); break;
    case 4: push_apply_kernel<4><<<grid, 256, 0, st>>>(p); break;
    case 8: push_apply_kernel<8><<<grid, 256, 0, st>>>(p); break;
    default: push_apply_kernel<0><<<grid, 256, 0, st>>>(p); break;
  }
  return (int)cudaGetLastError();
}

int geeps_ps_pull(const GeepsPullParams* params, int max_ctas, void* stream) {
  const GeepsPullParams& p = *params;
  if (p.n_ranks < 1 || p.n_ranks > GEEPS_MAX_RANKS) return (int)cudaErrorInvalidValue;
  long long max_owned = 0;
  for (int s = 0; s < p.n_ranks; ++s) if (p.n_owned[s] > max_owned) max_owned = p.n_owned[s];
  pull_kernel<<<pick_grid(max_owned, max_ctas), 256, 0, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}

int geeps_flag_signal(const GeepsFlagList* list, int index, int stamp, void* stream) {
  flag_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(*list, index, stamp);
  return (int)cudaGetLastError();
}

int geeps_flag_wait(const int* flags, int n, int stamp, unsigned long long budget_ns, int* status,
                    void* stream) {
  if (n > 32) return (int)cudaErrorInvalidValue;
  flag_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, n, stamp, budget_ns, status);
  return (int)cudaGetLastError();
}

int geeps_f32_to_bf16(const float* src, void* dst, long long n, void* stream) {
  if (n <= 0) return 0;
  long long blocks = ((n >> 2) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  f32_to_bf16_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(src, (__nv_bfloat16*)dst, n);
  return (int)cudaGetLastError();
}

}  // extern "C"
