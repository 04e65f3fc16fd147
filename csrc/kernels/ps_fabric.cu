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
// `failed` CTAs (an expired in-kernel wait: their rows were skipped) add a high bit to the counter, and
// *any_failed tells the last CTA whether any CTA of the launch did, so that it never stamps a clock that
// was not applied everywhere.
constexpr int kCtaFailBit = 1 << 20;
__device__ __forceinline__ bool last_cta_arrive(int* counter, bool failed = false, bool* any_failed = nullptr) {
  __syncthreads();
  bool last = false;
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int prev = atomicAdd(counter, 1 + (failed ? kCtaFailBit : 0));
    if ((prev & (kCtaFailBit - 1)) == (int)gridDim.x - 1) {
      __threadfence_system();
      if (any_failed) *any_failed = failed || prev >= kCtaFailBit;
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
  const int clock_stamp = p.clock_stamp + (p.clock_ref != nullptr ? *p.clock_ref : 0);
  if (p.push_ready != nullptr && (int)threadIdx.x < p.n_ranks) {
    int seen = 0;
    if (!geeps_wait_ge(p.push_ready + threadIdx.x, clock_stamp, p.wait_budget_ns, &seen)) {
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
    // apply + publish of one owned row, given the reduced update of this lane's four values
    auto finish_row = [&](long long i, long long grow, float4 g) {
      const long long goff = grow * GEEPS_ROW_FLOATS + lane * 4;  // offset in full-table buffers
      const long long loff = i * GEEPS_ROW_FLOATS + lane * 4;     // offset in shard-local buffers
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
      const uint2 h = make_uint2(pack_bf16x2(w.x, w.y), pack_bf16x2(w.z, w.w));
      if (p.master16 != nullptr) *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.master16) + loff) = h;
      // ---- fused publish into every worker's parameter cache ----
      if (p.publish) {
        const bool fp32_too = grow >= p.fp32_from_row;   // weights consumed in bf16 only skip two thirds of the bytes
        if (p.upd_mc != nullptr) {
          // one store per row reaches every worker's cache through the switch
          if (fp32_too && p.cache_mc != nullptr) multimem_st_f4(p.cache_mc + goff, w);
          if (p.cache16_mc != nullptr) multimem_st_bf16x4(static_cast<__nv_bfloat16*>(p.cache16_mc) + goff, h);
        } else {
          for (int q = 0; q < p.n_ranks; ++q) {
            if (fp32_too && p.cache[q] != nullptr) st_f4(p.cache[q] + goff, w);
            if (p.cache16[q] != nullptr) *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.cache16[q]) + goff) = h;
          }
        }
      }
    };
    auto row_of = [&](long long i, long long* grow) -> bool {
      *grow = p.row_start + i * p.row_stride;  // row id inside the table
      if (*grow < 0 || *grow >= p.total_rows) {
        if (lane == 0) geeps_report(p.status, GEEPS_ERR_BOUNDS, KID_PUSH_APPLY, (int)i, (int)*grow);
        return false;
      }
      return true;
    };
    if (p.upd_mc != nullptr) {
      // Through the switch one load per row returns the sum over all workers, so a warp has a single request in
      // flight per row where the peer-load path has one per worker: four rows are requested before the first is
      // applied, to cover the round trip through the switch.
      constexpr int U = 4;
      for (long long i0 = warp0; i0 < p.n_owned; i0 += nwarps * U) {
        float4 g[U];
        long long grow[U];
        bool valid[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * nwarps;
          valid[u] = i < p.n_owned && row_of(i, &grow[u]);
          if (valid[u]) g[u] = multimem_ld_reduce_f4(p.upd_mc + grow[u] * GEEPS_ROW_FLOATS + lane * 4);
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (valid[u]) finish_row(i0 + u * nwarps, grow[u], g[u]);
      }
    } else {
      for (long long i = warp0; i < p.n_owned; i += nwarps) {
        long long grow;
        if (!row_of(i, &grow)) continue;
        const long long goff = grow * GEEPS_ROW_FLOATS + lane * 4;
        finish_row(i, grow, (NR > 0) ? reduce_fixed_order<(NR > 0 ? NR : 1)>(p, goff, strong) : reduce_dyn(p, goff, strong));
      }
    }
  }
  // ---- stamp: rows (or at least the master) are globally visible ----
  bool any_failed = false;
  if (last_cta_arrive(p.cta_counter, !ok, &any_failed)) {
    if (!any_failed) {
      if (p.global_clock != nullptr) st_release_sys(p.global_clock, clock_stamp);
      if (p.publish)
        for (int q = 0; q < p.n_ranks; ++q)
          if (p.data_age[q] != nullptr) st_release_sys(p.data_age[q] + p.rank, clock_stamp);
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
      if (grow < p.row_from) continue;
      float4 w = ld_f4_peer(p.master[s] + i * GEEPS_ROW_FLOATS + lane * 4);
      const long long goff = (grow - p.row_base) * GEEPS_ROW_FLOATS + lane * 4;
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
__global__ void flag_signal_kernel(GeepsFlagList list, int index, int stamp, const int* clock_ref) {
  if (clock_ref != nullptr) stamp += *clock_ref;
  if (threadIdx.x < list.n && list.ptr[threadIdx.x] != nullptr) {
    __threadfence_system();
    st_release_sys(list.ptr[threadIdx.x] + index, stamp);
  }
}

// Wait until flags[i] >= stamp for all i < n; record TIMEOUT in status otherwise.
__global__ void flag_wait_kernel(const int* flags, int n, int stamp, unsigned long long budget_ns,
                                 int* status, const int* clock_ref) {
  if (clock_ref != nullptr) stamp += *clock_ref;
  if ((int)threadIdx.x < n) {
    int seen = 0;
    if (!geeps_wait_ge(flags + threadIdx.x, stamp, budget_ns, &seen))
      geeps_report(status, GEEPS_ERR_TIMEOUT, KID_FLAG_WAIT, (int)threadIdx.x, seen);
  }
}

// The same wait, followed (on success) by a stamp into slot `index` of each listed array.
__global__ void clock_advance_kernel(int* clock) {
  if (threadIdx.x == 0) *clock += 1;
}

__global__ void flag_wait_signal_kernel(const int* flags, int n, int stamp, unsigned long long budget_ns,
                                        int* status, GeepsFlagList then, int index, const int* clock_ref) {
  __shared__ int s_fail;
  if (clock_ref != nullptr) stamp += *clock_ref;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if ((int)threadIdx.x < n) {
    int seen = 0;
    if (!geeps_wait_ge(flags + threadIdx.x, stamp, budget_ns, &seen)) {
      geeps_report(status, GEEPS_ERR_TIMEOUT, KID_FLAG_WAIT, (int)threadIdx.x, seen);
      s_fail = 1;
    }
  }
  __syncthreads();
  if (!s_fail && (int)threadIdx.x < then.n && then.ptr[threadIdx.x] != nullptr) {
    st_release_sys(then.ptr[threadIdx.x] + index, stamp);
    __threadfence_system();
  }
}

// Gather with read-my-updates (see kernels.h).  One warp per row; the row's owning shard follows from the
// partitioning (range: idx / ceil(rows / shards); round robin: idx % shards).
__global__ void __launch_bounds__(256)
row_gather_rmw_kernel(const GeepsRmwReadParams p) {
  struct __align__(16) IndexPair { long long id0; long long id1; };
  const IndexPair* index = static_cast<const IndexPair*>(p.index);
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  const long long per = p.partition_per > 0 ? p.partition_per : (p.total_rows + p.n_ranks - 1) / p.n_ranks;
  const int clock = p.clock + (p.clock_ref != nullptr ? *p.clock_ref : 0);
  for (long long i = warp0; i < p.num_rows; i += nwarps) {
    IndexPair ip;
    if (lane == 0) ip = index[i];
    ip.id0 = __shfl_sync(0xffffffffu, ip.id0, 0);
    ip.id1 = __shfl_sync(0xffffffffu, ip.id1, 0);
    if (ip.id0 < 0 || ip.id0 >= p.dst_rows || ip.id1 < 0 || ip.id1 >= p.total_rows) {
      if (lane == 0) geeps_report(p.status, GEEPS_ERR_BOUNDS, KID_ROW_GATHER, (int)i, (int)(ip.id1));
      continue;
    }
    const long long app_val0 = ip.id0 * GEEPS_ROW_FLOATS + lane * 4;
    const int shard = p.partition_kind == 1 ? (int)(ip.id1 % p.n_ranks) : (int)(per ? ip.id1 / per : 0);
    const float* src = p.cache + ip.id1 * GEEPS_ROW_FLOATS + lane * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    bool done = false;
    // the flag words are read by lane 0 and broadcast, so that the whole warp takes the same decisions
    for (int attempt = 0; attempt < 16 && !done; ++attempt) {
      // stamp = (latest clock the shard has published) + 1; own clocks stamp .. clock-1 are still missing
      int age = 0;
      if (lane == 0) age = ld_acquire_sys(p.data_age + shard);
      age = __shfl_sync(0xffffffffu, age, 0);
      v = ld_f4_peer(src);
      int first = age > clock - (p.ring_slots - 1) ? age : clock - (p.ring_slots - 1);
      if (first < 0) first = 0;
      for (int k = first; k < clock; ++k) {
        const float a = k < p.additive_below_clock ? 1.f : p.alpha;
        const float4 u = ld_f4_cg(p.ring + ((long long)(k % p.ring_slots) * p.total_rows + ip.id1) * GEEPS_ROW_FLOATS + lane * 4);
        v.x += a * u.x; v.y += a * u.y; v.z += a * u.z; v.w += a * u.w;
      }
      __threadfence_system();
      int begun = 0, waited_ok = 1;
      if (lane == 0) {
        begun = ld_acquire_sys(p.publish_begin + shard);
        // a publish started while the row was being read: wait for it to complete, then read again
        if (begun > age) { int seen = 0; waited_ok = geeps_wait_ge(p.data_age + shard, begun, p.wait_budget_ns, &seen) ? 1 : 0; }
      }
      begun = __shfl_sync(0xffffffffu, begun, 0);
      waited_ok = __shfl_sync(0xffffffffu, waited_ok, 0);
      if (begun <= age) done = true;
      else if (!waited_ok) break;
    }
    if (!done) {
      if (lane == 0) geeps_report(p.status, GEEPS_ERR_TIMEOUT, KID_ROW_GATHER, shard, (int)i);
      continue;
    }
    float* d = p.dst + app_val0;
    if (app_val0 + 4 <= p.num_vals_limit) st_f4(d, v);
    else {
      const float e[4] = {v.x, v.y, v.z, v.w};
      for (int j = 0; j < 4 && app_val0 + j < p.num_vals_limit; ++j) d[j] = e[j];
    }
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
  if (max_ctas <= 0) max_ctas = geeps_sm_count() * 4;
  if (blocks > max_ctas) blocks = max_ctas;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace

extern "C" {

int geeps_ps_push_apply(const GeepsPushApplyParams* params, int max_ctas, void* stream) {
  const GeepsPushApplyParams& p = *params;
  if (p.n_ranks < 1 || p.n_ranks > GEEPS_MAX_RANKS) return (int)cudaErrorInvalidValue;
  int grid = pick_grid(p.n_owned, max_ctas);
  if (grid >= kCtaFailBit) grid = kCtaFailBit - 1;
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

int geeps_flag_signal_rel(const GeepsFlagList* list, int index, int stamp_rel, const int* clock_ref, void* stream) {
  flag_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(*list, index, stamp_rel, clock_ref);
  return (int)cudaGetLastError();
}
int geeps_flag_signal(const GeepsFlagList* list, int index, int stamp, void* stream) {
  return geeps_flag_signal_rel(list, index, stamp, nullptr, stream);
}

int geeps_flag_wait_rel(const int* flags, int n, int stamp_rel, const int* clock_ref, unsigned long long budget_ns,
                        int* status, void* stream) {
  if (n > 32) return (int)cudaErrorInvalidValue;
  flag_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, n, stamp_rel, budget_ns, status, clock_ref);
  return (int)cudaGetLastError();
}
int geeps_flag_wait(const int* flags, int n, int stamp, unsigned long long budget_ns, int* status,
                    void* stream) {
  return geeps_flag_wait_rel(flags, n, stamp, nullptr, budget_ns, status, stream);
}

int geeps_clock_advance(int* clock, void* stream) {
  clock_advance_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(clock);
  return (int)cudaGetLastError();
}

int geeps_flag_wait_signal_rel(const int* flags, int n, int stamp_rel, const int* clock_ref,
                               unsigned long long budget_ns, int* status, const GeepsFlagList* then, int index,
                               void* stream) {
  if (n > 32 || then->n > 32) return (int)cudaErrorInvalidValue;
  flag_wait_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, n, stamp_rel, budget_ns, status, *then, index,
                                                              clock_ref);
  return (int)cudaGetLastError();
}
int geeps_flag_wait_signal(const int* flags, int n, int stamp, unsigned long long budget_ns, int* status,
                           const GeepsFlagList* then, int index, void* stream) {
  return geeps_flag_wait_signal_rel(flags, n, stamp, nullptr, budget_ns, status, then, index, stream);
}

int geeps_row_gather_rmw(const GeepsRmwReadParams* params, void* stream) {
  const GeepsRmwReadParams& p = *params;
  if (p.num_rows <= 0) return 0;
  if (p.n_ranks < 1 || p.n_ranks > GEEPS_MAX_RANKS || p.ring_slots < 1) return (int)cudaErrorInvalidValue;
  row_gather_rmw_kernel<<<pick_grid(p.num_rows, geeps_sm_count() * 8), 256, 0, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}

int geeps_f32_to_bf16(const float* src, void* dst, long long n, void* stream) {
  if (n <= 0) return 0;
  long long blocks = ((n >> 2) + 255) / 256;
  if (blocks > geeps_sm_count() * 8) blocks = geeps_sm_count() * 8;
  if (blocks < 1) blocks = 1;
  f32_to_bf16_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(src, (__nv_bfloat16*)dst, n);
  return (int)cudaGetLastError();
}

}  // extern "C"
