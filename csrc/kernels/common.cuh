// Shared device helpers for every sm_100a kernel in this library.
//
// Conventions used by all kernels:
//  * A parameter-server row is 128 fp32 values = 512 bytes (same row shape as
//    include/geeps-user-defined-types.hpp:55-57 of the reference).
//  * No kernel traps, asserts or spins forever.  A wait that runs out of its
//    time budget, or an index that fails a bounds check, records a code in a
//    caller-provided 4-word status block and the kernel returns normally.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define GEEPS_ROW_FLOATS 128
#define GEEPS_ROW_BYTES 512

// status[0] = first error code (0 = ok), status[1] = kernel id,
// status[2] = detail (flag index / row index), status[3] = observed value.
enum GeepsStatusCode : int {
  GEEPS_OK = 0,
  GEEPS_ERR_TIMEOUT = 1,       // a bounded wait expired
  GEEPS_ERR_BOUNDS = 2,        // an index failed a software bounds check
  GEEPS_ERR_ALIGN = 3,         // a pointer failed an alignment check
};

enum GeepsKernelId : int {
  KID_ROW_GATHER = 1, KID_ROW_SCATTER = 2, KID_ROW_SCATTER_ADD = 3, KID_ROW_AXPY = 4,
  KID_PUSH_APPLY = 10, KID_PULL = 11, KID_PUSHPULL = 12, KID_FLAG_WAIT = 13,
  KID_GEMM_TC = 20, KID_GEMM_SIMT = 21, KID_PULL_GEMM = 22, KID_CONV_TC = 23,
};

// Number of SMs of the current device (cudaDevAttrMultiProcessorCount), read once per device and cached:
// grids are sized from it, never from a literal.
inline int geeps_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); dev = 0; }
  int n = cached[dev];
  if (n <= 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) { cudaGetLastError(); n = 148; }
    cached[dev] = n;
  }
  return n;
}

__device__ __forceinline__ void geeps_report(int* status, int code, int kid, int detail, int seen) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = kid;
    status[2] = detail;
    status[3] = seen;
    __threadfence_system();
  }
}

__device__ __forceinline__ uint64_t geeps_globaltimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- system-scope flag words (monotone clock stamps; wait for >= expected) ----
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_relaxed_sys(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Spin until *flag >= expected or budget_ns elapses.  Returns true on success.
// The polls are relaxed loads spaced by a sleep that backs off to 4 us, and one acquire load orders the
// data behind the flag once it has been seen: a waiting warp shares its SM with compute kernels (the
// persistent tensor-core kernels assign tiles statically, so one slowed SM slows the whole kernel), and
// system-scope acquires issued every microsecond were measurably slowing them.
__device__ __forceinline__ bool geeps_wait_ge(const int* flag, int expected, uint64_t budget_ns,
                                              int* seen_out) {
  int v = ld_acquire_sys(flag);
  if (v >= expected) { if (seen_out) *seen_out = v; return true; }
  const uint64_t t0 = geeps_globaltimer();
  unsigned backoff = 64;
  for (;;) {
    v = ld_relaxed_sys(flag);
    if (v >= expected) {
      v = ld_acquire_sys(flag);
      if (seen_out) *seen_out = v;
      return true;
    }
    if (geeps_globaltimer() - t0 > budget_ns) { if (seen_out) *seen_out = v; return false; }
    __nanosleep(backoff);
    if (backoff < 4096) backoff <<= 1;
  }
}

// 16-byte vector helpers
__device__ __forceinline__ float4 ld_f4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st_f4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ float4 ld_f4_nc_stream(const float* p) {
  float4 v;
  asm volatile("ld.global.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
// Weak 16-byte load that bypasses the (non-coherent) L1 and is served from L2 / the peer.  Correct for data
// that was completely written before this kernel started or before a flag this kernel's stream waited on
// (stream order and the release / acquire on the flag order those writes before this load).
__device__ __forceinline__ float4 ld_f4_cg(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
// Volatile-strength peer load: data written by another GPU during this kernel must
// not be served from a stale L1 line.
__device__ __forceinline__ float4 ld_f4_peer(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

// ---- NVSwitch multicast (multimem) accesses through a multicast mapping: 16-byte aligned addresses ----
// sum over every bound device of the float4 at this offset, added in the switch
__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float* p) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
// store to every bound device
__device__ __forceinline__ void multimem_st_f4(float* p, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void multimem_st_bf16x4(void* p, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.bf16x2 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
