// Row-batch movement kernels: gather, scatter, scatter-add and axpy over 512-byte rows.
//
// These cover the three device kernels of the reference
// (src/common/row-op-util.cu:39-55 gather "assign_rows_to_double_index",
//  :74-90 scatter "assign_rows_from_double_index", :109-125 scatter-add
//  "add_rows_from_double_index") and its cuBLAS saxpy call used for the
// read-my-writes replay (src/client/clientlib-data.cpp:137-149).
//
// Shape of the work here: one warp moves one row per step - 32 lanes x one
// 16-byte vector = 512 B, fully coalesced - instead of one thread per fp32
// element; indices are 64-bit; each index pair is read once per row (by lane
// broadcast), not once per element.  Nothing synchronises the stream.
#include "common.cuh"
#include "kernels.h"

namespace {

struct __align__(16) IndexPair { long long id0; long long id1; };

enum RowOpKind { ROW_GATHER = 0, ROW_SCATTER = 1, ROW_SCATTER_ADD = 2 };

// dst/src are row arrays.  For each i < num_rows:
//   gather     : dst[(id0+dst_off)] = src[(id1+src_off)]   (dst is the app buffer)
//   scatter    : dst[(id1+dst_off)] = src[(id0+src_off)]   (src is the app buffer)
//   scatter_add: dst[(id1+dst_off)] += src[(id0+src_off)]
// Values whose flat position in the *app buffer* is >= num_vals_limit are left
// untouched (row-op-util.cu:51,121 semantics).  Rows outside [0,dst_rows) /
// [0,src_rows) are skipped and reported.
template <int KIND>
__global__ void __launch_bounds__(256)
row_op_kernel(float* __restrict__ dst, const float* __restrict__ src,
              const IndexPair* __restrict__ index, long long num_rows,
              long long dst_off, long long src_off, long long num_vals_limit,
              long long dst_rows, long long src_rows, int* status, float alpha) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long i = warp0; i < num_rows; i += nwarps) {
    IndexPair ip;
    if (lane == 0) ip = index[i];
    ip.id0 = __shfl_sync(0xffffffffu, ip.id0, 0);
    ip.id1 = __shfl_sync(0xffffffffu, ip.id1, 0);
    long long drow, srow, app_row;
    if (KIND == ROW_GATHER) { drow = ip.id0 + dst_off; srow = ip.id1 + src_off; app_row = drow; }
    else                    { drow = ip.id1 + dst_off; srow = ip.id0 + src_off; app_row = srow; }
    if (drow < 0 || drow >= dst_rows || srow < 0 || srow >= src_rows) {
      if (lane == 0) geeps_report(status, GEEPS_ERR_BOUNDS,
                                  KIND == ROW_GATHER ? KID_ROW_GATHER : KIND == ROW_SCATTER ? KID_ROW_SCATTER : KID_ROW_SCATTER_ADD,
                                  (int)i, (int)(drow < 0 || drow >= dst_rows ? drow : srow));
      continue;
    }
    const long long app_val0 = app_row * GEEPS_ROW_FLOATS + lane * 4;
    if (app_val0 >= num_vals_limit) continue;
    float* d = dst + drow * GEEPS_ROW_FLOATS + lane * 4;
    const float* s = src + srow * GEEPS_ROW_FLOATS + lane * 4;
    if (app_val0 + 4 <= num_vals_limit) {
      float4 v = ld_f4(s);
      if (KIND == ROW_SCATTER_ADD) {
        float4 o = ld_f4(d);
        v.x = o.x + alpha * v.x; v.y = o.y + alpha * v.y; v.z = o.z + alpha * v.z; v.w = o.w + alpha * v.w;
      }
      st_f4(d, v);
    } else {  // ragged tail of the limit
      for (int e = 0; e < 4 && app_val0 + e < num_vals_limit; ++e) {
        if (KIND == ROW_SCATTER_ADD) d[e] += alpha * s[e]; else d[e] = s[e];
      }
    }
  }
}

// y[i] += alpha * x[i] over n floats (n multiple of 4 handled vectorised, tail scalar)
__global__ void __launch_bounds__(256)
axpy_kernel(float* __restrict__ y, const float* __restrict__ x, float alpha, long long n) {
  const long long n4 = n >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 a = ld_f4(x + i * 4), b = ld_f4(y + i * 4);
    b.x += alpha * a.x; b.y += alpha * a.y; b.z += alpha * a.z; b.w += alpha * a.w;
    st_f4(y + i * 4, b);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    long long i = (n4 << 2) + threadIdx.x;
    y[i] += alpha * x[i];
  }
}

inline int grid_for_rows(long long rows, int warps_per_block) {
  long long blocks = (rows + warps_per_block - 1) / warps_per_block;
  const long long cap = (long long)geeps_sm_count() * 8;  // 8 resident 256-thread CTAs per SM
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

template <int KIND>
int launch_row_op(float* dst, const float* src, const void* index, long long num_rows,
                  long long dst_off, long long src_off, long long num_vals_limit,
                  long long dst_rows, long long src_rows, int* status, cudaStream_t stream, float alpha = 1.f) {
  if (num_rows <= 0) return 0;
  row_op_kernel<KIND><<<grid_for_rows(num_rows, 8), 256, 0, stream>>>(
      dst, src, static_cast<const IndexPair*>(index), num_rows, dst_off, src_off, num_vals_limit,
      dst_rows, src_rows, status, alpha);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

int geeps_row_gather(float* dst, const float* src, const void* index, long long num_rows,
                     long long dst_off, long long src_off, long long num_vals_limit,
                     long long dst_rows, long long src_rows, int* status, void* stream) {
  return launch_row_op<ROW_GATHER>(dst, src, index, num_rows, dst_off, src_off, num_vals_limit,
                                   dst_rows, src_rows, status, (cudaStream_t)stream);
}
int geeps_row_scatter(float* dst, const float* src, const void* index, long long num_rows,
                      long long dst_off, long long src_off, long long num_vals_limit,
                      long long dst_rows, long long src_rows, int* status, void* stream) {
  return launch_row_op<ROW_SCATTER>(dst, src, index, num_rows, dst_off, src_off, num_vals_limit,
                                    dst_rows, src_rows, status, (cudaStream_t)stream);
}
int geeps_row_scatter_add(float* dst, const float* src, const void* index, long long num_rows,
                          long long dst_off, long long src_off, long long num_vals_limit,
                          long long dst_rows, long long src_rows, int* status, void* stream) {
  return launch_row_op<ROW_SCATTER_ADD>(dst, src, index, num_rows, dst_off, src_off,
                                        num_vals_limit, dst_rows, src_rows, status,
                                        (cudaStream_t)stream);
}
int geeps_row_scatter_axpy(float* dst, const float* src, const void* index, long long num_rows,
                           long long dst_off, long long src_off, long long num_vals_limit,
                           long long dst_rows, long long src_rows, float alpha, int* status, void* stream) {
  return launch_row_op<ROW_SCATTER_ADD>(dst, src, index, num_rows, dst_off, src_off,
                                        num_vals_limit, dst_rows, src_rows, status,
                                        (cudaStream_t)stream, alpha);
}
int geeps_axpy(float* y, const float* x, float alpha, long long n, void* stream) {
  if (n <= 0) return 0;
  long long blocks = ((n >> 2) + 255) / 256;
  if (blocks > geeps_sm_count() * 8) blocks = geeps_sm_count() * 8;
  if (blocks < 1) blocks = 1;
  axpy_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(y, x, alpha, n);
  return (int)cudaGetLastError();
}

}  // extern "C"
