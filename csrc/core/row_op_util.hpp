// Host-side row operations: the CPU counterparts of the device kernels in
// kernels/row_ops.cu and kernels/ps_fabric.cu.  They are the correctness oracle for those
// kernels and the data path of the CPU / TCP mode.
//
// Same operations as the reference's src/common/row-op-util.hpp:64-139 (add_row_batch and the
// three *_double_index_cpu functions) plus the server-side optimizer, which the reference
// leaves to the application (its server only adds: src/server/tablet-server.cpp:119-134).
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "geeps-user-defined-types.hpp"
#include "internal_config.hpp"

namespace geeps_b200 {

// (position in the application buffer, position in the cache / oplog)
struct DoubleIndex {
  int64_t id0;
  int64_t id1;
  DoubleIndex(int64_t a = 0, int64_t b = 0) : id0(a), id1(b) {}
};

inline void cpu_add(size_t n, const val_t* a, const val_t* b, val_t* y) {
  for (size_t i = 0; i < n; ++i) y[i] = a[i] + b[i];
}
inline void cpu_axpy(size_t n, val_t alpha, const val_t* x, val_t* y) {
  for (size_t i = 0; i < n; ++i) y[i] += alpha * x[i];
}
// y[r] += x[r] over whole rows
inline void add_row_batch(RowData* y, const RowData* x, size_t rows) {
  cpu_axpy(rows * ROW_DATA_SIZE, 1.f, reinterpret_cast<const val_t*>(x), reinterpret_cast<val_t*>(y));
}

// y[id0 + off0] = x[id1 + off1]   (cache -> application buffer); values at flat position
// >= num_vals_limit of the application buffer stay untouched.
inline void assign_rows_to_double_index_cpu(RowData* y, const RowData* x, const DoubleIndex* index, size_t n,
                                            size_t off0, size_t off1, size_t num_vals_limit) {
  for (size_t i = 0; i < n; ++i) {
    const size_t yr = index[i].id0 + off0, xr = index[i].id1 + off1;
    for (size_t v = 0; v < ROW_DATA_SIZE; ++v)
      if (yr * ROW_DATA_SIZE + v < num_vals_limit) y[yr].data[v] = x[xr].data[v];
  }
}
// y[id1 + off1] = x[id0 + off0]   (application buffer -> cache)
inline void assign_rows_from_double_index_cpu(RowData* y, const RowData* x, const DoubleIndex* index, size_t n,
                                              size_t off0, size_t off1, size_t num_vals_limit) {
  for (size_t i = 0; i < n; ++i) {
    const size_t xr = index[i].id0 + off0, yr = index[i].id1 + off1;
    for (size_t v = 0; v < ROW_DATA_SIZE; ++v)
      if (xr * ROW_DATA_SIZE + v < num_vals_limit) y[yr].data[v] = x[xr].data[v];
  }
}
// y[id1 + off1] += x[id0 + off0]  (application update buffer -> oplog / cache)
inline void add_rows_from_double_index_cpu(RowData* y, const RowData* x, const DoubleIndex* index, size_t n,
                                           size_t off0, size_t off1, size_t num_vals_limit) {
  for (size_t i = 0; i < n; ++i) {
    const size_t xr = index[i].id0 + off0, yr = index[i].id1 + off1;
    for (size_t v = 0; v < ROW_DATA_SIZE; ++v)
      if (xr * ROW_DATA_SIZE + v < num_vals_limit) y[yr].data[v] += x[xr].data[v];
  }
}

// y[id1 + off1] += alpha * x[id0 + off0]
inline void axpy_rows_from_double_index_cpu(RowData* y, const RowData* x, const DoubleIndex* index, size_t n,
                                            size_t off0, size_t off1, size_t num_vals_limit, val_t alpha) {
  for (size_t i = 0; i < n; ++i) {
    const size_t xr = index[i].id0 + off0, yr = index[i].id1 + off1;
    for (size_t v = 0; v < ROW_DATA_SIZE; ++v)
      if (xr * ROW_DATA_SIZE + v < num_vals_limit) y[yr].data[v] += alpha * x[xr].data[v];
  }
}

struct OptimizerParams {
  float lr = 0.01f, momentum = 0.9f, weight_decay = 0.f, grad_scale = 1.f;
};
// Momentum SGD with weight decay on fp32 master rows (Caffe convention), applied once per
// clock to the update summed over workers:  v = mu*v + lr*(g*scale + wd*p);  p -= v.
inline void cpu_sgd_momentum(size_t n, val_t* p, val_t* v, const val_t* g, const OptimizerParams& o) {
  for (size_t i = 0; i < n; ++i) {
    v[i] = o.momentum * v[i] + o.lr * (g[i] * o.grad_scale + o.weight_decay * p[i]);
    p[i] -= v[i];
  }
}

}  // namespace geeps_b200
