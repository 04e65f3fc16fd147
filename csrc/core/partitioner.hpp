// Row -> server-shard placement.  Rows of a table are numbered by their position `i` in the
// table's parameter cache (0 .. n-1); a partitioner maps i to the owning shard and to the
// row's position inside that shard.
//
//   range        equal contiguous chunks, the reference's only live policy
//                (src/client/clientlib-viter.cpp:674-682); with `align` > 1 every chunk is a whole number of
//                align-row groups (a weight matrix whose rows span several table rows then never straddles
//                two shards)
//   round_robin  i mod num_shards, the hash policy that only exists in the reference's dead
//                metadata server (src/server/metadata-server.cpp:129-134)
//
// Both describe a shard's rows as an arithmetic sequence start + k*stride, which is what the
// device kernels take.
#pragma once
#include <stddef.h>

namespace geeps_b200 {

enum PartitionKind { PARTITION_RANGE = 0, PARTITION_ROUND_ROBIN = 1 };

struct ShardRange {
  size_t start = 0;    // cache index of the shard's first row
  size_t stride = 1;   // distance between consecutive rows of the shard
  size_t count = 0;    // number of rows owned
};

class Partitioner {
 public:
  Partitioner(int kind = PARTITION_RANGE, size_t num_rows = 0, size_t num_shards = 1, size_t align = 1)
      : kind_(kind), n_(num_rows), s_(num_shards ? num_shards : 1), align_(align ? align : 1) {}
  // rows per shard of the range policy
  size_t per() const {
    const size_t p = (n_ + s_ - 1) / s_;
    return (p + align_ - 1) / align_ * align_;
  }
  size_t num_rows() const { return n_; }
  size_t num_shards() const { return s_; }
  int kind() const { return kind_; }

  ShardRange range_of(size_t shard) const {
    ShardRange r;
    if (kind_ == PARTITION_ROUND_ROBIN) {
      r.start = shard;
      r.stride = s_;
      r.count = n_ > shard ? (n_ - shard + s_ - 1) / s_ : 0;
    } else {
      const size_t p = per();
      r.start = shard * p < n_ ? shard * p : n_;
      r.stride = 1;
      const size_t end = (shard + 1) * p < n_ ? (shard + 1) * p : n_;
      r.count = end - r.start;
    }
    return r;
  }
  size_t shard_of(size_t i) const {
    if (kind_ == PARTITION_ROUND_ROBIN) return i % s_;
    const size_t p = per();
    return p ? i / p : 0;
  }
  size_t local_index(size_t i) const {
    if (kind_ == PARTITION_ROUND_ROBIN) return i / s_;
    const size_t p = per();
    return p ? i % p : 0;
  }
  size_t global_index(size_t shard, size_t local) const {
    ShardRange r = range_of(shard);
    return r.start + local * r.stride;
  }

 private:
  int kind_;
  size_t n_, s_, align_;
};

}  // namespace geeps_b200
