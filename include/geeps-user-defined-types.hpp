#ifndef GEEPS_B200_USER_DEFINED_TYPES_HPP_
#define GEEPS_B200_USER_DEFINED_TYPES_HPP_
// Row layout and scalar types of the parameter server.  A row is 128 fp32 values
// (512 bytes) - the same shape the reference fixes in
// include/geeps-user-defined-types.hpp:41-73 - because every kernel moves one row per warp
// as 32 x 16-byte vectors.
#include <stddef.h>
#include <stdint.h>
#include <string.h>

typedef float val_t;
typedef size_t row_idx_t;
typedef size_t col_idx_t;
typedef size_t table_id_t;
typedef int iter_t;
typedef unsigned int uint;

#define ROW_DATA_SIZE 128

struct ArrayData {
  val_t data[ROW_DATA_SIZE];
  void init() { memset(data, 0, sizeof(data)); }
  ArrayData() { init(); }
  // Flat archive hook (used by the snapshot writer): (de)serialises the 128 values.
  template <class Archive>
  void serialize(Archive& ar, const unsigned int /*version*/) {
    for (int i = 0; i < ROW_DATA_SIZE; ++i) ar & data[i];
  }
};

typedef ArrayData RowData;
typedef ArrayData RowOpVal;

#endif  // GEEPS_B200_USER_DEFINED_TYPES_HPP_
