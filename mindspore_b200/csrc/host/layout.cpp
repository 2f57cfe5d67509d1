// Tensor-layout algebra and redistribution operator inference (host C++).
//
// A layout is (device_matrix, tensor_map, tensor_shape): tensor_map[i] = k shards tensor dim i along the
// device-matrix dim counted from the right (device_matrix[n-1-k]); -1 means the dim is not sharded.
// Redistribution between two layouts over the same device matrix is inferred as a sequence of
//   SplitByAxis   (each rank keeps its chunk: StridedSlice)
//   PermuteByAxis (AlltoAll, or AllGather + Split when all-to-all is disabled)
//   ConcatByAxis  (AllGather along a tensor dim)
// in the greedy order of the reference (ccsrc/frontend/parallel/tensor_layout/redistribution_operator_infer.cc
// :98-231): first every split that needs no communication, then permutes, then concats, repeated until the
// maps agree.  Group membership follows ccsrc/frontend/parallel/device_matrix.cc:58-190.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>

#define MSB_API extern "C" __attribute__((visibility("default")))

namespace {

enum OpType : int32_t { kSplit = 1, kConcat = 2, kPermute = 3 };

struct Op {
  int32_t type, a, b, dev_dim, count;
};

bool dev_dim_used(const std::vector<int>& map, int k) {
  return std::find(map.begin(), map.end(), k) != map.end();
}

}  // namespace

// ops_out: 5 ints per op {type, arg_a, arg_b, dev_dim, split_count}:
//   Split  : a = tensor dim, b = unused
//   Concat : a = tensor dim
//   Permute: a = tensor dim to split (gets dev_dim), b = tensor dim to concat (loses dev_dim)
// Returns the number of ops, -1 if the capacity is too small, -2 on invalid input.
MSB_API int msb_redistribution_infer(const int32_t* dev_matrix, int n_dev, const int32_t* from_map,
                                     const int32_t* to_map, int rank_dims, int enable_alltoall, int32_t* ops_out,
                                     int capacity) {
  if (n_dev <= 0 || rank_dims < 0) return -2;
  std::vector<int> cur(from_map, from_map + rank_dims), dst(to_map, to_map + rank_dims);
  for (int i = 0; i < rank_dims; ++i) {
    if (cur[i] < -1 || cur[i] >= n_dev || dst[i] < -1 || dst[i] >= n_dev) return -2;
  }
  std::vector<Op> ops;
  auto size_of = [&](int k) { return dev_matrix[n_dev - 1 - k]; };
  int guard = 0;
  while (cur != dst && guard++ < 4 * (rank_dims + n_dev) + 8) {
    bool progressed = false;
    // 1. splits that need no data from other ranks: target wants dev dim k on dim i, k currently unused
    for (int i = 0; i < rank_dims; ++i) {
      if (cur[i] == -1 && dst[i] != -1 && !dev_dim_used(cur, dst[i])) {
        ops.push_back({kSplit, i, -1, dst[i], size_of(dst[i])});
        cur[i] = dst[i];
        progressed = true;
      }
    }
    if (cur == dst) break;
    // 2. permutes: dev dim k must move from tensor dim j to tensor dim i
    for (int i = 0; i < rank_dims; ++i) {
      if (cur[i] == -1 && dst[i] != -1) {
        const int k = dst[i];
        int j = -1;
        for (int t = 0; t < rank_dims; ++t)
          if (cur[t] == k) j = t;
        if (j >= 0) {
          if (enable_alltoall) {
            ops.push_back({kPermute, i, j, k, size_of(k)});
          } else {
            ops.push_back({kConcat, j, -1, k, size_of(k)});
            ops.push_back({kSplit, i, -1, k, size_of(k)});
          }
          cur[j] = -1;
          cur[i] = k;
          progressed = true;
        }
      }
    }
    if (cur == dst) break;
    // 3. concats: dim i is sharded on k but the target wants something else there
    for (int i = 0; i < rank_dims; ++i) {
      if (cur[i] != -1 && cur[i] != dst[i]) {
        ops.push_back({kConcat, i, -1, cur[i], size_of(cur[i])});
        cur[i] = -1;
        progressed = true;
      }
    }
    if (!progressed) return -2;
  }
  if (cur != dst) return -2;
  if (static_cast<int>(ops.size()) > capacity) return -1;
  for (size_t t = 0; t < ops.size(); ++t) {
    ops_out[5 * t + 0] = ops[t].type;
    ops_out[5 * t + 1] = ops[t].a;
    ops_out[5 * t + 2] = ops[t].b;
    ops_out[5 * t + 3] = ops[t].dev_dim;
    ops_out[5 * t + 4] = ops[t].count;
  }
  return static_cast<int>(ops.size());
}

// Ranks whose device-matrix coordinates equal `rank`'s except along the listed device dims (indices from the
// right).  Output sorted ascending, offset by base_rank.  Returns the count (or -1 if capacity is too small).
MSB_API int msb_group_ranks(const int32_t* dev_matrix, int n_dev, int rank, const int32_t* dev_dims, int n_dims,
                            int base_rank, int32_t* out, int capacity) {
  std::vector<int> coord(n_dev);
  int r = rank;
  for (int a = n_dev - 1; a >= 0; --a) {
    coord[a] = r % dev_matrix[a];
    r /= dev_matrix[a];
  }
  std::vector<char> free_axis(n_dev, 0);
  for (int t = 0; t < n_dims; ++t) {
    const int a = n_dev - 1 - dev_dims[t];
    if (a < 0 || a >= n_dev) return -2;
    free_axis[a] = 1;
  }
  std::vector<int> result;
  std::vector<int> c(coord);
  // odometer over the free axes
  std::vector<int> axes;
  for (int a = 0; a < n_dev; ++a)
    if (free_axis[a]) axes.push_back(a);
  long long total = 1;
  for (int a : axes) total *= dev_matrix[a];
  for (long long idx = 0; idx < total; ++idx) {
    long long t = idx;
    for (int q = static_cast<int>(axes.size()) - 1; q >= 0; --q) {
      c[axes[q]] = static_cast<int>(t % dev_matrix[axes[q]]);
      t /= dev_matrix[axes[q]];
    }
    int v = 0;
    for (int a = 0; a < n_dev; ++a) v = v * dev_matrix[a] + c[a];
    result.push_back(v + base_rank);
  }
  std::sort(result.begin(), result.end());
  if (static_cast<int>(result.size()) > capacity) return -1;
  std::copy(result.begin(), result.end(), out);
  return static_cast<int>(result.size());
}

// Communication volume (elements moved per rank) of an inferred op list on a tensor of the given per-rank
// slice size; AlltoAll is charged 2x and AllGather/ReduceScatter 0.5x like the reference's cost model
// (tensor_layout/tensor_redistribution.h:32-33).
MSB_API double msb_redistribution_cost(const int32_t* ops, int n_ops, double slice_elems) {
  double cost = 0.0, cur = slice_elems;
  for (int t = 0; t < n_ops; ++t) {
    const int type = ops[5 * t], cnt = ops[5 * t + 4];
    if (type == kSplit) {
      cur /= cnt;
    } else if (type == kConcat) {
      cost += 0.5 * cur * (cnt - 1);
      cur *= cnt;
    } else if (type == kPermute) {
      cost += 2.0 * cur * (cnt - 1) / cnt;
    }
  }
  return cost;
}
