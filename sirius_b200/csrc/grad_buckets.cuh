// Gradient buckets for the data-parallel all-reduce overlapped with backward (the c10d Reducer's buckets,
// pytorch/torch_col/csrc/dist_ext.{h,cc}): the flat gradient buffer is cut at unit boundaries (a unit = a block or
// layer of the model, in forward order) into ranges of at least `min_elems`, listed in the order backward completes
// them (last units first). An executor records a bucket's event on its main stream once the last kernel that writes
// into the range has been enqueued there (side-stream work joined before); a communication stream waits for it.
#pragma once
#include <vector>

#include "common.cuh"

namespace srt {

struct GradBuckets {
  struct Bucket { size_t off, count; int first_unit; cudaEvent_t ev; };
  std::vector<Bucket> list;
  int next = 0;  // next bucket to become ready in the current backward pass

  ~GradBuckets() {
    for (auto& b : list) if (b.ev) cudaEventDestroy(b.ev);
  }
  // unit_start[u]: offset of unit u's first gradient (ascending); everything before unit 0 belongs to the last bucket.
  int build(const std::vector<size_t>& unit_start, size_t n_flat, size_t min_elems) {
    for (auto& b : list) if (b.ev) cudaEventDestroy(b.ev);
    list.clear();
    size_t end = n_flat;
    for (int u = (int)unit_start.size() - 1; u > 0; --u) {
      if (end - unit_start[u] >= min_elems) {
        list.push_back({unit_start[u], end - unit_start[u], u, nullptr});
        end = unit_start[u];
      }
    }
    list.push_back({0, end, -1, nullptr});
    for (auto& b : list) SRT_CHECK_CUDA(cudaEventCreateWithFlags(&b.ev, cudaEventDisableTiming));
    return SRT_OK;
  }
  void begin_backward() { next = 0; }
  // Call after unit u's backward is fully enqueued on `st`.
  int unit_done(int u, cudaStream_t st) {
    if (next + 1 < (int)list.size() && list[next].first_unit == u) {
      SRT_CHECK_CUDA(cudaEventRecord(list[next].ev, st));
      ++next;
    }
    return SRT_OK;
  }
  // Call at the very end of backward: the remaining bucket (embeddings, first units) is final.
  int all_done(cudaStream_t st) {
    SRT_CHECK_CUDA(cudaEventRecord(list.back().ev, st));
    next = (int)list.size();
    return SRT_OK;
  }
};

}  // namespace srt
