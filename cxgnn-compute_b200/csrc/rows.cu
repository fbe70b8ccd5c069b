// out[i, :] = in[rows[i], :] for rows of `row_bytes` bytes: the pack step of the needed-rows feature
// exchange between GPUs (the reference's "densify" step gathers the rows a peer asked for before sending
// them, test/1-kernels/test_mgpu_model.py:227-331). A group of lanes copies one row with 16-byte accesses
// (4- or 2-byte accesses when the row size or the pointers do not allow 16), rows are dealt to groups
// grid-stride. Pure HBM copy: algorithmic bytes = 2 * n_rows * row_bytes + 8 * n_rows.
#include "common.cuh"

namespace cxg {
namespace {

constexpr int kThreads = 256;

template <typename V>
__global__ void __launch_bounds__(kThreads) gather_rows_kernel(const V *in, const int64_t *rows, V *out, int64_t n_rows,
                                                               int vecs_per_row, int group) {
  const int lane = threadIdx.x % group;
  const int64_t groups = static_cast<int64_t>(gridDim.x) * (kThreads / group);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(kThreads / group) + threadIdx.x / group; i < n_rows; i += groups) {
    const V *src = in + __ldg(rows + i) * vecs_per_row;
    V *dst = out + i * vecs_per_row;
    for (int c = lane; c < vecs_per_row; c += group) dst[c] = __ldg(src + c);
  }
}

template <typename V>
void launch(const void *in, const int64_t *rows, void *out, int64_t n_rows, int64_t row_bytes, cudaStream_t st) {
  const int vecs = static_cast<int>(row_bytes / sizeof(V));
  int group = 1;
  while (group < vecs && group < 32) group <<= 1;
  const int64_t want = (n_rows + kThreads / group - 1) / (kThreads / group);
  const unsigned grid = static_cast<unsigned>(want < kNumSM * 16 ? want : kNumSM * 16);
  gather_rows_kernel<V><<<grid, kThreads, 0, st>>>(static_cast<const V *>(in), rows, static_cast<V *>(out), n_rows, vecs,
                                                   group);
}

}  // namespace
}  // namespace cxg

using namespace cxg;

extern "C" int cxg_gather_rows(const void *in, const int64_t *rows, void *out, int64_t n_rows, int64_t row_bytes,
                               void *stream) {
  CXG_REQUIRE(n_rows >= 0 && row_bytes > 0 && row_bytes % 2 == 0 && row_bytes <= (1 << 20), CXG_EINVAL,
              "cxg_gather_rows: bad sizes (row_bytes must be even)");
  if (n_rows == 0) return CXG_OK;
  CXG_REQUIRE(in && rows && out, CXG_ENULL, "cxg_gather_rows: NULL argument");
  cudaStream_t st = as_stream(stream);
  const uintptr_t both = reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) | static_cast<uintptr_t>(row_bytes);
  if (both % 16 == 0)
    launch<uint4>(in, rows, out, n_rows, row_bytes, st);
  else if (both % 4 == 0)
    launch<uint32_t>(in, rows, out, n_rows, row_bytes, st);
  else
    launch<uint16_t>(in, rows, out, n_rows, row_bytes, st);
  count_launches(1);
  return check_launch("cxg_gather_rows");
}
