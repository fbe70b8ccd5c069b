// Column sums of a row-major matrix with a fixed order of additions: out[c] = sum_r x[r, c].
//
// This is the gradient of a layer's bias (MyGATConv / MyGCNConv add `bias` to every output row,
// cxgnncomp/graph_conv.py:493-494, 543-545, 622-623; autograd turns that into a sum over the rows of the upstream
// gradient). Two kernels, no atomics: CTA b owns a contiguous chunk of rows and leaves one partial row,
// a second kernel adds the partial rows in CTA order. The result has the same bits on every run.
#include "common.cuh"

namespace cxg {
namespace {

constexpr int kCsThreads = 256;
constexpr int kCsCtas = kNumSM * 8;

template <typename T>
__device__ __forceinline__ float cs_load(const T *p);
template <>
__device__ __forceinline__ float cs_load<float>(const float *p) {
  return __ldg(p);
}
template <>
__device__ __forceinline__ float cs_load<__nv_bfloat16>(const __nv_bfloat16 *p) {
  return __bfloat162float(*p);
}

// Stage 1: thread (sub, col) adds x[r, col] over the chunk's rows r = first + sub + j * nsub in four interleaved
// accumulators (j mod 4) joined as (a0 + a1) + (a2 + a3); the nsub sums of a column are added in sub order.
template <typename T>
__global__ void __launch_bounds__(kCsThreads) column_sum_partial(const T *x, float *part, int64_t n_row, int width) {
  __shared__ float sh[kCsThreads];
  const int nsub = width <= kCsThreads ? kCsThreads / width : 1;
  const int64_t per = (n_row + gridDim.x - 1) / gridDim.x;
  const int64_t first = blockIdx.x * per, last = min(n_row, first + per);
  for (int col0 = 0; col0 < width; col0 += kCsThreads) {
    const int sub = width <= kCsThreads ? threadIdx.x / width : 0;
    const int col = col0 + (width <= kCsThreads ? threadIdx.x % width : threadIdx.x);
    const bool on = col < width && sub < nsub;
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    if (on) {
      int64_t r = first + sub;
      for (; r + 3 * static_cast<int64_t>(nsub) < last; r += 4 * nsub) {
        float f[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) f[u] = cs_load<T>(x + (r + static_cast<int64_t>(u) * nsub) * width + col);
#pragma unroll
        for (int u = 0; u < 4; ++u) a[u] += f[u];
      }
      for (int u = 0; r < last; r += nsub, ++u) a[u] += cs_load<T>(x + r * width + col);
    }
    float s = (a[0] + a[1]) + (a[2] + a[3]);
    sh[threadIdx.x] = s;
    __syncthreads();
    if (on && sub == 0) {
      for (int u = 1; u < nsub; ++u) s += sh[u * width + threadIdx.x];
      part[static_cast<int64_t>(blockIdx.x) * width + col] = s;
    }
    __syncthreads();
  }
}

// Stage 2: one warp per column; lane l adds the partials of CTAs l, l + 32, ... in order, the 32 lane sums are
// joined by a shuffle tree.
__global__ void __launch_bounds__(kCsThreads) column_sum_final(const float *part, float *out, int n_part, int width) {
  const int lane = threadIdx.x & 31;
  const int col = (blockIdx.x * kCsThreads + threadIdx.x) >> 5;
  if (col >= width) return;
  float s = 0.f;
  for (int b = lane; b < n_part; b += 32) s += part[static_cast<int64_t>(b) * width + col];
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) out[col] = s;
}

}  // namespace
}  // namespace cxg

using namespace cxg;

extern "C" int cxg_column_sum_workspace_size(int width, size_t *bytes) {
  CXG_REQUIRE(bytes != nullptr, CXG_ENULL, "cxg_column_sum_workspace_size: bytes is NULL");
  CXG_REQUIRE(width > 0, CXG_EINVAL, "cxg_column_sum_workspace_size: width %d", width);
  *bytes = static_cast<size_t>(kCsCtas) * width * sizeof(float);
  return CXG_OK;
}

extern "C" int cxg_column_sum(const void *x, int dtype, int64_t n_row, int width, float *out, void *workspace,
                              size_t workspace_bytes, void *stream) {
  CXG_REQUIRE(n_row >= 0 && width > 0 && (dtype == CXG_F32 || dtype == CXG_BF16), CXG_EINVAL,
              "cxg_column_sum: bad arguments");
  CXG_REQUIRE(out != nullptr && (n_row == 0 || x != nullptr), CXG_ENULL, "cxg_column_sum: NULL argument");
  size_t need = 0;
  cxg_column_sum_workspace_size(width, &need);
  CXG_REQUIRE(workspace != nullptr && workspace_bytes >= need, CXG_EWORKSPACE,
              "cxg_column_sum: workspace %zu bytes, need %zu", workspace_bytes, need);
  cudaStream_t st = as_stream(stream);
  float *part = static_cast<float *>(workspace);
  // every CTA writes its partial row (zeros when its chunk is empty), so the second stage reads no stale value
  if (dtype == CXG_F32)
    column_sum_partial<float><<<kCsCtas, kCsThreads, 0, st>>>(static_cast<const float *>(x), part, n_row, width);
  else
    column_sum_partial<__nv_bfloat16><<<kCsCtas, kCsThreads, 0, st>>>(static_cast<const __nv_bfloat16 *>(x), part,
                                                                      n_row, width);
  column_sum_final<<<(width * 32 + kCsThreads - 1) / kCsThreads, kCsThreads, 0, st>>>(part, out, kCsCtas, width);
  count_launches(2);
  return check_launch("cxg_column_sum");
}
