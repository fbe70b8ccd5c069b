// Relational (RGCN) helpers for sm_100a that do not need the tensor cores:
//   * pad_rel / pad_rel_idx   relation-bucket padding      (src/cpp/src/stitch_kernel.cu:3-53)
//   * typed linear, exact fp32, one warp per row           (src/cpp/src/rel_spmm.cu:231-358:
//     typed_linear_kernel, _s2e, _s2d), also the exact-fp32 mode of the typed matmul
//   * aggr_rgcn_direct: y[d] = sum_e x[idx[e]] . W[rel[e]]  (rel_spmm.cu:138-181,442-467)
//   * rel_schedule on the host                              (src/cpp/src/schedule.cu:5-63)
#include <vector>

#include "common.cuh"

namespace cxg {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__global__ void pad_rel_kernel(int64_t *rel, int64_t *idx, const int64_t *count, int thres, int num_rel, int64_t base) {
  const int tid = blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= num_rel * (thres - 1)) return;
  const int which = tid / (thres - 1);
  const int mod = static_cast<int>(count[which] % thres);
  const int64_t pos = base + tid;
  // slot of relation `which` becomes a member of it while the bucket is short of a multiple of thres
  rel[pos] = ((tid % (thres - 1)) < (thres - mod) && mod != 0) ? which : num_rel;
  if (idx != nullptr) idx[pos] = -1;
}

// One warp per position m: out[oc(m), :] (+)= a[ia(m), :] . W[rel(m)]  with fp32 fma in k order.
// RelT is int32 (typed_linear* of the reference) or int64 (typed matmul); rows whose relation
// lies outside [0, num_rel) or whose source index lies outside [0, m_valid) are padding.
// MODE 0: store, 1: add to what is there, 2: atomic add (rows may repeat).
template <typename T, typename RelT, int MODE>
__global__ void __launch_bounds__(kThreads) typed_linear_rows(const T *a, const T *w, T *out, const RelT *rel,
                                                              const int64_t *src, const int64_t *dst, int64_t m,
                                                              int64_t m_valid, int k, int n, int num_rel,
                                                              int out_follows_src) {
  extern __shared__ float sh[];  // one row of a per warp
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t pos = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  if (pos >= m) return;
  const int64_t r = static_cast<int64_t>(rel[pos]);
  if (r < 0 || r >= num_rel) return;
  const int64_t ia = src != nullptr ? src[pos] : pos;
  if (ia < 0 || ia >= m_valid) return;
  const int64_t oc = dst != nullptr ? dst[pos] : (out_follows_src ? ia : pos);
  float *row = sh + warp * k;
  for (int i = lane; i < k; i += 32) row[i] = to_f32(a[ia * k + i]);
  __syncwarp();
  const T *wr = w + r * static_cast<int64_t>(k) * n;
  for (int j = lane; j < n; j += 32) {
    float acc = 0.f;
    for (int kk = 0; kk < k; ++kk) acc = fmaf(row[kk], to_f32(wr[static_cast<int64_t>(kk) * n + j]), acc);
    T *o = out + oc * n + j;
    if (MODE == 0)
      *o = from_f32<T>(acc);
    else if (MODE == 1)
      *o = from_f32<T>(to_f32(*o) + acc);
    else
      atomicAdd(reinterpret_cast<float *>(o), acc);  // fp32 only (checked on the host)
  }
}

// y[d, :] = sum over row d of x[idx[e], :] . W[rel[e]]; one warp per destination, lane j owns
// output columns j, j+32, ... (up to 4 of them).
template <typename IdxT>
__global__ void __launch_bounds__(kThreads) rgcn_direct_rows(const void *ptr, int ptr_bytes, const IdxT *idx,
                                                             const int32_t *rel, const float *x, const float *w,
                                                             float *y, int64_t n_dst, int k, int n) {
  extern __shared__ float sh[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t d = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  if (d >= n_dst) return;
  float *row = sh + warp * k;
  const int64_t b = load_ptr(ptr, d, ptr_bytes), e = load_ptr(ptr, d + 1, ptr_bytes);
  for (int j0 = 0; j0 < n; j0 += 128) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int64_t i = b; i < e; ++i) {
      const int64_t s = static_cast<int64_t>(idx[i]);
      const float *wr = w + static_cast<int64_t>(rel[i]) * k * n;
      __syncwarp();
      for (int c = lane; c < k; c += 32) row[c] = __ldg(x + s * k + c);
      __syncwarp();
      for (int kk = 0; kk < k; ++kk) {
        const float xv = row[kk];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int j = j0 + lane + 32 * q;
          if (j < n) acc[q] = fmaf(xv, __ldg(wr + static_cast<int64_t>(kk) * n + j), acc[q]);
        }
      }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int j = j0 + lane + 32 * q;
      if (j < n) y[d * n + j] = acc[q];
    }
  }
}

template <typename T, typename RelT>
void launch_typed_rows(int mode, unsigned grid, size_t smem, cudaStream_t st, const T *a, const T *w, T *out,
                       const RelT *rel, const int64_t *src, const int64_t *dst, int64_t m, int64_t m_valid, int k, int n,
                       int num_rel, int follows) {
  if (mode == 0)
    typed_linear_rows<T, RelT, 0><<<grid, kThreads, smem, st>>>(a, w, out, rel, src, dst, m, m_valid, k, n, num_rel, follows);
  else if (mode == 1)
    typed_linear_rows<T, RelT, 1><<<grid, kThreads, smem, st>>>(a, w, out, rel, src, dst, m, m_valid, k, n, num_rel, follows);
  else
    typed_linear_rows<T, RelT, 2><<<grid, kThreads, smem, st>>>(a, w, out, rel, src, dst, m, m_valid, k, n, num_rel, follows);
}

}  // namespace

// Exact-fp32 typed matmul rows, shared with typed_mm.cu.
int typed_rows_launch(const void *a, const void *w, void *out, const void *rel, int rel_bytes, const int64_t *src,
                      const int64_t *dst, int64_t m, int64_t m_valid, int k, int n, int num_rel, int dtype, int mode,
                      int out_follows_src, cudaStream_t st) {
  const size_t smem = static_cast<size_t>(kWarps) * k * sizeof(float);
  if (smem > 48 * 1024) return set_error(CXG_ELIMIT, "typed linear: K = %d too wide for the per-warp row buffer", k);
  if (mode == 2 && dtype != CXG_F32) return set_error(CXG_EUNSUPPORTED, "typed linear: atomic output needs fp32");
  const unsigned grid = static_cast<unsigned>((m + kWarps - 1) / kWarps);
  if (dtype == CXG_F32) {
    auto A = static_cast<const float *>(a), W = static_cast<const float *>(w);
    auto O = static_cast<float *>(out);
    if (rel_bytes == 4)
      launch_typed_rows<float, int32_t>(mode, grid, smem, st, A, W, O, static_cast<const int32_t *>(rel), src, dst, m,
                                        m_valid, k, n, num_rel, out_follows_src);
    else
      launch_typed_rows<float, int64_t>(mode, grid, smem, st, A, W, O, static_cast<const int64_t *>(rel), src, dst, m,
                                        m_valid, k, n, num_rel, out_follows_src);
  } else {
    auto A = static_cast<const __nv_bfloat16 *>(a), W = static_cast<const __nv_bfloat16 *>(w);
    auto O = static_cast<__nv_bfloat16 *>(out);
    if (rel_bytes == 4)
      launch_typed_rows<__nv_bfloat16, int32_t>(mode, grid, smem, st, A, W, O, static_cast<const int32_t *>(rel), src,
                                                dst, m, m_valid, k, n, num_rel, out_follows_src);
    else
      launch_typed_rows<__nv_bfloat16, int64_t>(mode, grid, smem, st, A, W, O, static_cast<const int64_t *>(rel), src,
                                                dst, m, m_valid, k, n, num_rel, out_follows_src);
  }
  count_launches(1);
  return check_launch("typed linear rows");
}

}  // namespace cxg

using namespace cxg;

extern "C" int cxg_pad_rel(int64_t *rel, int64_t *idx, const int64_t *count, int thres, int num_rel, int64_t base,
                           void *stream) {
  CXG_REQUIRE(thres > 1 && num_rel > 0 && base >= 0, CXG_EINVAL, "cxg_pad_rel: thres=%d num_rel=%d", thres, num_rel);
  CXG_REQUIRE(rel != nullptr && count != nullptr, CXG_ENULL, "cxg_pad_rel: NULL argument");
  const int n = num_rel * (thres - 1);
  pad_rel_kernel<<<(n + 63) / 64, 64, 0, as_stream(stream)>>>(rel, idx, count, thres, num_rel, base);
  count_launches(1);
  return check_launch("cxg_pad_rel");
}

extern "C" int cxg_typed_linear(const float *x, const float *w, float *out, const int32_t *types, const int64_t *src,
                                const int64_t *dst, int64_t num, int64_t n_rows_x, int k, int n, int num_rel,
                                void *stream) {
  CXG_REQUIRE(num >= 0 && k > 0 && n > 0 && num_rel > 0, CXG_EINVAL, "cxg_typed_linear: bad sizes");
  if (num == 0) return CXG_OK;
  CXG_REQUIRE(x && w && out && types, CXG_ENULL, "cxg_typed_linear: NULL argument");
  CXG_REQUIRE(dst == nullptr || src != nullptr, CXG_EINVAL, "cxg_typed_linear: dst needs src");
  // out += for typed_linear / _s2e (one writer per row), atomic for _s2d (rows repeat)
  return typed_rows_launch(x, w, out, types, 4, src, dst, num, n_rows_x, k, n, num_rel, CXG_F32, dst ? 2 : 1, 0,
                           as_stream(stream));
}

extern "C" int cxg_rgcn_direct(const void *ptr, const void *idx, int ptr_bytes, int idx_bytes, const int32_t *rel,
                               const float *x, const float *w, float *y, int64_t n_dst, int k, int n, void *stream) {
  CXG_REQUIRE(n_dst >= 0 && k > 0 && n > 0, CXG_EINVAL, "cxg_rgcn_direct: bad sizes");
  CXG_REQUIRE((ptr_bytes == 4 || ptr_bytes == 8) && (idx_bytes == 4 || idx_bytes == 8), CXG_EINVAL,
              "cxg_rgcn_direct: index widths");
  if (n_dst == 0) return CXG_OK;
  CXG_REQUIRE(ptr && x && w && y, CXG_ENULL, "cxg_rgcn_direct: NULL argument");
  const size_t smem = static_cast<size_t>(kWarps) * k * sizeof(float);
  CXG_REQUIRE(smem <= 48 * 1024, CXG_ELIMIT, "cxg_rgcn_direct: K = %d too wide", k);
  const unsigned grid = static_cast<unsigned>((n_dst + kWarps - 1) / kWarps);
  cudaStream_t st = as_stream(stream);
  if (idx_bytes == 8)
    rgcn_direct_rows<int64_t><<<grid, kThreads, smem, st>>>(ptr, ptr_bytes, static_cast<const int64_t *>(idx), rel, x, w,
                                                            y, n_dst, k, n);
  else
    rgcn_direct_rows<int32_t><<<grid, kThreads, smem, st>>>(ptr, ptr_bytes, static_cast<const int32_t *>(idx), rel, x, w,
                                                            y, n_dst, k, n);
  count_launches(1);
  return check_launch("cxg_rgcn_direct");
}

// Host-side: per-relation sub-graphs. For relation r the rows that own at least one edge of r,
// their edges in CSR order and the row ids; n_in_layer[r * num_layer + l] = kept rows among the
// first num_node_in_layer[l] rows. Outputs are caller-allocated: sub_ptr [num_rel][n_dst + 1],
// sub_idx [num_rel][nnz], sub_target [num_rel][n_dst] (row-major), counts[num_rel][2] =
// (rows kept, edges kept). All pointers are HOST pointers.
extern "C" int cxg_rel_schedule_host(const int64_t *ptr_host, const int64_t *idx_host, const int32_t *rel_host,
                                     int64_t n_dst, const int64_t *num_node_in_layer_host, int num_layer, int num_rel,
                                     int64_t *sub_ptr_host, int64_t *sub_idx_host, int64_t *sub_target_host,
                                     int64_t *counts_host, int64_t *n_in_layer_host) {
  CXG_REQUIRE(n_dst >= 0 && num_rel > 0 && num_layer >= 0, CXG_EINVAL, "cxg_rel_schedule_host: bad sizes");
  CXG_REQUIRE(ptr_host && (idx_host || ptr_host[n_dst] == 0) && sub_ptr_host && sub_idx_host && sub_target_host &&
                  counts_host,
              CXG_ENULL, "cxg_rel_schedule_host: NULL argument");
  const int64_t nnz = ptr_host[n_dst];
  for (int r = 0; r < num_rel; ++r) {
    int64_t *sp = sub_ptr_host + static_cast<int64_t>(r) * (n_dst + 1);
    int64_t *si = sub_idx_host + static_cast<int64_t>(r) * nnz;
    int64_t *stg = sub_target_host + static_cast<int64_t>(r) * n_dst;
    int64_t rows = 0, edges = 0;
    int layer = 0;
    sp[0] = 0;
    for (int64_t i = 0; i < n_dst; ++i) {
      const int64_t before = edges;
      for (int64_t j = ptr_host[i]; j < ptr_host[i + 1]; ++j)
        if (rel_host[j] == r) si[edges++] = idx_host[j];
      if (edges > before) {
        stg[rows] = i;
        sp[++rows] = edges;
      }
      while (layer < num_layer && i == num_node_in_layer_host[layer] - 1) {
        n_in_layer_host[static_cast<int64_t>(r) * num_layer + layer] = rows;
        ++layer;
      }
    }
    counts_host[2 * r] = rows;
    counts_host[2 * r + 1] = edges;
  }
  return CXG_OK;
}

// topo_sort (src/cpp/src/schedule.cu:72-124) on host arrays: a breadth-first release of the nodes whose
// remaining in-degree is 0. When nothing is releasable and nodes remain, one pass over the nodes
// releases every node of remaining degree 1 and, if any node has a larger degree, the first node of
// the smallest such degree, which is how the reference walks through cycles. `order` receives the
// nodes in release order; *n_order the number released (n_node unless the walk got stuck).
extern "C" int cxg_topo_sort_host(const int64_t *ptr_host, const int64_t *idx_host, const int64_t *degree_host,
                                  int64_t n_node, int64_t *order_host, int64_t *n_order) {
  CXG_REQUIRE(n_node >= 0, CXG_EINVAL, "cxg_topo_sort_host: bad size");
  CXG_REQUIRE(n_order != nullptr, CXG_ENULL, "cxg_topo_sort_host: n_order is NULL");
  *n_order = 0;
  if (n_node == 0) return CXG_OK;
  CXG_REQUIRE(ptr_host && idx_host && degree_host && order_host, CXG_ENULL, "cxg_topo_sort_host: NULL argument");
  std::vector<int64_t> left(degree_host, degree_host + n_node);
  std::vector<int64_t> ready;  // FIFO: `head` is the next node to release
  ready.reserve(static_cast<size_t>(n_node));
  size_t head = 0;
  for (int64_t v = 0; v < n_node; ++v)
    if (left[v] == 0) ready.push_back(v);
  int64_t done = 0;
  while (done < n_node) {
    for (; head < ready.size() && done < n_node; ++head) {
      const int64_t v = ready[head];
      order_host[done++] = v;
      for (int64_t e = ptr_host[v]; e < ptr_host[v + 1]; ++e)
        if (--left[idx_host[e]] == 0) ready.push_back(idx_host[e]);
    }
    if (done >= n_node) break;
    int64_t best = n_node, pick = -1;
    for (int64_t v = 0; v < n_node; ++v) {
      if (left[v] > 1 && left[v] < best) {
        best = left[v];
        pick = v;
      } else if (left[v] == 1) {
        left[v] = 0;
        ready.push_back(v);
      }
    }
    if (pick >= 0) {
      left[pick] = 0;
      ready.push_back(pick);
    } else if (head == ready.size()) {
      break;
    }
  }
  *n_order = done;
  return CXG_OK;
}
