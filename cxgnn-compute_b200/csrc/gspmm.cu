// Generalised SpMM of the dgSPARSE surface (GSpMM_u / GSpMM_u_e, src/cpp/include/dgsparse.h:14-131,
// src/cpp/src/dgsparse.cu:324-475):
//   y[r, c] = REDUCE over the edges e of row r of COMPUTE(val[e], x[idx[e], c])
// REDUCE in {sum, max, min, mean}, COMPUTE in {add: v + x, sub: x - v, mul: v * x, div: x / v}; without
// edge values the operand is x itself. The accumulator starts at 0 / INT_MIN / INT_MAX (as floats, like
// the reference's init()), rows without edges give 0, and mean divides the sum by the edge count.
// Edges are reduced in CSR order with one accumulator per column, so the result is reproducible.
//
// One group of G lanes owns a row (G = smallest power of two that covers feat / 4 vectors, at most 32),
// each lane keeps 4 columns per 128-column panel in registers and loads x as 16-byte vectors when
// feat % 4 == 0 (scalar loads otherwise); the edge loop is unrolled by 4 so that four neighbour rows are
// in flight per lane.
#include <limits.h>

#include "common.cuh"

namespace cxg {
namespace {

constexpr int kThreads = 256;

struct GArgs {
  const void *ptr;
  const void *idx;
  const float *val;
  const float *x;
  float *y;
  int64_t n_dst;
  int feat;
  int ptr_bytes;
};

template <int COP>
__device__ __forceinline__ float compute(float v, float x) {
  if (COP == CXG_COP_ADD) return __fadd_rn(v, x);
  if (COP == CXG_COP_SUB) return __fsub_rn(x, v);
  if (COP == CXG_COP_MUL) return __fmul_rn(v, x);
  return __fdiv_rn(x, v);
}

template <int ROP>
__device__ __forceinline__ float reduce(float acc, float t) {
  if (ROP == CXG_ROP_MAX) return acc < t ? t : acc;
  if (ROP == CXG_ROP_MIN) return acc < t ? acc : t;
  return __fadd_rn(acc, t);
}

// sum / mean of products contract to one fused multiply-add, as nvcc compiles the reference's acc + v * x
template <int ROP, int COP, bool HASVAL>
__device__ __forceinline__ float step(float acc, float v, float x) {
  if (!HASVAL) return reduce<ROP>(acc, x);
  if ((ROP == CXG_ROP_SUM || ROP == CXG_ROP_MEAN) && COP == CXG_COP_MUL) return fmaf(v, x, acc);
  return reduce<ROP>(acc, compute<COP>(v, x));
}

template <int ROP>
__device__ __forceinline__ float initial() {
  if (ROP == CXG_ROP_MAX) return static_cast<float>(INT_MIN);
  if (ROP == CXG_ROP_MIN) return static_cast<float>(INT_MAX);
  return 0.f;
}

// VEC: 4 consecutive columns per lane and step (16-byte loads); otherwise one column per lane and step.
template <typename IdxT, int ROP, int COP, bool HASVAL, bool VEC>
__global__ void __launch_bounds__(kThreads) gspmm_rows(GArgs a, int group) {
  const int lane_in_group = threadIdx.x % group;
  const int64_t row = (blockIdx.x * static_cast<int64_t>(kThreads) + threadIdx.x) / group;
  if (row >= a.n_dst) return;
  const int64_t lo = load_ptr(a.ptr, row, a.ptr_bytes), hi = load_ptr(a.ptr, row + 1, a.ptr_bytes);
  const IdxT *idx = static_cast<const IdxT *>(a.idx);
  constexpr int W = VEC ? 4 : 1;
  for (int c0 = lane_in_group * W; c0 < a.feat; c0 += group * W) {
    float acc[W];
#pragma unroll
    for (int j = 0; j < W; ++j) acc[j] = hi > lo ? initial<ROP>() : 0.f;
    int64_t e = lo;
    for (; e + 4 <= hi; e += 4) {
      float xv[4][W], v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float *p = a.x + static_cast<int64_t>(__ldg(idx + e + u)) * a.feat + c0;
        v[u] = HASVAL ? __ldg(a.val + e + u) : 0.f;
        if (VEC) {
          const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
          xv[u][0] = t.x, xv[u][W > 1 ? 1 : 0] = t.y, xv[u][W > 2 ? 2 : 0] = t.z, xv[u][W > 3 ? 3 : 0] = t.w;
        } else {
          xv[u][0] = __ldg(p);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < W; ++j) acc[j] = step<ROP, COP, HASVAL>(acc[j], v[u], xv[u][j]);
    }
    for (; e < hi; ++e) {
      const float *p = a.x + static_cast<int64_t>(__ldg(idx + e)) * a.feat + c0;
      const float v = HASVAL ? __ldg(a.val + e) : 0.f;
#pragma unroll
      for (int j = 0; j < W; ++j) {
        const float xj = __ldg(p + j);
        acc[j] = step<ROP, COP, HASVAL>(acc[j], v, xj);
      }
    }
    if (ROP == CXG_ROP_MEAN && hi > lo) {
      const float d = static_cast<float>(hi - lo);
#pragma unroll
      for (int j = 0; j < W; ++j) acc[j] = __fdiv_rn(acc[j], d);
    }
    float *o = a.y + row * a.feat + c0;
    if (VEC)
      *reinterpret_cast<float4 *>(o) = make_float4(acc[0], acc[W > 1 ? 1 : 0], acc[W > 2 ? 2 : 0], acc[W > 3 ? 3 : 0]);
    else
      o[0] = acc[0];
  }
}

template <typename IdxT, int ROP, int COP, bool HASVAL>
void launch_vec(const GArgs &a, cudaStream_t st) {
  const bool vec = a.feat % 4 == 0 && reinterpret_cast<uintptr_t>(a.x) % 16 == 0 && reinterpret_cast<uintptr_t>(a.y) % 16 == 0;
  const int per_row = vec ? a.feat / 4 : a.feat;
  int group = 1;
  while (group < per_row && group < 32) group <<= 1;
  const int rows_per_block = kThreads / group;
  const unsigned grid = static_cast<unsigned>((a.n_dst + rows_per_block - 1) / rows_per_block);
  if (vec)
    gspmm_rows<IdxT, ROP, COP, HASVAL, true><<<grid, kThreads, 0, st>>>(a, group);
  else
    gspmm_rows<IdxT, ROP, COP, HASVAL, false><<<grid, kThreads, 0, st>>>(a, group);
}

template <typename IdxT, int ROP>
void launch_cop(const GArgs &a, int cop, cudaStream_t st) {
  if (a.val == nullptr) return launch_vec<IdxT, ROP, CXG_COP_MUL, false>(a, st);
  switch (cop) {
    case CXG_COP_ADD: return launch_vec<IdxT, ROP, CXG_COP_ADD, true>(a, st);
    case CXG_COP_SUB: return launch_vec<IdxT, ROP, CXG_COP_SUB, true>(a, st);
    case CXG_COP_MUL: return launch_vec<IdxT, ROP, CXG_COP_MUL, true>(a, st);
    default: return launch_vec<IdxT, ROP, CXG_COP_DIV, true>(a, st);
  }
}

template <typename IdxT>
void launch_rop(const GArgs &a, int rop, int cop, cudaStream_t st) {
  switch (rop) {
    case CXG_ROP_SUM: return launch_cop<IdxT, CXG_ROP_SUM>(a, cop, st);
    case CXG_ROP_MAX: return launch_cop<IdxT, CXG_ROP_MAX>(a, cop, st);
    case CXG_ROP_MIN: return launch_cop<IdxT, CXG_ROP_MIN>(a, cop, st);
    default: return launch_cop<IdxT, CXG_ROP_MEAN>(a, cop, st);
  }
}

}  // namespace
}  // namespace cxg

using namespace cxg;

extern "C" int cxg_gspmm_csr(const void *ptr, const void *idx, int ptr_bytes, int idx_bytes, const float *val, const float *x,
                             float *y, int64_t n_dst, int feat, int reduce_op, int compute_op, void *stream) {
  CXG_REQUIRE(n_dst >= 0 && feat > 0, CXG_EINVAL, "cxg_gspmm_csr: bad sizes");
  CXG_REQUIRE((ptr_bytes == 4 || ptr_bytes == 8) && (idx_bytes == 4 || idx_bytes == 8), CXG_EINVAL,
              "cxg_gspmm_csr: index widths must be 4 or 8");
  CXG_REQUIRE(reduce_op >= CXG_ROP_SUM && reduce_op <= CXG_ROP_MEAN, CXG_EINVAL, "cxg_gspmm_csr: reduce_op %d", reduce_op);
  CXG_REQUIRE(val == nullptr || (compute_op >= CXG_COP_ADD && compute_op <= CXG_COP_DIV), CXG_EINVAL,
              "cxg_gspmm_csr: compute_op %d", compute_op);
  if (n_dst == 0) return CXG_OK;
  CXG_REQUIRE(ptr && idx && x && y, CXG_ENULL, "cxg_gspmm_csr: NULL argument");
  GArgs a;
  a.ptr = ptr, a.idx = idx, a.val = val, a.x = x, a.y = y, a.n_dst = n_dst, a.feat = feat, a.ptr_bytes = ptr_bytes;
  cudaStream_t st = as_stream(stream);
  if (idx_bytes == 8)
    launch_rop<int64_t>(a, reduce_op, compute_op, st);
  else
    launch_rop<int32_t>(a, reduce_op, compute_op, st);
  count_launches(1);
  return check_launch("cxg_gspmm_csr");
}
