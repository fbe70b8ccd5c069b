// Backward of the CSR SpMM:  dX[s(e),h,:] += v[e,h] * dY[t(r),h,:]   (divided by the row's
// edge count for mean) and, on request, dV[e,h] = <dY[t(r),h,:], X[s(e),h,:]>.
//
// Replaces gen_bwd_sum / gen_bwd_mean / gen_bwd_sum_edge_value{,_multi_head}{,_edge_grad}
// (src/cpp/src/aggr_kernel.cu:188-491), run_spmm_sharedmem_bwd* (spmm_kernel.cu:799-1046),
// selective_aggr_bwd_kernel / target_aggr_backward (aggr_kernel.cu:523-607) and
// aggr_rel_bwd (src/cpp/src/rel_spmm.cu:72-104).
//
// Like the reference this is a scatter: the gradient row of a destination is held
// in registers and pushed to every source of the row. The push is one 128-bit
// vector reduction (`red.global.add.v4.f32`) per lane instead of four scalar
// atomicAdds, and the work is cut into tiles of consecutive edges rather than rows,
// so a hub row does not serialise on one warp. The order of the additions into dX
// is not fixed (it is not in the reference either), so dX is reproducible only up
// to fp32 rounding; dV has a fixed order.
#include "common.cuh"

namespace cxg {
namespace {

constexpr int kThreads = 256;
constexpr int kSegment = 256;  // edges per work item

struct BwdArgs {
  const void *ptr;
  const void *idx;
  const void *dy;
  const void *x;  // forward input, only for dV
  float *dx;
  float *dval;
  const float *edge_val;
  const uint8_t *edge_mask;
  const int32_t *edge_rel;
  const int64_t *targets;
  int64_t n_dst;
  int64_t rel_stride;
  int width, feat, heads, ptr_bytes, reduce;
};

__device__ __forceinline__ void red_add_v4(float *addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

// One group of G lanes per tile of kSegment consecutive edges, whatever rows they belong to: the
// work is balanced by edges, so a hub row is spread over as many groups as it has tiles. The group
// finds the row of its first edge by binary search in ptr, then walks its edges in CSR order and
// reloads the gradient row whenever the walk enters a new row (the row ends of the next G rows
// are kept one per lane). E = elements per lane and vector (4 for fp32, 8 for bf16 gradients, 1
// for the scalar path).
template <typename VT, typename T, typename IdxT, int G, int VALMODE, bool EDGE_GRAD>
__global__ void __launch_bounds__(kThreads) spmm_bwd_tiles(BwdArgs a) {
  constexpr int E = VT::kElems;
  constexpr int kGroupsPerBlock = kThreads / G;
  const int lane = threadIdx.x & 31;
  const int lg = lane & (G - 1);
  const unsigned gmask = (G == 32) ? 0xffffffffu : (((1u << G) - 1u) << (lane & ~(G - 1)));
  const int nvec = a.width / E;
  const IdxT *idx = reinterpret_cast<const IdxT *>(a.idx);
  const T *dy = reinterpret_cast<const T *>(a.dy);
  const T *x = reinterpret_cast<const T *>(a.x);
  const int64_t e_first = load_ptr(a.ptr, 0, a.ptr_bytes), e_last = load_ptr(a.ptr, a.n_dst, a.ptr_bytes);
  const int64_t tile = static_cast<int64_t>(blockIdx.x) * kGroupsPerBlock + threadIdx.x / G;
  const int64_t sb = e_first + tile * kSegment;
  if (sb >= e_last) return;
  const int64_t se = min(e_last, sb + static_cast<int64_t>(kSegment));
  // row0 = last row whose first edge is <= sb (rows without edges in front of it are skipped)
  int64_t lo = 0, hi = a.n_dst;  // invariant: ptr[lo] <= sb < ptr[hi]
  while (hi - lo > 1) {
    const int64_t mid = (lo + hi) >> 1;
    if (load_ptr(a.ptr, mid, a.ptr_bytes) <= sb)
      lo = mid;
    else
      hi = mid;
  }
  const int64_t row0 = lo;
  const int lanes_per_head = a.feat / E;  // a power of two when dV is asked for

  for (int v0 = 0; v0 < nvec; v0 += G) {
    const int v = v0 + lg;
    const bool on = v < nvec;
    const int col = v * E;
    const int head = on ? col / a.feat : 0;
    // walk state: `row` owns the edges up to row_end; lane l keeps the end of row cache_base + l
    int64_t row = row0, cache_base = row0;
    int64_t my_end = load_ptr(a.ptr, min(cache_base + lg, a.n_dst - 1) + 1, a.ptr_bytes);
    int64_t row_end = __shfl_sync(gmask, my_end, 0, G);
    bool fresh = true;  // the gradient row of `row` is not loaded yet
    float g[E];
    for (int64_t e0 = sb; e0 < se; e0 += G) {
      int64_t my_nid = -1;
      float my_val = 1.f;
      const int64_t e = e0 + lg;
      if (e < se) {
        const bool keep = a.edge_mask == nullptr || a.edge_mask[e] != 0;
        if (keep) {
          my_nid = static_cast<int64_t>(__ldg(idx + e));
          if (a.edge_rel != nullptr) my_nid += static_cast<int64_t>(__ldg(a.edge_rel + e)) * a.rel_stride;
        }
        if (VALMODE == 1) my_val = __ldg(a.edge_val + e);
      }
      const int64_t left = se - e0;
      const int cnt = left < G ? static_cast<int>(left) : G;
      for (int j = 0; j < cnt; ++j) {
        const int64_t ej = e0 + j;
        while (ej >= row_end) {  // uniform over the group
          ++row;
          if (row - cache_base == G) {
            cache_base = row;
            my_end = load_ptr(a.ptr, min(cache_base + lg, a.n_dst - 1) + 1, a.ptr_bytes);
          }
          row_end = __shfl_sync(gmask, my_end, static_cast<int>(row - cache_base), G);
          fresh = true;
        }
        if (fresh) {
          fresh = false;
          const int64_t g_row = a.targets != nullptr ? __ldg(a.targets + row) : row;
#pragma unroll
          for (int i = 0; i < E; ++i) g[i] = 0.f;
          if (on) {
            VT::to_float(g, VT::load(dy + g_row * a.width + col));
            if (a.reduce == CXG_MEAN) {
              const float inv = 1.f / static_cast<float>(row_end - load_ptr(a.ptr, row, a.ptr_bytes));
#pragma unroll
              for (int i = 0; i < E; ++i) g[i] *= inv;
            }
          }
        }
        const int64_t nid = __shfl_sync(gmask, my_nid, j, G);
        float val = 1.f;
        if (VALMODE == 1) val = __shfl_sync(gmask, my_val, j, G);
        if (VALMODE == 2 && on) val = __ldg(a.edge_val + ej * a.heads + head);
        if (nid < 0) continue;
        if (a.dx != nullptr && on) {
          float *dst = a.dx + nid * a.width + col;
          if (E % 4 == 0) {
#pragma unroll
            for (int i = 0; i < E; i += 4)
              red_add_v4(dst + i, g[i] * val, g[(i + 1) % E] * val, g[(i + 2) % E] * val, g[(i + 3) % E] * val);
          } else {
#pragma unroll
            for (int i = 0; i < E; ++i) atomicAdd(dst + i, g[i] * val);
          }
        }
        if (EDGE_GRAD) {
          float dot = 0.f;
          if (on) {
            float xv[E];
            VT::to_float(xv, VT::load(x + nid * a.width + col));
#pragma unroll
            for (int i = 0; i < E; ++i) dot = fmaf(g[i], xv[i], dot);
          }
          // tree over the lanes of one head (xor butterflies stay inside the aligned block of
          // lanes_per_head lanes)
          for (int o = lanes_per_head >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(gmask, dot, o, G);
          if (on && (lg % lanes_per_head) == 0) a.dval[ej * a.heads + head] = dot;  // a head never straddles two passes
        }
      }
    }
  }
}

template <typename VT, typename T, typename IdxT, int G>
void launch_bwd2(const BwdArgs &a, int valmode, bool edge_grad, dim3 grid, cudaStream_t st) {
#define CXG_BWD(VM, EG) spmm_bwd_tiles<VT, T, IdxT, G, VM, EG><<<grid, kThreads, 0, st>>>(a)
  if (!edge_grad) {
    if (valmode == 0)
      CXG_BWD(0, false);
    else if (valmode == 1)
      CXG_BWD(1, false);
    else
      CXG_BWD(2, false);
  } else {
    if (valmode == 0)
      CXG_BWD(0, true);
    else if (valmode == 1)
      CXG_BWD(1, true);
    else
      CXG_BWD(2, true);
  }
#undef CXG_BWD
}

template <typename T, typename IdxT>
int launch_bwd(const BwdArgs &a, int valmode, bool edge_grad, int64_t nnz, cudaStream_t st) {
  constexpr int E = Vec<T>::kElems;
  bool vector_ok = (a.width % E == 0) && (a.feat % E == 0) &&
                   (reinterpret_cast<uintptr_t>(a.dy) % 16 == 0) &&
                   (a.x == nullptr || reinterpret_cast<uintptr_t>(a.x) % 16 == 0) &&
                   (a.dx == nullptr || reinterpret_cast<uintptr_t>(a.dx) % 16 == 0);
  if (edge_grad) {
    // The per-head tree needs a power-of-two number of lanes per head inside one pass.
    int lph = vector_ok ? a.feat / E : a.feat;
    bool pow2 = lph > 0 && (lph & (lph - 1)) == 0;
    if (!pow2 || lph > 32)
      return set_error(CXG_EUNSUPPORTED,
                       "cxg_spmm_csr_backward: edge gradients need feat/%d (=%d) to be a power of "
                       "two <= 32",
                       vector_ok ? E : 1, lph);
  }
  int G = 32;
  if (vector_ok) {
    int nvec = a.width / E;
    if (nvec <= 8)
      G = 8;
    else if (nvec <= 16)
      G = 16;
  }
  // one group per tile of kSegment edges; nnz bounds the edge count (tiles past ptr[n_dst] return)
  const int64_t groups_per_block = kThreads / G;
  const int64_t tiles = (nnz + kSegment - 1) / kSegment;
  dim3 grid(static_cast<unsigned>((tiles + groups_per_block - 1) / groups_per_block));
  if (!vector_ok)
    launch_bwd2<Scalar<T>, T, IdxT, 32>(a, valmode, edge_grad, grid, st);
  else if (G == 8)
    launch_bwd2<Vec<T>, T, IdxT, 8>(a, valmode, edge_grad, grid, st);
  else if (G == 16)
    launch_bwd2<Vec<T>, T, IdxT, 16>(a, valmode, edge_grad, grid, st);
  else
    launch_bwd2<Vec<T>, T, IdxT, 32>(a, valmode, edge_grad, grid, st);
  return CXG_OK;
}

}  // namespace
}  // namespace cxg

using namespace cxg;

extern "C" int cxg_spmm_csr_backward(const cxg_spmm_desc *d, const void *dy, float *dx, float *dval,
                                     void *stream) {
  CXG_REQUIRE(d != nullptr, CXG_ENULL, "cxg_spmm_csr_backward: desc is NULL");
  CXG_REQUIRE(d->n_dst >= 0 && d->nnz >= 0 && d->feat > 0 && d->heads > 0, CXG_EINVAL,
              "cxg_spmm_csr_backward: bad sizes");
  CXG_REQUIRE(d->dtype == CXG_F32 || d->dtype == CXG_BF16, CXG_EINVAL,
              "cxg_spmm_csr_backward: dtype %d", d->dtype);
  CXG_REQUIRE((d->ptr_bytes == 4 || d->ptr_bytes == 8) && (d->idx_bytes == 4 || d->idx_bytes == 8),
              CXG_EINVAL, "cxg_spmm_csr_backward: index widths %d/%d", d->ptr_bytes, d->idx_bytes);
  CXG_REQUIRE(d->reduce == CXG_SUM || d->reduce == CXG_MEAN, CXG_EINVAL,
              "cxg_spmm_csr_backward: reduce %d", d->reduce);
  if (d->n_dst == 0 || d->nnz == 0) return CXG_OK;
  CXG_REQUIRE(d->ptr != nullptr && d->idx != nullptr && dy != nullptr, CXG_ENULL,
              "cxg_spmm_csr_backward: ptr, idx or dy is NULL");
  CXG_REQUIRE(dx != nullptr || dval != nullptr, CXG_ENULL,
              "cxg_spmm_csr_backward: neither dx nor dval requested");
  CXG_REQUIRE(dval == nullptr || d->x != nullptr, CXG_ENULL,
              "cxg_spmm_csr_backward: dval needs the forward input x");
  CXG_REQUIRE(d->edge_rel == nullptr || d->rel_stride > 0, CXG_EINVAL,
              "cxg_spmm_csr_backward: edge_rel needs rel_stride > 0");
  BwdArgs a;
  a.ptr = d->ptr;
  a.idx = d->idx;
  a.dy = dy;
  a.x = d->x;
  a.dx = dx;
  a.dval = dval;
  a.edge_val = d->edge_val;
  a.edge_mask = d->edge_mask;
  a.edge_rel = d->edge_rel;
  a.targets = d->targets;
  a.n_dst = d->n_dst;
  a.rel_stride = d->rel_stride;
  a.feat = d->feat;
  a.heads = d->heads;
  a.width = d->feat * d->heads;
  a.ptr_bytes = d->ptr_bytes;
  a.reduce = d->reduce;
  int valmode = d->edge_val == nullptr ? 0 : (d->heads == 1 ? 1 : 2);
  bool edge_grad = dval != nullptr;
  cudaStream_t st = as_stream(stream);
  int rc;
  if (d->dtype == CXG_F32)
    rc = d->idx_bytes == 8 ? launch_bwd<float, int64_t>(a, valmode, edge_grad, d->nnz, st)
                           : launch_bwd<float, int32_t>(a, valmode, edge_grad, d->nnz, st);
  else
    rc = d->idx_bytes == 8 ? launch_bwd<__nv_bfloat16, int64_t>(a, valmode, edge_grad, d->nnz, st)
                           : launch_bwd<__nv_bfloat16, int32_t>(a, valmode, edge_grad, d->nnz, st);
  if (rc != CXG_OK) return rc;
  count_launches(1);
  return check_launch("cxg_spmm_csr_backward");
}
