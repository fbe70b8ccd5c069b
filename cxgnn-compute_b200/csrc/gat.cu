// Attention-side kernels of the GAT path for sm_100a: edge softmax forward / backward,
// SDDMM on an edge list, and the small per-edge helpers that travel with them.
//
// Replaces edge_softmax_fwd / edge_softmax_bwd (src/cpp/src/edge_softmax.cu:3-95),
// sddmm_multihead (src/cpp/src/sddmm_kernel.cu:3-25), gen_edge_value_degree and spmv_csr
// (edge_softmax.cu:186-232), gather_fwd / gather_bwd (src/cpp/src/aggr.cu:42-62).
//
// Edge softmax. The reference runs one warp per (destination, head) and walks the row three
// times with 4-byte accesses strided by the head count. Here one warp owns a destination and
// carries up to four heads at once, so the source id of an edge is read once per pass and the
// per-head scores of a source are one 16-byte sector. The arithmetic per (destination, head)
// keeps the reference's order: lane l takes edges l, l+32, ...; the row maximum starts at
// -100000; the row sum adds the lanes' partial sums with the shuffle-down tree 16, 8, 4, 2, 1;
// the quotient is an exact fp32 division. Rows with more than kHeavyRow edges are handed to a
// second kernel that puts a thread-block cluster of 8 CTAs on each of them (their sums join warps through
// shared memory and CTAs through distributed shared memory, in a fixed order).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace cxg {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kHeavyRow = 1024;      // rows above this many edges get a whole CTA
constexpr int kHeavyThreads = 1024;  // threads of that CTA
constexpr int kHeavyWarps = kHeavyThreads / 32;
constexpr int kHeavyCluster = 8;     // CTAs (one thread-block cluster) that share such a row
constexpr int kHC = 4;  // heads carried together

struct SoftmaxArgs {
  const void *ptr;
  const void *idx;
  const float *att_dst;
  const float *att_src;
  const float *grad;     // backward: d(out)
  float *out;            // forward: written; backward: read
  uint8_t *mask;         // forward: written; backward: read
  float *grad_dst;
  float *grad_src;
  int64_t n_dst;
  int heads, ptr_bytes;
  float slope;
  int32_t *hdr;          // [0] number of heavy rows
  int64_t *heavy;        // heavy row ids
  int max_heavy;
};

__device__ __forceinline__ float warp_tree_sum(float v) {
  // lane 0 ends with ((v0+v16)+(v8+v24))+..., the reference's shfl_down order
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
  return __shfl_sync(0xffffffffu, v, 0);
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum / max over all threads of a cluster (kHeavyCluster CTAs of kHeavyThreads threads) of kHC values per
// thread at once; every thread receives the results. Warps are joined through shared memory, CTAs through
// distributed shared memory, both in a fixed order. sh: [kHeavyWarps][kHC] floats, cl: [kHC] floats.
template <bool MAX>
__device__ __forceinline__ void cluster_reduce(float (&v)[4], float *sh, float *cl) {
  static_assert(kHC == 4, "reductions carry four heads");
#pragma unroll
  for (int k = 0; k < kHC; ++k)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float t = __shfl_xor_sync(0xffffffffu, v[k], o);
      v[k] = MAX ? fmaxf(v[k], t) : v[k] + t;
    }
  __syncthreads();
  if ((threadIdx.x & 31) == 0)
#pragma unroll
    for (int k = 0; k < kHC; ++k) sh[(threadIdx.x >> 5) * kHC + k] = v[k];
  __syncthreads();
  if (threadIdx.x < kHC) {
    float r = sh[threadIdx.x];
    for (int w = 1; w < kHeavyWarps; ++w) r = MAX ? fmaxf(r, sh[w * kHC + threadIdx.x]) : r + sh[w * kHC + threadIdx.x];
    cl[threadIdx.x] = r;
  }
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();
#pragma unroll
  for (int k = 0; k < kHC; ++k) {
    float r = cluster.map_shared_rank(cl, 0)[k];
    for (int c = 1; c < kHeavyCluster; ++c) {
      const float t = cluster.map_shared_rank(cl, c)[k];
      r = MAX ? fmaxf(r, t) : r + t;
    }
    v[k] = r;
  }
  cluster.sync();  // nobody overwrites cl while a peer still reads it
}

// Forward for one row; the STEP threads that share the row take edges first+k*STEP.
// HEAVY = false: one warp, reference summation order. HEAVY = true: one CTA.
template <typename IdxT, bool HEAVY>
__device__ __forceinline__ void softmax_fwd_row(const SoftmaxArgs &a, int64_t d, int first, float *sh, float *cl) {
  constexpr int STEP = HEAVY ? kHeavyThreads * kHeavyCluster : 32;
  const IdxT *idx = reinterpret_cast<const IdxT *>(a.idx);
  const int H = a.heads;
  const int64_t b = load_ptr(a.ptr, d, a.ptr_bytes), e = load_ptr(a.ptr, d + 1, a.ptr_bytes);
  if (!HEAVY && e - b <= 32) {
    // at most one edge per lane: the three passes collapse into one, every value stays in registers and is
    // written once (same operations in the same order as below, so the same bits)
    const int64_t i = b + first;
    const bool has = i < e;
    const int64_t s = has ? static_cast<int64_t>(__ldg(idx + i)) : 0;
    for (int h0 = 0; h0 < H; h0 += kHC) {
      float t[kHC], mx[kHC], p[kHC], sum[kHC];
#pragma unroll
      for (int k = 0; k < kHC; ++k) {
        t[k] = 0.f;
        mx[k] = -100000.f;
        if (has && h0 + k < H) {
          t[k] = __ldg(a.att_dst + d * H + h0 + k) + __ldg(a.att_src + s * H + h0 + k);
          t[k] = fmaxf(t[k], t[k] * a.slope);
          mx[k] = fmaxf(mx[k], t[k]);
        }
        mx[k] = warp_max(mx[k]);
        p[k] = has && h0 + k < H ? expf(t[k] - mx[k]) : 0.f;
        sum[k] = warp_tree_sum(p[k]);
      }
      if (has)
#pragma unroll
        for (int k = 0; k < kHC; ++k)
          if (h0 + k < H) {
            a.out[i * H + h0 + k] = __fdiv_rn(p[k], sum[k]);
            a.mask[i * H + h0 + k] = t[k] > 0.f;
          }
    }
    return;
  }
  for (int h0 = 0; h0 < H; h0 += kHC) {
    float dv[kHC], mx[kHC], part[kHC];
#pragma unroll
    for (int k = 0; k < kHC; ++k) {
      dv[k] = h0 + k < H ? __ldg(a.att_dst + d * H + h0 + k) : 0.f;
      mx[k] = -100000.f;
      part[k] = 0.f;
    }
    for (int64_t i = b + first; i < e; i += STEP) {
      const int64_t s = static_cast<int64_t>(__ldg(idx + i));
#pragma unroll
      for (int k = 0; k < kHC; ++k)
        if (h0 + k < H) {
          float t = dv[k] + __ldg(a.att_src + s * H + h0 + k);
          t = fmaxf(t, t * a.slope);
          a.out[i * H + h0 + k] = t;
          a.mask[i * H + h0 + k] = t > 0.f;
          mx[k] = fmaxf(mx[k], t);
        }
    }
    if (HEAVY) {
      cluster_reduce<true>(mx, sh, cl);
    } else {
#pragma unroll
      for (int k = 0; k < kHC; ++k) mx[k] = warp_max(mx[k]);
    }
    for (int64_t i = b + first; i < e; i += STEP) {
#pragma unroll
      for (int k = 0; k < kHC; ++k)
        if (h0 + k < H) {
          const float p = expf(a.out[i * H + h0 + k] - mx[k]);
          a.out[i * H + h0 + k] = p;
          part[k] += p;
        }
    }
    if (HEAVY) {
      cluster_reduce<false>(part, sh, cl);
    } else {
#pragma unroll
      for (int k = 0; k < kHC; ++k) part[k] = warp_tree_sum(part[k]);
    }
    for (int64_t i = b + first; i < e; i += STEP) {
#pragma unroll
      for (int k = 0; k < kHC; ++k)
        if (h0 + k < H) a.out[i * H + h0 + k] = __fdiv_rn(a.out[i * H + h0 + k], part[k]);
    }
  }
}

// Backward for one row (edge_softmax.cu:44-95): s = sum out*g; tmp = out*(g-s), times
// slope where the forward pre-activation was not positive; grad_src[src] += tmp;
// grad_dst = sum tmp, written only when the row has both signs (it is 0 otherwise).
template <typename IdxT, bool HEAVY>
__device__ __forceinline__ void softmax_bwd_row(const SoftmaxArgs &a, int64_t d, int first, float *sh, float *cl) {
  constexpr int STEP = HEAVY ? kHeavyThreads * kHeavyCluster : 32;
  const IdxT *idx = reinterpret_cast<const IdxT *>(a.idx);
  const int H = a.heads;
  const int64_t b = load_ptr(a.ptr, d, a.ptr_bytes), e = load_ptr(a.ptr, d + 1, a.ptr_bytes);
  if (!HEAVY && e - b <= 32) {
    // at most one edge per lane: out, grad and mask are read once (same operations in the same order as below)
    const int64_t i = b + first;
    const bool has = i < e;
    const int64_t src = has ? static_cast<int64_t>(__ldg(idx + i)) : 0;
    for (int h0 = 0; h0 < H; h0 += kHC) {
#pragma unroll
      for (int k = 0; k < kHC; ++k) {
        const bool on = has && h0 + k < H;
        const float o = on ? a.out[i * H + h0 + k] : 0.f;
        const float g = on ? a.grad[i * H + h0 + k] : 0.f;
        const float sk = warp_tree_sum(on ? o * g : 0.f);
        float tmp = 0.f, ps = 0.f, ng = 0.f;
        if (on) {
          tmp = o * (g - sk);
          if (!a.mask[i * H + h0 + k]) {
            tmp *= a.slope;
            ng = 1.f;
          } else {
            ps = 1.f;
          }
          atomicAdd(a.grad_src + src * H + h0 + k, tmp);
        }
        const float dg = warp_tree_sum(tmp);
        ps = warp_tree_sum(ps);
        ng = warp_tree_sum(ng);
        if (first == 0 && h0 + k < H && ps > 0.f && ng > 0.f) a.grad_dst[d * H + h0 + k] = dg;
      }
    }
    return;
  }
  for (int h0 = 0; h0 < H; h0 += kHC) {
    float s[kHC], dg[kHC], pos[kHC], neg[kHC];
#pragma unroll
    for (int k = 0; k < kHC; ++k) s[k] = dg[k] = pos[k] = neg[k] = 0.f;
    for (int64_t i = b + first; i < e; i += STEP)
#pragma unroll
      for (int k = 0; k < kHC; ++k)
        if (h0 + k < H) s[k] += a.out[i * H + h0 + k] * a.grad[i * H + h0 + k];
    if (HEAVY) {
      cluster_reduce<false>(s, sh, cl);
    } else {
#pragma unroll
      for (int k = 0; k < kHC; ++k) s[k] = warp_tree_sum(s[k]);
    }
    for (int64_t i = b + first; i < e; i += STEP) {
      const int64_t src = static_cast<int64_t>(__ldg(idx + i));
#pragma unroll
      for (int k = 0; k < kHC; ++k)
        if (h0 + k < H) {
          float tmp = a.out[i * H + h0 + k] * (a.grad[i * H + h0 + k] - s[k]);
          if (!a.mask[i * H + h0 + k]) {
            tmp *= a.slope;
            neg[k] = 1.f;
          } else {
            pos[k] = 1.f;
          }
          dg[k] += tmp;
          atomicAdd(a.grad_src + src * H + h0 + k, tmp);
        }
    }
    if (HEAVY) {
      cluster_reduce<false>(dg, sh, cl);
      cluster_reduce<false>(pos, sh, cl);
      cluster_reduce<false>(neg, sh, cl);
    } else {
#pragma unroll
      for (int k = 0; k < kHC; ++k) {
        dg[k] = warp_tree_sum(dg[k]);
        pos[k] = warp_tree_sum(pos[k]);
        neg[k] = warp_tree_sum(neg[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < kHC; ++k)
      if (first == 0 && h0 + k < H && pos[k] > 0.f && neg[k] > 0.f) a.grad_dst[d * H + h0 + k] = dg[k];
  }
}

template <typename IdxT, bool BWD>
__global__ void __launch_bounds__(kThreads) edge_softmax_rows(SoftmaxArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t d = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  if (d >= a.n_dst) return;
  const int64_t deg = load_ptr(a.ptr, d + 1, a.ptr_bytes) - load_ptr(a.ptr, d, a.ptr_bytes);
  if (deg > kHeavyRow) {  // left to the CTA-per-row kernel
    if (lane == 0) {
      int slot = atomicAdd(a.hdr, 1);
      if (slot < a.max_heavy) a.heavy[slot] = d;
    }
    return;
  }
  if (BWD)
    softmax_bwd_row<IdxT, false>(a, d, lane, nullptr, nullptr);
  else
    softmax_fwd_row<IdxT, false>(a, d, lane, nullptr, nullptr);
}

// Rows above kHeavyRow edges: one thread-block cluster per row (launched with cluster dimension kHeavyCluster).
template <typename IdxT, bool BWD>
__global__ void __launch_bounds__(kHeavyThreads) edge_softmax_heavy(SoftmaxArgs a) {
  __shared__ float sh[kHeavyWarps * kHC];
  __shared__ float cl[kHC];
  cg::cluster_group cluster = cg::this_cluster();
  const int n = min(a.hdr[0], a.max_heavy);
  const int first = static_cast<int>(cluster.block_rank()) * kHeavyThreads + threadIdx.x;
  const int n_clusters = gridDim.x / kHeavyCluster;
  for (int i = blockIdx.x / kHeavyCluster; i < n; i += n_clusters) {  // uniform over the cluster
    if (BWD)
      softmax_bwd_row<IdxT, true>(a, a.heavy[i], first, sh, cl);
    else
      softmax_fwd_row<IdxT, true>(a, a.heavy[i], first, sh, cl);
  }
}

template <typename IdxT, bool BWD>
cudaError_t launch_heavy(const SoftmaxArgs &a, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((kNumSM / kHeavyCluster) * kHeavyCluster);  // 144 CTAs = 18 clusters
  cfg.blockDim = dim3(kHeavyThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kHeavyCluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, edge_softmax_heavy<IdxT, BWD>, a);
}

// out[e,h] = <src_feat[src[e],h,:], dst_feat[dst[e],(h),:]>; one warp per edge, the lanes of a
// head add their products with a shuffle tree.
template <typename IdxT>
__global__ void __launch_bounds__(kThreads) sddmm_coo(const IdxT *src, const IdxT *dst, const float *src_feat,
                                                     const float *dst_feat, float *out, int64_t n_edge, int feat,
                                                     int heads, int per_head) {
  const int lane = threadIdx.x & 31;
  const int64_t e = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  if (e >= n_edge) return;
  const int64_t s = static_cast<int64_t>(src[e]), d = static_cast<int64_t>(dst[e]);
  for (int h = 0; h < heads; ++h) {
    const float *pa = src_feat + (s * heads + h) * feat;
    const float *pb = dst_feat + (per_head ? (d * heads + h) : d) * static_cast<int64_t>(feat);
    float r = 0.f;
    for (int i = lane; i < feat; i += 32) r = fmaf(__ldg(pa + i), __ldg(pb + i), r);
    r = warp_tree_sum(r);
    if (lane == 0) out[e * heads + h] = r;
  }
}

__global__ void edge_value_degree_kernel(const void *ptr, int ptr_bytes, float *out, int64_t n_dst) {
  const int lane = threadIdx.x & 31;
  const int64_t d = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  if (d >= n_dst) return;
  const int64_t b = load_ptr(ptr, d, ptr_bytes), e = load_ptr(ptr, d + 1, ptr_bytes);
  if (e <= b) return;
  const float v = 1.f / static_cast<float>(e - b);
  for (int64_t i = b + lane; i < e; i += 32) out[i] = v;
}

template <typename IdxT>
__global__ void spmv_kernel(const void *ptr, int ptr_bytes, const IdxT *idx, const float *x, float *y,
                            int64_t n_dst) {
  const int lane = threadIdx.x & 31;
  const int64_t d = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  if (d >= n_dst) return;
  const int64_t b = load_ptr(ptr, d, ptr_bytes), e = load_ptr(ptr, d + 1, ptr_bytes);
  float v = 0.f;
  for (int64_t i = b + lane; i < e; i += 32) v += __ldg(x + static_cast<int64_t>(idx[i]));
  v = warp_tree_sum(v);
  if (lane == 0) y[d] = v;
}

// out[dest[e], :] += x_edge[e, :] (forward) / grad_edge[e, :] = grad_out[dest[e], :] (backward)
template <typename IdxT, bool BWD>
__global__ void gather_kernel(const float *in, const IdxT *dest, float *out, int64_t n_edge, int feat) {
  const int64_t total = n_edge * feat;
  for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < total;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e = t / feat;
    const int c = static_cast<int>(t - e * feat);
    const int64_t v = static_cast<int64_t>(dest[e]);
    if (BWD)
      out[t] = in[v * feat + c];
    else
      atomicAdd(out + v * feat + c, in[t]);
  }
}

int softmax_common(SoftmaxArgs &a, const void *ptr, const void *idx, int ptr_bytes, int idx_bytes, int64_t n_dst,
                   int64_t nnz, int heads, void *workspace, size_t ws_bytes, const char *who) {
  CXG_REQUIRE(n_dst >= 0 && nnz >= 0 && heads > 0, CXG_EINVAL, "%s: bad sizes", who);
  CXG_REQUIRE((ptr_bytes == 4 || ptr_bytes == 8) && (idx_bytes == 4 || idx_bytes == 8), CXG_EINVAL,
              "%s: index widths %d/%d", who, ptr_bytes, idx_bytes);
  const int64_t max_heavy = nnz / kHeavyRow + 1;
  const size_t need = 256 + static_cast<size_t>(max_heavy) * sizeof(int64_t);
  CXG_REQUIRE(workspace != nullptr && ws_bytes >= need, CXG_EWORKSPACE, "%s: workspace %zu bytes, need %zu", who,
              ws_bytes, need);
  CXG_REQUIRE(max_heavy <= INT32_MAX, CXG_ELIMIT, "%s: too many long rows", who);
  a.ptr = ptr, a.idx = idx, a.n_dst = n_dst, a.heads = heads, a.ptr_bytes = ptr_bytes;
  a.hdr = reinterpret_cast<int32_t *>(workspace);
  a.heavy = reinterpret_cast<int64_t *>(reinterpret_cast<char *>(workspace) + 256);
  a.max_heavy = static_cast<int>(max_heavy);
  return CXG_OK;
}

}  // namespace
}  // namespace cxg

using namespace cxg;

extern "C" int cxg_edge_softmax_workspace_size(int64_t n_dst, int64_t nnz, size_t *bytes) {
  CXG_REQUIRE(bytes != nullptr, CXG_ENULL, "cxg_edge_softmax_workspace_size: bytes is NULL");
  CXG_REQUIRE(n_dst >= 0 && nnz >= 0, CXG_EINVAL, "cxg_edge_softmax_workspace_size: bad sizes");
  *bytes = 256 + static_cast<size_t>(nnz / kHeavyRow + 1) * sizeof(int64_t);
  return CXG_OK;
}

extern "C" int cxg_edge_softmax_forward(const void *ptr, const void *idx, int ptr_bytes, int idx_bytes,
                                        const float *att_dst, const float *att_src, float *out, uint8_t *mask,
                                        int64_t n_dst, int64_t nnz, int heads, float slope, void *workspace,
                                        size_t workspace_bytes, void *stream) {
  SoftmaxArgs a = {};
  int rc = softmax_common(a, ptr, idx, ptr_bytes, idx_bytes, n_dst, nnz, heads, workspace, workspace_bytes,
                          "cxg_edge_softmax_forward");
  if (rc != CXG_OK) return rc;
  if (n_dst == 0 || nnz == 0) return CXG_OK;
  CXG_REQUIRE(ptr && idx && att_dst && att_src && out && mask, CXG_ENULL, "cxg_edge_softmax_forward: NULL argument");
  a.att_dst = att_dst, a.att_src = att_src, a.out = out, a.mask = mask, a.slope = slope;
  cudaStream_t st = as_stream(stream);
  if (cudaMemsetAsync(a.hdr, 0, 256, st) != cudaSuccess) return check_launch("cxg_edge_softmax_forward: memset");
  const unsigned grid = static_cast<unsigned>((n_dst + kWarps - 1) / kWarps);
  if (idx_bytes == 8) {
    edge_softmax_rows<int64_t, false><<<grid, kThreads, 0, st>>>(a);
    if (launch_heavy<int64_t, false>(a, st) != cudaSuccess) return check_launch("edge_softmax_heavy");
  } else {
    edge_softmax_rows<int32_t, false><<<grid, kThreads, 0, st>>>(a);
    if (launch_heavy<int32_t, false>(a, st) != cudaSuccess) return check_launch("edge_softmax_heavy");
  }
  count_launches(2);
  return check_launch("cxg_edge_softmax_forward");
}

extern "C" int cxg_edge_softmax_backward(const void *ptr, const void *idx, int ptr_bytes, int idx_bytes,
                                         const float *grad, const uint8_t *mask, const float *out, float *grad_dst,
                                         float *grad_src, int64_t n_dst, int64_t nnz, int heads, float slope,
                                         void *workspace, size_t workspace_bytes, void *stream) {
  SoftmaxArgs a = {};
  int rc = softmax_common(a, ptr, idx, ptr_bytes, idx_bytes, n_dst, nnz, heads, workspace, workspace_bytes,
                          "cxg_edge_softmax_backward");
  if (rc != CXG_OK) return rc;
  if (n_dst == 0 || nnz == 0) return CXG_OK;
  CXG_REQUIRE(ptr && idx && grad && mask && out && grad_dst && grad_src, CXG_ENULL,
              "cxg_edge_softmax_backward: NULL argument");
  a.grad = grad, a.mask = const_cast<uint8_t *>(mask), a.out = const_cast<float *>(out);
  a.grad_dst = grad_dst, a.grad_src = grad_src, a.slope = slope;
  cudaStream_t st = as_stream(stream);
  if (cudaMemsetAsync(a.hdr, 0, 256, st) != cudaSuccess) return check_launch("cxg_edge_softmax_backward: memset");
  const unsigned grid = static_cast<unsigned>((n_dst + kWarps - 1) / kWarps);
  if (idx_bytes == 8) {
    edge_softmax_rows<int64_t, true><<<grid, kThreads, 0, st>>>(a);
    if (launch_heavy<int64_t, true>(a, st) != cudaSuccess) return check_launch("edge_softmax_heavy");
  } else {
    edge_softmax_rows<int32_t, true><<<grid, kThreads, 0, st>>>(a);
    if (launch_heavy<int32_t, true>(a, st) != cudaSuccess) return check_launch("edge_softmax_heavy");
  }
  count_launches(2);
  return check_launch("cxg_edge_softmax_backward");
}

extern "C" int cxg_sddmm_coo(const void *src, const void *dst, int idx_bytes, const float *src_feat,
                             const float *dst_feat, float *out, int64_t n_edge, int feat, int heads,
                             int dst_per_head, void *stream) {
  CXG_REQUIRE(n_edge >= 0 && feat > 0 && heads > 0, CXG_EINVAL, "cxg_sddmm_coo: bad sizes");
  CXG_REQUIRE(idx_bytes == 4 || idx_bytes == 8, CXG_EINVAL, "cxg_sddmm_coo: idx_bytes %d", idx_bytes);
  if (n_edge == 0) return CXG_OK;
  CXG_REQUIRE(src && dst && src_feat && dst_feat && out, CXG_ENULL, "cxg_sddmm_coo: NULL argument");
  const unsigned grid = static_cast<unsigned>((n_edge + kWarps - 1) / kWarps);
  cudaStream_t st = as_stream(stream);
  if (idx_bytes == 8)
    sddmm_coo<int64_t><<<grid, kThreads, 0, st>>>(static_cast<const int64_t *>(src), static_cast<const int64_t *>(dst),
                                                  src_feat, dst_feat, out, n_edge, feat, heads, dst_per_head);
  else
    sddmm_coo<int32_t><<<grid, kThreads, 0, st>>>(static_cast<const int32_t *>(src), static_cast<const int32_t *>(dst),
                                                  src_feat, dst_feat, out, n_edge, feat, heads, dst_per_head);
  count_launches(1);
  return check_launch("cxg_sddmm_coo");
}

extern "C" int cxg_edge_value_degree(const void *ptr, int ptr_bytes, float *out, int64_t n_dst, void *stream) {
  CXG_REQUIRE(n_dst >= 0 && (ptr_bytes == 4 || ptr_bytes == 8), CXG_EINVAL, "cxg_edge_value_degree: bad arguments");
  if (n_dst == 0) return CXG_OK;
  CXG_REQUIRE(ptr && out, CXG_ENULL, "cxg_edge_value_degree: NULL argument");
  const unsigned grid = static_cast<unsigned>((n_dst + kWarps - 1) / kWarps);
  edge_value_degree_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(ptr, ptr_bytes, out, n_dst);
  count_launches(1);
  return check_launch("cxg_edge_value_degree");
}

extern "C" int cxg_spmv_csr(const void *ptr, const void *idx, int ptr_bytes, int idx_bytes, const float *x, float *y,
                            int64_t n_dst, void *stream) {
  CXG_REQUIRE(n_dst >= 0 && (ptr_bytes == 4 || ptr_bytes == 8) && (idx_bytes == 4 || idx_bytes == 8), CXG_EINVAL,
              "cxg_spmv_csr: bad arguments");
  if (n_dst == 0) return CXG_OK;
  CXG_REQUIRE(ptr && idx && x && y, CXG_ENULL, "cxg_spmv_csr: NULL argument");
  const unsigned grid = static_cast<unsigned>((n_dst + kWarps - 1) / kWarps);
  if (idx_bytes == 8)
    spmv_kernel<int64_t><<<grid, kThreads, 0, as_stream(stream)>>>(ptr, ptr_bytes, static_cast<const int64_t *>(idx), x,
                                                                  y, n_dst);
  else
    spmv_kernel<int32_t><<<grid, kThreads, 0, as_stream(stream)>>>(ptr, ptr_bytes, static_cast<const int32_t *>(idx), x,
                                                                  y, n_dst);
  count_launches(1);
  return check_launch("cxg_spmv_csr");
}

namespace cxg {
namespace {
// out[r, f] = sum over h (in head order, one fp32 accumulator) of in[r, h, f]
template <typename T>
__global__ void head_sum_kernel(const T *in, T *out, int64_t n_row, int heads, int feat) {
  const int64_t total = n_row * feat;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / feat;
    const int f = static_cast<int>(i - r * feat);
    const T *p = in + r * heads * feat + f;
    float acc = to_f32(p[0]);
    for (int h = 1; h < heads; ++h) acc += to_f32(p[static_cast<int64_t>(h) * feat]);
    out[i] = from_f32<T>(acc);
  }
}
}  // namespace
}  // namespace cxg

namespace cxg {
namespace {
// alpha_src[n, h] = <feat[n, h, :], att_src[h, :]> for all n; alpha_dst[n, h] = <feat[n, h, :], att_dst[h, :]> for
// n < n_dst: both attention scores of a GAT layer in one pass over the transformed features. One thread per
// (node, head), the products of a row added in index order.
__global__ void __launch_bounds__(kThreads) gat_scores_kernel(const float *feat, const float *att_src, const float *att_dst,
                                                              float *alpha_src, float *alpha_dst, int64_t n_src,
                                                              int64_t n_dst, int heads, int c) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(kThreads) + threadIdx.x;
  if (i >= n_src * heads) return;
  const int h = static_cast<int>(i % heads);
  const int64_t n = i / heads;
  const float *f = feat + i * c, *as = att_src + h * c, *ad = att_dst + h * c;
  float s = 0.f, d = 0.f;
  if (c % 4 == 0) {
    for (int j = 0; j < c; j += 4) {
      const float4 v = __ldg(reinterpret_cast<const float4 *>(f + j));
      s = fmaf(v.x, __ldg(as + j), s), d = fmaf(v.x, __ldg(ad + j), d);
      s = fmaf(v.y, __ldg(as + j + 1), s), d = fmaf(v.y, __ldg(ad + j + 1), d);
      s = fmaf(v.z, __ldg(as + j + 2), s), d = fmaf(v.z, __ldg(ad + j + 2), d);
      s = fmaf(v.w, __ldg(as + j + 3), s), d = fmaf(v.w, __ldg(ad + j + 3), d);
    }
  } else {
    for (int j = 0; j < c; ++j) {
      const float v = __ldg(f + j);
      s = fmaf(v, __ldg(as + j), s), d = fmaf(v, __ldg(ad + j), d);
    }
  }
  alpha_src[i] = s;
  if (n < n_dst) alpha_dst[i] = d;
}

// grad_feat[n, h, :] = g_src[n, h] * att_src[h, :] + (n < n_dst ? g_dst[n, h] * att_dst[h, :] : 0)
__global__ void __launch_bounds__(kThreads) gat_scores_bwd_kernel(const float *g_src, const float *g_dst,
                                                                  const float *att_src, const float *att_dst,
                                                                  float *grad_feat, int64_t n_src, int64_t n_dst,
                                                                  int heads, int c) {
  const int64_t total = n_src * heads * c;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(kThreads) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t nh = i / c;
    const int j = static_cast<int>(i - nh * c);
    const int h = static_cast<int>(nh % heads);
    float v = __ldg(g_src + nh) * __ldg(att_src + h * c + j);
    if (nh / heads < n_dst) v = fmaf(__ldg(g_dst + nh), __ldg(att_dst + h * c + j), v);
    grad_feat[i] = v;
  }
}
}  // namespace
}  // namespace cxg

extern "C" int cxg_gat_scores(const float *feat, const float *att_src, const float *att_dst, float *alpha_src,
                              float *alpha_dst, int64_t n_src, int64_t n_dst, int heads, int c, void *stream) {
  CXG_REQUIRE(n_src >= 0 && n_dst >= 0 && n_dst <= n_src && heads > 0 && c > 0, CXG_EINVAL, "cxg_gat_scores: bad sizes");
  if (n_src == 0) return CXG_OK;
  CXG_REQUIRE(feat && att_src && att_dst && alpha_src && (alpha_dst || n_dst == 0), CXG_ENULL,
              "cxg_gat_scores: NULL argument");
  CXG_REQUIRE(c % 4 != 0 || reinterpret_cast<uintptr_t>(feat) % 16 == 0, CXG_EINVAL, "cxg_gat_scores: feat alignment");
  const unsigned grid = static_cast<unsigned>((n_src * heads + kThreads - 1) / kThreads);
  gat_scores_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(feat, att_src, att_dst, alpha_src, alpha_dst, n_src, n_dst,
                                                             heads, c);
  count_launches(1);
  return check_launch("cxg_gat_scores");
}

extern "C" int cxg_gat_scores_backward(const float *g_src, const float *g_dst, const float *att_src, const float *att_dst,
                                       float *grad_feat, int64_t n_src, int64_t n_dst, int heads, int c, void *stream) {
  CXG_REQUIRE(n_src >= 0 && n_dst >= 0 && n_dst <= n_src && heads > 0 && c > 0, CXG_EINVAL,
              "cxg_gat_scores_backward: bad sizes");
  if (n_src == 0) return CXG_OK;
  CXG_REQUIRE(g_src && (g_dst || n_dst == 0) && att_src && att_dst && grad_feat, CXG_ENULL,
              "cxg_gat_scores_backward: NULL argument");
  const int64_t want = (n_src * heads * c + kThreads - 1) / kThreads;
  const unsigned grid = static_cast<unsigned>(want < kNumSM * 32 ? want : kNumSM * 32);
  gat_scores_bwd_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(g_src, g_dst, att_src, att_dst, grad_feat, n_src, n_dst,
                                                                 heads, c);
  count_launches(1);
  return check_launch("cxg_gat_scores_backward");
}

namespace cxg {
namespace {
constexpr int kAttGradCtas = kNumSM * 8;

// Stage 1 of the attention-vector gradients: CTA b owns a contiguous chunk of rows; thread (sub, col) adds
// g[r, h(col)] * feat[r, col] over the chunk's rows r = first + sub + j * nsub in four interleaved accumulators
// (j mod 4) that are joined as (a0 + a1) + (a2 + a3); the nsub sums of a column are added in sub order and written
// to part[b][0 | 1][col] (0: att_src, 1: att_dst).
__global__ void __launch_bounds__(kThreads) gat_att_grad_partial(const float *feat, const float *g_src, const float *g_dst,
                                                                 float *part, int64_t n_src, int64_t n_dst, int heads,
                                                                 int c) {
  __shared__ float sh[2][kThreads];
  const int width = heads * c;
  const int nsub = width <= kThreads ? kThreads / width : 1;
  const int64_t per = (n_src + gridDim.x - 1) / gridDim.x;
  const int64_t first = blockIdx.x * per, last = min(n_src, first + per);
  for (int col0 = 0; col0 < width; col0 += kThreads) {
    const int sub = threadIdx.x / width, col = col0 + (width <= kThreads ? threadIdx.x % width : threadIdx.x);
    const bool on = col < width && sub < nsub;
    const int h = on ? col / c : 0;
    float as[4] = {0.f, 0.f, 0.f, 0.f}, ad[4] = {0.f, 0.f, 0.f, 0.f};
    if (on) {
      int64_t r = first + sub;
      for (; r + 3 * nsub < last; r += 4 * nsub) {
        float f[4], gs[4], gd[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int64_t ru = r + u * nsub;
          f[u] = __ldg(feat + ru * width + col);
          gs[u] = __ldg(g_src + ru * heads + h);
          gd[u] = ru < n_dst ? __ldg(g_dst + ru * heads + h) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          as[u] = fmaf(gs[u], f[u], as[u]);
          ad[u] = fmaf(gd[u], f[u], ad[u]);
        }
      }
      for (int u = 0; r < last; r += nsub, ++u) {
        const float f = __ldg(feat + r * width + col);
        as[u] = fmaf(__ldg(g_src + r * heads + h), f, as[u]);
        if (r < n_dst) ad[u] = fmaf(__ldg(g_dst + r * heads + h), f, ad[u]);
      }
    }
    float a_s = (as[0] + as[1]) + (as[2] + as[3]), a_d = (ad[0] + ad[1]) + (ad[2] + ad[3]);
    sh[0][threadIdx.x] = a_s;
    sh[1][threadIdx.x] = a_d;
    __syncthreads();
    if (on && sub == 0) {
      for (int u = 1; u < nsub; ++u) {
        a_s += sh[0][u * width + threadIdx.x];
        a_d += sh[1][u * width + threadIdx.x];
      }
      part[(static_cast<int64_t>(blockIdx.x) * 2) * width + col] = a_s;
      part[(static_cast<int64_t>(blockIdx.x) * 2 + 1) * width + col] = a_d;
    }
    __syncthreads();
  }
}

// Stage 2: one warp per column; lane l adds the partials of CTAs l, l + 32, ... in order, the 32 lane sums are
// joined by a shuffle tree.
__global__ void __launch_bounds__(kThreads) gat_att_grad_final(const float *part, float *grad_att_src, float *grad_att_dst,
                                                               int n_part, int width) {
  const int lane = threadIdx.x & 31;
  const int col = (blockIdx.x * kThreads + threadIdx.x) >> 5;
  if (col >= width) return;
  float as = 0.f, ad = 0.f;
  for (int b = lane; b < n_part; b += 32) {
    as += part[(static_cast<int64_t>(b) * 2) * width + col];
    ad += part[(static_cast<int64_t>(b) * 2 + 1) * width + col];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    as += __shfl_down_sync(0xffffffffu, as, o);
    ad += __shfl_down_sync(0xffffffffu, ad, o);
  }
  if (lane == 0) {
    grad_att_src[col] = as;
    grad_att_dst[col] = ad;
  }
}
}  // namespace
}  // namespace cxg

extern "C" int cxg_gat_att_grad_workspace_size(int heads, int c, size_t *bytes) {
  CXG_REQUIRE(bytes != nullptr && heads > 0 && c > 0, CXG_EINVAL, "cxg_gat_att_grad_workspace_size: bad arguments");
  *bytes = static_cast<size_t>(kAttGradCtas) * 2 * heads * c * sizeof(float);
  return CXG_OK;
}

extern "C" int cxg_gat_att_grad(const float *feat, const float *g_src, const float *g_dst, float *grad_att_src,
                                float *grad_att_dst, int64_t n_src, int64_t n_dst, int heads, int c, void *workspace,
                                size_t workspace_bytes, void *stream) {
  CXG_REQUIRE(n_src >= 0 && n_dst >= 0 && n_dst <= n_src && heads > 0 && c > 0, CXG_EINVAL, "cxg_gat_att_grad: bad sizes");
  CXG_REQUIRE(grad_att_src && grad_att_dst, CXG_ENULL, "cxg_gat_att_grad: NULL output");
  CXG_REQUIRE(n_src == 0 || (feat && g_src && (g_dst || n_dst == 0)), CXG_ENULL, "cxg_gat_att_grad: NULL argument");
  size_t need = 0;
  cxg_gat_att_grad_workspace_size(heads, c, &need);
  CXG_REQUIRE(workspace != nullptr && workspace_bytes >= need, CXG_EWORKSPACE,
              "cxg_gat_att_grad: workspace %zu bytes, need %zu", workspace_bytes, need);
  cudaStream_t st = as_stream(stream);
  const int width = heads * c;
  float *part = static_cast<float *>(workspace);
  gat_att_grad_partial<<<kAttGradCtas, kThreads, 0, st>>>(feat, g_src, g_dst, part, n_src, n_dst, heads, c);
  gat_att_grad_final<<<(width * 32 + kThreads - 1) / kThreads, kThreads, 0, st>>>(part, grad_att_src, grad_att_dst,
                                                                                  kAttGradCtas, width);
  count_launches(2);
  return check_launch("cxg_gat_att_grad");
}

extern "C" int cxg_head_sum(const void *in, void *out, int64_t n_row, int heads, int feat, int dtype, void *stream) {
  CXG_REQUIRE(n_row >= 0 && heads > 0 && feat > 0 && (dtype == CXG_F32 || dtype == CXG_BF16), CXG_EINVAL,
              "cxg_head_sum: bad arguments");
  if (n_row == 0) return CXG_OK;
  CXG_REQUIRE(in && out, CXG_ENULL, "cxg_head_sum: NULL argument");
  const int64_t want = (n_row * feat + kThreads - 1) / kThreads;
  const unsigned grid = static_cast<unsigned>(want < kNumSM * 32 ? want : kNumSM * 32);
  cudaStream_t st = as_stream(stream);
  if (dtype == CXG_F32)
    head_sum_kernel<float><<<grid, kThreads, 0, st>>>(static_cast<const float *>(in), static_cast<float *>(out), n_row,
                                                      heads, feat);
  else
    head_sum_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>(static_cast<const __nv_bfloat16 *>(in),
                                                              static_cast<__nv_bfloat16 *>(out), n_row, heads, feat);
  count_launches(1);
  return check_launch("cxg_head_sum");
}

extern "C" int cxg_gather_edges(const float *in, const void *dest, int idx_bytes, float *out, int64_t n_edge, int feat,
                                int backward, void *stream) {
  CXG_REQUIRE(n_edge >= 0 && feat > 0 && (idx_bytes == 4 || idx_bytes == 8), CXG_EINVAL,
              "cxg_gather_edges: bad arguments");
  if (n_edge == 0) return CXG_OK;
  CXG_REQUIRE(in && dest && out, CXG_ENULL, "cxg_gather_edges: NULL argument");
  const int64_t total = n_edge * feat;
  const int64_t want = (total + kThreads - 1) / kThreads;
  const unsigned grid = static_cast<unsigned>(want < kNumSM * 32 ? want : kNumSM * 32);
  cudaStream_t st = as_stream(stream);
#define CXG_GATHER(I, B) \
  gather_kernel<I, B><<<grid, kThreads, 0, st>>>(in, static_cast<const I *>(dest), out, n_edge, feat)
  if (idx_bytes == 8) {
    if (backward)
      CXG_GATHER(int64_t, true);
    else
      CXG_GATHER(int64_t, false);
  } else {
    if (backward)
      CXG_GATHER(int32_t, true);
    else
      CXG_GATHER(int32_t, false);
  }
#undef CXG_GATHER
  count_launches(1);
  return check_launch("cxg_gather_edges");
}
