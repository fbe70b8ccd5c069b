// CSR SpMM forward for sm_100a:  y[t(r),h,:] (+)= red_{e in row r} v[e,h] * x[s(e),h,:]
//
// One kernel covers what the reference spreads over gen_fwd_sum / gen_fwd_mean /
// gen_fwd_sum_edge_value{,_multi_head} (src/cpp/src/aggr_kernel.cu:3-186),
// run_spmm_sharedmem* (src/cpp/src/spmm_kernel.cu:231-512),
// selective_aggr_fwd_kernel / target_aggr (aggr_kernel.cu:493-581) and
// aggr_rel_fwd (src/cpp/src/rel_spmm.cu:8-35).
//
// Schedule. A row is owned by a "group" of G lanes (G = 8/16/32, the fewest lanes
// whose 16-byte vectors cover the row), so a 512-byte fp32 row at F=128 is one
// coalesced 128-bit load per lane and every neighbour id is read once (the
// reference reads it once per 32-column slice). Neighbour ids are fetched G at a
// time, coalesced, and handed round by shuffle; feature rows are fetched kUnroll
// at a time so several 512-byte gathers are in flight per group, then added in
// CSR order, which keeps the sum bit-identical to a sequential loop.
//
// Power-law rows. Rows with more than `split` edges are cut into segments of
// `split` edges by a plan pass; segments are spread over a fixed set of CTAs,
// their fp32 partial rows go to scratch memory and a last pass adds them in
// segment order. No atomics touch feature data, so results are reproducible.
#include "common.cuh"
#include "spmm_stream.cuh"

namespace cxg {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kUnroll = 8;
constexpr int kDefaultSplit = 256;
constexpr int kRowsPerGroup = 4;
#ifndef CXG_SPMM_MIN_BLOCKS
#define CXG_SPMM_MIN_BLOCKS 3  // resident CTAs per SM the row kernel is compiled for (register cap)
#endif
constexpr int kHeavyBlocksPerSM = 4;

// Header words at the start of the workspace.
enum { kHdrNumHeavy = 0, kHdrNumChunks = 1, kHdrWords = 64 };

struct SpmmArgs {
  const void *ptr;
  const void *idx;
  const void *x;
  void *y;
  const float *edge_val;
  const uint8_t *edge_mask;
  const int32_t *edge_rel;
  const int64_t *targets;
  int64_t n_dst;
  int64_t rel_stride;
  int width;  // heads * feat: elements per feature row
  int feat;   // elements per head
  int heads;
  int ptr_bytes;
  int reduce;
  int accumulate;
  int split;
  // plan (lives in the caller's workspace)
  int32_t *hdr;
  int64_t *heavy_row;
  int32_t *heavy_base;
  int32_t *chunk_slot;
  float *partials;
  int max_heavy;
  int max_chunks;
  int heavy_blocks;
};

// ---------------------------------------------------------------------------
// Plan: which rows are long, and which segment belongs to which long row.
// ---------------------------------------------------------------------------
__global__ void spmm_plan_rows(SpmmArgs a) {
  int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (r >= a.n_dst) return;
  int64_t deg = load_ptr(a.ptr, r + 1, a.ptr_bytes) - load_ptr(a.ptr, r, a.ptr_bytes);
  if (deg <= a.split) return;
  int nch = static_cast<int>((deg + a.split - 1) / a.split);
  int slot = atomicAdd(a.hdr + kHdrNumHeavy, 1);
  int base = atomicAdd(a.hdr + kHdrNumChunks, nch);
  if (slot < a.max_heavy) {
    a.heavy_row[slot] = r;
    a.heavy_base[slot] = base;
  }
}

__global__ void spmm_plan_chunks(SpmmArgs a) {
  int n_heavy = min(a.hdr[kHdrNumHeavy], a.max_heavy);
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  int n_warps = (gridDim.x * blockDim.x) >> 5;
  for (int slot = warp; slot < n_heavy; slot += n_warps) {
    int64_t r = a.heavy_row[slot];
    int64_t deg = load_ptr(a.ptr, r + 1, a.ptr_bytes) - load_ptr(a.ptr, r, a.ptr_bytes);
    int nch = static_cast<int>((deg + a.split - 1) / a.split);
    int base = a.heavy_base[slot];
    for (int k = lane; k < nch; k += 32)
      if (base + k < a.max_chunks) a.chunk_slot[base + k] = slot;
  }
}

// ---------------------------------------------------------------------------
// Edge stream. idx (and the optional per-edge arrays) are read exactly once, so
// they are loaded with an L2 evict-first policy and do not displace feature rows.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

__device__ __forceinline__ int64_t load_stream(const int64_t *p, uint64_t pol) {
  int64_t v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.s64 %0, [%1], %2;" : "=l"(v) : "l"(p), "l"(pol));
  return v;
}

__device__ __forceinline__ int64_t load_stream(const int32_t *p, uint64_t pol) {
  int32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.s32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(pol));
  return static_cast<int64_t>(v);
}

// Source row (or -1 when the edge is masked out) and single-head value of edge e.
template <typename IdxT, int VALMODE>
__device__ __forceinline__ void load_edge(const SpmmArgs &a, int64_t e, uint64_t pol, int64_t &nid,
                                          float &val) {
  const IdxT *idx = reinterpret_cast<const IdxT *>(a.idx);
  bool keep = a.edge_mask == nullptr || a.edge_mask[e] != 0;
  nid = -1;
  if (keep) {
    nid = load_stream(idx + e, pol);
    if (a.edge_rel != nullptr) nid += static_cast<int64_t>(__ldg(a.edge_rel + e)) * a.rel_stride;
  }
  if (VALMODE == 1) val = __ldg(a.edge_val + e);
}

// ---------------------------------------------------------------------------
// Sum of edges [e_begin, e_end) into acc, CSR order, for the NV vectors of this
// lane. VALMODE: 0 none, 1 one value per edge, 2 one value per (edge, head).
// (nid0, val0) is this lane's edge of the first batch, already loaded by the
// caller; the ids of batch b+1 are requested before the rows of batch b, so the
// index stream never sits on the critical path.
// ---------------------------------------------------------------------------
template <typename VT, typename T, typename IdxT, int G, int NV, int VALMODE>
__device__ __forceinline__ void aggregate_segment(const SpmmArgs &a, int64_t e_begin, int64_t e_end,
                                                  int lg, unsigned gmask, uint64_t pol, int64_t nid0,
                                                  float val0, const int (&col)[NV], const bool (&on)[NV],
                                                  const int (&head)[NV], float (&acc)[NV][VT::kElems]) {
  const T *x = reinterpret_cast<const T *>(a.x);
  int64_t my_nid = nid0;
  float my_val = val0;
  for (int64_t e0 = e_begin; e0 < e_end; e0 += G) {
    int64_t next_nid = -1;
    float next_val = 0.f;
    if (e0 + G + lg < e_end) load_edge<IdxT, VALMODE>(a, e0 + G + lg, pol, next_nid, next_val);
    int64_t left = e_end - e0;
    int cnt = left < G ? static_cast<int>(left) : G;
    for (int j = 0; j < cnt; j += kUnroll) {
      typename VT::Raw v[kUnroll][NV];
      int64_t nid[kUnroll];
      float val[kUnroll][NV];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        int src = j + u;
        nid[u] = __shfl_sync(gmask, my_nid, src & (G - 1), G);
        if (VALMODE == 1) val[u][0] = __shfl_sync(gmask, my_val, src & (G - 1), G);
        if (src >= cnt) nid[u] = -1;
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (nid[u] >= 0) {
#pragma unroll
          for (int k = 0; k < NV; ++k) {
            if (on[k]) {
              v[u][k] = VT::load(x + nid[u] * a.width + col[k]);
              if (VALMODE == 2) val[u][k] = __ldg(a.edge_val + (e0 + j + u) * a.heads + head[k]);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (nid[u] >= 0) {
#pragma unroll
          for (int k = 0; k < NV; ++k) {
            if (on[k]) {
              if (VALMODE == 0)
                VT::add(acc[k], v[u][k]);
              else if (VALMODE == 1)
                VT::fma(acc[k], v[u][k], val[u][0]);
              else
                VT::fma(acc[k], v[u][k], val[u][k]);
            }
          }
        }
      }
    }
    my_nid = next_nid;
    my_val = next_val;
  }
}

// Blocks [0, heavy_blocks) walk the segments of long rows (grid-stride); every
// other block owns a tile of kGroupsPerBlock * kRowsPerGroup consecutive short
// rows. A group handles kRowsPerGroup rows of the tile one after the other; the
// row pointers of all of them are fetched up front and the first ids of row k+1
// are requested before the features of row k.
template <typename VT, typename T, typename IdxT, int G, int NV, int VALMODE>
__global__ void __launch_bounds__(kThreads, CXG_SPMM_MIN_BLOCKS) spmm_rows(SpmmArgs a) {
  constexpr int E = VT::kElems;
  constexpr int kGroupsPerBlock = kThreads / G;
  const int lane = threadIdx.x & 31;
  const int lg = lane & (G - 1);
  const unsigned gmask = (G == 32) ? 0xffffffffu : (((1u << G) - 1u) << (lane & ~(G - 1)));
  const int group_in_block = threadIdx.x / G;
  const int nvec = a.width / E;  // vectors per feature row
  const uint64_t pol = policy_evict_first();
  T *y = reinterpret_cast<T *>(a.y);
  const bool heavy = static_cast<int>(blockIdx.x) < a.heavy_blocks;

  int64_t task = 0, task_end = 0, task_step = 1;
  int64_t rb[kRowsPerGroup], re[kRowsPerGroup];
  if (heavy) {
    task = static_cast<int64_t>(blockIdx.x) * kGroupsPerBlock + group_in_block;
    task_end = min(a.hdr[kHdrNumChunks], a.max_chunks);
    task_step = static_cast<int64_t>(a.heavy_blocks) * kGroupsPerBlock;
  } else {
    int64_t tile0 = (static_cast<int64_t>(blockIdx.x) - a.heavy_blocks) * kGroupsPerBlock * kRowsPerGroup;
    task = tile0 + group_in_block;
    task_step = kGroupsPerBlock;
    task_end = min(a.n_dst, tile0 + static_cast<int64_t>(kGroupsPerBlock) * kRowsPerGroup);
#pragma unroll
    for (int k = 0; k < kRowsPerGroup; ++k) {
      int64_t r = task + static_cast<int64_t>(k) * kGroupsPerBlock;
      rb[k] = re[k] = 0;
      if (r < task_end) {
        rb[k] = load_ptr(a.ptr, r, a.ptr_bytes);
        re[k] = load_ptr(a.ptr, r + 1, a.ptr_bytes);
      }
    }
  }

  // Range and first-batch ids of the task after the current one.
  int64_t nxt_begin = 0, nxt_end = 0, nxt_row = -1, nxt_nid = -1;
  float nxt_val = 0.f;
  auto fetch_heavy = [&](int64_t t) {
    nxt_row = -1;
    nxt_nid = -1;
    if (t >= task_end) return;
    int slot = a.chunk_slot[t];
    nxt_row = a.heavy_row[slot];
    int c = static_cast<int>(t) - a.heavy_base[slot];
    int64_t b = load_ptr(a.ptr, nxt_row, a.ptr_bytes);
    int64_t e = load_ptr(a.ptr, nxt_row + 1, a.ptr_bytes);
    nxt_begin = b + static_cast<int64_t>(c) * a.split;
    nxt_end = min(e, nxt_begin + a.split);
    if (nxt_begin + lg < nxt_end) load_edge<IdxT, VALMODE>(a, nxt_begin + lg, pol, nxt_nid, nxt_val);
  };
  auto fetch_light = [&](int64_t t, int64_t b, int64_t e) {
    nxt_row = t;
    nxt_nid = -1;
    nxt_begin = b;
    nxt_end = (e - b > a.split) ? b : e;  // long row: left to the heavy blocks
    if (nxt_begin + lg < nxt_end) load_edge<IdxT, VALMODE>(a, nxt_begin + lg, pol, nxt_nid, nxt_val);
  };

  auto run = [&](int64_t row, int64_t e_begin, int64_t e_end, int64_t nid0, float val0, int64_t cur) {
    const int64_t deg = heavy ? 1 : e_end - e_begin;
    // Column passes: G*NV vectors per pass (one pass whenever the row fits).
    for (int v0 = 0; v0 < nvec; v0 += G * NV) {
      int col[NV], head[NV];
      bool on[NV];
      float acc[NV][E];
#pragma unroll
      for (int q = 0; q < NV; ++q) {
        int v = v0 + lg + q * G;
        on[q] = v < nvec;
        col[q] = v * E;
        head[q] = on[q] ? col[q] / a.feat : 0;
#pragma unroll
        for (int i = 0; i < E; ++i) acc[q][i] = 0.f;
      }
      int64_t n0 = nid0;
      float w0 = val0;
      if (v0 > 0 && e_begin + lg < e_end) load_edge<IdxT, VALMODE>(a, e_begin + lg, pol, n0, w0);
      aggregate_segment<VT, T, IdxT, G, NV, VALMODE>(a, e_begin, e_end, lg, gmask, pol, n0, w0, col, on,
                                                     head, acc);
      if (heavy) {
        float *partial = a.partials + cur * a.width;
#pragma unroll
        for (int q = 0; q < NV; ++q)
          if (on[q]) {
            if (E % 4 == 0) {
#pragma unroll
              for (int i = 0; i < E; i += 4)
                *reinterpret_cast<float4 *>(partial + col[q] + i) =
                    make_float4(acc[q][i], acc[q][(i + 1) % E], acc[q][(i + 2) % E], acc[q][(i + 3) % E]);
            } else {
#pragma unroll
              for (int i = 0; i < E; ++i) partial[col[q] + i] = acc[q][i];
            }
          }
      } else {
        int64_t out_row = a.targets != nullptr ? __ldg(a.targets + row) : row;
        T *yr = y + out_row * a.width;
#pragma unroll
        for (int q = 0; q < NV; ++q)
          if (on[q]) {
            if (a.reduce == CXG_MEAN) {
              float d = static_cast<float>(deg);
#pragma unroll
              for (int i = 0; i < E; ++i) acc[q][i] = deg > 0 ? __fdiv_rn(acc[q][i], d) : 0.f;
            }
            if (a.accumulate) {
              float old[E];
              VT::to_float(old, VT::load_plain(yr + col[q]));
#pragma unroll
              for (int i = 0; i < E; ++i) acc[q][i] += old[i];
            }
            VT::store_stream(yr + col[q], VT::from_float(acc[q]));
          }
      }
    }
  };

  if (heavy) {
    fetch_heavy(task);
    while (task < task_end) {
      const int64_t row = nxt_row, e_begin = nxt_begin, e_end = nxt_end, nid0 = nxt_nid, cur = task;
      const float val0 = nxt_val;
      task += task_step;
      fetch_heavy(task);
      run(row, e_begin, e_end, nid0, val0, cur);
    }
  } else {
    fetch_light(task, rb[0], re[0]);
#pragma unroll
    for (int k = 0; k < kRowsPerGroup; ++k) {
      const int64_t row = nxt_row, e_begin = nxt_begin, e_end = nxt_end, nid0 = nxt_nid;
      const float val0 = nxt_val;
      const bool live = row < task_end && (re[k] - rb[k] <= a.split);
      if (k + 1 < kRowsPerGroup)
        fetch_light(task + static_cast<int64_t>(k + 1) * kGroupsPerBlock, rb[k + 1 < kRowsPerGroup ? k + 1 : k],
                    re[k + 1 < kRowsPerGroup ? k + 1 : k]);
      if (live) run(row, e_begin, e_end, nid0, val0, 0);
    }
  }
}

// Adds the partial rows of each long row in segment order. The segments of a
// row are dealt to the 8 warps of the CTA in contiguous blocks (a function of the
// segment count only), each warp adds its block in order, warp 0 adds the 8
// results in order.
template <typename T>
__global__ void __launch_bounds__(kThreads) spmm_reduce_long_rows(SpmmArgs a) {
  __shared__ float stage[kWarps][32];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int n_heavy = min(a.hdr[kHdrNumHeavy], a.max_heavy);
  T *y = reinterpret_cast<T *>(a.y);
  for (int slot = blockIdx.x; slot < n_heavy; slot += gridDim.x) {
    int64_t row = a.heavy_row[slot];
    int64_t deg = load_ptr(a.ptr, row + 1, a.ptr_bytes) - load_ptr(a.ptr, row, a.ptr_bytes);
    int nch = static_cast<int>((deg + a.split - 1) / a.split);
    const float *p = a.partials + static_cast<int64_t>(a.heavy_base[slot]) * a.width;
    int kb = static_cast<int>(static_cast<int64_t>(nch) * warp / kWarps);
    int ke = static_cast<int>(static_cast<int64_t>(nch) * (warp + 1) / kWarps);
    int64_t out_row = a.targets != nullptr ? a.targets[row] : row;
    for (int c0 = 0; c0 < a.width; c0 += 32) {
      int c = c0 + lane;
      float s = 0.f;
      if (c < a.width) {
        int k = kb;
        for (; k + 8 <= ke; k += 8) {
          float t[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) t[u] = p[static_cast<int64_t>(k + u) * a.width + c];
#pragma unroll
          for (int u = 0; u < 8; ++u) s += t[u];
        }
        for (; k < ke; ++k) s += p[static_cast<int64_t>(k) * a.width + c];
      }
      stage[warp][lane] = s;
      __syncthreads();
      if (warp == 0 && c < a.width) {
        // Warps whose block is empty hold 0; blocks are in segment order.
        float r = stage[0][lane];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) r += stage[w][lane];
        if (a.reduce == CXG_MEAN) r = __fdiv_rn(r, static_cast<float>(deg));
        T *dst = y + out_row * a.width + c;
        if (a.accumulate) r += to_f32(*dst);
        *dst = from_f32<T>(r);
      }
      __syncthreads();
    }
  }
}

template <typename VT, typename T, typename IdxT, int G, int NV>
void launch_rows_val(const SpmmArgs &a, int valmode, dim3 grid, cudaStream_t st) {
  if (valmode == 0)
    spmm_rows<VT, T, IdxT, G, NV, 0><<<grid, kThreads, 0, st>>>(a);
  else if (valmode == 1)
    spmm_rows<VT, T, IdxT, G, NV, 1><<<grid, kThreads, 0, st>>>(a);
  else
    spmm_rows<VT, T, IdxT, G, NV, 2><<<grid, kThreads, 0, st>>>(a);
}

template <typename T, typename IdxT>
void launch_rows(SpmmArgs &a, int valmode, cudaStream_t st) {
  constexpr int E = Vec<T>::kElems;
  const bool vector_ok = (a.width % E == 0) && (a.feat % E == 0 || a.heads == 1) &&
                         (reinterpret_cast<uintptr_t>(a.x) % 16 == 0) &&
                         (reinterpret_cast<uintptr_t>(a.y) % 16 == 0);
  int G = 32, NV = 1;
  if (vector_ok) {
    int nvec = a.width / E;
    if (nvec <= 8)
      G = 8;
    else if (nvec <= 16)
      G = 16;
    else if (nvec > 32)
      NV = 2;
  }
  int64_t rows_per_block = static_cast<int64_t>(kThreads / G) * kRowsPerGroup;
  int64_t light_blocks = (a.n_dst + rows_per_block - 1) / rows_per_block;
  dim3 grid(static_cast<unsigned>(a.heavy_blocks + light_blocks));
  if (!vector_ok) {
    launch_rows_val<Scalar<T>, T, IdxT, 32, 1>(a, valmode, grid, st);
  } else if (G == 8) {
    launch_rows_val<Vec<T>, T, IdxT, 8, 1>(a, valmode, grid, st);
  } else if (G == 16) {
    launch_rows_val<Vec<T>, T, IdxT, 16, 1>(a, valmode, grid, st);
  } else if (NV == 1) {
    launch_rows_val<Vec<T>, T, IdxT, 32, 1>(a, valmode, grid, st);
  } else {
    launch_rows_val<Vec<T>, T, IdxT, 32, 2>(a, valmode, grid, st);
  }
}

struct WorkspaceLayout {
  size_t hdr, heavy_row, heavy_base, chunk_slot, partials, total;
  int max_heavy, max_chunks;
};

int plan_layout(int64_t n_dst, int64_t nnz, int64_t width, int split, WorkspaceLayout *L) {
  // A long row has more than `split` edges, so there are fewer than nnz/split of
  // them, and sum(ceil(deg/split)) <= nnz/split + (number of long rows).
  int64_t max_heavy = nnz / split + 1;
  if (max_heavy > n_dst) max_heavy = n_dst;
  int64_t max_chunks = nnz / split + max_heavy + 1;
  if (max_chunks > INT32_MAX || max_heavy > INT32_MAX) return CXG_ELIMIT;
  size_t off = 0;
  L->hdr = off;
  off = align_up(off + kHdrWords * sizeof(int32_t), 256);
  L->heavy_row = off;
  off = align_up(off + max_heavy * sizeof(int64_t), 256);
  L->heavy_base = off;
  off = align_up(off + max_heavy * sizeof(int32_t), 256);
  L->chunk_slot = off;
  off = align_up(off + max_chunks * sizeof(int32_t), 256);
  L->partials = off;
  off = align_up(off + static_cast<size_t>(max_chunks) * width * sizeof(float), 256);
  L->total = off;
  L->max_heavy = static_cast<int>(max_heavy);
  L->max_chunks = static_cast<int>(max_chunks);
  return CXG_OK;
}

}  // namespace
}  // namespace cxg

using namespace cxg;

extern "C" int cxg_spmm_csr_workspace_size(int64_t n_dst, int64_t nnz, int32_t feat, int32_t heads,
                                           int32_t split_edges, size_t *bytes) {
  CXG_REQUIRE(bytes != nullptr, CXG_ENULL, "cxg_spmm_csr_workspace_size: bytes is NULL");
  CXG_REQUIRE(n_dst >= 0 && nnz >= 0 && feat > 0 && heads > 0 && split_edges >= 0, CXG_EINVAL,
              "cxg_spmm_csr_workspace_size: bad sizes n_dst=%lld nnz=%lld feat=%d heads=%d",
              (long long)n_dst, (long long)nnz, feat, heads);
  int split = split_edges > 0 ? split_edges : kDefaultSplit;
  WorkspaceLayout L;
  int rc = plan_layout(n_dst, nnz, static_cast<int64_t>(feat) * heads, split, &L);
  CXG_REQUIRE(rc == CXG_OK, rc, "cxg_spmm_csr_workspace_size: graph too large for 32-bit segment ids");
  // the streaming path tiles the edge array; its smallest automatic tile is 64 edges
  StreamLayout S;
  int tile = split_edges > 0 ? split_edges : 64;
  rc = stream_layout(nnz, static_cast<int64_t>(feat) * heads, tile, &S);
  CXG_REQUIRE(rc == CXG_OK, rc, "cxg_spmm_csr_workspace_size: graph too large for 32-bit tile ids");
  *bytes = L.total > S.total ? L.total : S.total;
  return CXG_OK;
}

extern "C" int cxg_spmm_csr(const cxg_spmm_desc *d, void *workspace, size_t workspace_bytes,
                            void *stream) {
  CXG_REQUIRE(d != nullptr, CXG_ENULL, "cxg_spmm_csr: desc is NULL");
  CXG_REQUIRE(d->n_dst >= 0 && d->nnz >= 0, CXG_EINVAL, "cxg_spmm_csr: negative n_dst or nnz");
  CXG_REQUIRE(d->feat > 0 && d->heads > 0, CXG_EINVAL, "cxg_spmm_csr: feat=%d heads=%d", d->feat,
              d->heads);
  CXG_REQUIRE(d->dtype == CXG_F32 || d->dtype == CXG_BF16, CXG_EINVAL, "cxg_spmm_csr: dtype %d",
              d->dtype);
  CXG_REQUIRE(d->ptr_bytes == 4 || d->ptr_bytes == 8, CXG_EINVAL, "cxg_spmm_csr: ptr_bytes %d",
              d->ptr_bytes);
  CXG_REQUIRE(d->idx_bytes == 4 || d->idx_bytes == 8, CXG_EINVAL, "cxg_spmm_csr: idx_bytes %d",
              d->idx_bytes);
  CXG_REQUIRE(d->reduce == CXG_SUM || d->reduce == CXG_MEAN, CXG_EINVAL, "cxg_spmm_csr: reduce %d",
              d->reduce);
  CXG_REQUIRE(!(d->reduce == CXG_MEAN && d->edge_val != nullptr), CXG_EUNSUPPORTED,
              "cxg_spmm_csr: mean with edge values is rejected (the reference asserts on it, "
              "src/cpp/src/aggr.cu:158,163)");
  CXG_REQUIRE(d->split_edges >= 0, CXG_EINVAL, "cxg_spmm_csr: split_edges %d", d->split_edges);
  if (d->n_dst == 0) return CXG_OK;
  CXG_REQUIRE(d->ptr != nullptr && d->y != nullptr, CXG_ENULL, "cxg_spmm_csr: ptr or y is NULL");
  CXG_REQUIRE(d->nnz == 0 || (d->idx != nullptr && d->x != nullptr), CXG_ENULL,
              "cxg_spmm_csr: idx or x is NULL");
  CXG_REQUIRE(d->edge_rel == nullptr || d->rel_stride > 0, CXG_EINVAL,
              "cxg_spmm_csr: edge_rel needs rel_stride > 0");

  if (stream_eligible(d)) {
    CXG_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0, CXG_EINVAL,
                "cxg_spmm_csr: workspace must be 16-byte aligned");
    return stream_launch(d, workspace, workspace_bytes, as_stream(stream));
  }
  SpmmArgs a;
  a.ptr = d->ptr;
  a.idx = d->idx;
  a.x = d->x;
  a.y = d->y;
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
  a.accumulate = (d->flags & CXG_SPMM_ACCUMULATE) ? 1 : 0;
  a.split = d->split_edges > 0 ? d->split_edges : kDefaultSplit;

  WorkspaceLayout L;
  int rc = plan_layout(d->n_dst, d->nnz, a.width, a.split, &L);
  CXG_REQUIRE(rc == CXG_OK, rc, "cxg_spmm_csr: graph too large for 32-bit segment ids");
  CXG_REQUIRE(workspace != nullptr && workspace_bytes >= L.total, CXG_EWORKSPACE,
              "cxg_spmm_csr: workspace %zu bytes, need %zu", workspace_bytes, L.total);
  CXG_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0, CXG_EINVAL,
              "cxg_spmm_csr: workspace must be 16-byte aligned");
  char *ws = reinterpret_cast<char *>(workspace);
  a.hdr = reinterpret_cast<int32_t *>(ws + L.hdr);
  a.heavy_row = reinterpret_cast<int64_t *>(ws + L.heavy_row);
  a.heavy_base = reinterpret_cast<int32_t *>(ws + L.heavy_base);
  a.chunk_slot = reinterpret_cast<int32_t *>(ws + L.chunk_slot);
  a.partials = reinterpret_cast<float *>(ws + L.partials);
  a.max_heavy = L.max_heavy;
  a.max_chunks = L.max_chunks;
  // No row can be long when the whole graph has no more than `split` edges.
  const bool may_split = d->nnz > a.split;
  a.heavy_blocks = may_split ? kNumSM * kHeavyBlocksPerSM : 0;

  cudaStream_t st = as_stream(stream);
  // the header (plan counters, error word 63 read by cxg_spmm_csr_status) starts from zero on every call
  if (cudaMemsetAsync(a.hdr, 0, kHdrWords * sizeof(int32_t), st) != cudaSuccess)
    return check_launch("cxg_spmm_csr: clearing the plan header");
  if (may_split) {
    unsigned pb = static_cast<unsigned>((d->n_dst + kThreads - 1) / kThreads);
    spmm_plan_rows<<<pb, kThreads, 0, st>>>(a);
    spmm_plan_chunks<<<kNumSM, kThreads, 0, st>>>(a);
  }
  int valmode = d->edge_val == nullptr ? 0 : (d->heads == 1 ? 1 : 2);
  if (d->dtype == CXG_F32) {
    if (d->idx_bytes == 8)
      launch_rows<float, int64_t>(a, valmode, st);
    else
      launch_rows<float, int32_t>(a, valmode, st);
  } else {
    if (d->idx_bytes == 8)
      launch_rows<__nv_bfloat16, int64_t>(a, valmode, st);
    else
      launch_rows<__nv_bfloat16, int32_t>(a, valmode, st);
  }
  if (may_split) {
    if (d->dtype == CXG_F32)
      spmm_reduce_long_rows<float><<<kNumSM * 2, kThreads, 0, st>>>(a);
    else
      spmm_reduce_long_rows<__nv_bfloat16><<<kNumSM * 2, kThreads, 0, st>>>(a);
  }
  count_launches(may_split ? 4 : 1);
  return check_launch("cxg_spmm_csr");
}
