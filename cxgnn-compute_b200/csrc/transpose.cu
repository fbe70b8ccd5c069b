// CSR transpose on the device: a stable counting sort of the edges by source id.
//
// dX = A^T dY is a forward aggregation over the transposed graph, so the backward of every
// SpMM can run on the deterministic forward kernel instead of scattering with atomics (which
// is what the reference does: gen_bwd_* in src/cpp/src/aggr_kernel.cu:188-249, and what its
// AggrOP sidesteps by assuming a symmetric graph, cxgnncomp/graph_conv.py:57-77). This file
// builds that transposed graph from (ptr, idx):
//   t_ptr[s] .. t_ptr[s+1]  the transposed edges of source s,
//   t_idx[j]                the destination (forward row) of transposed edge j,
//   t_eid[j]                the forward edge it came from (to permute edge values),
// ordered by (source, forward edge id): within a source row the destinations ascend, exactly
// what a stable sort of idx gives.
//
// The sort is a least-significant-digit radix sort with 8-bit digits over the source ids
// (as many passes as the ids have bytes), values = forward edge ids. A pass is four launches:
//   radix_hist     per-tile digit counts           -> counts[digit][tile]
//   scan_blocks    exclusive scan of 2048-entry blocks of counts + one total per block
//   scan_totals    exclusive scan of the block totals (one CTA)
//   radix_scatter  every element to  counts[digit][tile] + block total + its rank among the
//                  tile's earlier elements of the same digit (ranks by warp match + ordered
//                  per-warp counters, so equal keys keep their order: the sort is stable and
//                  the result does not depend on scheduling)
// No atomics on global memory, no spin waits. All scratch comes from the caller.
#include "common.cuh"

namespace cxg {
namespace {

constexpr int kRadixBits = 8;
constexpr int kRadix = 1 << kRadixBits;
constexpr int kTThreads = 256;
constexpr int kTWarps = kTThreads / 32;
constexpr int kItems = 8;                          // elements per thread and tile
constexpr int kTileElems = kTThreads * kItems;     // 2048
constexpr int kScanBlock = 2048;                   // entries of `counts` per scan block

struct TransposeArgs {
  const void *ptr;
  const void *idx;
  int64_t n_dst, n_src, nnz;
  int64_t n_tiles;   // tiles of kTileElems edges
  int64_t n_counts;  // kRadix * n_tiles
  int64_t n_blocks;  // scan blocks over counts
  int ptr_bytes, idx_bytes;
  uint32_t *keys[2];
  void *vals[2];
  int32_t *counts;
  int32_t *totals;
  int64_t *t_ptr;
  void *t_idx;
  void *t_eid;
  float *inv_deg;
};

__device__ __forceinline__ int64_t edge_total(const TransposeArgs &a) {
  const int64_t e = load_ptr(a.ptr, a.n_dst, a.ptr_bytes);
  return e < a.nnz ? (e < 0 ? 0 : e) : a.nnz;  // never beyond what the caller declared
}

// Key of element i in pass 0 comes from idx, later from the key buffer of the previous pass.
template <typename IdxT, bool FIRST>
__device__ __forceinline__ uint32_t load_key(const TransposeArgs &a, int in, int64_t i) {
  if (FIRST) return static_cast<uint32_t>(__ldg(reinterpret_cast<const IdxT *>(a.idx) + i));
  return a.keys[in][i];
}

template <typename IdxT, bool FIRST>
__global__ void __launch_bounds__(kTThreads) radix_hist(TransposeArgs a, int in, int shift) {
  __shared__ int32_t hist[kRadix];
  hist[threadIdx.x] = 0;
  __syncthreads();
  const int64_t e_total = edge_total(a);
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTileElems;
#pragma unroll
  for (int k = 0; k < kItems; ++k) {
    const int64_t i = base + k * kTThreads + threadIdx.x;
    if (i < e_total) atomicAdd(&hist[(load_key<IdxT, FIRST>(a, in, i) >> shift) & (kRadix - 1)], 1);
  }
  __syncthreads();
  a.counts[static_cast<int64_t>(threadIdx.x) * a.n_tiles + blockIdx.x] = hist[threadIdx.x];
}

// Exclusive scan of one block of kScanBlock entries in place; the block's sum goes to totals[block].
__global__ void __launch_bounds__(kTThreads) scan_blocks(int32_t *data, int64_t n, int32_t *totals) {
  __shared__ int32_t warp_sum[kTWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanBlock + threadIdx.x * kItems;
  int32_t v[kItems];
  int32_t sum = 0;
#pragma unroll
  for (int k = 0; k < kItems; ++k) {
    v[k] = base + k < n ? data[base + k] : 0;
    sum += v[k];
  }
  int32_t inc = sum;  // inclusive scan of the per-thread sums inside the warp
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int32_t t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_sum[warp] = inc;
  __syncthreads();
  int32_t before = 0;
#pragma unroll
  for (int w = 0; w < kTWarps; ++w)
    if (w < warp) before += warp_sum[w];
  int32_t run = before + inc - sum;
#pragma unroll
  for (int k = 0; k < kItems; ++k) {
    if (base + k < n) data[base + k] = run;
    run += v[k];
  }
  if (threadIdx.x == kTThreads - 1) totals[blockIdx.x] = run;
}

// Exclusive scan of the block totals by one CTA, kTThreads entries at a time with a running carry.
__global__ void __launch_bounds__(kTThreads) scan_totals(int32_t *totals, int64_t n) {
  __shared__ int32_t warp_sum[kTWarps];
  __shared__ int32_t carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int64_t base = 0; base < n; base += kTThreads) {
    const int64_t i = base + threadIdx.x;
    const int32_t v = i < n ? totals[i] : 0;
    int32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    if (lane == 31) warp_sum[warp] = inc;
    __syncthreads();
    int32_t before = carry_s;
#pragma unroll
    for (int w = 0; w < kTWarps; ++w)
      if (w < warp) before += warp_sum[w];
    if (i < n) totals[i] = before + inc - v;
    __syncthreads();
    if (threadIdx.x == kTThreads - 1) carry_s = before + inc;
    __syncthreads();
  }
}

// Warp w of a CTA owns the elements [w*256, (w+1)*256) of the tile, eight rounds of 32 consecutive
// elements. The rank of an element among the tile's earlier elements of its digit is
//   (elements of that digit in earlier warps) + (in earlier rounds of this warp) + (in lower lanes).
template <typename IdxT, typename ValT, bool FIRST, bool WRITE_KEYS>
__global__ void __launch_bounds__(kTThreads) radix_scatter(TransposeArgs a, int in, int shift) {
  __shared__ int32_t cnt[kTWarps][kRadix];  // per warp: elements of each digit seen so far
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int d = lane; d < kRadix; d += 32) cnt[warp][d] = 0;
  __syncwarp();
  const int64_t e_total = edge_total(a);
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTileElems + warp * (kTileElems / kTWarps);
  if (static_cast<int64_t>(blockIdx.x) * kTileElems >= e_total) return;
  const ValT *vin = reinterpret_cast<const ValT *>(a.vals[in]);
  uint32_t key[kItems];
  ValT val[kItems];
  int32_t rank[kItems];
  const uint32_t lower = (1u << lane) - 1u;
#pragma unroll
  for (int k = 0; k < kItems; ++k) {
    const int64_t i = base + k * 32 + lane;
    const bool ok = i < e_total;
    key[k] = ok ? load_key<IdxT, FIRST>(a, in, i) : 0u;
    val[k] = FIRST ? static_cast<ValT>(i) : (ok ? vin[i] : ValT(0));
    const uint32_t d = ok ? ((key[k] >> shift) & (kRadix - 1)) : kRadix;  // kRadix: not an element
    const uint32_t peers = __match_any_sync(0xffffffffu, d);
    int32_t prior = 0;
    if (ok) prior = cnt[warp][d];
    __syncwarp();
    if (ok && (peers & lower) == 0) cnt[warp][d] = prior + __popc(peers);  // lowest lane of the group
    __syncwarp();
    rank[k] = prior + __popc(peers & lower);
  }
  __syncthreads();
  // digit d = threadIdx.x: turn the per-warp counts into exclusive prefixes over the warps and add the
  // tile's global base for that digit
  {
    const int d = threadIdx.x;
    const int64_t ci = static_cast<int64_t>(d) * a.n_tiles + blockIdx.x;
    int32_t run = a.counts[ci] + a.totals[ci / kScanBlock];
#pragma unroll
    for (int w = 0; w < kTWarps; ++w) {
      const int32_t c = cnt[w][d];
      cnt[w][d] = run;
      run += c;
    }
  }
  __syncthreads();
  uint32_t *kout = a.keys[in ^ 1];
  ValT *vout = reinterpret_cast<ValT *>(a.vals[in ^ 1]);
#pragma unroll
  for (int k = 0; k < kItems; ++k) {
    const int64_t i = base + k * 32 + lane;
    if (i < e_total) {
      const uint32_t d = (key[k] >> shift) & (kRadix - 1);
      const int64_t pos = static_cast<int64_t>(cnt[warp][d]) + rank[k];
      if (WRITE_KEYS) kout[pos] = key[k];
      vout[pos] = val[k];
    }
  }
}

// Row that owns forward edge e (ptr[r] <= e < ptr[r+1]).
__device__ __forceinline__ int64_t owner_row(const void *ptr, int ptr_bytes, int64_t n_dst, int64_t e) {
  int64_t lo = 0, hi = n_dst;
  while (hi - lo > 1) {
    const int64_t mid = (lo + hi) >> 1;
    if (load_ptr(ptr, mid, ptr_bytes) <= e)
      lo = mid;
    else
      hi = mid;
  }
  return lo;
}

// After the last pass: sorted keys in keys[buf], forward edge ids in vals[buf]. Writes t_eid, t_idx, the row
// boundaries t_ptr and (optionally) 1 / in-degree per forward row.
template <typename ValT, typename OutT>
__global__ void __launch_bounds__(kTThreads) transpose_finish(TransposeArgs a, int buf) {
  const int64_t e_total = edge_total(a);
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * kTThreads + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * kTThreads;
  const uint32_t *keys = a.keys[buf];
  const ValT *vals = reinterpret_cast<const ValT *>(a.vals[buf]);
  OutT *t_idx = reinterpret_cast<OutT *>(a.t_idx);
  OutT *t_eid = reinterpret_cast<OutT *>(a.t_eid);
  for (int64_t j = tid; j < e_total; j += nthreads) {
    const int64_t s = keys[j];
    const int64_t prev = j == 0 ? -1 : static_cast<int64_t>(keys[j - 1]);
    for (int64_t q = prev + 1; q <= s; ++q) a.t_ptr[q] = j;  // sources without edges share the boundary
    const int64_t e = static_cast<int64_t>(vals[j]);
    if (t_eid != nullptr) t_eid[j] = static_cast<OutT>(e);
    t_idx[j] = static_cast<OutT>(owner_row(a.ptr, a.ptr_bytes, a.n_dst, e));
  }
  // slots behind the last edge are defined too, so that they can be used as gather indices
  for (int64_t j = e_total + tid; j < a.nnz; j += nthreads) {
    if (t_eid != nullptr) t_eid[j] = 0;
    t_idx[j] = 0;
  }
  // boundaries behind the last source that has an edge (all of them when there is no edge)
  const int64_t last = e_total == 0 ? -1 : static_cast<int64_t>(keys[e_total - 1]);
  for (int64_t q = last + 1 + tid; q <= a.n_src; q += nthreads) a.t_ptr[q] = e_total;
  if (a.inv_deg != nullptr)
    for (int64_t r = tid; r < a.n_dst; r += nthreads) {
      const int64_t deg = load_ptr(a.ptr, r + 1, a.ptr_bytes) - load_ptr(a.ptr, r, a.ptr_bytes);
      a.inv_deg[r] = 1.f / static_cast<float>(deg > 0 ? deg : 1);
    }
}

struct TransposeLayout {
  size_t keys[2], vals[2], counts, totals, total;
  int64_t n_tiles, n_counts, n_blocks;
  int val_bytes;
};

int transpose_layout(int64_t nnz, TransposeLayout *L) {
  L->n_tiles = (nnz + kTileElems - 1) / kTileElems;
  if (L->n_tiles < 1) L->n_tiles = 1;
  L->n_counts = L->n_tiles * kRadix;
  L->n_blocks = (L->n_counts + kScanBlock - 1) / kScanBlock;
  L->val_bytes = 4;  // edge ids and prefix sums are 32-bit: nnz < 2^31 is checked by the caller
  size_t off = 0;
  for (int b = 0; b < 2; ++b) {
    L->keys[b] = off;
    off = align_up(off + static_cast<size_t>(nnz) * sizeof(uint32_t), 256);
  }
  for (int b = 0; b < 2; ++b) {
    L->vals[b] = off;
    off = align_up(off + static_cast<size_t>(nnz) * L->val_bytes, 256);
  }
  L->counts = off;
  off = align_up(off + static_cast<size_t>(L->n_counts) * sizeof(int32_t), 256);
  L->totals = off;
  off = align_up(off + static_cast<size_t>(L->n_blocks) * sizeof(int32_t), 256);
  L->total = off;
  return CXG_OK;
}

template <typename IdxT, typename ValT>
void run_passes(const TransposeArgs &a, int passes, cudaStream_t st) {
  const unsigned tiles = static_cast<unsigned>(a.n_tiles);
  const unsigned blocks = static_cast<unsigned>(a.n_blocks);
  for (int p = 0; p < passes; ++p) {
    const int in = (p + 1) & 1;  // pass p writes buffer p & 1 and reads the other one (pass 0 reads idx)
    const int shift = p * kRadixBits;
    if (p == 0)
      radix_hist<IdxT, true><<<tiles, kTThreads, 0, st>>>(a, in, shift);
    else
      radix_hist<IdxT, false><<<tiles, kTThreads, 0, st>>>(a, in, shift);
    scan_blocks<<<blocks, kTThreads, 0, st>>>(a.counts, a.n_counts, a.totals);
    scan_totals<<<1, kTThreads, 0, st>>>(a.totals, a.n_blocks);
    if (p == 0)
      radix_scatter<IdxT, ValT, true, true><<<tiles, kTThreads, 0, st>>>(a, in, shift);
    else
      radix_scatter<IdxT, ValT, false, true><<<tiles, kTThreads, 0, st>>>(a, in, shift);
  }
}

}  // namespace
}  // namespace cxg

using namespace cxg;

extern "C" int cxg_csr_transpose_workspace_size(int64_t nnz, size_t *bytes) {
  CXG_REQUIRE(bytes != nullptr, CXG_ENULL, "cxg_csr_transpose_workspace_size: bytes is NULL");
  CXG_REQUIRE(nnz >= 0, CXG_EINVAL, "cxg_csr_transpose_workspace_size: nnz %lld", (long long)nnz);
  TransposeLayout L;
  transpose_layout(nnz, &L);
  *bytes = L.total;
  return CXG_OK;
}

extern "C" int cxg_csr_transpose(const void *ptr, const void *idx, int ptr_bytes, int idx_bytes, int64_t n_dst,
                                 int64_t n_src, int64_t nnz, int64_t *t_ptr, void *t_idx, void *t_eid,
                                 float *inv_deg, void *workspace, size_t workspace_bytes, void *stream) {
  CXG_REQUIRE(n_dst >= 0 && n_src >= 0 && nnz >= 0, CXG_EINVAL, "cxg_csr_transpose: negative size");
  CXG_REQUIRE((ptr_bytes == 4 || ptr_bytes == 8) && (idx_bytes == 4 || idx_bytes == 8), CXG_EINVAL,
              "cxg_csr_transpose: index widths %d/%d", ptr_bytes, idx_bytes);
  CXG_REQUIRE(n_src < (1ll << 32), CXG_ELIMIT, "cxg_csr_transpose: %lld sources, keys are 32-bit", (long long)n_src);
  CXG_REQUIRE(nnz < (1ll << 31), CXG_ELIMIT, "cxg_csr_transpose: %lld edges, edge ids and offsets are 32-bit",
              (long long)nnz);
  CXG_REQUIRE(t_ptr != nullptr, CXG_ENULL, "cxg_csr_transpose: t_ptr is NULL");
  CXG_REQUIRE(ptr != nullptr || n_dst == 0, CXG_ENULL, "cxg_csr_transpose: ptr is NULL");
  cudaStream_t st = as_stream(stream);
  if (n_dst == 0 || nnz == 0) {  // no edge: every transposed row is empty
    if (cudaMemsetAsync(t_ptr, 0, (n_src + 1) * sizeof(int64_t), st) != cudaSuccess)
      return check_launch("cxg_csr_transpose: clearing t_ptr");
    if (nnz > 0 && t_idx != nullptr) cudaMemsetAsync(t_idx, 0, nnz * idx_bytes, st);
    if (nnz > 0 && t_eid != nullptr) cudaMemsetAsync(t_eid, 0, nnz * idx_bytes, st);
    if (inv_deg != nullptr && n_dst > 0) {
      TransposeArgs a = {};
      a.ptr = ptr, a.n_dst = n_dst, a.n_src = -1, a.nnz = 0, a.ptr_bytes = ptr_bytes, a.t_ptr = t_ptr, a.inv_deg = inv_deg;
      transpose_finish<uint32_t, int32_t><<<kNumSM, kTThreads, 0, st>>>(a, 0);
      count_launches(1);
    }
    return check_launch("cxg_csr_transpose");
  }
  CXG_REQUIRE(idx != nullptr && t_idx != nullptr, CXG_ENULL, "cxg_csr_transpose: idx or t_idx is NULL");
  TransposeLayout L;
  transpose_layout(nnz, &L);
  CXG_REQUIRE(workspace != nullptr && workspace_bytes >= L.total, CXG_EWORKSPACE,
              "cxg_csr_transpose: workspace %zu bytes, need %zu", workspace_bytes, L.total);
  CXG_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0, CXG_EINVAL,
              "cxg_csr_transpose: workspace must be 16-byte aligned");
  char *ws = reinterpret_cast<char *>(workspace);
  TransposeArgs a;
  a.ptr = ptr, a.idx = idx, a.n_dst = n_dst, a.n_src = n_src, a.nnz = nnz;
  a.n_tiles = L.n_tiles, a.n_counts = L.n_counts, a.n_blocks = L.n_blocks;
  a.ptr_bytes = ptr_bytes, a.idx_bytes = idx_bytes;
  for (int b = 0; b < 2; ++b) {
    a.keys[b] = reinterpret_cast<uint32_t *>(ws + L.keys[b]);
    a.vals[b] = ws + L.vals[b];
  }
  a.counts = reinterpret_cast<int32_t *>(ws + L.counts);
  a.totals = reinterpret_cast<int32_t *>(ws + L.totals);
  a.t_ptr = t_ptr, a.t_idx = t_idx, a.t_eid = t_eid, a.inv_deg = inv_deg;

  int bits = 0;
  while (bits < 32 && (static_cast<uint64_t>(n_src > 0 ? n_src - 1 : 0) >> bits) != 0) ++bits;
  int passes = (bits + kRadixBits - 1) / kRadixBits;
  if (passes < 1) passes = 1;
  if (idx_bytes == 8)
    run_passes<int64_t, uint32_t>(a, passes, st);
  else
    run_passes<int32_t, uint32_t>(a, passes, st);
  const int buf = (passes - 1) & 1;
  int64_t fin = (nnz + kTThreads - 1) / kTThreads;
  if (fin > kNumSM * 32) fin = kNumSM * 32;
  if (fin < 1) fin = 1;
  if (idx_bytes == 8)
    transpose_finish<uint32_t, int64_t><<<static_cast<unsigned>(fin), kTThreads, 0, st>>>(a, buf);
  else
    transpose_finish<uint32_t, int32_t><<<static_cast<unsigned>(fin), kTThreads, 0, st>>>(a, buf);
  count_launches(passes * 4 + 1);
  return check_launch("cxg_csr_transpose");
}
