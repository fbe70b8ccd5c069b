// Neighbour sampling for mini-batch training in the CSR_Layer batch format: for every frontier node pick
// min(degree, fanout) of its in-neighbours uniformly without replacement. (In the reference this step is
// the external loader's `neighbor_sample`, called from cxgnncomp/data_preparation.py:214-215 and
// test/ae/E2_spmm/perf-spmm.py:45-46; its output is the batch that model.py:55-71 consumes.)
//
// The draw is a pure function of (seed, node id): Floyd's subset algorithm over the positions
// 0 .. degree-1 of the node's CSR row with a counter-based generator (splitmix64 of seed, node and draw
// number), the chosen positions then sorted so that the sampled row keeps the CSR order of the full row.
// One thread per frontier node; the chosen positions (at most 64) live in registers / local memory.
#include "common.cuh"

namespace cxg {
namespace {

constexpr int kThreads = 128;
constexpr int kMaxFanout = 64;

__host__ __device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// uniform integer in [0, bound) from the high 32 bits of a hash (multiply-shift)
__host__ __device__ __forceinline__ int64_t bounded(uint64_t h, int64_t bound) {
  return static_cast<int64_t>(((h >> 32) * static_cast<uint64_t>(bound)) >> 32);
}

template <typename IdxT>
__global__ void __launch_bounds__(kThreads) sample_rows(const void *gptr, int ptr_bytes, const IdxT *gidx,
                                                        const int64_t *frontier, int64_t n_front, int fanout,
                                                        const int64_t *out_ptr, int64_t *out, uint64_t seed) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(kThreads) + threadIdx.x;
  if (i >= n_front) return;
  const int64_t v = frontier[i];
  const int64_t lo = load_ptr(gptr, v, ptr_bytes), deg = load_ptr(gptr, v + 1, ptr_bytes) - lo;
  int64_t *o = out + out_ptr[i];
  if (deg <= fanout) {
    for (int64_t j = 0; j < deg; ++j) o[j] = static_cast<int64_t>(gidx[lo + j]);
    return;
  }
  // deg > fanout: Floyd's algorithm needs bound < 2^32 for the multiply-shift draw
  int64_t pick[kMaxFanout];
  int k = 0;
  const uint64_t base = splitmix64(seed ^ (static_cast<uint64_t>(v) * 0xD1B54A32D192ED03ull));
  for (int64_t j = deg - fanout; j < deg; ++j) {
    int64_t t = bounded(splitmix64(base + static_cast<uint64_t>(k)), j + 1);
    bool seen = false;
    for (int q = 0; q < k; ++q) seen |= pick[q] == t;
    if (seen) t = j;
    // insert keeping pick[0..k) ascending
    int q = k;
    for (; q > 0 && pick[q - 1] > t; --q) pick[q] = pick[q - 1];
    pick[q] = t;
    ++k;
  }
  for (int q = 0; q < fanout; ++q) o[q] = static_cast<int64_t>(gidx[lo + pick[q]]);
}

}  // namespace
}  // namespace cxg

using namespace cxg;

extern "C" int cxg_sample_neighbors(const void *graph_ptr, const void *graph_idx, int ptr_bytes, int idx_bytes,
                                    const int64_t *frontier, int64_t n_front, int fanout, const int64_t *out_ptr,
                                    int64_t *out, uint64_t seed, void *stream) {
  CXG_REQUIRE(n_front >= 0, CXG_EINVAL, "cxg_sample_neighbors: bad size");
  CXG_REQUIRE(fanout >= 1 && fanout <= kMaxFanout, CXG_EUNSUPPORTED, "cxg_sample_neighbors: fanout %d not in [1, %d]", fanout,
              kMaxFanout);
  CXG_REQUIRE((ptr_bytes == 4 || ptr_bytes == 8) && (idx_bytes == 4 || idx_bytes == 8), CXG_EINVAL,
              "cxg_sample_neighbors: index widths must be 4 or 8");
  if (n_front == 0) return CXG_OK;
  CXG_REQUIRE(graph_ptr && graph_idx && frontier && out_ptr && out, CXG_ENULL, "cxg_sample_neighbors: NULL argument");
  const unsigned grid = static_cast<unsigned>((n_front + kThreads - 1) / kThreads);
  cudaStream_t st = as_stream(stream);
  if (idx_bytes == 8)
    sample_rows<int64_t><<<grid, kThreads, 0, st>>>(graph_ptr, ptr_bytes, static_cast<const int64_t *>(graph_idx), frontier,
                                                    n_front, fanout, out_ptr, out, seed);
  else
    sample_rows<int32_t><<<grid, kThreads, 0, st>>>(graph_ptr, ptr_bytes, static_cast<const int32_t *>(graph_idx), frontier,
                                                    n_front, fanout, out_ptr, out, seed);
  count_launches(1);
  return check_launch("cxg_sample_neighbors");
}

namespace cxg {
namespace {

// Renumbering of sampled neighbours into batch-local ids, step 1: every sampled global id that has no local
// id yet (local_of < 0) is claimed once (atomicCAS on its table entry, -1 -> -2) and appended to `fresh`
// (order of arrival; the caller sorts the list, so the batch does not depend on that order).
__global__ void __launch_bounds__(256) claim_fresh_kernel(const int64_t *picked, int64_t n, int64_t *local_of,
                                                          int64_t *fresh, unsigned long long *n_fresh) {
  for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t v = picked[i];
    if (local_of[v] == -1) {
      const unsigned long long old = atomicCAS(reinterpret_cast<unsigned long long *>(local_of + v),
                                               static_cast<unsigned long long>(-1ll), static_cast<unsigned long long>(-2ll));
      if (old == static_cast<unsigned long long>(-1ll)) fresh[atomicAdd(n_fresh, 1ull)] = v;
    }
  }
}

// step 2 (after the caller has sorted fresh[0 .. n_fresh)): local_of[fresh[i]] = base + i
__global__ void __launch_bounds__(256) number_fresh_kernel(const int64_t *fresh, int64_t n_fresh, int64_t base,
                                                           int64_t *local_of) {
  const int64_t i = blockIdx.x * 256ll + threadIdx.x;
  if (i < n_fresh) local_of[fresh[i]] = base + i;
}

// step 3: out[i] = local_of[picked[i]]
__global__ void __launch_bounds__(256) translate_kernel(const int64_t *picked, int64_t n, const int64_t *local_of,
                                                        int64_t *out) {
  for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * 256)
    out[i] = local_of[picked[i]];
}

unsigned grid_for(int64_t n) {
  const int64_t want = (n + 255) / 256;
  return static_cast<unsigned>(want < kNumSM * 16 ? (want > 0 ? want : 1) : kNumSM * 16);
}

}  // namespace
}  // namespace cxg

namespace cxg {
namespace {
__global__ void __launch_bounds__(256) sample_counts_kernel(const void *gptr, int ptr_bytes, const int64_t *frontier,
                                                            int64_t n_front, int fanout, int64_t *counts) {
  const int64_t i = blockIdx.x * 256ll + threadIdx.x;
  if (i >= n_front) return;
  const int64_t v = frontier[i];
  const int64_t deg = load_ptr(gptr, v + 1, ptr_bytes) - load_ptr(gptr, v, ptr_bytes);
  counts[i] = deg < fanout ? deg : fanout;
}
}  // namespace
}  // namespace cxg

extern "C" int cxg_sample_counts(const void *graph_ptr, int ptr_bytes, const int64_t *frontier, int64_t n_front,
                                 int fanout, int64_t *counts, void *stream) {
  CXG_REQUIRE(n_front >= 0 && fanout >= 1 && (ptr_bytes == 4 || ptr_bytes == 8), CXG_EINVAL,
              "cxg_sample_counts: bad arguments");
  if (n_front == 0) return CXG_OK;
  CXG_REQUIRE(graph_ptr && frontier && counts, CXG_ENULL, "cxg_sample_counts: NULL argument");
  sample_counts_kernel<<<static_cast<unsigned>((n_front + 255) / 256), 256, 0, as_stream(stream)>>>(
      graph_ptr, ptr_bytes, frontier, n_front, fanout, counts);
  count_launches(1);
  return check_launch("cxg_sample_counts");
}

extern "C" int cxg_renumber_claim(const int64_t *picked, int64_t n_picked, int64_t *local_of, int64_t *fresh,
                                  int64_t *n_fresh, void *stream) {
  CXG_REQUIRE(n_picked >= 0, CXG_EINVAL, "cxg_renumber_claim: bad size");
  CXG_REQUIRE(local_of && fresh && n_fresh && (picked || n_picked == 0), CXG_ENULL, "cxg_renumber_claim: NULL argument");
  cudaStream_t st = as_stream(stream);
  if (cudaMemsetAsync(n_fresh, 0, sizeof(int64_t), st) != cudaSuccess) return check_launch("cxg_renumber_claim: memset");
  if (n_picked == 0) return CXG_OK;
  claim_fresh_kernel<<<grid_for(n_picked), 256, 0, st>>>(picked, n_picked, local_of, fresh,
                                                        reinterpret_cast<unsigned long long *>(n_fresh));
  count_launches(1);
  return check_launch("cxg_renumber_claim");
}

extern "C" int cxg_renumber_assign(const int64_t *fresh_sorted, int64_t n_fresh, int64_t base, const int64_t *picked,
                                   int64_t n_picked, int64_t *local_of, int64_t *out, void *stream) {
  CXG_REQUIRE(n_fresh >= 0 && n_picked >= 0 && base >= 0, CXG_EINVAL, "cxg_renumber_assign: bad sizes");
  CXG_REQUIRE(local_of && (fresh_sorted || n_fresh == 0) && ((picked && out) || n_picked == 0), CXG_ENULL,
              "cxg_renumber_assign: NULL argument");
  cudaStream_t st = as_stream(stream);
  if (n_fresh > 0) {
    number_fresh_kernel<<<static_cast<unsigned>((n_fresh + 255) / 256), 256, 0, st>>>(fresh_sorted, n_fresh, base, local_of);
    count_launches(1);
  }
  if (n_picked > 0) {
    translate_kernel<<<grid_for(n_picked), 256, 0, st>>>(picked, n_picked, local_of, out);
    count_launches(1);
  }
  return check_launch("cxg_renumber_assign");
}
