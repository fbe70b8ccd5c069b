// out[i, :] = in[rows[i], :] for rows of `row_bytes` bytes: the pack step of the needed-rows feature
// exchange between GPUs (the reference's "densify" step gathers the rows a peer asked for before sending
// them, test/1-kernels/test_mgpu_model.py:227-331). A group of lanes copies one row with 16-byte accesses
// (4- or 2-byte accesses when the row size or the pointers do not allow 16), rows are dealt to groups
// grid-stride. Pure HBM copy: algorithmic bytes = 2 * n_rows * row_bytes + 8 * n_rows.
#include <string.h>

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

// out_q[i - seg_start[q], :] = in[rows[i], :] for the peer q whose segment [seg_start[q], seg_start[q+1]) holds i:
// the pack step of the needed-rows exchange writing straight into the receivers' feature buffers (plain 16-byte
// stores through peer-mapped pointers over NVLink), so no send buffer and no separate transfer are needed.
constexpr int kMaxPeers = 16;
struct PutArgs {
  void *base[kMaxPeers];        // where the first row for peer q goes (a mapping of q's memory in this context)
  int64_t seg_start[kMaxPeers + 1];
  int order[kMaxPeers];         // peers that receive rows, rotated so that senders start at different receivers
  int n_peer;
};

// Work is dealt in chunks of kPutChunk rows that rotate over the peers (chunk c belongs to peer order[c % n_act],
// rows [c / n_act * kPutChunk, +kPutChunk) of that peer's segment), so at every moment this GPU writes to all
// peers and, with every sender doing the same from a different starting peer, every receiver is written to by
// all senders at once instead of one receiver at a time.
constexpr int kPutChunk = 64;

__global__ void __launch_bounds__(kThreads) put_rows_kernel(const uint4 *in, const int64_t *rows, PutArgs a, int vecs_per_row,
                                                            int group, int n_act, int64_t chunks_per_peer) {
  const int lane = threadIdx.x % group;
  const int gpb = kThreads / group;  // row groups per block
  const int64_t total = chunks_per_peer * n_act * (kPutChunk / 1);
  // flat index t = (chunk, row in chunk); groups stride over it
  for (int64_t t = blockIdx.x * static_cast<int64_t>(gpb) + threadIdx.x / group; t < total;
       t += static_cast<int64_t>(gridDim.x) * gpb) {
    const int64_t c = t / kPutChunk;
    const int q = a.order[c % n_act];
    const int64_t j = (c / n_act) * kPutChunk + (t % kPutChunk);  // row inside peer q's segment
    const int64_t i = a.seg_start[q] + j;
    if (i >= a.seg_start[q + 1]) continue;
    const uint4 *src = in + __ldg(rows + i) * vecs_per_row;
    uint4 *dst = static_cast<uint4 *>(a.base[q]) + j * vecs_per_row;
    for (int v = lane; v < vecs_per_row; v += group) dst[v] = __ldg(src + v);
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

// ---- peer mappings: a buffer of another process's GPU mapped into the CURRENT device's context ----------------
// (cudaIpcOpenMemHandle with lazy peer access, opened by the device that will read or write the memory; a mapping
// opened in another context of this process is not reachable from this device's kernels or copy engines at NVLink
// speed).
extern "C" int cxg_ipc_export(const void *ptr, unsigned char *handle64, int64_t *offset_bytes) {
  CXG_REQUIRE(ptr && handle64 && offset_bytes, CXG_ENULL, "cxg_ipc_export: NULL argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void *>(ptr));
  if (e != cudaSuccess) return set_error(CXG_ECUDA, "cxg_ipc_export: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  // the handle names the whole allocation that holds ptr: find its base through the driver's address-range query
  typedef int (*RangeFn)(unsigned long long *, size_t *, unsigned long long);
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult qr;
  e = cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qr);
  if (e != cudaSuccess || fn == nullptr || qr != cudaDriverEntryPointSuccess) {
    cudaGetLastError();
    return set_error(CXG_ECUDA, "cxg_ipc_export: cuMemGetAddressRange is not available");
  }
  unsigned long long base = 0;
  size_t size = 0;
  if (reinterpret_cast<RangeFn>(fn)(&base, &size, reinterpret_cast<unsigned long long>(ptr)) != 0)
    return set_error(CXG_ECUDA, "cxg_ipc_export: address range query failed");
  memcpy(handle64, &h, 64);
  *offset_bytes = static_cast<int64_t>(reinterpret_cast<unsigned long long>(ptr) - base);
  return CXG_OK;
}

extern "C" int cxg_ipc_open(const unsigned char *handle64, void **base) {
  CXG_REQUIRE(handle64 && base, CXG_ENULL, "cxg_ipc_open: NULL argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void *p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return set_error(CXG_ECUDA, "cxg_ipc_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  }
  // probe through the copy engine: an unusable mapping is reported here as an error code, before any kernel
  // dereferences it
  unsigned char probe[16];
  e = cudaMemcpy(probe, p, sizeof(probe), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) {
    cudaGetLastError();
    cudaIpcCloseMemHandle(p);
    return set_error(CXG_ECUDA, "cxg_ipc_open: the mapping cannot be read: %s", cudaGetErrorString(e));
  }
  *base = p;
  return CXG_OK;
}

extern "C" int cxg_ipc_close(void *base) {
  if (base == nullptr) return CXG_OK;
  cudaError_t e = cudaIpcCloseMemHandle(base);
  if (e != cudaSuccess) return set_error(CXG_ECUDA, "cxg_ipc_close: %s", cudaGetErrorString(e));
  return CXG_OK;
}

extern "C" int cxg_copy_async(void *dst, const void *src, int64_t bytes, void *stream) {
  CXG_REQUIRE(bytes >= 0, CXG_EINVAL, "cxg_copy_async: negative size");
  if (bytes == 0) return CXG_OK;
  CXG_REQUIRE(dst && src, CXG_ENULL, "cxg_copy_async: NULL argument");
  cudaError_t e = cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyDeviceToDevice, as_stream(stream));
  if (e != cudaSuccess) return set_error(CXG_ECUDA, "cxg_copy_async: %s", cudaGetErrorString(e));
  return CXG_OK;
}

extern "C" int cxg_put_rows(const void *in, const int64_t *rows, void *const *peer_base_host,
                            const int64_t *seg_start_host, int n_peer, int64_t row_bytes, void *stream) {
  CXG_REQUIRE(n_peer > 0 && n_peer <= kMaxPeers, CXG_ELIMIT, "cxg_put_rows: %d peers, at most %d", n_peer, kMaxPeers);
  CXG_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0 && row_bytes <= (1 << 20), CXG_EINVAL,
              "cxg_put_rows: rows must be a multiple of 16 bytes");
  CXG_REQUIRE(peer_base_host && seg_start_host, CXG_ENULL, "cxg_put_rows: NULL argument");
  PutArgs a;
  a.n_peer = n_peer;
  for (int q = 0; q <= n_peer; ++q) a.seg_start[q] = seg_start_host[q];
  for (int q = 0; q < n_peer; ++q) {
    a.base[q] = peer_base_host[q];
    CXG_REQUIRE(a.seg_start[q + 1] >= a.seg_start[q], CXG_EINVAL, "cxg_put_rows: segment starts must ascend");
    CXG_REQUIRE(a.seg_start[q + 1] == a.seg_start[q] || (a.base[q] && reinterpret_cast<uintptr_t>(a.base[q]) % 16 == 0),
                CXG_EINVAL, "cxg_put_rows: destination of peer %d is NULL or not 16-byte aligned", q);
  }
  const int64_t n_rows = a.seg_start[n_peer];
  if (n_rows == 0) return CXG_OK;
  CXG_REQUIRE(in && rows && reinterpret_cast<uintptr_t>(in) % 16 == 0, CXG_EINVAL, "cxg_put_rows: in must be 16-byte aligned");
  const int vecs = static_cast<int>(row_bytes / 16);
  int group = 1;
  while (group < vecs && group < 32) group <<= 1;
  // receivers in rotated order: the first one after this rank (the rank whose own segment is empty), and so on
  int self = 0;
  for (int q = 0; q < n_peer; ++q)
    if (a.seg_start[q + 1] == a.seg_start[q]) self = q;  // with several empty segments any of them will do
  int n_act = 0;
  int64_t max_cnt = 0;
  for (int k = 1; k <= n_peer; ++k) {
    const int q = (self + k) % n_peer;
    const int64_t cnt = a.seg_start[q + 1] - a.seg_start[q];
    if (cnt == 0) continue;
    a.order[n_act++] = q;
    if (cnt > max_cnt) max_cnt = cnt;
  }
  const int64_t chunks_per_peer = (max_cnt + kPutChunk - 1) / kPutChunk;
  const int64_t total = chunks_per_peer * n_act * kPutChunk;
  const int64_t want = (total + kThreads / group - 1) / (kThreads / group);
  const unsigned grid = static_cast<unsigned>(want < kNumSM * 16 ? want : kNumSM * 16);
  put_rows_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(static_cast<const uint4 *>(in), rows, a, vecs, group, n_act,
                                                            chunks_per_peer);
  count_launches(1);
  return check_launch("cxg_put_rows");
}

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
