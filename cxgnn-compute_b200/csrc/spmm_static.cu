// cxg_spmm_csr_static: the CSR SpMM forward for callers that cannot provide scratch memory.
//
// cxg_spmm_csr needs a workspace (tile table and partial sums of rows that cross tile
// borders) and, like every entry point of this library, leaves its allocation to the
// caller. Some callers have no way to do that: a plugin loaded into a host program whose
// own memory pool already holds the whole device and offers plugins no scratch hook; a
// serving loop that must not run into the device-wide synchronisation a cudaMalloc or
// cudaFree brings; a binding through an FFI that can pass the tensors of the operator but
// nothing else. For them this file keeps ONE fixed scratch array in device memory, owned
// by the library itself, and runs the same kernels on it.
//
// Consequences of the array being static:
//   * it exists once per GPU that loads the library and stays for the life of the process
//     (kStaticScratchBytes on each such GPU, used or not);
//   * requests whose scratch need exceeds it are refused with CXG_ELIMIT;
//   * every call uses the same bytes. Nothing is assumed about their previous contents
//     (the plan kernel of each call rewrites the counters it relies on), but two calls that
//     overlap on the GPU -- different streams, or different host threads on one device --
//     overwrite each other's partial sums. Calls must be ordered on the device.
//
// In host code the array's name is only a host-side handle, not a device address. The
// address is looked up with cudaGetSymbolAddress, once per device with that device current,
// by the first call made on that device. No cudaMalloc, cudaFree or other allocating routine is
// called.
#include <mutex>

#include "common.cuh"
#include "spmm_stream.cuh"

namespace cxg {
namespace {

constexpr size_t kStaticScratchBytes = 32u << 20;  // 32 MiB per GPU
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_spmm_static_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
void *g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device (looked up on first use).
int static_scratch(void **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_error(CXG_ECUDA, "cxg_spmm_csr_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices)
    return set_error(CXG_ELIMIT, "cxg_spmm_csr_static: device ordinal %d beyond the %d supported", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_spmm_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return set_error(CXG_ECUDA, "cxg_spmm_csr_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return CXG_OK;
}

}  // namespace
}  // namespace cxg

using namespace cxg;

static_assert(kStaticScratchBytes == CXG_SPMM_STATIC_SCRATCH_BYTES, "header and array size must agree");

extern "C" int cxg_spmm_csr_static(const cxg_spmm_desc *d, void *stream) {
  CXG_REQUIRE(d != nullptr, CXG_ENULL, "cxg_spmm_csr_static: desc is NULL");
  CXG_REQUIRE(d->n_dst >= 0 && d->nnz >= 0 && d->feat > 0 && d->heads > 0, CXG_EINVAL,
              "cxg_spmm_csr_static: bad sizes n_dst=%lld nnz=%lld feat=%d heads=%d", (long long)d->n_dst,
              (long long)d->nnz, d->feat, d->heads);
  // Scratch this request needs: exact for the tiled kernel, the published upper bound otherwise.
  size_t need = 0;
  if (stream_eligible(d)) {
    StreamLayout L;
    int rc = stream_layout(d->nnz, static_cast<int64_t>(d->feat) * d->heads, stream_tile_edges(d), &L);
    CXG_REQUIRE(rc == CXG_OK, rc, "cxg_spmm_csr_static: graph too large for 32-bit tile ids");
    need = L.total;
  } else {
    int rc = cxg_spmm_csr_workspace_size(d->n_dst, d->nnz, d->feat, d->heads, d->split_edges, &need);
    if (rc != CXG_OK) return rc;
  }
  CXG_REQUIRE(need <= kStaticScratchBytes, CXG_ELIMIT,
              "cxg_spmm_csr_static: this graph needs %zu bytes of scratch, the built-in array holds %zu; use "
              "cxg_spmm_csr with a caller-provided workspace",
              need, kStaticScratchBytes);
  void *scratch = nullptr;
  int rc = static_scratch(&scratch);
  if (rc != CXG_OK) return rc;
  return cxg_spmm_csr(d, scratch, kStaticScratchBytes, stream);
}

extern "C" int cxg_spmm_csr_static_status(void *stream) {
  void *scratch = nullptr;
  int rc = static_scratch(&scratch);
  if (rc != CXG_OK) return rc;
  return cxg_spmm_csr_status(scratch, stream);
}
