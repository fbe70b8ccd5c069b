// Error reporting shared by every entry point of the C ABI. The reference ends
// the process on a failed check (src/cpp/include/common.h:16-37: exit(1), or
// cudaDeviceReset + abort); here a failure is a negative return code plus a
// message kept per calling thread.
#include "common.cuh"

namespace cxg {

static thread_local char g_last_error[512] = "";

int set_error(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

static long long g_launches = 0;

void count_launches(int n) { __atomic_fetch_add(&g_launches, static_cast<long long>(n), __ATOMIC_RELAXED); }

static long long g_wait_cycles = 0;  // 0 = default

long long wait_limit_cycles() {
  const long long v = __atomic_load_n(&g_wait_cycles, __ATOMIC_RELAXED);
  return v > 0 ? v : (1ll << 31);  // ~1 s: a wait that long is a fault, not latency
}

int check_launch(const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return CXG_OK;
  return set_error(CXG_ECUDA, "%s: %s", what, cudaGetErrorString(e));
}

}  // namespace cxg

extern "C" const char *cxg_last_error_string(void) { return cxg::g_last_error; }

extern "C" int cxg_abi_version(void) { return 1; }

extern "C" long long cxg_kernel_launch_count(void) {
  return __atomic_load_n(&cxg::g_launches, __ATOMIC_RELAXED);
}

namespace {
// Reads one 32-bit word of a device workspace after everything queued on `stream` has run.
int read_status_word(const void *workspace, size_t word, void *stream, const char *who) {
  if (workspace == nullptr) return cxg::set_error(CXG_ENULL, "%s: workspace is NULL", who);
  int32_t v = 0;
  cudaStream_t st = cxg::as_stream(stream);
  cudaError_t e = cudaMemcpyAsync(&v, static_cast<const int32_t *>(workspace) + word, sizeof(v), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cxg::set_error(CXG_ECUDA, "%s: %s", who, cudaGetErrorString(e));
  if (v == 2)
    return cxg::set_error(CXG_EINVAL, "%s: ptr[n_dst] exceeds the declared nnz; only the declared edges were read and the result is incomplete", who);
  if (v != 0) return cxg::set_error(CXG_ETIMEOUT, "%s: a bounded device-side wait ran out; the result is incomplete", who);
  return CXG_OK;
}
}  // namespace

extern "C" int cxg_set_wait_limit_cycles(long long cycles) {
  if (cycles < 0) return cxg::set_error(CXG_EINVAL, "cxg_set_wait_limit_cycles: %lld", cycles);
  __atomic_store_n(&cxg::g_wait_cycles, cycles, __ATOMIC_RELAXED);
  return CXG_OK;
}

extern "C" int cxg_spmm_csr_status(const void *workspace, void *stream) {
  return read_status_word(workspace, 63, stream, "cxg_spmm_csr_status");
}

extern "C" int cxg_typed_matmul_status(const void *workspace, void *stream) {
  return read_status_word(workspace, 0, stream, "cxg_typed_matmul_status");
}
