// Typed (relation-bucketed) matmul for RGCN on the 5th-generation tensor cores:
//   C[oc(m), :] = A[ia(m), :] . W[rel(tile of m)]      for positions m = 0 .. M-1
// where every aligned block of 128 positions holds one relation (that is what the padding of
// TypedLinearE2EOP.preprocess guarantees, cxgnncomp/typed_linear.py:74-87), ia gathers the rows of
// A and oc scatters the rows of C. It replaces the four Triton kernels behind typed_matmul
// (cxgnncomp/codegen/triton_typed_matmul.py:145-749: no index / single index / single index with
// sequential output / source + destination index), whose tl.dot is a TF32 mma.sync on Ampere.
//
// One CTA (128 threads) owns one 128-position tile at a time:
//   1. the 128 gathered rows of A are copied into shared memory in the K-major "core matrix"
//      layout the tensor core reads without swizzle (8 rows x 16 bytes per core matrix), padding
//      rows as zeros; W[rel] (pre-transposed once to [N][K]) is copied the same way when the
//      relation differs from the previous tile's;
//   2. one thread issues K/16 (bf16) or K/8 (tf32) `tcgen05.mma` instructions with M = 128,
//      N = n, accumulating fp32 in tensor memory, and commits them to an mbarrier;
//   3. after the barrier each warp reads its 32 accumulator lanes with `tcgen05.ld`, converts and
//      writes the rows of C to their scattered destinations.
// The work is HBM-bound at RGCN shapes (K = 128, N = 64: 43 flop per byte in bf16), so several
// small CTAs per SM overlap each other's copy / MMA / store phases instead of a warp-specialised
// pipeline inside one CTA.
//
// Waits are bounded: if the MMA barrier does not complete within about a second the CTA records
// an error, releases its tensor memory and returns.
#include "common.cuh"

namespace cxg {

int typed_rows_launch(const void *a, const void *w, void *out, const void *rel, int rel_bytes, const int64_t *src,
                      const int64_t *dst, int64_t m, int64_t m_valid, int k, int n, int num_rel, int dtype, int mode,
                      int out_follows_src, cudaStream_t st);

namespace {

constexpr int kTileM = 128;
constexpr int kMmThreads = 128;
constexpr long long kWaitCycles = 1ll << 31;

struct TmmArgs {
  const void *a;
  const void *wt;  // [R][N][K], K contiguous
  void *c;
  const int64_t *rel;
  const int64_t *src;
  const int64_t *dst;
  int64_t m, m_valid;
  int k, n, num_rel, out_follows_src;
  int tmem_cols;
  int32_t *status;  // [0] error flag
};

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// Shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 bytes,
// `lbo` bytes between core matrices along K, `sbo` bytes between 8-row groups.
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3fff);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3fff) << 32;
  d |= 1ull << 46;  // descriptor version of sm_100
  return d;
}

// Instruction descriptor: fp32 accumulate, A and B of format `fmt` (1 = bf16, 2 = tf32), both K-major.
__device__ __forceinline__ uint32_t make_idesc(int fmt, int m, int n) {
  uint32_t d = 0;
  d |= 1u << 4;                                 // D format: f32
  d |= static_cast<uint32_t>(fmt) << 7;         // A format
  d |= static_cast<uint32_t>(fmt) << 10;        // B format
  d |= static_cast<uint32_t>(n >> 3) << 17;     // N / 8
  d |= static_cast<uint32_t>(m >> 4) << 24;     // M / 16
  return d;
}

template <bool TF32>
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  if (TF32)
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// W [R][K][N] -> Wt [R][N][K]
template <typename T>
__global__ void transpose_w(const T *w, T *wt, int num_rel, int k, int n) {
  const int64_t total = static_cast<int64_t>(num_rel) * k * n;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / (static_cast<int64_t>(k) * n);
    const int rem = static_cast<int>(i - r * k * n);
    const int nn = rem / k, kk = rem - nn * k;
    wt[i] = w[(r * k + kk) * n + nn];
  }
}

// T = __nv_bfloat16 (kind::f16, 16 K per instruction) or float (kind::tf32, 8 K per instruction).
template <typename T>
__global__ void __launch_bounds__(kMmThreads) typed_mm_tc(TmmArgs a) {
  constexpr bool TF32 = sizeof(T) == 4;
  constexpr int EPC = 16 / sizeof(T);  // elements per 16-byte chunk
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t mma_bar;
  __shared__ uint32_t tmem_base_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunks = a.k / EPC;             // 16-byte chunks per row
  const uint32_t lbo = 128;                 // next core matrix along K
  const uint32_t sbo = chunks * 128;        // next 8-row group
  uint8_t *smem_a = smem;                   // 128 rows
  uint8_t *smem_b = smem + static_cast<size_t>(kTileM) * a.k * sizeof(T);  // n rows
  const uint32_t bar = smem_addr(&mma_bar);

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)),
                 "r"(static_cast<uint32_t>(a.tmem_cols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_slot;
  const uint32_t idesc = make_idesc(TF32 ? 2 : 1, kTileM, a.n);

  const T *A = static_cast<const T *>(a.a);
  const T *Wt = static_cast<const T *>(a.wt);
  T *C = static_cast<T *>(a.c);
  const int64_t n_tiles = (a.m + kTileM - 1) / kTileM;
  int64_t loaded_rel = -1;
  uint32_t parity = 0;
  bool dead = false;

  for (int64_t tile = blockIdx.x; tile < n_tiles && !dead; tile += gridDim.x) {
    const int64_t m0 = tile * kTileM;
    const int64_t r = a.rel[m0];
    if (r < 0 || r >= a.num_rel) continue;  // a tile of padding only
    // ---- A: thread t copies 16-byte chunks; 8 consecutive threads take 8 consecutive rows of
    // one chunk column, so a warp writes 512 contiguous bytes of shared memory.
    const int r8 = tid & 7, c_lo = tid >> 3;  // c_lo in [0,16)
    for (int g = 0; g < kTileM / 8; ++g) {
      const int64_t pos = m0 + g * 8 + r8;
      int64_t ia = -1;
      if (pos < a.m) ia = a.src != nullptr ? a.src[pos] : pos;
      const bool ok = ia >= 0 && ia < a.m_valid;
      for (int c = c_lo; c < chunks; c += 16) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (ok) v = __ldg(reinterpret_cast<const uint4 *>(A + ia * a.k) + c);
        *reinterpret_cast<uint4 *>(smem_a + static_cast<size_t>(g) * sbo + c * 128 + r8 * 16) = v;
      }
    }
    if (r != loaded_rel) {
      const T *wr = Wt + r * static_cast<int64_t>(a.n) * a.k;
      for (int g = 0; g < a.n / 8; ++g)
        for (int c = c_lo; c < chunks; c += 16)
          *reinterpret_cast<uint4 *>(smem_b + static_cast<size_t>(g) * sbo + c * 128 + r8 * 16) =
              __ldg(reinterpret_cast<const uint4 *>(wr + static_cast<int64_t>(g * 8 + r8) * a.k) + c);
      loaded_rel = r;
    }
    // make the generic-proxy writes visible to the tensor core (async proxy)
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a0 = smem_addr(smem_a), b0 = smem_addr(smem_b);
      const int steps = chunks / 2;  // two chunks (32 bytes) of K per instruction
      for (int j = 0; j < steps; ++j)
        mma_ss<TF32>(tmem_d, make_desc(a0 + j * 256, lbo, sbo), make_desc(b0 + j * 256, lbo, sbo), idesc, j > 0 ? 1u : 0u);
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    }
    // ---- wait for the accumulators
    if (!mbar_try_wait(bar, parity)) {
      const long long t0 = clock64();
      while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > kWaitCycles) {
          dead = true;
          break;
        }
      }
    }
    if (dead) {
      atomicExch(a.status, 1);
      break;
    }
    parity ^= 1u;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // ---- epilogue: warp w owns accumulator lanes 32w .. 32w+31 = tile rows
    const int64_t pos = m0 + warp * 32 + lane;
    int64_t oc = -1;
    if (pos < a.m) {
      const int64_t ia = a.src != nullptr ? a.src[pos] : pos;
      if (ia >= 0 && ia < a.m_valid) oc = a.dst != nullptr ? a.dst[pos] : (a.out_follows_src ? ia : pos);
    }
    const uint32_t taddr = tmem_d + (static_cast<uint32_t>(warp * 32) << 16);
    for (int c0 = 0; c0 < a.n; c0 += 8) {
      uint32_t v[8];
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                   : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                   : "r"(taddr + c0));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (oc >= 0) {
        T *o = C + oc * a.n + c0;
        if (TF32) {
          *reinterpret_cast<uint4 *>(o) = make_uint4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<uint4 *>(o + 4) = make_uint4(v[4], v[5], v[6], v[7]);
        } else {
          uint32_t p[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(v[2 * q]), __uint_as_float(v[2 * q + 1]));
            p[q] = *reinterpret_cast<uint32_t *>(&t);
          }
          *reinterpret_cast<uint4 *>(o) = make_uint4(p[0], p[1], p[2], p[3]);
        }
      }
    }
    // the next tile overwrites shared and tensor memory: order this tile's reads before it
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
  }

  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d),
                 "r"(static_cast<uint32_t>(a.tmem_cols))
                 : "memory");
}

}  // namespace
}  // namespace cxg

using namespace cxg;

extern "C" int cxg_typed_matmul_workspace_size(int num_rel, int k, int n, int dtype, size_t *bytes) {
  CXG_REQUIRE(bytes != nullptr, CXG_ENULL, "cxg_typed_matmul_workspace_size: bytes is NULL");
  CXG_REQUIRE(num_rel > 0 && k > 0 && n > 0 && (dtype == CXG_F32 || dtype == CXG_BF16), CXG_EINVAL,
              "cxg_typed_matmul_workspace_size: bad arguments");
  *bytes = 256 + align_up(static_cast<size_t>(num_rel) * k * n * (dtype == CXG_F32 ? 4 : 2), 256);
  return CXG_OK;
}

extern "C" int cxg_typed_matmul(const void *a, const void *w, void *c, const int64_t *rel, const int64_t *src_idx,
                                const int64_t *dst_idx, int64_t m, int64_t m_valid, int k, int n, int num_rel, int dtype,
                                int precision, int seq_output, void *workspace, size_t workspace_bytes, void *stream) {
  CXG_REQUIRE(m >= 0 && m_valid >= 0 && k > 0 && n > 0 && num_rel > 0, CXG_EINVAL, "cxg_typed_matmul: bad sizes");
  CXG_REQUIRE(dtype == CXG_F32 || dtype == CXG_BF16, CXG_EINVAL, "cxg_typed_matmul: dtype %d", dtype);
  CXG_REQUIRE(precision == 0 || precision == 1, CXG_EINVAL, "cxg_typed_matmul: precision %d", precision);
  if (m == 0) return CXG_OK;
  CXG_REQUIRE(a && w && c && rel, CXG_ENULL, "cxg_typed_matmul: NULL argument");
  cudaStream_t st = as_stream(stream);
  const int follows = (src_idx != nullptr && dst_idx == nullptr && !seq_output) ? 1 : 0;
  if (precision == 0)  // exact fp32 accumulation of every product, no tensor cores
    return typed_rows_launch(a, w, c, rel, 8, src_idx, dst_idx, m, m_valid, k, n, num_rel, dtype, 0, follows, st);

  const int elem = dtype == CXG_F32 ? 4 : 2;
  const int epc = 16 / elem;
  CXG_REQUIRE(k % (2 * epc) == 0, CXG_EUNSUPPORTED, "cxg_typed_matmul: K = %d must be a multiple of %d on the tensor path",
              k, 2 * epc);
  CXG_REQUIRE(n % 16 == 0 && n >= 16 && n <= 256, CXG_EUNSUPPORTED,
              "cxg_typed_matmul: N = %d must be a multiple of 16 in [16, 256] on the tensor path", n);
  const size_t smem = static_cast<size_t>(kTileM + n) * k * elem;
  CXG_REQUIRE(smem <= 200 * 1024, CXG_ELIMIT, "cxg_typed_matmul: tile of %zu bytes exceeds shared memory", smem);
  CXG_REQUIRE(reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0 && (k * elem) % 16 == 0 &&
                  (n * elem) % 16 == 0,
              CXG_EINVAL, "cxg_typed_matmul: A, C and their rows must be 16-byte aligned");
  size_t need = 0;
  cxg_typed_matmul_workspace_size(num_rel, k, n, dtype, &need);
  CXG_REQUIRE(workspace != nullptr && workspace_bytes >= need, CXG_EWORKSPACE,
              "cxg_typed_matmul: workspace %zu bytes, need %zu", workspace_bytes, need);
  CXG_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0, CXG_EINVAL, "cxg_typed_matmul: workspace alignment");

  TmmArgs t;
  t.a = a, t.c = c, t.rel = rel, t.src = src_idx, t.dst = dst_idx;
  t.m = m, t.m_valid = m_valid, t.k = k, t.n = n, t.num_rel = num_rel, t.out_follows_src = follows;
  t.status = reinterpret_cast<int32_t *>(workspace);
  void *wt = reinterpret_cast<char *>(workspace) + 256;
  t.wt = wt;
  int cols = 32;
  while (cols < n) cols <<= 1;
  t.tmem_cols = cols;
  if (cudaMemsetAsync(t.status, 0, 256, st) != cudaSuccess) return check_launch("cxg_typed_matmul: memset");
  const int64_t n_tiles = (m + kTileM - 1) / kTileM;
  // CTAs per SM: limited by shared memory and by 512 tensor-memory columns
  int per_sm = static_cast<int>((220 * 1024) / (smem + 1024));
  if (per_sm > 512 / cols) per_sm = 512 / cols;
  if (per_sm > 8) per_sm = 8;
  if (per_sm < 1) per_sm = 1;
  int64_t grid = static_cast<int64_t>(kNumSM) * per_sm;
  if (grid > n_tiles) grid = n_tiles;
  cudaError_t e;
  if (dtype == CXG_F32) {
    transpose_w<float><<<kNumSM, 256, 0, st>>>(static_cast<const float *>(w), static_cast<float *>(wt), num_rel, k, n);
    e = cudaFuncSetAttribute(typed_mm_tc<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e == cudaSuccess) typed_mm_tc<float><<<static_cast<unsigned>(grid), kMmThreads, smem, st>>>(t);
  } else {
    transpose_w<__nv_bfloat16><<<kNumSM, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(w),
                                                       static_cast<__nv_bfloat16 *>(wt), num_rel, k, n);
    e = cudaFuncSetAttribute(typed_mm_tc<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem));
    if (e == cudaSuccess) typed_mm_tc<__nv_bfloat16><<<static_cast<unsigned>(grid), kMmThreads, smem, st>>>(t);
  }
  if (e != cudaSuccess) return set_error(CXG_ECUDA, "cxg_typed_matmul: %s", cudaGetErrorString(e));
  count_launches(2);
  return check_launch("cxg_typed_matmul");
}
