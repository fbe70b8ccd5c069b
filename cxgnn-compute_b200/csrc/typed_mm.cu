// Typed (relation-bucketed) matmul for RGCN on the 5th-generation tensor cores:
//   C[oc(m), :] = A[ia(m), :] . W[rel(tile of m)]      for positions m = 0 .. M-1
// where every aligned block of 128 positions holds one relation (that is what the padding of
// TypedLinearE2EOP.preprocess guarantees, cxgnncomp/typed_linear.py:74-87), ia gathers the rows of
// A and oc scatters the rows of C. It replaces the four Triton kernels behind typed_matmul
// (cxgnncomp/codegen/triton_typed_matmul.py:145-749: no index / single index / single index with
// sequential output / source + destination index), whose tl.dot is a TF32 mma.sync on Ampere.
//
// A persistent, warp-specialised CTA per SM owns a contiguous range of 128-position tiles (so the
// relation changes at most num_rel times per CTA) and runs three roles that meet only at mbarriers:
//   * 4 or 8 producer warps gather the 128 rows of A of a tile with 16-byte `cp.async` copies into
//     one stage of a shared-memory ring, in the K-major "core matrix" layout the tensor core reads
//     without swizzle (8 rows x 16 bytes per core matrix; padding rows are zero-filled by a copy
//     of size 0), and hand the stage over with `cp.async.mbarrier.arrive.noinc`: the barrier counts
//     a thread's arrival when its copies have landed, so a producer never waits for its own
//     copies and up to `stages` tiles are in flight per CTA (waiting with `cp.async.wait_group`
//     plus a proxy fence in the producer serialised copy and MMA latency and was 13-19 % slower).
//     The thread that issues the MMAs executes the generic-to-async proxy fence after the barrier.
//     The op is memory-bound at RGCN shapes (K = 128, N = 64: 43 flop per byte in bf16). W[rel]
//     (pre-transposed once to [N][K]) is copied the same way when the relation changes, after
//     the MMAs that read the previous one have drained;
//   * one thread issues K/16 (bf16) or K/8 (tf32) `tcgen05.mma` instructions per tile with M = 128,
//     N = n, accumulating fp32 in one of two tensor-memory buffers, and commits them to the
//     barrier that frees the stage and to the one that hands the accumulator to the epilogue;
//   * 8 epilogue warps (4 in the error-compensated mode, where converter warps take the other four places)
//     read their 32 accumulator lanes with `tcgen05.ld` - two groups of four warps, each group one half of the
//     columns, 64 (fp32: 32) columns per round trip to tensor memory - convert, and write (or atomically add)
//     the rows of C at their scattered destinations while the next tile's MMAs run into the other buffer.
//     (With four warps and one round trip per 16 columns the epilogue bounded the kernel: 0.28 us per 16
//     columns of a tile, 5.5 us per 256-column tile of the dense mode.)
//
// fp32 inputs have two tensor-core modes. Plain TF32 (precision 1) feeds the fp32 words to `kind::tf32` as they
// are, like the reference's tl.dot: products carry 10 mantissa bits (about 6e-4 relative on these shapes). The
// error-compensated mode (precision 2, "3xTF32") splits every operand into hi = tf32(v) and lo = tf32(v - hi) and
// accumulates A_hi.W_lo + A_lo.W_hi + A_hi.W_hi into the same tensor-memory accumulator, which restores fp32
// accuracy (about 1e-6) while the tensor pipe, idle most of the time on this memory-bound op, absorbs the two
// extra instructions. W is split once by the transposing pre-pass; a tile of A is split in shared memory by
// converter warps between the producers and the MMA thread (raw -> hi in place, lo into the second half of
// the stage). To keep several stages in flight with stages twice as large, the K dimension is cut into blocks:
// the pipeline unit is (tile, K-block) and all blocks of a tile accumulate into one accumulator buffer.
//
// Dense mode (CXG_TMM_ALL_RELATIONS): C[r * m_valid + i, :] = A[i, :] . W[r] for every row i and EVERY relation r, the
// "transform all nodes with every relation's weight" step of the transform-first RGCN schedule
// (TypedLinearS2DMMAggrOP, cxgnncomp/typed_linear.py:191-221, which the reference runs as num_rel torch.mm calls).
// No index arrays: a CTA owns P consecutive relations (as many as fit: their weights side by side are one B operand
// of P * N columns, P * N <= 256) and the row tiles of one group; W is copied once per CTA, a tile of A is
// multiplied by all P weights with one set of MMAs, and the num_rel / P CTAs of a group walk the same tiles at the
// same time, so a tile of A comes from HBM once and from L2 for the other relation sets.
//
// Every wait is bounded: a role that waits longer than about a second raises a CTA-wide abort
// flag and an error status; all roles then leave their loops, the copies in flight are waited
// for, the tensor memory is released and the kernel returns.
#include <cuda.h>  // CUtensorMap and its enums; the encoder is obtained through the runtime, nothing links libcuda

#include "common.cuh"

namespace cxg {

int typed_rows_launch(const void *a, const void *w, void *out, const void *rel, int rel_bytes, const int64_t *src,
                      const int64_t *dst, int64_t m, int64_t m_valid, int k, int n, int num_rel, int dtype, int mode,
                      int out_follows_src, cudaStream_t st);

namespace {

constexpr int kTileM = 128;
constexpr int kEpiWarps = 4;
constexpr int kMaxProdWarps = 8;  // producer warps: 8 for 4-byte elements, 4 for 2-byte ones (measured)
#ifndef CXG_TMM_CONV_WARPS
#define CXG_TMM_CONV_WARPS 4
#endif
constexpr int kConvWarps = CXG_TMM_CONV_WARPS;  // converter warps of the error-compensated fp32 mode
constexpr int kMmaWarp = kEpiWarps;                              // warp 4
constexpr int kMaxStages = 6;
constexpr int kRpi = 8, kCpi = 32 / kRpi;  // rows / chunks per warp copy instruction
constexpr int kSmemBudget = 226 * 1024;

struct TmmArgs {
  const void *a;
  const void *wt;  // [R][N][K], K contiguous
  void *c;
  const int64_t *rel;
  const int64_t *src;
  const int64_t *dst;
  int64_t m, m_valid;
  int k, n, num_rel, out_follows_src;
  int atomic;  // add the rows into a float32 C with vector reductions instead of storing them
  int tmem_cols;  // columns of ONE accumulator buffer (two are allocated)
  int stages;     // shared-memory stages of A
  int kb;         // K-block: columns of A per pipeline unit (= k unless the stage would not fit several times)
  int dense;       // dense mode: relations per CTA (0 = off); n is then dense * ncols (see below)
  int ncols;       // columns of C per relation (= n outside dense mode)
  int test_stall;  // test hook: the producers never hand over the first tile, so the waits for it run out
  long long wait_cycles;  // limit of one barrier wait
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

// The same for a tile that the bulk tensor copy unit (TMA) wrote with its 128-byte swizzle: rows of 128 bytes (one
// swizzle span of K), 8-row groups 1024 bytes apart, the 16-byte chunks of a row permuted by (row % 8). The tile must
// start on a 1024-byte boundary; K advances inside the span by adding bytes to `addr`.
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3fff);
  d |= 1ull << 16;                                   // leading offset: unused with a swizzle, canonical value 1
  d |= static_cast<uint64_t>(1024 >> 4) << 32;       // next 8-row group
  d |= 1ull << 46;                                   // descriptor version of sm_100
  d |= 2ull << 61;                                   // layout type: 128-byte swizzle
  return d;
}

// One tiled 2-D bulk tensor copy global -> shared (x = element column, y = row of the tensor map's matrix); its bytes
// are counted on `bar`. x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Four rows of the tensor map's matrix (any four: y0 .. y3), columns [x, x + box width), into 4 x 128 consecutive
// bytes of shared memory (tile::gather4; the map's box is one row high). Rows outside the matrix arrive as zeros.
__device__ __forceinline__ void tma_gather4(uint32_t dst, const CUtensorMap *map, int x, int y0, int y1, int y2, int y3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, "
      "%6, %7}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3)
      : "memory");
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

__device__ __forceinline__ float to_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}

__device__ __forceinline__ float trunc_tf32(float v) { return __uint_as_float(__float_as_uint(v) & 0xffffe000u); }

// W [R][K][N] -> Wt [R][N][K]; with `wt_lo` (fp32 only) the two TF32 terms hi = tf32(w), lo = tf32(w - hi).
template <typename T>
__global__ void transpose_w(const T *w, T *wt, T *wt_lo, int num_rel, int k, int n) {
  const int64_t total = static_cast<int64_t>(num_rel) * k * n;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / (static_cast<int64_t>(k) * n);
    const int rem = static_cast<int>(i - r * k * n);
    const int nn = rem / k, kk = rem - nn * k;
    const T v = w[(r * k + kk) * n + nn];
    if constexpr (sizeof(T) == 4) {
      if (wt_lo != nullptr) {
        const float hi = to_tf32(v);
        wt[i] = hi;
        wt_lo[i] = to_tf32(v - hi);
        continue;
      }
    }
    wt[i] = v;
  }
}

struct Barriers {
  uint64_t full[kMaxStages];   // producers -> MMA (or -> converters): the stage holds a unit (one arrival per producer thread)
  uint64_t conv[kMaxStages];   // converters -> MMA: hi / lo halves of the stage are written (128 arrivals)
  uint64_t empty[kMaxStages];  // MMA -> producers: the MMAs that read the stage are done (1 commit)
  uint64_t acc_full[2];        // MMA -> epilogue (1 commit)
  uint64_t acc_empty[2];       // epilogue -> MMA (128 arrivals)
};

// Bounded wait on phase `parity`; false after a time-out here or an abort raised by another role.
__device__ __forceinline__ bool wait_bar(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int32_t *status,
                                         long long limit) {
  const uint32_t b = smem_addr(bar);
  if (mbar_try_wait(b, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(b, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > limit) {
      *abort_flag = 1;
      atomicExch(status, 1);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// 16-byte asynchronous copy; CA = through L1 (adjacent lanes' chunks merge into one request per line, which
// is what a gather of re-used rows wants), otherwise L2 only (faster when every row is read once).
template <bool CA>
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, int bytes) {
  if (CA)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
  else
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

// 16 consecutive 32-bit columns of this warp's 32 accumulator lanes; completion is awaited by the caller
__device__ __forceinline__ void tmem_ld16(uint32_t *v, uint32_t taddr) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
}

__device__ __forceinline__ void st_global_v4(void *p, uint4 v) {
  asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// PW producer warps; each copies 128 / PW rows of a tile, kSlots of them per thread. X3: error-compensated
// fp32 (three TF32 products per term), with kConvWarps converter warps behind the producers.
// TMA: (dense mode) the tiles of A are not gathered by the producers' 16-byte copies but fetched by the bulk tensor copy
// unit, boxes of 128 rows x 128 bytes with the 128-byte swizzle, issued by one producer thread. The converters of the
// compensated mode work element by element, so they keep whatever layout the stage has.
template <typename T, bool CA, int PW, bool X3, bool TMA>
__global__ void __launch_bounds__(32 * (kEpiWarps + 1 + PW + (X3 ? kConvWarps : kEpiWarps)), 1)
    typed_mm_tc(TmmArgs a, const __grid_constant__ CUtensorMap tmap_a) {
  constexpr int kProdWarps = PW;
  constexpr int kRowsPerProdWarp = kTileM / kProdWarps;
  constexpr int kSlots = kRowsPerProdWarp / kRpi;
  constexpr int kIdx = kSlots < 4 ? 4 : kSlots;  // row indices a producer thread keeps (four for a gathering bulk copy)
  constexpr bool TF32 = sizeof(T) == 4;
  constexpr int EPC = 16 / sizeof(T);  // elements per 16-byte chunk
  constexpr int kFirstConvWarp = kMmaWarp + 1 + PW;
  // Without converter warps a second group of four epilogue warps sits in their place: the two groups share a
  // tile's accumulator by columns (a warp reads the tensor-memory lanes 32 * (warp % 4) .. + 31, whatever its group).
  constexpr bool E2 = !X3;
  constexpr int kEpiAll = E2 ? 2 * kEpiWarps : kEpiWarps;
  static_assert(!X3 || TF32, "the error-compensated mode is for fp32 inputs");
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) Barriers bars;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_slot;
  volatile int *abort_flag = &abort_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunks = a.k / EPC;             // 16-byte chunks per full row (layout of W in shared memory)
  const int chunks_blk = a.kb / EPC;        // 16-byte chunks per row of one K-block (layout of a stage of A)
  const int nkb = a.k / a.kb;               // K-blocks per tile
  const uint32_t lbo = 128;                 // next core matrix along K
  const uint32_t sbo_a = chunks_blk * 128;  // next 8-row group inside a stage of A
  const uint32_t sbo_b = chunks * 128;      // next 8-row group of W
  const int S = a.stages;
  const size_t half_bytes = static_cast<size_t>(kTileM) * a.kb * sizeof(T);  // one [128][kb] tile
  const size_t a_bytes = X3 ? 2 * half_bytes : half_bytes;                   // a stage: raw / hi (+ lo)
  const size_t w_bytes = static_cast<size_t>(a.n) * a.k * sizeof(T);        // n rows of W[rel]^T
  uint8_t *smem_b = smem;                                    // W (hi), then W lo in the compensated mode
  uint8_t *smem_a = smem + (X3 ? 2 * w_bytes : w_bytes);     // S stages
  if (TMA) smem_a += (1024u - (smem_addr(smem_a) & 1023u)) & 1023u;  // swizzled tiles start on 1024-byte boundaries

  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)),
                 "r"(static_cast<uint32_t>(2 * a.tmem_cols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    abort_slot = 0;
    for (int s = 0; s < kMaxStages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.full[s])), "r"(32 * kProdWarps) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.conv[s])), "r"(32 * kConvWarps) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&bars.empty[s])) : "memory");
    }
    for (int b = 0; b < 2; ++b) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&bars.acc_full[b])) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.acc_empty[b])), "r"(32 * kEpiAll) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_slot;

  const T *A = static_cast<const T *>(a.a);
  const int64_t n_tiles = (a.m + kTileM - 1) / kTileM;
  const bool dense = a.dense != 0;
  const int rel_sets = dense ? a.num_rel / a.dense : 1;                   // CTAs per group of row tiles
  const int64_t dense_rel = dense ? (blockIdx.x % rel_sets) * a.dense : 0;  // first relation of this CTA in dense mode
  const int64_t part = dense ? blockIdx.x / rel_sets : blockIdx.x, parts = dense ? gridDim.x / rel_sets : gridDim.x;
  const int64_t tile_lo = n_tiles * part / parts, tile_hi = n_tiles * (part + 1) / parts;
  // relation of a tile: the position array's, or the CTA's own in dense mode
  auto rel_of = [&](int64_t tile) -> int64_t { return tile < tile_hi ? (dense ? dense_rel : a.rel[tile * kTileM]) : -1; };

  if (warp > kMmaWarp && warp < kFirstConvWarp) {
    // ================= producers: gather A (and W on a relation change) =================
    const int pw = warp - kMmaWarp - 1;          // producer warp: owns rows pw * kRowsPerProdWarp .. of every tile
    // one copy instruction of a warp covers kRpi rows x kCpi consecutive 16-byte chunks
    const int rsub = lane / kCpi, cq = lane % kCpi;
    const T *Wt = static_cast<const T *>(a.wt);
    int64_t loaded_rel = -1;
    int64_t it = 0;        // units (tile, K-block) issued by this CTA
    bool alive = true;
    // the relation and the row indices of a tile are fetched one tile ahead, off the critical path
    auto fetch = [&](int64_t tile, int64_t &r, int64_t (&ia)[kIdx]) {
      const int64_t m0 = tile * kTileM;
      r = rel_of(tile);
#pragma unroll
      for (int gi = 0; gi < kIdx; ++gi) {
        // warp pw owns kRowsPerProdWarp rows; with gathering bulk tensor copies lane l of warp 0 asks for rows 4l .. 4l+3
        const bool g4 = TMA && !dense;
        const int64_t pos = g4 ? m0 + 4 * lane + gi : m0 + pw * kRowsPerProdWarp + gi * kRpi + rsub;
        ia[gi] = -1;
        if (g4 ? gi >= 4 : gi >= kSlots) continue;
        if (tile < tile_hi && pos < a.m) ia[gi] = a.src != nullptr ? a.src[pos] : pos;
      }
    };
    int64_t r_next, ia_next[kIdx];
    fetch(tile_lo, r_next, ia_next);
    for (int64_t tile = tile_lo; tile < tile_hi && alive; ++tile) {
      const int64_t r = r_next;
      int64_t ia[kIdx];
#pragma unroll
      for (int gi = 0; gi < kIdx; ++gi) ia[gi] = ia_next[gi];
      fetch(tile + 1, r_next, ia_next);
      if (r < 0 || r >= a.num_rel) continue;  // a tile of padding only
      if (r != loaded_rel) {
        // every MMA issued so far reads the old W: let them finish
        for (int64_t j = (it > S ? it - S : 0); j < it && alive; ++j)
          alive = wait_bar(&bars.empty[j % S], static_cast<uint32_t>((j / S) & 1), abort_flag, a.status, a.wait_cycles);
        if (!alive) break;
        const int64_t w_elems = static_cast<int64_t>(a.ncols) * a.k;  // one relation's weight (dense: P of them in a row)
        const uint32_t b0 = smem_addr(smem_b);
        for (int part = 0; part < (X3 ? 2 : 1); ++part) {  // hi, then lo
          const T *wr = Wt + (part * static_cast<int64_t>(a.num_rel) + r) * w_elems;
          const uint32_t bp = b0 + part * static_cast<uint32_t>(w_bytes);
          for (int row = pw * kRpi + rsub; row < a.n; row += kProdWarps * kRpi)
            for (int c = cq; c < chunks; c += kCpi)
              cp_async16<false>(bp + (row >> 3) * sbo_b + c * 128 + (row & 7) * 16, wr + static_cast<int64_t>(row) * a.k + c * EPC, 16);
        }
        loaded_rel = r;
      }
      for (int kb = 0; kb < nkb && alive; ++kb) {
        const int s = static_cast<int>(it % S);
        if (it >= S) {
          alive = wait_bar(&bars.empty[s], static_cast<uint32_t>(((it / S) - 1) & 1), abort_flag, a.status, a.wait_cycles);
          if (!alive) break;
        }
        const uint32_t a0 = smem_addr(smem_a + s * a_bytes);
        if (TMA) {
          // one thread announces the tile's bytes on the stage barrier and asks the copy unit for its boxes (rows past
          // the end of A arrive as zeros); its own arrival below comes after the announcement, so the phase cannot
          // complete without the bytes
          const uint32_t bar = smem_addr(&bars.full[s]);
          const int span = 128 / static_cast<int>(sizeof(T));  // elements of K per 128-byte swizzle span
          if (pw == 0 && lane == 0)
            asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar),
                         "r"(static_cast<uint32_t>(half_bytes))
                         : "memory");
          if (dense) {
            if (pw == 0 && lane == 0)
              for (int h = 0; h * span < a.kb; ++h)
                tma_load_2d(a0 + h * (kTileM * 128), &tmap_a, kb * a.kb + h * span, static_cast<int>(tile * kTileM), bar);
          } else if (pw == 0) {
            // gathered rows: every lane of the first producer warp asks for its four rows of every span; a position
            // without a row (padding, index out of range) names the row past the matrix and receives zeros
            __syncwarp();  // the announcement above precedes every request
            int y[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              y[i] = (ia[i] >= 0 && ia[i] < a.m_valid) ? static_cast<int>(ia[i]) : static_cast<int>(a.m_valid);
            for (int h = 0; h * span < a.kb; ++h)
              tma_gather4(a0 + h * (kTileM * 128) + lane * 512, &tmap_a, kb * a.kb + h * span, y[0], y[1], y[2], y[3], bar);
          }
        } else {
#pragma unroll
          for (int gi = 0; gi < kSlots; ++gi) {
            const int row = pw * kRowsPerProdWarp + gi * kRpi + rsub;  // row of the tile
            const bool ok = ia[gi] >= 0 && ia[gi] < a.m_valid;
            const T *src_row = ok ? A + ia[gi] * a.k + kb * a.kb : A;
            const int bytes = ok ? 16 : 0;  // size 0 writes zeros
            const uint32_t d0 = a0 + (row >> 3) * sbo_a + (row & 7) * 16;
            for (int c = cq; c < chunks_blk; c += kCpi) cp_async16<CA>(d0 + c * 128, src_row + c * EPC, bytes);
          }
        }
        // the unit's full barrier counts this thread's arrival when all copies it has issued so far (this unit's
        // rows, and W when it was re-copied) have landed: the producer never waits for its own copies
        if (!(a.test_stall && it == 0))
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&bars.full[s])) : "memory");
        ++it;
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (X3 && warp >= kFirstConvWarp) {
    // ================= converters: raw fp32 stage -> hi (in place) and lo (second half) =================
    const int ct = tid - 32 * kFirstConvWarp;  // 0 .. 32 * kConvWarps - 1
    const int n16 = static_cast<int>(half_bytes / 16);
    int64_t it = 0;
    bool alive = true;
    for (int64_t tile = tile_lo; tile < tile_hi && alive; ++tile) {
      const int64_t r = rel_of(tile);
      if (r < 0 || r >= a.num_rel) continue;
      for (int kb = 0; kb < nkb && alive; ++kb) {
        const int s = static_cast<int>(it % S);
        alive = wait_bar(&bars.full[s], static_cast<uint32_t>((it / S) & 1), abort_flag, a.status, a.wait_cycles);
        if (!alive) break;
        float4 *hi = reinterpret_cast<float4 *>(smem_a + s * a_bytes);
        float4 *lo = reinterpret_cast<float4 *>(smem_a + s * a_bytes + half_bytes);
        for (int c = ct; c < n16; c += 32 * kConvWarps) {
          // hi = the upper 19 bits of v, lo = the upper 19 bits of v - hi: both are exact TF32 values (one
          // logic op each instead of a conversion instruction), v - hi is exact in fp32
          const float4 v = hi[c];
          float4 h, l;
          h.x = trunc_tf32(v.x), h.y = trunc_tf32(v.y), h.z = trunc_tf32(v.z), h.w = trunc_tf32(v.w);
          l.x = trunc_tf32(v.x - h.x), l.y = trunc_tf32(v.y - h.y), l.z = trunc_tf32(v.z - h.z), l.w = trunc_tf32(v.w - h.w);
          hi[c] = h;
          lo[c] = l;
        }
        // these generic-proxy writes are read by the tensor core through the async proxy
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(&bars.conv[s]);
        ++it;
      }
    }
  } else if (warp == kMmaWarp) {
    // ================= MMA issuer =================
    if (lane == 0) {
      const uint32_t idesc = make_idesc(TF32 ? 2 : 1, kTileM, a.n);
      const uint32_t b0 = smem_addr(smem_b);
      const int steps = chunks_blk / 2;  // two chunks (32 bytes) of K per instruction
      int64_t it = 0, tile_it = 0;
      bool alive = true;
      int64_t r_next = rel_of(tile_lo);
      for (int64_t tile = tile_lo; tile < tile_hi && alive; ++tile) {
        const int64_t r = r_next;
        r_next = rel_of(tile + 1);
        if (r < 0 || r >= a.num_rel) continue;
        const int buf = static_cast<int>(tile_it & 1);
        const uint32_t d = tmem_d + buf * a.tmem_cols;
        for (int kb = 0; kb < nkb && alive; ++kb) {
          const int s = static_cast<int>(it % S);
          alive = wait_bar(X3 ? &bars.conv[s] : &bars.full[s], static_cast<uint32_t>((it / S) & 1), abort_flag, a.status,
                           a.wait_cycles);
          if (alive && kb == 0 && tile_it >= 2)
            alive = wait_bar(&bars.acc_empty[buf], static_cast<uint32_t>(((tile_it >> 1) - 1) & 1), abort_flag, a.status,
                             a.wait_cycles);
          if (!alive) break;
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a0 = smem_addr(smem_a + s * a_bytes);
          const uint32_t bk = b0 + kb * chunks_blk * 128;  // this K-block's columns of W
          for (int j = 0; j < steps; ++j) {
            const uint32_t first = (kb > 0 || j > 0) ? 1u : 0u;
            if (X3) {
              const uint32_t ao = TMA ? (j >> 2) * (kTileM * 128) + (j & 3) * 32 : j * 256;  // as in the plain branch below
              const uint64_t da_hi = TMA ? make_desc_sw128(a0 + ao) : make_desc(a0 + ao, lbo, sbo_a);
              const uint64_t da_lo = TMA ? make_desc_sw128(a0 + static_cast<uint32_t>(half_bytes) + ao)
                                         : make_desc(a0 + static_cast<uint32_t>(half_bytes) + ao, lbo, sbo_a);
              const uint64_t db_hi = make_desc(bk + j * 256, lbo, sbo_b);
              const uint64_t db_lo = make_desc(bk + static_cast<uint32_t>(w_bytes) + j * 256, lbo, sbo_b);
              mma_ss<TF32>(d, da_hi, db_lo, idesc, first);  // the two small terms first, the large one last
              mma_ss<TF32>(d, da_lo, db_hi, idesc, 1u);
              mma_ss<TF32>(d, da_hi, db_hi, idesc, 1u);
            } else if (TMA) {
              // step j reads 32 bytes of K: span j / 4 of the stage (16 KiB each), 32-byte offset j % 4 inside it
              mma_ss<TF32>(d, make_desc_sw128(a0 + (j >> 2) * (kTileM * 128) + (j & 3) * 32),
                           make_desc(bk + j * 256, lbo, sbo_b), idesc, first);
            } else {
              mma_ss<TF32>(d, make_desc(a0 + j * 256, lbo, sbo_a), make_desc(bk + j * 256, lbo, sbo_b), idesc, first);
            }
          }
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                           smem_addr(&bars.empty[s]))
                       : "memory");
          ++it;
        }
        if (!alive) break;
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                         smem_addr(&bars.acc_full[buf]))
                     : "memory");
        ++tile_it;
      }
      // the epilogue of the last tiles must be over before the tensor memory goes away: it arrives on
      // acc_empty, which the final __syncthreads of the epilogue warps also orders.
    }
    __syncwarp();
  } else {
    // ================= epilogue: a warp owns accumulator lanes 32 * (warp % 4) .. + 31 = tile rows =================
    T *C = static_cast<T *>(a.c);
    const int quarter = warp & 3;
    const int grp = (E2 && warp >= kFirstConvWarp) ? 1 : 0;
    // columns of this group: the first or the second half of the accumulator, in units of 16
    const int n_half = E2 ? ((a.n / 16 + 1) / 2) * 16 : a.n;
    const int c_lo = grp ? n_half : 0, c_hi = grp ? a.n : n_half;
    const int rel_lo = dense ? c_lo / a.ncols : 0, cc_lo = dense ? c_lo % a.ncols : c_lo;
    int64_t it = 0;
    bool alive = true;
    // relation, source and destination index of this thread's row, fetched one tile ahead
    auto fetch = [&](int64_t tile, int64_t &r, int64_t &sv, int64_t &dv) {
      const int64_t m0 = tile * kTileM, pos = m0 + quarter * 32 + lane;
      r = rel_of(tile);
      sv = -1, dv = -1;
      if (tile < tile_hi && pos < a.m) {
        sv = a.src != nullptr ? a.src[pos] : pos;
        dv = a.dst != nullptr ? a.dst[pos] : -2;  // -2: no destination index
        if (dense) dv = dense_rel * a.m_valid + pos;  // row of the [num_rel * m_valid, ncols] table, first relation
      }
    };
    int64_t r_next, sv_next, dv_next;
    fetch(tile_lo, r_next, sv_next, dv_next);
    for (int64_t tile = tile_lo; tile < tile_hi && alive; ++tile) {
      const int64_t r = r_next, sv = sv_next, dv = dv_next;
      fetch(tile + 1, r_next, sv_next, dv_next);
      if (r < 0 || r >= a.num_rel) continue;
      int64_t oc = -1;
      if (sv >= 0 && sv < a.m_valid) oc = dv != -2 ? dv : (a.out_follows_src ? sv : tile * kTileM + quarter * 32 + lane);
      const int buf = static_cast<int>(it & 1);
      alive = wait_bar(&bars.acc_full[buf], static_cast<uint32_t>((it >> 1) & 1), abort_flag, a.status, a.wait_cycles);
      if (!alive) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem_d + (static_cast<uint32_t>(quarter * 32) << 16) + buf * a.tmem_cols;
      if (a.atomic) {
        if (c_lo >= c_hi) {  // nothing for this group (n = 16): only hand the buffer back
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          mbar_arrive(&bars.acc_empty[buf]);
        }
        for (int c0 = c_lo; c0 < c_hi; c0 += 16) {
          uint32_t v[16];
          tmem_ld16(v, taddr + c0);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (c0 + 16 >= c_hi) {  // the accumulator buffer is in registers: give it back to the MMA thread
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&bars.acc_empty[buf]);
          }
          if (oc >= 0) {
            float *o = static_cast<float *>(a.c) + oc * a.n + c0;
#pragma unroll
            for (int q = 0; q < 4; ++q)
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + 4 * q), "f"(__uint_as_float(v[4 * q])),
                           "f"(__uint_as_float(v[4 * q + 1])), "f"(__uint_as_float(v[4 * q + 2])),
                           "f"(__uint_as_float(v[4 * q + 3]))
                           : "memory");
          }
        }
      } else {
        // Store epilogue. The accumulator is read in groups of 64 (32) columns (four (two) loads in flight, one wait),
        // so that a tile of n columns costs n / 64 round trips to tensor memory instead of n / 16. Two adjacent
        // lanes trade 16-byte quads so that one store instruction of the pair writes one whole 32-byte sector.
        const bool odd = lane & 1;
        const int64_t oc_a = __shfl_sync(0xffffffffu, oc, lane & ~1), oc_b = __shfl_sync(0xffffffffu, oc, lane | 1);
        // dense mode: columns [j * ncols, (j + 1) * ncols) of the accumulator are relation dense_rel + j, whose rows
        // start j * m_valid rows further down the table; cc = column inside the relation's row
        const int64_t rel_step = dense ? a.m_valid * a.ncols : 0;
        T *row_a = C + oc_a * a.ncols + rel_lo * rel_step, *row_b = C + oc_b * a.ncols + rel_lo * rel_step;
        int cc = cc_lo;
        constexpr int GU = TF32 ? 2 : 4;  // loads of 16 columns per round trip (fp32 kernels have fewer registers per thread)
        if (c_lo >= c_hi) {  // nothing for this group (n = 16): only hand the buffer back
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          mbar_arrive(&bars.acc_empty[buf]);
        }
        for (int g0 = c_lo; g0 < c_hi; g0 += 16 * GU) {
          uint32_t v[16 * GU];
#pragma unroll
          for (int u = 0; u < GU; ++u)
            if (g0 + 16 * u < c_hi) tmem_ld16(v + 16 * u, taddr + g0 + 16 * u);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (g0 + 16 * GU >= c_hi) {  // the accumulator buffer is in registers: give it back to the MMA thread
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&bars.acc_empty[buf]);
          }
#pragma unroll
          for (int u = 0; u < GU; ++u) {
            if (g0 + 16 * u >= c_hi) break;
            constexpr int NQ = TF32 ? 4 : 2;
            uint4 q[NQ];
            if (TF32) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                q[j % NQ] = make_uint4(v[16 * u + 4 * j], v[16 * u + 4 * j + 1], v[16 * u + 4 * j + 2], v[16 * u + 4 * j + 3]);
            } else {
              uint32_t p[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(v[16 * u + 2 * j]), __uint_as_float(v[16 * u + 2 * j + 1]));
                p[j] = *reinterpret_cast<uint32_t *>(&t);
              }
              q[0] = make_uint4(p[0], p[1], p[2], p[3]);
              q[1] = make_uint4(p[4], p[5], p[6], p[7]);
            }
            constexpr int QE = 16 / sizeof(T);  // elements per quad
#pragma unroll
            for (int h = 0; h < NQ / 2; ++h) {
              const uint4 keep = odd ? q[2 * h + 1] : q[2 * h], send = odd ? q[2 * h] : q[2 * h + 1];
              uint4 got;
              got.x = __shfl_xor_sync(0xffffffffu, send.x, 1);
              got.y = __shfl_xor_sync(0xffffffffu, send.y, 1);
              got.z = __shfl_xor_sync(0xffffffffu, send.z, 1);
              got.w = __shfl_xor_sync(0xffffffffu, send.w, 1);
              const int col = cc + (2 * h + (odd ? 1 : 0)) * QE;
              // row of the even lane: its own quad 2h, and its quad 2h+1 written by the odd lane. (One store
              // instruction for both lanes, so that the two halves leave as one sector.)
              const uint4 va = odd ? got : keep, vb = odd ? keep : got;
              if (oc_a >= 0) st_global_v4(row_a + col, va);
              if (oc_b >= 0) st_global_v4(row_b + col, vb);
            }
            cc += 16;
            if (dense && cc == a.ncols) {  // next relation of this CTA
              cc = 0;
              row_a += rel_step;
              row_b += rel_step;
            }
          }
        }
      }
      ++it;
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d),
                 "r"(static_cast<uint32_t>(2 * a.tmem_cols))
                 : "memory");
  }
}

}  // namespace
}  // namespace cxg

using namespace cxg;

namespace {

// Tensor map of a row-major [rows][k] matrix of bf16 or fp32 elements for boxes of 128 rows x one 128-byte swizzle
// span of columns (64 / 32 elements). False when the driver's encoder is not available or refuses the arguments.
bool encode_a_map(CUtensorMap *map, const void *base, int64_t rows, int k, int elem, int box_rows) {
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                               const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn fn = nullptr;
  static bool looked = false;
  if (!looked) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
    else
      (void)cudaGetLastError();
    looked = true;
  }
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * elem};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elem), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, elem == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" int cxg_typed_matmul_workspace_size(int num_rel, int k, int n, int dtype, size_t *bytes) {
  CXG_REQUIRE(bytes != nullptr, CXG_ENULL, "cxg_typed_matmul_workspace_size: bytes is NULL");
  CXG_REQUIRE(num_rel > 0 && k > 0 && n > 0 && (dtype == CXG_F32 || dtype == CXG_BF16), CXG_EINVAL,
              "cxg_typed_matmul_workspace_size: bad arguments");
  // status words + W transposed; fp32 keeps room for the hi and lo parts of the error-compensated mode
  *bytes = 256 + align_up(static_cast<size_t>(num_rel) * k * n * (dtype == CXG_F32 ? 8 : 2), 256);
  return CXG_OK;
}

extern "C" int cxg_typed_matmul(const void *a, const void *w, void *c, const int64_t *rel, const int64_t *src_idx,
                                const int64_t *dst_idx, int64_t m, int64_t m_valid, int k, int n, int num_rel, int dtype,
                                int precision, int flags, void *workspace, size_t workspace_bytes, void *stream) {
  const int seq_output = (flags & CXG_TMM_SEQ_OUTPUT) ? 1 : 0;
  const int atomic = (flags & CXG_TMM_ATOMIC_F32) ? 1 : 0;
  const int dense = (flags & CXG_TMM_ALL_RELATIONS) ? 1 : 0;
  CXG_REQUIRE(m >= 0 && m_valid >= 0 && k > 0 && n > 0 && num_rel > 0, CXG_EINVAL, "cxg_typed_matmul: bad sizes");
  CXG_REQUIRE(dtype == CXG_F32 || dtype == CXG_BF16, CXG_EINVAL, "cxg_typed_matmul: dtype %d", dtype);
  CXG_REQUIRE(precision >= 0 && precision <= 2, CXG_EINVAL, "cxg_typed_matmul: precision %d", precision);
  if (m == 0) return CXG_OK;
  CXG_REQUIRE(a && w && c && (rel || dense), CXG_ENULL, "cxg_typed_matmul: NULL argument");
  if (dense) {
    CXG_REQUIRE(precision != 0 && !atomic && src_idx == nullptr && dst_idx == nullptr && m == m_valid, CXG_EUNSUPPORTED,
                "cxg_typed_matmul: CXG_TMM_ALL_RELATIONS takes no index arrays, m == m_valid, a tensor-core precision");
    CXG_REQUIRE(num_rel <= kNumSM, CXG_ELIMIT, "cxg_typed_matmul: %d relations, at most %d in dense mode", num_rel, kNumSM);
  }
  cudaStream_t st = as_stream(stream);
  const int follows = (src_idx != nullptr && dst_idx == nullptr && !seq_output) ? 1 : 0;
  if (precision == 0) {  // exact fp32 accumulation of every product, no tensor cores
    CXG_REQUIRE(!atomic || dtype == CXG_F32, CXG_EUNSUPPORTED, "cxg_typed_matmul: exact mode adds atomically in fp32 only");
    return typed_rows_launch(a, w, c, rel, 8, src_idx, dst_idx, m, m_valid, k, n, num_rel, dtype, atomic ? 2 : 0, follows,
                             st);
  }
  const bool x3 = precision == 2 && dtype == CXG_F32;  // bf16 inputs have nothing to compensate
  const int ncols = n;  // columns of C per relation
  int rel_per_cta = 0;
  if (dense) {
    // as many relations side by side as divide num_rel, fit 256 accumulator columns and leave shared memory for at
    // least three stages of A next to their weights
    const size_t elem_b = dtype == CXG_F32 ? 4 : 2;
    for (int p = 1; p <= num_rel; ++p) {
      if (num_rel % p != 0 || p * ncols > 256) continue;
      const size_t wb = static_cast<size_t>(p) * ncols * k * elem_b * (x3 ? 2 : 1);
      const size_t stage = static_cast<size_t>(kTileM) * (k < 32 ? k : 32) * elem_b * (x3 ? 2 : 1);
      if (wb + 3 * stage <= static_cast<size_t>(kSmemBudget)) rel_per_cta = p;
    }
    CXG_REQUIRE(rel_per_cta > 0, CXG_EUNSUPPORTED, "cxg_typed_matmul: K = %d, N = %d is too large for the dense mode", k, n);
    n = rel_per_cta * ncols;
  }
  if (x3 && static_cast<size_t>(n) * k * 8 + static_cast<size_t>(kTileM) * 8 * 8 > static_cast<size_t>(kSmemBudget)) {
    // both TF32 terms of W[rel] do not fit in shared memory next to one stage: the exact kernel keeps the accuracy
    CXG_REQUIRE(!dense, CXG_EUNSUPPORTED, "cxg_typed_matmul: K = %d, N = %d is too large for the dense fp32 mode", k, n);
    CXG_REQUIRE(!atomic || dtype == CXG_F32, CXG_EUNSUPPORTED, "cxg_typed_matmul: exact mode adds atomically in fp32 only");
    return typed_rows_launch(a, w, c, rel, 8, src_idx, dst_idx, m, m_valid, k, n, num_rel, dtype, atomic ? 2 : 0, follows,
                             st);
  }

  const int elem = dtype == CXG_F32 ? 4 : 2;
  const int epc = 16 / elem;
  CXG_REQUIRE(k % (2 * epc) == 0, CXG_EUNSUPPORTED, "cxg_typed_matmul: K = %d must be a multiple of %d on the tensor path",
              k, 2 * epc);
  CXG_REQUIRE(n % 16 == 0 && n >= 16 && n <= 256, CXG_EUNSUPPORTED,
              "cxg_typed_matmul: N = %d must be a multiple of 16 in [16, 256] on the tensor path", n);
  const size_t b_bytes = static_cast<size_t>(n) * k * elem * (x3 ? 2 : 1);
  // K-block: the whole row when a stage then fits at least `want` times next to W, else halved while it stays a
  // multiple of one instruction's K (32 bytes)
  auto stage_bytes = [&](int kb) { return static_cast<size_t>(kTileM) * kb * elem * (x3 ? 2 : 1); };
  int kb = k;
  // (compensated dense mode: three stages of K-block 32 measured 7 % faster than six of K-block 16)
  const int want = dense ? 3 : (x3 ? 4 : 1);
  while (b_bytes + want * stage_bytes(kb) > static_cast<size_t>(kSmemBudget) && kb % (4 * epc) == 0) kb /= 2;
  const size_t a_bytes = stage_bytes(kb);
  CXG_REQUIRE(a_bytes + b_bytes <= static_cast<size_t>(kSmemBudget), CXG_ELIMIT,
              "cxg_typed_matmul: one stage of %zu bytes plus W of %zu bytes exceeds shared memory", a_bytes, b_bytes);
  // Dense mode: the tiles of A are contiguous row blocks, which the bulk tensor copy unit fetches as swizzled boxes of
  // 128 rows x 128 bytes, one to four per K-block (CXG_TMM_NO_TMA keeps the 16-byte copies, for comparison)
  CUtensorMap tmap;
  memset(&tmap, 0, sizeof(tmap));
  // Rows gathered by index and read once can go through the same copy unit in its gathering form (tile::gather4: four
  // rows of 128 bytes per request, box one row high) with CXG_TMM_GATHER4. It is not the default: one request per
  // 512 bytes keeps the copy unit busier than the 16-byte copies keep the producers (config 4, per-edge matmul:
  // 3.47 vs 2.07 ms in bf16, 6.95 vs 3.73 ms in TF32).
  const bool ca = src_idx != nullptr && m_valid * 2 <= m;
  const bool tma = (dense || (!ca && (flags & CXG_TMM_GATHER4))) && (kb * elem) % 128 == 0 && kb * elem <= 512 &&
                   !(flags & CXG_TMM_NO_TMA) &&
                   m < (1ll << 31) && m_valid < (1ll << 31) - 1 && m_valid > 0 &&
                   encode_a_map(&tmap, a, m_valid, k, elem, dense ? kTileM : 1);
  const size_t tma_pad = tma ? 1024 : 0;  // the stages start on a 1024-byte boundary
  int stages = static_cast<int>((kSmemBudget - b_bytes - tma_pad) / a_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  const size_t smem = b_bytes + tma_pad + stages * a_bytes;
  CXG_REQUIRE(reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0 && (k * elem) % 16 == 0 &&
                  (n * elem) % 16 == 0,
              CXG_EINVAL, "cxg_typed_matmul: A, C and their rows must be 16-byte aligned");
  size_t need = 0;
  cxg_typed_matmul_workspace_size(num_rel, k, ncols, dtype, &need);
  CXG_REQUIRE(workspace != nullptr && workspace_bytes >= need, CXG_EWORKSPACE,
              "cxg_typed_matmul: workspace %zu bytes, need %zu", workspace_bytes, need);
  CXG_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0, CXG_EINVAL, "cxg_typed_matmul: workspace alignment");

  TmmArgs t;
  t.a = a, t.c = c, t.rel = rel, t.src = src_idx, t.dst = dst_idx;
  t.m = m, t.m_valid = m_valid, t.k = k, t.n = n, t.num_rel = num_rel, t.out_follows_src = follows;
  t.atomic = atomic;
  t.dense = rel_per_cta;
  t.ncols = ncols;
  t.test_stall = (flags & CXG_TMM_TEST_STALL) ? 1 : 0;
  t.wait_cycles = wait_limit_cycles();
  t.status = reinterpret_cast<int32_t *>(workspace);
  void *wt = reinterpret_cast<char *>(workspace) + 256;
  t.wt = wt;
  int cols = 32;
  while (cols < n) cols <<= 1;
  t.tmem_cols = cols;  // two buffers: 2 * cols <= 512
  t.stages = stages;
  t.kb = kb;
  if (cudaMemsetAsync(t.status, 0, 256, st) != cudaSuccess) return check_launch("cxg_typed_matmul: memset");
  const int64_t n_tiles = (m + kTileM - 1) / kTileM;
  // one persistent CTA per SM (its shared-memory ring fills the SM), contiguous tile ranges
  int64_t grid = kNumSM;
  if (grid > n_tiles) grid = n_tiles;
  if (dense) {  // num_rel / rel_per_cta CTAs per group of row tiles
    const int sets = num_rel / rel_per_cta;
    int64_t groups = kNumSM / sets;
    if (groups > n_tiles) groups = n_tiles;
    grid = groups * sets;
  }
  // rows that are gathered several times each go through L1 (`ca` above), rows read once bypass it
  // (rows read once: L1-allocating copies measured 4-6 % slower on the dense mode as well)
  cudaError_t e = cudaSuccess;
  auto launch = [&](auto kernel, int warps) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e == cudaSuccess) kernel<<<static_cast<unsigned>(grid), 32 * warps, smem, st>>>(t, tmap);
  };
  if (dtype == CXG_F32) {
    float *wt_f = static_cast<float *>(wt);
    transpose_w<float><<<kNumSM, 256, 0, st>>>(static_cast<const float *>(w), wt_f,
                                               x3 ? wt_f + static_cast<size_t>(num_rel) * k * ncols : nullptr, num_rel, k,
                                               ncols);
    constexpr int kW = kEpiWarps + 1 + 8;
    if (x3) {
      if (tma)
        launch(typed_mm_tc<float, false, 8, true, true>, kW + kConvWarps);
      else if (ca)
        launch(typed_mm_tc<float, true, 8, true, false>, kW + kConvWarps);
      else
        launch(typed_mm_tc<float, false, 8, true, false>, kW + kConvWarps);
    } else {
      if (tma)
        launch(typed_mm_tc<float, false, 8, false, true>, kW + kEpiWarps);
      else if (ca)
        launch(typed_mm_tc<float, true, 8, false, false>, kW + kEpiWarps);
      else
        launch(typed_mm_tc<float, false, 8, false, false>, kW + kEpiWarps);
    }
  } else {
    transpose_w<__nv_bfloat16><<<kNumSM, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(w),
                                                       static_cast<__nv_bfloat16 *>(wt), nullptr, num_rel, k, ncols);
    constexpr int kW = kEpiWarps + 1 + 4;
    if (tma)
      launch(typed_mm_tc<__nv_bfloat16, false, 4, false, true>, kW + kEpiWarps);
    else if (ca)
      launch(typed_mm_tc<__nv_bfloat16, true, 4, false, false>, kW + kEpiWarps);
    else
      launch(typed_mm_tc<__nv_bfloat16, false, 4, false, false>, kW + kEpiWarps);
  }
  if (e != cudaSuccess) return set_error(CXG_ECUDA, "cxg_typed_matmul: %s", cudaGetErrorString(e));
  count_launches(2);
  return check_launch("cxg_typed_matmul");
}
