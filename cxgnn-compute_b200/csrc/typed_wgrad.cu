// Weight gradient of the typed (relation-bucketed) linear on the 5th-generation tensor cores:
//   dW[r] = sum over the positions m of relation r of  x[ix(m), :]^T (outer) g[ig(m), :]          [num_rel, K, N]
// with the positions sorted by relation and padded so that every aligned block of 128 positions holds one relation
// (TypedLinearE2EOP.preprocess, cxgnncomp/typed_linear.py:74-87). The reference computes it as one torch.mm per
// relation over row sets (typed_linear.py:115-137); here it is one launch: a contraction over POSITIONS.
//
// The contraction index is the row of both operands, so both are "MN-major" for the tensor core: a tile of 128
// positions of x ([128][K]) is the A operand A[m = column of x][k = position], a tile of g ([128][N]) the B operand.
// A tile is laid out in a 128-byte swizzle: per 128-byte span of a row one block of 128 rows x 128 bytes (row p at
// p * 128, its chunks permuted by the row number), the spans 16 KiB apart. The producers put it there themselves with
// 16-byte asynchronous copies (the rows are gathered by index).
//
// A persistent CTA per SM owns a contiguous range of tiles and accumulates consecutive tiles of one relation in
// tensor memory; when the relation changes (or the range ends) the epilogue warps flush the [K][N] accumulator to
// a partial slot of this CTA. A second kernel adds the slots of every relation in (CTA, slot) order: no atomics,
// the same bits on every run.
//
// fp32 inputs: plain TF32 products (precision 1) or, like the forward, error-compensated ones (precision 2): four
// converter warps split both tiles of a stage into hi = upper 19 bits and lo = upper 19 bits of (v - hi), and the
// tensor core accumulates A_hi.B_lo + A_lo.B_hi + A_hi.B_hi.
//
// Every wait is bounded; a role that waits too long raises a CTA-wide abort flag and an error status.
#include "common.cuh"

namespace cxg {
namespace {

constexpr int kProdWarps = 8;
constexpr int kConvWarps = 4;
constexpr int kEpiWarps = 4;    // warps 0..3: tensor-memory lanes 32 * warp .. + 31
constexpr int kMmaWarp = kEpiWarps;
constexpr int kFirstProd = kMmaWarp + 1;
constexpr int kFirstConv = kFirstProd + kProdWarps;
constexpr int kMaxStages = 4;
constexpr int kSmemBudget = 225 * 1024;

struct WgArgs {
  const void *x;       // [*, k]
  const void *g;       // [*, n]
  const int64_t *rel;  // [m] relation of every position (constant per aligned block of 128)
  const int64_t *idx;    // [m] row of x of every position, or NULL (position = row)
  const int64_t *idx_g;  // [m] row of g of every position, or NULL (the row of x)
  int64_t m, x_rows, g_rows;  // positions; rows with an index in [0, x_rows) / [0, g_rows) exist, others count as zero rows
  int k, n, num_rel;
  int stages, slots;
  int chunk_tiles;     // tiles summed in one tensor-memory accumulator before the epilogue takes it over
  int test_stall;      // test hook: the producers never hand over their first tile, so the waits for it run out
  float *partial;      // [grid][slots][k][n]
  int32_t *slot_rel;   // [grid][slots]: relation of a flushed slot, -1 when unused
  int32_t *status;
  long long wait_cycles;
};

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// MN-major operand in a 128-byte swizzled layout: rows of 128 bytes (one per step of the contraction index), `lbo`
// bytes between 128-byte spans along M / N. 16-bit elements: groups of 8 rows 1024 bytes apart, the 16-byte chunks of
// a row permuted by row % 8 (layout type 2). 32-bit elements have their own form, the only one the tensor core takes
// for MN-major TF32 operands: groups of 4 rows 512 bytes apart, the 32-byte chunks of a row permuted by row % 4
// (layout type 1, "128-byte swizzle with a 32-byte base").
template <bool W32>
__device__ __forceinline__ uint64_t make_desc_mn_sw128(uint32_t addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3fff);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((W32 ? 512 : 1024) >> 4) << 32;
  d |= 1ull << 46;  // descriptor version of sm_100
  d |= (W32 ? 1ull : 2ull) << 61;
  return d;
}

// Byte offset of 16-byte chunk c16 of row p inside a span of either layout.
template <bool W32>
__device__ __forceinline__ uint32_t swizzled_offset(int p, int c16) {
  if (W32) return p * 128 + ((((c16 >> 1) ^ (p & 3)) << 5) | ((c16 & 1) << 4));
  return p * 128 + ((c16 ^ (p & 7)) << 4);
}

// fp32 accumulate, A and B of format `fmt` (1 = bf16, 2 = tf32), both MN-major.
__device__ __forceinline__ uint32_t make_idesc_mn(int fmt, int m, int n) {
  uint32_t d = 0;
  d |= 1u << 4;
  d |= static_cast<uint32_t>(fmt) << 7;
  d |= static_cast<uint32_t>(fmt) << 10;
  d |= 1u << 15;  // A is MN-major
  d |= 1u << 16;  // B is MN-major
  d |= static_cast<uint32_t>(n >> 3) << 17;
  d |= static_cast<uint32_t>(m >> 4) << 24;
  return d;
}

template <bool TF32>
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  if (TF32)
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
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

__device__ __forceinline__ void commit_to(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ float trunc_tf32(float v) { return __uint_as_float(__float_as_uint(v) & 0xffffe000u); }

struct Barriers {
  uint64_t full[kMaxStages];   // producers -> MMA (or converters): 256 arrivals
  uint64_t conv[kMaxStages];   // converters -> MMA: 128 arrivals
  uint64_t empty[kMaxStages];  // MMA -> producers: 1 commit
  uint64_t acc_full[2];        // MMA -> epilogue: the accumulator buffer holds a finished chunk (1 commit)
  uint64_t acc_empty[2];       // epilogue -> MMA: the buffer has been read (128 arrivals)
};

// X3: error-compensated fp32. T = float or __nv_bfloat16. kPos = positions per tile, the contraction length of one
// pipeline unit: 128, or 64 in the compensated mode, whose stages hold every tile twice.
template <typename T, bool X3>
__global__ void __launch_bounds__(32 * (kEpiWarps + 1 + kProdWarps + (X3 ? kConvWarps : 0)), 1) typed_wgrad_tc(WgArgs a) {
  constexpr bool TF32 = sizeof(T) == 4;
  constexpr int kPos = X3 ? 64 : 128;
  constexpr int kSpan = 128 * kPos;  // bytes of one 128-byte span of a tile (kPos rows)
  constexpr int kInstrK = TF32 ? 8 : 16;  // positions per MMA
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) Barriers bars;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_slot;
  volatile int *abort_flag = &abort_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int spans_x = a.k * static_cast<int>(sizeof(T)) / 128, spans_g = a.n * static_cast<int>(sizeof(T)) / 128;
  const uint32_t half_bytes = static_cast<uint32_t>(spans_x + spans_g) * kSpan;  // raw (or hi) tiles of x and g
  const uint32_t stage_bytes = X3 ? 2 * half_bytes : half_bytes;
  const int S = a.stages;
  uint8_t *smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);  // swizzled tiles: 1024-byte boundaries
  int tmem_cols = 32;
  while (tmem_cols < a.n) tmem_cols <<= 1;

  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)),
                 "r"(static_cast<uint32_t>(2 * tmem_cols))
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
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.acc_empty[b])), "r"(32 * kEpiWarps) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_slot;

  const int64_t n_tiles = (a.m + kPos - 1) / kPos;
  const int64_t tile_lo = n_tiles * blockIdx.x / gridDim.x, tile_hi = n_tiles * (blockIdx.x + 1) / gridDim.x;
  auto rel_of = [&](int64_t tile) -> int64_t { return tile < tile_hi ? a.rel[tile * kPos] : -1; };
  auto valid_rel = [&](int64_t r) { return r >= 0 && r < a.num_rel; };

  if (warp >= kFirstProd && warp < kFirstConv) {
    // ================= producers: gather the rows of x and g of a tile into the swizzled layout =================
    const int pt = tid - 32 * kFirstProd;  // 0 .. 255
    const int c16 = pt & 7;                // 16-byte chunk inside a 128-byte span
    const int prow = pt >> 3;              // row inside a pass of 32 rows
    const uint8_t *X = static_cast<const uint8_t *>(a.x), *G = static_cast<const uint8_t *>(a.g);
    const int64_t xrow_bytes = static_cast<int64_t>(a.k) * sizeof(T), grow_bytes = static_cast<int64_t>(a.n) * sizeof(T);
    constexpr int kPass = kPos / 32;  // passes of 32 rows per tile
    auto fetch = [&](int64_t tile, int64_t (&ia)[kPass], int64_t (&ig)[kPass]) {
#pragma unroll
      for (int q = 0; q < kPass; ++q) {
        const int64_t pos = tile * kPos + q * 32 + prow;
        ia[q] = -1, ig[q] = -1;
        if (tile < tile_hi && pos < a.m) {
          ia[q] = a.idx != nullptr ? a.idx[pos] : pos;
          ig[q] = a.idx_g != nullptr ? a.idx_g[pos] : ia[q];
        }
      }
    };
    int64_t ia_next[kPass], ig_next[kPass];
    fetch(tile_lo, ia_next, ig_next);
    int64_t it = 0;
    bool alive = true;
    for (int64_t tile = tile_lo; tile < tile_hi && alive; ++tile) {
      int64_t ia[kPass], ig[kPass];
#pragma unroll
      for (int q = 0; q < kPass; ++q) ia[q] = ia_next[q], ig[q] = ig_next[q];
      fetch(tile + 1, ia_next, ig_next);
      if (!valid_rel(rel_of(tile))) continue;  // a tile of padding only
      const int s = static_cast<int>(it % S);
      if (it >= S) {
        alive = wait_bar(&bars.empty[s], static_cast<uint32_t>(((it / S) - 1) & 1), abort_flag, a.status, a.wait_cycles);
        if (!alive) break;
      }
      const uint32_t st0 = smem_addr(smem + static_cast<size_t>(s) * stage_bytes);
#pragma unroll
      for (int q = 0; q < kPass; ++q) {
        const int p = q * 32 + prow;
        // a position contributes only when both of its rows exist; size 0 writes zeros
        const bool ok = ia[q] >= 0 && ia[q] < a.x_rows && ig[q] >= 0 && ig[q] < a.g_rows;
        const int bytes = ok ? 16 : 0;
        const uint32_t d0 = st0 + swizzled_offset<TF32>(p, c16);
        const uint8_t *xs = ok ? X + ia[q] * xrow_bytes + c16 * 16 : X;
        const uint8_t *gs = ok ? G + ig[q] * grow_bytes + c16 * 16 : G;
        for (int j = 0; j < spans_x; ++j)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d0 + j * kSpan), "l"(xs + j * 128), "r"(bytes) : "memory");
        for (int j = 0; j < spans_g; ++j)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d0 + (spans_x + j) * kSpan), "l"(gs + j * 128), "r"(bytes)
                       : "memory");
      }
      if (!(a.test_stall && it == 0))
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&bars.full[s])) : "memory");
      ++it;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (X3 && warp >= kFirstConv) {
    // ================= converters: raw fp32 tiles -> hi (in place) and lo (second half of the stage) =================
    const int ct = tid - 32 * kFirstConv;
    const int n16 = static_cast<int>(half_bytes / 16);
    int64_t it = 0;
    bool alive = true;
    for (int64_t tile = tile_lo; tile < tile_hi && alive; ++tile) {
      if (!valid_rel(rel_of(tile))) continue;
      const int s = static_cast<int>(it % S);
      alive = wait_bar(&bars.full[s], static_cast<uint32_t>((it / S) & 1), abort_flag, a.status, a.wait_cycles);
      if (!alive) break;
      float4 *hi = reinterpret_cast<float4 *>(smem + static_cast<size_t>(s) * stage_bytes);
      float4 *lo = reinterpret_cast<float4 *>(smem + static_cast<size_t>(s) * stage_bytes + half_bytes);
      for (int c = ct; c < n16; c += 32 * kConvWarps) {
        const float4 v = hi[c];
        float4 h, l;
        h.x = trunc_tf32(v.x), h.y = trunc_tf32(v.y), h.z = trunc_tf32(v.z), h.w = trunc_tf32(v.w);
        l.x = trunc_tf32(v.x - h.x), l.y = trunc_tf32(v.y - h.y), l.z = trunc_tf32(v.z - h.z), l.w = trunc_tf32(v.w - h.w);
        hi[c] = h;
        lo[c] = l;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(&bars.conv[s]);
      ++it;
    }
  } else if (warp == kMmaWarp) {
    // ================= MMA issuer =================
    // The tensor core's fp32 accumulation loses a little on every addition (the error grows linearly with the number
    // of positions summed in one accumulator), so an accumulator takes at most `chunk_tiles` tiles; the epilogue adds
    // the chunks of a relation with ordinary fp32 additions. Two accumulator buffers alternate.
    if (lane == 0) {
      const uint32_t idesc = make_idesc_mn(TF32 ? 2 : 1, a.k, a.n);
      const uint32_t step_bytes = kInstrK * 128;  // the next kInstrK positions of a span
      int64_t it = 0, chunk = 0;
      int in_chunk = 0;
      bool alive = true, open = false;  // open: the current accumulator holds tiles of relation `cur`
      int64_t cur = -1;
      for (int64_t tile = tile_lo; tile < tile_hi && alive; ++tile) {
        const int64_t r = rel_of(tile);
        if (!valid_rel(r)) continue;
        if (open && (r != cur || in_chunk == a.chunk_tiles)) {  // hand the chunk to the epilogue
          commit_to(&bars.acc_full[chunk & 1]);
          open = false;
          ++chunk;
        }
        const int buf = static_cast<int>(chunk & 1);
        if (!open) {
          if (chunk >= 2) {  // the epilogue has read the chunk that used this buffer before
            alive = wait_bar(&bars.acc_empty[buf], static_cast<uint32_t>(((chunk >> 1) - 1) & 1), abort_flag, a.status,
                             a.wait_cycles);
            if (!alive) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          }
          cur = r;
          in_chunk = 0;
        }
        const uint32_t d = tmem_d + buf * tmem_cols;
        const int s = static_cast<int>(it % S);
        alive = wait_bar(X3 ? &bars.conv[s] : &bars.full[s], static_cast<uint32_t>((it / S) & 1), abort_flag, a.status,
                         a.wait_cycles);
        if (!alive) break;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t x0 = smem_addr(smem + static_cast<size_t>(s) * stage_bytes);
        const uint32_t g0 = x0 + spans_x * kSpan;
        for (int j = 0; j < kPos / kInstrK; ++j) {
          const uint32_t first = (open || j > 0) ? 1u : 0u;
          const uint32_t off = j * step_bytes;
          if (X3) {
            const uint64_t xa = make_desc_mn_sw128<TF32>(x0 + off, kSpan), xl = make_desc_mn_sw128<TF32>(x0 + half_bytes + off, kSpan);
            const uint64_t ga = make_desc_mn_sw128<TF32>(g0 + off, kSpan), gl = make_desc_mn_sw128<TF32>(g0 + half_bytes + off, kSpan);
            mma_ss<TF32>(d, xa, gl, idesc, first);  // the two small terms first, the large one last
            mma_ss<TF32>(d, xl, ga, idesc, 1u);
            mma_ss<TF32>(d, xa, ga, idesc, 1u);
          } else {
            mma_ss<TF32>(d, make_desc_mn_sw128<TF32>(x0 + off, kSpan), make_desc_mn_sw128<TF32>(g0 + off, kSpan), idesc, first);
          }
        }
        commit_to(&bars.empty[s]);
        open = true;
        ++in_chunk;
        ++it;
      }
      if (alive && open) commit_to(&bars.acc_full[chunk & 1]);
    }
    __syncwarp();
  } else if (warp < kEpiWarps) {
    // ================= epilogue: add every chunk's accumulator into the relation segment's slot of this CTA =================
    // the chunks and segments are found by walking the same tile range as the MMA thread
    int64_t chunk = 0, seg = 0, cur = -1;
    int in_chunk = 0;
    bool alive = true, open = false, seg_started = false;
    const int row = warp * 32 + lane;  // row of dW[r] = column of x
    auto take_chunk = [&]() {
      const int buf = static_cast<int>(chunk & 1);
      alive = wait_bar(&bars.acc_full[buf], static_cast<uint32_t>((chunk >> 1) & 1), abort_flag, a.status, a.wait_cycles);
      if (!alive) return;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float *out = a.partial + ((static_cast<int64_t>(blockIdx.x) * a.slots + seg) * a.k + row) * a.n;
      const uint32_t taddr = tmem_d + (static_cast<uint32_t>(warp * 32) << 16) + buf * tmem_cols;
      for (int c0 = 0; c0 < a.n; c0 += 16) {
        uint32_t v[16];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
              "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr + c0));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < a.k) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float4 acc = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]),
                                     __uint_as_float(v[4 * q + 3]));
            float4 *dst = reinterpret_cast<float4 *>(out + c0 + 4 * q);
            if (seg_started) {  // a later chunk of the segment: ordinary fp32 additions, in chunk order
              const float4 old = *dst;
              acc.x += old.x, acc.y += old.y, acc.z += old.z, acc.w += old.w;
            }
            *dst = acc;
          }
        }
      }
      if (tid == 0 && !seg_started) a.slot_rel[static_cast<int64_t>(blockIdx.x) * a.slots + seg] = static_cast<int32_t>(cur);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(&bars.acc_empty[buf]);
      seg_started = true;
      ++chunk;
    };
    for (int64_t tile = tile_lo; tile < tile_hi && alive; ++tile) {
      const int64_t r = rel_of(tile);
      if (!valid_rel(r)) continue;
      if (open && (r != cur || in_chunk == a.chunk_tiles)) {
        take_chunk();
        if (!alive) break;
        open = false;
        if (r != cur) {
          ++seg;
          seg_started = false;
        }
      }
      if (!open) in_chunk = 0;
      cur = r;
      open = true;
      ++in_chunk;
    }
    if (alive && open) take_chunk();
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(static_cast<uint32_t>(2 * tmem_cols))
                 : "memory");
  }
}

// dW[r][i] = sum of partial[cta][slot][i] over the slots whose relation is r, in (cta, slot) order.
__global__ void __launch_bounds__(256) wgrad_reduce(const float *partial, const int32_t *slot_rel, float *dw, int n_slots,
                                                    int num_rel, int64_t kn) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int r = blockIdx.y;
  if (i >= kn || r >= num_rel) return;
  float s = 0.f;
  for (int q = 0; q < n_slots; ++q)
    if (slot_rel[q] == r) s += partial[static_cast<int64_t>(q) * kn + i];
  dw[static_cast<int64_t>(r) * kn + i] = s;
}

__global__ void wgrad_clear(int32_t *slot_rel, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) slot_rel[i] = -1;
}

struct WgLayout {
  size_t status, slot_rel, partial, total;
  int grid, slots;
};

void wgrad_layout(int num_rel, int k, int n, WgLayout *L) {
  L->grid = kNumSM;
  L->slots = num_rel + 1;  // a contiguous range of sorted tiles meets every relation at most once, plus one
  size_t off = 0;
  L->status = off;
  off = align_up(off + 256, 256);
  L->slot_rel = off;
  off = align_up(off + static_cast<size_t>(L->grid) * L->slots * sizeof(int32_t), 256);
  L->partial = off;
  off = align_up(off + static_cast<size_t>(L->grid) * L->slots * k * n * sizeof(float), 256);
  L->total = off;
}

}  // namespace
}  // namespace cxg

using namespace cxg;

extern "C" int cxg_typed_wgrad_workspace_size(int num_rel, int k, int n, size_t *bytes) {
  CXG_REQUIRE(bytes != nullptr, CXG_ENULL, "cxg_typed_wgrad_workspace_size: bytes is NULL");
  CXG_REQUIRE(num_rel > 0 && k > 0 && n > 0, CXG_EINVAL, "cxg_typed_wgrad_workspace_size: bad sizes");
  WgLayout L;
  wgrad_layout(num_rel, k, n, &L);
  *bytes = L.total;
  return CXG_OK;
}

extern "C" int cxg_typed_wgrad(const void *x, const void *g, const int64_t *rel, const int64_t *idx, const int64_t *idx_g,
                               int64_t m, int64_t x_rows, int64_t g_rows, int k, int n, int num_rel, int dtype,
                               int precision, uint32_t flags, float *dw, void *workspace, size_t workspace_bytes,
                               void *stream) {
  CXG_REQUIRE(m >= 0 && x_rows >= 0 && g_rows >= 0 && k > 0 && n > 0 && num_rel > 0, CXG_EINVAL,
              "cxg_typed_wgrad: bad sizes");
  CXG_REQUIRE(dtype == CXG_F32 || dtype == CXG_BF16, CXG_EINVAL, "cxg_typed_wgrad: dtype %d", dtype);
  CXG_REQUIRE(precision == 1 || precision == 2, CXG_EINVAL, "cxg_typed_wgrad: precision %d (1 = plain, 2 = compensated)",
              precision);
  CXG_REQUIRE(dw != nullptr, CXG_ENULL, "cxg_typed_wgrad: dw is NULL");
  const int elem = dtype == CXG_F32 ? 4 : 2;
  CXG_REQUIRE(k == 128 && (n * elem) % 128 == 0 && n % 16 == 0 && n <= 256, CXG_EUNSUPPORTED,
              "cxg_typed_wgrad: K = %d must be 128 and N = %d a multiple of %d up to 256", k, n, 128 / elem);
  cudaStream_t st = as_stream(stream);
  const int64_t kn = static_cast<int64_t>(k) * n;
  if (m == 0) {
    if (cudaMemsetAsync(dw, 0, static_cast<size_t>(num_rel) * kn * sizeof(float), st) != cudaSuccess)
      return check_launch("cxg_typed_wgrad: memset");
    return CXG_OK;
  }
  CXG_REQUIRE(x && g && rel, CXG_ENULL, "cxg_typed_wgrad: NULL argument");
  CXG_REQUIRE(reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(g) % 16 == 0, CXG_EINVAL,
              "cxg_typed_wgrad: x and g must be 16-byte aligned");
  WgLayout L;
  wgrad_layout(num_rel, k, n, &L);
  CXG_REQUIRE(workspace != nullptr && workspace_bytes >= L.total, CXG_EWORKSPACE,
              "cxg_typed_wgrad: workspace %zu bytes, need %zu", workspace_bytes, L.total);
  CXG_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0, CXG_EINVAL, "cxg_typed_wgrad: workspace alignment");
  const bool x3 = precision == 2 && dtype == CXG_F32;
  const int pos = x3 ? 64 : 128;  // positions per tile, as in the kernel
  const size_t half = static_cast<size_t>(k + n) * elem / 128 * (128 * pos);
  const size_t stage = x3 ? 2 * half : half;
  int stages = static_cast<int>((kSmemBudget - 1024) / stage);
  if (stages > kMaxStages) stages = kMaxStages;
  CXG_REQUIRE(stages >= 1, CXG_EUNSUPPORTED, "cxg_typed_wgrad: one stage of %zu bytes exceeds shared memory", stage);
  const size_t smem = 1024 + stages * stage;

  char *ws = static_cast<char *>(workspace);
  WgArgs a;
  a.x = x, a.g = g, a.rel = rel, a.idx = idx, a.idx_g = idx_g, a.m = m, a.x_rows = x_rows, a.g_rows = g_rows;
  a.k = k, a.n = n, a.num_rel = num_rel, a.stages = stages, a.slots = L.slots;
  a.test_stall = (flags & CXG_WGRAD_TEST_STALL) ? 1 : 0;
  a.chunk_tiles = x3 ? 8 : 32;  // 512 / 4096 positions per accumulator: its error stays well below 1e-5 of fp32 / below
                                // the rounding of the plain products
  a.partial = reinterpret_cast<float *>(ws + L.partial);
  a.slot_rel = reinterpret_cast<int32_t *>(ws + L.slot_rel);
  a.status = reinterpret_cast<int32_t *>(ws + L.status);
  a.wait_cycles = wait_limit_cycles();
  if (cudaMemsetAsync(a.status, 0, 256, st) != cudaSuccess) return check_launch("cxg_typed_wgrad: memset");
  const int n_slots = L.grid * L.slots;
  wgrad_clear<<<(n_slots + 255) / 256, 256, 0, st>>>(a.slot_rel, n_slots);
  const int64_t n_tiles = (m + pos - 1) / pos;  // a last partial tile holds positions past the padded buckets
  const unsigned grid = static_cast<unsigned>(n_tiles < L.grid ? n_tiles : L.grid);
  cudaError_t e = cudaSuccess;
  auto launch = [&](auto kernel, int warps) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e == cudaSuccess) kernel<<<grid, 32 * warps, smem, st>>>(a);
  };
  constexpr int kW = kEpiWarps + 1 + kProdWarps;
  if (dtype == CXG_F32) {
    if (x3)
      launch(typed_wgrad_tc<float, true>, kW + kConvWarps);
    else
      launch(typed_wgrad_tc<float, false>, kW);
  } else {
    launch(typed_wgrad_tc<__nv_bfloat16, false>, kW);
  }
  if (e != cudaSuccess) return set_error(CXG_ECUDA, "cxg_typed_wgrad: %s", cudaGetErrorString(e));
  dim3 rg(static_cast<unsigned>((kn + 255) / 256), static_cast<unsigned>(num_rel));
  wgrad_reduce<<<rg, 256, 0, st>>>(a.partial, a.slot_rel, dw, n_slots, num_rel, kn);
  count_launches(3);
  return check_launch("cxg_typed_wgrad");
}

extern "C" int cxg_typed_wgrad_status(const void *workspace, void *stream) {
  CXG_REQUIRE(workspace != nullptr, CXG_ENULL, "cxg_typed_wgrad_status: workspace is NULL");
  int32_t word = 0;
  cudaStream_t st = as_stream(stream);
  if (cudaMemcpyAsync(&word, workspace, sizeof(word), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess)
    return check_launch("cxg_typed_wgrad_status");
  if (word != 0) return set_error(CXG_ETIMEOUT, "cxg_typed_wgrad: a bounded wait ran out");
  return CXG_OK;
}
