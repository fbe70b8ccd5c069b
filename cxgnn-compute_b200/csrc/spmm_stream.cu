// Edge-tiled streaming CSR SpMM for sm_100a (the fast path of cxg_spmm_csr).
//
// Work is cut by EDGES, not by rows: tile t owns edges [t*T, (t+1)*T) of the CSR
// edge array, whatever rows they belong to, so every warp gets the same number of
// 256/512-byte feature-row gathers no matter how skewed the degrees are (the
// reference gives each warp one row: src/cpp/src/aggr_kernel.cu:30-53).
//
// One warp walks its tile in CSR order:
//   * the source ids of a stage are fetched kStages stages ahead (coalesced);
//   * the feature rows of a stage are copied global -> shared asynchronously, either
//     with ONE bulk async copy per row issued by the lane that holds the row's id
//     (`cp.async.bulk`, completion counted on an mbarrier), or with 16-byte
//     `cp.async` copies; up to kStages stages per warp are in flight and no register
//     is held for them;
//   * the rows are added from shared memory strictly in edge order, the whole warp
//     on one row (32 lanes x 4/8/16 bytes), into one fp32 accumulator per column
//     (packed f32x2 adds);
//   * when the walk passes the end of a row the accumulator is written out and
//     reset; rows without edges get zeros on the way.
// Rows that lie inside one tile are therefore summed exactly like a sequential
// loop. A row that crosses tile borders leaves one partial per tile in scratch
// memory; a second kernel adds those partials in tile order (sequentially up to
// 64 of them; beyond that in blocks of 64 consecutive partials, one warp per block,
// whose sums are then added in block order), so results do not depend on scheduling
// and can be reproduced on a CPU given T.
#include <type_traits>

#include "common.cuh"
#include "spmm_stream.cuh"

namespace cxg {
namespace {

constexpr int kSWarps = 4;         // warps per CTA
constexpr int kSThreads = kSWarps * 32;
constexpr int kStages = 1;         // ring depth per warp (1: latency is hidden by other warps)
constexpr int kStageBytes = 8192;  // feature bytes per stage and warp
constexpr int kCtasPerSM = 6;
constexpr int kSeqPartials = 64;   // longer chains are added in ordered blocks of this many partials
constexpr int kFar = 1 << 30;      // "no row end in sight" in tile-relative positions

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bulk async copy of `bytes` (multiple of 16, both addresses 16-byte aligned) from
// global to this CTA's shared memory; completion is counted on `bar`.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ int64_t load_idx_stream(const int64_t *p) {
  int64_t v;
  asm volatile("ld.global.nc.L1::no_allocate.s64 %0, [%1];" : "=l"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ int64_t load_idx_stream(const int32_t *p) {
  int32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.s32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// CB bytes of a feature row: W 32-bit words in shared memory, EL fp32 values.
template <typename T, int CB>
struct Chunk;
template <int CB>
struct Chunk<float, CB> {
  static constexpr int kWords = CB / 4;
  static constexpr int kElems = CB / 4;
  __device__ __forceinline__ static void unpack(float *f, const uint32_t *w) {
#pragma unroll
    for (int i = 0; i < kWords; ++i) f[i] = __uint_as_float(w[i]);
  }
  __device__ __forceinline__ static void pack(uint32_t *w, const float *f) {
#pragma unroll
    for (int i = 0; i < kWords; ++i) w[i] = __float_as_uint(f[i]);
  }
};
template <int CB>
struct Chunk<__nv_bfloat16, CB> {
  static constexpr int kWords = CB / 4;
  static constexpr int kElems = CB / 2;
  __device__ __forceinline__ static void unpack(float *f, const uint32_t *w) {
#pragma unroll
    for (int i = 0; i < kWords; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ static void pack(uint32_t *w, const float *f) {
#pragma unroll
    for (int i = 0; i < kWords; ++i) {
      __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t *>(&t);
    }
  }
};

// W 32-bit words from a 32-bit shared-space address (always an LDS, 32-bit address math).
template <int W>
__device__ __forceinline__ void lds_words(uint32_t *w, uint32_t addr) {
  if (W == 1) {
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[0]) : "r"(addr));
  } else if (W == 2) {
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[W > 1 ? 1 : 0]) : "r"(addr));
  } else {
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(w[0]), "=r"(w[W > 1 ? 1 : 0]), "=r"(w[W > 2 ? 2 : 0]), "=r"(w[W > 3 ? 3 : 0])
                 : "r"(addr));
  }
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
template <int W>
__device__ __forceinline__ void ldg_words(uint32_t *w, const void *p) {
  if (W == 1) {
    w[0] = *reinterpret_cast<const uint32_t *>(p);
  } else if (W == 2) {
    uint2 v = *reinterpret_cast<const uint2 *>(p);
    w[0] = v.x, w[W > 1 ? 1 : 0] = v.y;
  } else {
    uint4 v = *reinterpret_cast<const uint4 *>(p);
    w[0] = v.x, w[W > 1 ? 1 : 0] = v.y, w[W > 2 ? 2 : 0] = v.z, w[W > 3 ? 3 : 0] = v.w;
  }
}
template <int W>
__device__ __forceinline__ void stg_words_stream(void *p, const uint32_t *w) {
  if (W == 1)
    __stcs(reinterpret_cast<unsigned int *>(p), w[0]);
  else if (W == 2)
    __stcs(reinterpret_cast<uint2 *>(p), make_uint2(w[0], w[W > 1 ? 1 : 0]));
  else
    __stcs(reinterpret_cast<uint4 *>(p), make_uint4(w[0], w[W > 1 ? 1 : 0], w[W > 2 ? 2 : 0], w[W > 3 ? 3 : 0]));
}

// EL fp32 accumulators kept as EL/2 packed pairs in 64-bit registers for the whole walk:
// sm_100 adds or multiply-adds two fp32 values per instruction (f32x2), each rounded like
// the scalar operation
// (plus one scalar when EL is odd), so that every add is one f32x2 instruction and no
// register shuffling is needed around it.
template <int EL>
struct PackedAcc {
  static constexpr int P = EL / 2;
  unsigned long long p[P > 0 ? P : 1];
  float s;
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < P; ++i) p[i] = 0ull;
    s = 0.f;
  }
  __device__ __forceinline__ static unsigned long long pack(float a, float b) {
    unsigned long long r;
    asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
  }
  __device__ __forceinline__ void add(const float *f) {
#pragma unroll
    for (int i = 0; i < P; ++i) asm("add.rn.f32x2 %0, %0, %1;" : "+l"(p[i]) : "l"(pack(f[2 * i], f[2 * i + 1])));
    if (EL & 1) s += f[EL - 1];
  }
  __device__ __forceinline__ void fma(const float *f, float v) {
    const unsigned long long vv = pack(v, v);
#pragma unroll
    for (int i = 0; i < P; ++i)
      asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(p[i]) : "l"(pack(f[2 * i], f[2 * i + 1])), "l"(vv));
    if (EL & 1) s = fmaf(f[EL - 1], v, s);
  }
  __device__ __forceinline__ void get(float *f) const {
#pragma unroll
    for (int i = 0; i < P; ++i) asm("mov.b64 {%0,%1}, %2;" : "=f"(f[2 * i]), "=f"(f[2 * i + 1]) : "l"(p[i]));
    if (EL & 1) f[EL - 1] = s;
  }
};

// Row r with ptr[r] <= pos < ptr[r+1], i.e. the row that owns edge `pos`.
__device__ __forceinline__ int64_t row_of_edge(const void *ptr, int ptr_bytes, int64_t n_dst, int64_t pos) {
  int64_t lo = 0, hi = n_dst;  // invariant: ptr[lo] <= pos < ptr[hi]
  while (hi - lo > 1) {
    int64_t mid = (lo + hi) >> 1;
    if (load_ptr(ptr, mid, ptr_bytes) <= pos)
      lo = mid;
    else
      hi = mid;
  }
  return lo;
}

// Edges the kernels walk: ptr[n_dst], but never more than the caller declared (the workspace and the idx
// array are only that large). A larger ptr[n_dst] is a caller error, recorded by the plan kernel.
__device__ __forceinline__ int64_t stream_edge_total(const StreamArgs &a) {
  const int64_t e = load_ptr(a.ptr, a.n_dst, a.ptr_bytes);
  return e > a.nnz ? a.nnz : e;
}

__global__ void spmm_stream_plan(StreamArgs a) {
  int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (t == 0) {
    a.hdr[kSHdrNumLong] = 0;
    a.hdr[kSHdrNumBlocks] = 0;
    a.hdr[kSHdrError] = load_ptr(a.ptr, a.n_dst, a.ptr_bytes) > a.nnz ? kSErrEdgeCount : kSErrNone;
  }
  if (t >= a.max_tiles) return;
  a.tail_row[t] = -1;  // no unfinished row unless the tile's walk says so
  int64_t e_total = stream_edge_total(a);
  int64_t pos = t * a.tile;
  if (pos >= e_total) return;
  a.tile_row[t] = row_of_edge(a.ptr, a.ptr_bytes, a.n_dst, pos);
}

template <typename T, int CB, int NV, int VALMODE, typename IdxT, bool TMA>
__global__ void __launch_bounds__(kSThreads, kCtasPerSM) spmm_stream(StreamArgs a) {
  using C = Chunk<T, CB>;
  constexpr int EL = C::kElems;
  constexpr int W = C::kWords;
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int row_bytes = a.width * static_cast<int>(sizeof(T));
  const int B = a.stage_edges;  // edges per stage, <= 32
  // per-warp shared memory: kStages mbarriers, per-stage edge values, per-stage row slots
  uint8_t *wbase = smem + static_cast<size_t>(warp) * a.warp_smem;
  uint64_t *bars = reinterpret_cast<uint64_t *>(wbase);
  float *svals = reinterpret_cast<float *>(wbase + 64);
  uint8_t *slots = wbase + a.slot_offset;
  const uint32_t slots_u32 = smem_u32(slots);
  const uint32_t svals_u32 = smem_u32(svals);
  const int vals_per_stage = VALMODE == 0 ? 0 : (VALMODE == 1 ? B : B * a.heads);
  const int val_stride = VALMODE == 0 ? 0 : (VALMODE == 1 ? 4 : 4 * a.heads);  // bytes of edge values per edge

  if (TMA) {
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < kStages; ++s) mbar_init(smem_u32(bars + s), 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
  }

  const IdxT *idx = reinterpret_cast<const IdxT *>(a.idx);
  const uint8_t *x = reinterpret_cast<const uint8_t *>(a.x);
  uint8_t *y = reinterpret_cast<uint8_t *>(a.y);
  const int64_t e_total = stream_edge_total(a);
  const int64_t n_tiles = (e_total + a.tile - 1) / a.tile;
  const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * kSWarps + warp;
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * kSWarps;

  // this lane's byte columns
  bool on[NV];
  int cbyte[NV], head[NV];
#pragma unroll
  for (int q = 0; q < NV; ++q) {
    cbyte[q] = (lane + 32 * q) * CB;
    on[q] = cbyte[q] < row_bytes;
    head[q] = on[q] ? (cbyte[q] / static_cast<int>(sizeof(T))) / a.feat : 0;
  }
  const int cbyte0 = cbyte[0], head0 = head[0];
  // cp.async variant, power-of-two rows: this lane's fixed 16 bytes inside a row
  const uint8_t *xlane = x + ((lane & ((row_bytes >> 4) - 1)) << 4);

  auto zero_row = [&](int64_t r) {
    if (a.accumulate) return;
    const int64_t out = a.targets != nullptr ? __ldg(a.targets + r) : r;
    uint32_t z[W];
#pragma unroll
    for (int i = 0; i < W; ++i) z[i] = 0u;
#pragma unroll
    for (int q = 0; q < NV; ++q)
      if (on[q]) stg_words_stream<W>(y + out * row_bytes + cbyte[q], z);
  };
  auto write_row = [&](int64_t r, float (&acc)[NV][EL], int deg) {
    const int64_t out = a.targets != nullptr ? __ldg(a.targets + r) : r;
#pragma unroll
    for (int q = 0; q < NV; ++q)
      if (on[q]) {
        uint8_t *dst = y + out * row_bytes + cbyte[q];
        if (a.reduce == CXG_MEAN) {
          const float d = static_cast<float>(deg);
#pragma unroll
          for (int i = 0; i < EL; ++i) acc[q][i] = __fdiv_rn(acc[q][i], d);
        }
        uint32_t w[W];
        if (a.accumulate) {
          float old[EL];
          ldg_words<W>(w, dst);
          C::unpack(old, w);
#pragma unroll
          for (int i = 0; i < EL; ++i) acc[q][i] += old[i];
        }
        C::pack(w, acc[q]);
        stg_words_stream<W>(dst, w);
      }
  };
  auto write_partial = [&](int64_t t, int which, float (&acc)[NV][EL]) {
    float *p = a.partials + (t * 2 + which) * a.width;
#pragma unroll
    for (int q = 0; q < NV; ++q)
      if (on[q]) {
        float *pq = p + cbyte[q] / static_cast<int>(sizeof(T));
        if (EL % 4 == 0) {
#pragma unroll
          for (int i = 0; i < EL; i += 4)
            *reinterpret_cast<float4 *>(pq + i) =
                make_float4(acc[q][i], acc[q][(i + 1) % EL], acc[q][(i + 2) % EL], acc[q][(i + 3) % EL]);
        } else if (EL % 2 == 0) {
#pragma unroll
          for (int i = 0; i < EL; i += 2) *reinterpret_cast<float2 *>(pq + i) = make_float2(acc[q][i], acc[q][(i + 1) % EL]);
        } else {
#pragma unroll
          for (int i = 0; i < EL; ++i) pq[i] = acc[q][i];
        }
      }
  };

  if (e_total == 0) {  // no edge at all: every row is empty
    for (int64_t r = gwarp; r < a.n_dst; r += nwarps) zero_row(r);
    return;
  }

  uint32_t phases = 0;  // bit s: parity the next wait on stage s expects
  bool dead = false;

  for (int64_t t = gwarp; t < n_tiles && !dead; t += nwarps) {
    const int64_t tb = t * a.tile;
    const int tile_len = static_cast<int>(min(static_cast<int64_t>(a.tile), e_total - tb));
    const int n_stage = (tile_len + B - 1) / B;
    int64_t row = a.tile_row[t];
    if (t == 0)
      for (int64_t r = 0; r < row; ++r) zero_row(r);  // leading rows without edges
    // Row ends as 32-bit positions relative to the tile: lane i holds the end of row
    // pbase + i, or kFar beyond the last row.
    int64_t pbase = row;
    auto load_ends = [&]() -> int {
      const int64_t r = pbase + lane;
      if (r >= a.n_dst) return kFar;
      const int64_t v = load_ptr(a.ptr, r + 1, a.ptr_bytes) - tb;
      return v > kFar ? kFar : static_cast<int>(v);
    };
    int pc = load_ends();
    int rrel = 0;  // row - pbase
    int rend = __shfl_sync(0xffffffffu, pc, 0);
    // tile-relative start of the current row; negative when it began in an earlier tile
    const int64_t rs64 = load_ptr(a.ptr, row, a.ptr_bytes) - tb;
    int rstart = rs64 < -kFar ? -kFar : static_cast<int>(rs64);
    const IdxT *idx_t = idx + tb;

    // Fills ring slot s with the rows of stage k; `nid` is this lane's source id.
    auto fill = [&](int k, int s, int64_t nid) {
      const int sbase = k * B;
      const int cnt = min(B, tile_len - sbase);
      if (VALMODE == 1) {
        if (lane < cnt) svals[s * vals_per_stage + lane] = __ldg(a.edge_val + tb + sbase + lane);
      } else if (VALMODE == 2) {
        for (int q = lane; q < cnt * a.heads; q += 32)
          svals[s * vals_per_stage + q] = __ldg(a.edge_val + (tb + sbase) * a.heads + q);
      }
      const uint32_t dst0 = slots_u32 + s * a.stage_bytes;
      if (TMA) {
        const uint32_t bar = smem_u32(bars + s);
        // order earlier generic-proxy reads of this slot before the async-proxy writes
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // (test hook: stage 0 of tile 0 announces 16 bytes that no copy delivers, so its wait must run out)
        if (lane == 0) mbar_expect_tx(bar, static_cast<uint32_t>(cnt * row_bytes) + ((a.test_stall && t == 0 && k == 0) ? 16u : 0u));
        __syncwarp();
        if (lane < cnt) bulk_g2s(dst0 + lane * row_bytes, x + nid * row_bytes, row_bytes, bar);
      } else {
        // 16-byte async copies, 32 per instruction: chunk c of the stage belongs to row c / cpr.
        // For power-of-two rows of up to 512 bytes a lane always copies the same 16 bytes of
        // the same relative row, so an instruction costs one shuffle and one 64-bit multiply-add.
        const int cpr = row_bytes >> 4;
        const int total = cnt * cpr;
        if (a.cpr_shift >= 0 && a.cpr_shift <= 5) {
          const int rpi = 32 >> a.cpr_shift;  // rows per instruction
          int j = lane >> a.cpr_shift;
          uint32_t dst = dst0 + (lane << 4);
#pragma unroll 8
          for (int c0 = 0; c0 < total; c0 += 32) {
            const int64_t nj = __shfl_sync(0xffffffffu, nid, j & 31);
            if (j < cnt) cp_async16(dst, xlane + nj * row_bytes);
            j += rpi;
            dst += 512;
          }
        } else {
          for (int c0 = 0; c0 < total; c0 += 32) {
            const int c = c0 + lane;
            const bool ok = c < total;
            const int j = ok ? (a.cpr_shift >= 0 ? (c >> a.cpr_shift) : (c / cpr)) : 0;
            const int64_t nj = __shfl_sync(0xffffffffu, nid, j);
            if (ok) cp_async16(dst0 + (c << 4), x + nj * row_bytes + ((c - j * cpr) << 4));
          }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
      }
    };
    auto load_nid = [&](int k) -> int64_t {
      const int pos = k * B + lane;
      int64_t nid = 0;
      if (lane < B && pos < tile_len) {
        nid = load_idx_stream(idx_t + pos);
        if (a.edge_rel != nullptr) nid += static_cast<int64_t>(__ldg(a.edge_rel + tb + pos)) * a.rel_stride;
      }
      return nid;
    };

    // prologue: up to kStages stages in flight
    {
      int64_t nids[kStages];
#pragma unroll
      for (int k = 0; k < kStages; ++k) nids[k] = load_nid(k);
#pragma unroll
      for (int k = 0; k < kStages; ++k) {
        if (k < n_stage)
          fill(k, k, nids[k]);
        else if (!TMA)
          asm volatile("cp.async.commit_group;" ::: "memory");
      }
    }

    PackedAcc<EL> pacc[NV];
#pragma unroll
    for (int q = 0; q < NV; ++q) pacc[q].zero();
    float acc[NV][EL];  // unpacked copy, only filled when a row or a partial is written

    int s = 0;
    for (int k = 0; k < n_stage; ++k) {
      const int64_t nid_next = load_nid(k + kStages);  // used after the walk below
      if (TMA) {
        const uint32_t bar = smem_u32(bars + s);
        const uint32_t parity = (phases >> s) & 1u;
        if (!mbar_try_wait(bar, parity)) {
          const long long t0 = clock64();
          while (!mbar_try_wait(bar, parity)) {
            if (clock64() - t0 > a.wait_cycles) {
              dead = true;
              break;
            }
          }
        }
        if (dead) {
          // Nothing else of this warp is in flight: one stage per warp, and the copies of that stage are what
          // the wait was for. The tile's tail_row keeps the -1 of the plan kernel and the fix-up kernels do
          // nothing once the error word is set.
          if (lane == 0) atomicExch(a.hdr + kSHdrError, kSErrTimeout);
          break;
        }
        phases ^= 1u << s;
      } else {
        // one group is committed per fill (empty ones included), so all but the newest
        // kStages - 1 groups being complete means stage k has landed
        asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 1) : "memory");
        __syncwarp();
      }
      const int sbase = k * B;  // tile-relative position of the stage's first edge
      const int send = min(sbase + B, tile_len);
      const uint32_t sl = slots_u32 + s * a.stage_bytes;  // 32-bit shared-space addresses
      const uint32_t sv = svals_u32 + s * vals_per_stage * 4;
      int pos = sbase;
      while (pos < send) {
        // edges of the current row inside this stage: added without any per-edge test,
        // four at a time (independent shared loads first), then two, then one
        const int stop = min(send, rend);
        uint32_t p = sl + (pos - sbase) * row_bytes + cbyte0;
        uint32_t pv = sv + (pos - sbase) * val_stride + head0 * 4;
        auto add_edges = [&](auto n_tag) {
          constexpr int N = decltype(n_tag)::value;
          uint32_t w[N][NV][W];
          float v[N][NV];
#pragma unroll
          for (int e = 0; e < N; ++e)
#pragma unroll
            for (int q = 0; q < NV; ++q)
              if (on[q]) {
                lds_words<W>(w[e][q], p + e * row_bytes + q * 32 * CB);
                if (VALMODE == 1) v[e][q] = lds_f32(pv + e * val_stride);
                if (VALMODE == 2) v[e][q] = lds_f32(pv + e * val_stride + (head[q] - head0) * 4);
              }
#pragma unroll
          for (int e = 0; e < N; ++e)
#pragma unroll
            for (int q = 0; q < NV; ++q)
              if (on[q]) {
                float f[EL];
                C::unpack(f, w[e][q]);
                if (VALMODE == 0)
                  pacc[q].add(f);
                else
                  pacc[q].fma(f, v[e][q]);
              }
          p += N * row_bytes;
          pv += N * val_stride;
          pos += N;
        };
        while (stop - pos >= 4) add_edges(std::integral_constant<int, 4>{});
        if (stop - pos >= 2) add_edges(std::integral_constant<int, 2>{});
        if (stop - pos >= 1) add_edges(std::integral_constant<int, 1>{});
        if (pos == rend) {
          // the row ends here: write it out (to scratch when it began in an earlier tile)
#pragma unroll
          for (int q = 0; q < NV; ++q) pacc[q].get(acc[q]);
          if (rstart < 0)
            write_partial(t, 0, acc);
          else
            write_row(row, acc, rend - rstart);
#pragma unroll
          for (int q = 0; q < NV; ++q) pacc[q].zero();
          rstart = rend;
          for (;;) {
            ++row;
            if (++rrel == 32) {
              pbase = row;
              rrel = 0;
              pc = load_ends();
            }
            rend = __shfl_sync(0xffffffffu, pc, rrel);
            if (rend != rstart) break;
            zero_row(row);  // a row without edges
          }
        }
      }
      __syncwarp();
      if (k + kStages < n_stage)
        fill(k + kStages, s, nid_next);
      else if (!TMA)
        asm volatile("cp.async.commit_group;" ::: "memory");
      s = (s + 1 == kStages) ? 0 : s + 1;
    }
    if (dead) break;
    // what is left in the accumulators belongs to a row that continues in the next tile
    int64_t tail = -1;
    if (row < a.n_dst && rstart < tile_len && rend > tile_len) {
#pragma unroll
      for (int q = 0; q < NV; ++q) pacc[q].get(acc[q]);
      if (rstart < 0) {
        write_partial(t, 0, acc);  // the row covers this whole tile
      } else {
        write_partial(t, 1, acc);
        tail = row;
      }
    }
    if (lane == 0) a.tail_row[t] = tail;
  }
}

// ---------------------------------------------------------------------------------------------
// Lean variant of the walk for the shapes that carry the large graphs: rows of exactly 32 * CB bytes
// (128 / 256 / 512 bytes: every lane owns CB bytes of every row), no edge values, relations or targets,
// 16-byte cp.async staging, one stage per warp. Same tiles, same order of additions, same
// partials as spmm_stream (results are bit-identical); what differs is the instruction count per edge:
// tile-relative 32-bit positions and source ids, a running shared-memory pointer instead of per-run
// address arithmetic, no per-lane column predicates, and a full-stage copy loop without bounds tests.
// ---------------------------------------------------------------------------------------------
template <typename T, int CB>
struct FastAcc;

// fp32 rows: the shared-memory words are the addends; CB / 8 packed pairs.
template <int CB>
struct FastAcc<float, CB> {
  static constexpr int P = CB / 8 > 0 ? CB / 8 : 1;
  unsigned long long p[P];
  float s;  // CB == 4: one scalar
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < P; ++i) p[i] = 0ull;
    s = 0.f;
  }
  // adds the CB bytes at shared address `addr`
  __device__ __forceinline__ void add(uint32_t addr) {
    if (CB == 4) {
      s += lds_f32(addr);
    } else if (CB == 8) {
      unsigned long long v;
      asm volatile("ld.shared.b64 %0, [%1];" : "=l"(v) : "r"(addr));
      asm("add.rn.f32x2 %0, %0, %1;" : "+l"(p[0]) : "l"(v));
    } else {
      unsigned long long v0, v1;
      asm volatile("ld.shared.v2.b64 {%0,%1}, [%2];" : "=l"(v0), "=l"(v1) : "r"(addr));
      asm("add.rn.f32x2 %0, %0, %1;" : "+l"(p[0]) : "l"(v0));
      asm("add.rn.f32x2 %0, %0, %1;" : "+l"(p[P > 1 ? 1 : 0]) : "l"(v1));
    }
  }
  static constexpr int EL = CB / 4;
  __device__ __forceinline__ void get(float *f) const {
    if (CB == 4) {
      f[0] = s;
    } else {
#pragma unroll
      for (int i = 0; i < P; ++i) asm("mov.b64 {%0,%1}, %2;" : "=f"(f[2 * i]), "=f"(f[2 * i + 1]) : "l"(p[i]));
    }
  }
};

// bf16 rows: every 32-bit word holds two values; low half << 16 and high half masked are the fp32 addends.
template <int CB>
struct FastAcc<__nv_bfloat16, CB> {
  static constexpr int P = CB / 4;  // one packed pair per 32-bit word
  static constexpr int EL = CB / 2;
  unsigned long long p[P];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < P; ++i) p[i] = 0ull;
  }
  __device__ __forceinline__ void add(uint32_t addr) {
    uint32_t w[P];
    lds_words<P>(w, addr);
#pragma unroll
    for (int i = 0; i < P; ++i) {
      unsigned long long v;
      asm("mov.b64 %0, {%1,%2};" : "=l"(v) : "r"(w[i] << 16), "r"(w[i] & 0xffff0000u));
      asm("add.rn.f32x2 %0, %0, %1;" : "+l"(p[i]) : "l"(v));
    }
  }
  __device__ __forceinline__ void get(float *f) const {
#pragma unroll
    for (int i = 0; i < P; ++i) asm("mov.b64 {%0,%1}, %2;" : "=f"(f[2 * i]), "=f"(f[2 * i + 1]) : "l"(p[i]));
  }
};

// NS = stages in flight per warp: 2 (two stages of 4 KiB, the default) or 1 (the whole 8 KiB as one stage).
#ifndef CXG_FAST_CTAS
#define CXG_FAST_CTAS kCtasPerSM  // resident CTAs per SM of the lean walk (7 measured 25 % slower: more warps, more L2 misses)
#endif
// IDXS: the tile's source ids are not loaded by the lanes but staged by the bulk-copy unit (TMA): one
// `cp.async.bulk` of 512 bytes (128 int32 / 64 int64 ids) per chunk into a two-slot ring per warp, completion on an
// mbarrier, the next chunk (of this tile or of the warp's next tile) requested when a chunk is first read. The
// copy lanes then take the id of their row from shared memory instead of a shuffle. The waits are bounded like
// those of the bulk-row variant.
template <typename T, int CB, typename IdxT, bool ACC, int NS, bool IDXS>
__global__ void __launch_bounds__(kSThreads, CXG_FAST_CTAS) spmm_stream_fast(StreamArgs a) {
  using C = Chunk<T, CB>;
  using Acc = FastAcc<T, CB>;
  constexpr int EL = C::kElems;
  constexpr int W = C::kWords;
  constexpr int RB = 32 * CB;                        // bytes per row
  constexpr int B = (kStageBytes / NS) / RB > 32 ? 32 : (kStageBytes / NS) / RB;  // edges per stage
  constexpr int CPR = RB / 16;                       // 16-byte chunks per row
  constexpr int RPI = 32 / CPR;                      // rows per copy instruction
  constexpr int NCOPY = B * CPR / 32;                // copy instructions per full stage
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const uint32_t sl = smem_u32(smem + static_cast<size_t>(warp) * (NS * B * RB));  // NS stage slots of B rows
  const uint32_t my = sl + lane * CB;                // this lane's columns of the first slot's first row
  const IdxT *idx = reinterpret_cast<const IdxT *>(a.idx);
  const uint8_t *x = reinterpret_cast<const uint8_t *>(a.x);
  uint8_t *y = reinterpret_cast<uint8_t *>(a.y) + lane * CB;
  const int64_t e_total = stream_edge_total(a);
  const int64_t n_tiles = (e_total + a.tile - 1) / a.tile;
  const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * kSWarps + warp;
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * kSWarps;
  const bool mean = a.reduce == CXG_MEAN;
  // copy roles of this lane: row (lane / CPR) of every group of RPI rows, bytes [16 * (lane % CPR), +16) of it
  const int jrow = lane / CPR;
  const uint8_t *xlane = x + (lane % CPR) * 16;
  const uint32_t cdst = sl + lane * 16;
  // id ring (IDXS): two slots of kIdxChunkBytes per warp behind the row slots of all warps, then two barriers per warp
  constexpr int CH = kIdxChunkBytes / static_cast<int>(sizeof(IdxT));  // ids per chunk; a multiple of B
  const uint32_t ibuf = smem_u32(smem + static_cast<size_t>(kSWarps) * (NS * B * RB) + warp * (2 * kIdxChunkBytes));
  const uint32_t ibar = smem_u32(smem + static_cast<size_t>(kSWarps) * (NS * B * RB + 2 * kIdxChunkBytes) + warp * 16);
  uint32_t g_issue = 0, g_wait = 0;  // chunks requested / consumed by this warp so far (slot = number & 1)
  bool dead = false;
  if (IDXS) {
    if (lane == 0) {
      mbar_init(ibar, 1);
      mbar_init(ibar + 8, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
  }

  auto zero_row = [&](int64_t r) {
    if (ACC) return;  // y[r] += 0
    uint32_t z[W];
#pragma unroll
    for (int i = 0; i < W; ++i) z[i] = 0u;
    stg_words_stream<W>(y + r * RB, z);
  };

  if (e_total == 0) {
    for (int64_t r = gwarp; r < a.n_dst; r += nwarps) zero_row(r);
    return;
  }

  // requests chunk c of tile t2 into slot g_issue & 1; every lane of the warp has finished reading that slot (the
  // caller passed a __syncwarp since). The part that is a multiple of 16 bytes goes through the copy unit, the
  // last few ids of the graph's last tile (fewer than 16 bytes) through the lanes.
  auto request_chunk = [&](int64_t t2, int c) {
    const int64_t e0 = t2 * a.tile + static_cast<int64_t>(c) * CH;
    const int64_t left = min(static_cast<int64_t>(a.tile) - static_cast<int64_t>(c) * CH, e_total - e0);
    const int len = static_cast<int>(min(static_cast<int64_t>(CH), left));
    const uint32_t bulk = (static_cast<uint32_t>(len) * static_cast<uint32_t>(sizeof(IdxT))) & ~15u;
    const uint32_t slot = ibuf + (g_issue & 1u) * kIdxChunkBytes;
    const uint32_t bar = ibar + (g_issue & 1u) * 8;
    if (lane == 0) {
      mbar_expect_tx(bar, bulk + ((a.test_stall && g_issue == 0) ? 16u : 0u));
      if (bulk) bulk_g2s(slot, idx + e0, bulk, bar);
    }
    const int done = static_cast<int>(bulk / sizeof(IdxT));
    if (lane < len - done) {
      const uint32_t v = static_cast<uint32_t>(load_idx_stream(idx + e0 + done + lane));
      asm volatile("st.shared.b32 [%0], %1;" ::"r"(slot + (done + lane) * static_cast<uint32_t>(sizeof(IdxT))), "r"(v) : "memory");
    }
    ++g_issue;
  };
  if (IDXS && gwarp < n_tiles) request_chunk(gwarp, 0);

  for (int64_t t = gwarp; t < n_tiles; t += nwarps) {
    const int64_t tb = t * a.tile;
    const int tile_len = static_cast<int>(min(static_cast<int64_t>(a.tile), e_total - tb));
    const int n_stage = (tile_len + B - 1) / B;
    const int n_chunk = (tile_len + CH - 1) / CH;
    int64_t row = a.tile_row[t];
    if (t == 0)
      for (int64_t r = 0; r < row; ++r) zero_row(r);
    int64_t pbase = row;
    auto load_ends = [&]() -> int {
      const int64_t r = pbase + lane;
      if (r >= a.n_dst) return kFar;
      const int64_t v = load_ptr(a.ptr, r + 1, a.ptr_bytes) - tb;
      return v > kFar ? kFar : static_cast<int>(v);
    };
    int pc = load_ends();
    int rrel = 0;
    int rend = __shfl_sync(0xffffffffu, pc, 0);
    const int64_t rs64 = load_ptr(a.ptr, row, a.ptr_bytes) - tb;
    int rstart = rs64 < -kFar ? -kFar : static_cast<int>(rs64);
    const IdxT *idx_t = idx + tb;

    auto load_nid = [&](int k) -> uint32_t {
      if (IDXS) return 0u;
      const int pos = k * B + lane;
      return (lane < B && pos < tile_len) ? static_cast<uint32_t>(load_idx_stream(idx_t + pos)) : 0u;
    };
    // stage k goes to slot k % NS; exactly one group is committed per call (an empty one past the last stage), so
    // "all but the newest NS - 1 groups complete" means stage k has landed
    auto fill = [&](int k, uint32_t nid) {
      const int cnt = tile_len - k * B;
      const uint32_t dst = cdst + (NS == 1 ? 0 : (k & (NS - 1)) * (B * RB));
      uint32_t ids = 0;  // IDXS: shared address of the id of this lane's row of the stage's first copy group
      if (IDXS && cnt > 0 && !dead) {
        const int in_chunk = (k * B) % CH;
        if (in_chunk == 0) {  // first stage of a chunk: wait for it, then request the one after it
          const uint32_t bar = ibar + (g_wait & 1u) * 8;
          const uint32_t parity = (g_wait >> 1) & 1u;
          if (!mbar_try_wait(bar, parity)) {
            const long long t0 = clock64();
            while (!mbar_try_wait(bar, parity)) {
              if (clock64() - t0 > a.wait_cycles) {
                dead = true;
                break;
              }
            }
          }
          dead = __any_sync(0xffffffffu, dead);  // also orders the lanes' own id stores and the reads of the other slot
          ++g_wait;
          if (!dead) {
            const int c = (k * B) / CH;
            if (c + 1 < n_chunk)
              request_chunk(t, c + 1);
            else if (t + nwarps < n_tiles)
              request_chunk(t + nwarps, 0);
          }
        }
        ids = ibuf + ((g_wait - 1) & 1u) * kIdxChunkBytes + (in_chunk + jrow) * static_cast<uint32_t>(sizeof(IdxT));
      }
      if (IDXS && dead) {
        // the stage's copies are not issued; the group below stays empty
      } else if (cnt >= B) {  // full stage: no bounds test per copy
#pragma unroll
        for (int c = 0; c < NCOPY; ++c) {
          uint32_t nj;
          if (IDXS)
            asm volatile("ld.shared.b32 %0, [%1];" : "=r"(nj) : "r"(ids + c * RPI * static_cast<uint32_t>(sizeof(IdxT))));
          else
            nj = __shfl_sync(0xffffffffu, nid, c * RPI + jrow);
          cp_async16(dst + c * 512, xlane + static_cast<uint64_t>(nj) * RB);
        }
      } else if (cnt > 0) {
#pragma unroll
        for (int c = 0; c < NCOPY; ++c) {
          uint32_t nj = 0;
          if (IDXS) {
            if (c * RPI + jrow < cnt)
              asm volatile("ld.shared.b32 %0, [%1];" : "=r"(nj) : "r"(ids + c * RPI * static_cast<uint32_t>(sizeof(IdxT))));
          } else {
            nj = __shfl_sync(0xffffffffu, nid, (c * RPI + jrow) & 31);
          }
          if (c * RPI + jrow < cnt) cp_async16(dst + c * 512, xlane + static_cast<uint64_t>(nj) * RB);
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };

    fill(0, load_nid(0));
    if (NS == 2) fill(1, load_nid(1));
    Acc acc;
    acc.zero();
    float f[EL];

    for (int k = 0; k < n_stage; ++k) {
      if (IDXS && dead) break;
      const uint32_t nid_next = load_nid(k + NS);
      asm volatile("cp.async.wait_group %0;" ::"n"(NS - 1) : "memory");
      __syncwarp();
      const int sbase = k * B;
      const int send = min(sbase + B, tile_len);
      int pos = sbase;
      uint32_t p = my + (NS == 1 ? 0 : (k & (NS - 1)) * (B * RB));  // shared address of this lane's bytes of edge `pos`
      while (pos < send) {
        const int stop = min(send, rend);
        int n = stop - pos;
        pos = stop;
        for (; n >= 4; n -= 4) {
          acc.add(p);
          acc.add(p + RB);
          acc.add(p + 2 * RB);
          acc.add(p + 3 * RB);
          p += 4 * RB;
        }
        if (n & 2) {
          acc.add(p);
          acc.add(p + RB);
          p += 2 * RB;
        }
        if (n & 1) {
          acc.add(p);
          p += RB;
        }
        if (pos == rend) {
          acc.get(f);
          acc.zero();
          if (rstart < 0) {
            float *pp = a.partials + (t * 2) * (RB / static_cast<int>(sizeof(T))) + lane * EL;
#pragma unroll
            for (int i = 0; i < EL; ++i) pp[i] = f[i];
          } else {
            if (mean) {
              const float d = static_cast<float>(rend - rstart);
#pragma unroll
              for (int i = 0; i < EL; ++i) f[i] = __fdiv_rn(f[i], d);
            }
            uint32_t w[W];
            if (ACC) {  // y[row] += result (added after the division, as the general kernel does)
              float old[EL];
              ldg_words<W>(w, y + row * RB);
              C::unpack(old, w);
#pragma unroll
              for (int i = 0; i < EL; ++i) f[i] += old[i];
            }
            C::pack(w, f);
            stg_words_stream<W>(y + row * RB, w);
          }
          rstart = rend;
          for (;;) {
            ++row;
            if (++rrel == 32) {
              pbase = row;
              rrel = 0;
              pc = load_ends();
            }
            rend = __shfl_sync(0xffffffffu, pc, rrel);
            if (rend != rstart) break;
            zero_row(row);
          }
        }
      }
      __syncwarp();
      if (NS == 2)
        fill(k + 2, nid_next);  // also past the last stage: an empty group keeps the group count in step
      else if (k + 1 < n_stage)
        fill(k + 1, nid_next);
    }
    if (NS == 2) asm volatile("cp.async.wait_group 0;" ::: "memory");  // only empty groups are left
    if (IDXS && dead) {
      // An id chunk did not arrive within the limit. The row copies of this warp have been waited for above and no
      // other chunk is requested; the tile's tail_row keeps the -1 of the plan kernel and the fix-up kernels do
      // nothing once the error word is set.
      if (lane == 0) atomicExch(a.hdr + kSHdrError, kSErrTimeout);
      break;
    }
    int64_t tail = -1;
    if (row < a.n_dst && rstart < tile_len && rend > tile_len) {
      acc.get(f);
      const int which = rstart < 0 ? 0 : 1;
      float *pp = a.partials + (t * 2 + which) * (RB / static_cast<int>(sizeof(T))) + lane * EL;
#pragma unroll
      for (int i = 0; i < EL; ++i) pp[i] = f[i];
      if (which) tail = row;
    }
    if (lane == 0) a.tail_row[t] = tail;
  }
}

// VW consecutive fp32 partial columns (VW = 4 when the row width allows, else 1).
template <int VW>
struct PVec {
  float v[VW];
  __device__ __forceinline__ void load(const float *p) {
    if (VW == 4) {
      float4 t = *reinterpret_cast<const float4 *>(p);
      v[0] = t.x, v[VW > 1 ? 1 : 0] = t.y, v[VW > 2 ? 2 : 0] = t.z, v[VW > 3 ? 3 : 0] = t.w;
    } else {
      v[0] = *p;
    }
  }
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < VW; ++i) v[i] = 0.f;
  }
  __device__ __forceinline__ void add(const PVec &o) {
#pragma unroll
    for (int i = 0; i < VW; ++i) v[i] += o.v[i];
  }
};

template <typename T, int VW>
__device__ __forceinline__ void finish_row(const StreamArgs &a, PVec<VW> &s, T *dst, int64_t deg) {
#pragma unroll
  for (int i = 0; i < VW; ++i) {
    float r = s.v[i];
    if (a.reduce == CXG_MEAN) r = __fdiv_rn(r, static_cast<float>(deg));
    if (a.accumulate) r += to_f32(dst[i]);
    dst[i] = from_f32<T>(r);
  }
}

// Adds, for every row that began in tile t and ran on, its partial of tile t and the
// head partials of the following tiles, in tile order. Chains longer than
// kSeqPartials are left to spmm_stream_fix_long.
template <typename T, int VW>
__global__ void __launch_bounds__(256) spmm_stream_fix(StreamArgs a) {
  const int lane = threadIdx.x & 31;
  if (a.hdr[kSHdrError] != kSErrNone) return;  // the walk did not finish: the partials are not all there
  const int64_t e_total = stream_edge_total(a);
  const int64_t n_tiles = (e_total + a.tile - 1) / a.tile;
  const int64_t gwarp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  T *y = reinterpret_cast<T *>(a.y);
  for (int64_t t = gwarp; t < n_tiles; t += nwarps) {
    const int64_t r = a.tail_row[t];
    if (r < 0 || r >= a.n_dst) continue;
    const int64_t rb = load_ptr(a.ptr, r, a.ptr_bytes), re = min(load_ptr(a.ptr, r + 1, a.ptr_bytes), e_total);
    const int64_t t_last = (re - 1) / a.tile;
    const int64_t m = t_last - t + 1;  // partials in the chain
    if (m > kSeqPartials) {
      // left to the two long-chain kernels: claim a slot and one entry of the block table per 64 partials
      const int nb = static_cast<int>((m + kSeqPartials - 1) / kSeqPartials);
      int slot = 0, base = 0;
      if (lane == 0) {
        slot = atomicAdd(a.hdr + kSHdrNumLong, 1);
        base = atomicAdd(a.hdr + kSHdrNumBlocks, nb);
        if (slot < a.max_long) {
          a.long_tiles[slot] = t;
          a.long_base[slot] = base;
        }
      }
      slot = __shfl_sync(0xffffffffu, slot, 0);
      base = __shfl_sync(0xffffffffu, base, 0);
      if (slot < a.max_long)
        for (int b = lane; b < nb; b += 32)
          if (base + b < a.max_blocks) a.block_owner[base + b] = slot;
      continue;
    }
    const int64_t out = a.targets != nullptr ? a.targets[r] : r;
    for (int c = lane * VW; c < a.width; c += 32 * VW) {
      PVec<VW> s, v;
      s.load(a.partials + (t * 2 + 1) * a.width + c);
      for (int64_t u = t + 1; u <= t_last; ++u) {
        v.load(a.partials + (u * 2) * a.width + c);
        s.add(v);
      }
      finish_row<T, VW>(a, s, y + out * a.width + c, re - rb);
    }
  }
}

// Long chains, level 1: block g of the block table = partials [64 b, min(64 b + 64, m)) of the chain that owns
// it; one warp adds them in order and leaves the block's sum in block_sums[g].
template <int VW>
__global__ void __launch_bounds__(256) spmm_stream_fix_long_blocks(StreamArgs a) {
  if (a.hdr[kSHdrError] != kSErrNone) return;
  const int lane = threadIdx.x & 31;
  const int64_t e_total = stream_edge_total(a);
  const int n_blocks = min(a.hdr[kSHdrNumBlocks], a.max_blocks);
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int g = gwarp; g < n_blocks; g += nwarps) {
    const int slot = a.block_owner[g];
    const int64_t t = a.long_tiles[slot];
    const int64_t r = a.tail_row[t];
    if (r < 0 || r >= a.n_dst) continue;
    const int64_t re = min(load_ptr(a.ptr, r + 1, a.ptr_bytes), e_total);
    const int64_t m = (re - 1) / a.tile - t + 1;
    const int64_t kb = static_cast<int64_t>(g - a.long_base[slot]) * kSeqPartials;
    const int64_t ke = min(kb + kSeqPartials, m);
    for (int c = lane * VW; c < a.width; c += 32 * VW) {
      // chain element 0 is the tail partial of tile t, element k > 0 the head partial of tile t + k
      auto at = [&](int64_t k) { return a.partials + (k == 0 ? (t * 2 + 1) : ((t + k) * 2)) * a.width + c; };
      PVec<VW> s;
      s.load(at(kb));
      int64_t k = kb + 1;
      for (; k + 8 <= ke; k += 8) {
        PVec<VW> v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u].load(at(k + u));
#pragma unroll
        for (int u = 0; u < 8; ++u) s.add(v[u]);
      }
      for (; k < ke; ++k) {
        PVec<VW> v;
        v.load(at(k));
        s.add(v);
      }
#pragma unroll
      for (int u = 0; u < VW; ++u) a.block_sums[static_cast<int64_t>(g) * a.width + c + u] = s.v[u];
    }
  }
}

// Long chains, level 2: one warp per chain adds its block sums in block order and writes the row.
template <typename T, int VW>
__global__ void __launch_bounds__(256) spmm_stream_fix_long_rows(StreamArgs a) {
  if (a.hdr[kSHdrError] != kSErrNone) return;
  const int lane = threadIdx.x & 31;
  const int64_t e_total = stream_edge_total(a);
  const int n_long = min(a.hdr[kSHdrNumLong], a.max_long);
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  T *y = reinterpret_cast<T *>(a.y);
  for (int i = gwarp; i < n_long; i += nwarps) {
    const int64_t t = a.long_tiles[i];
    const int64_t r = a.tail_row[t];
    if (r < 0 || r >= a.n_dst) continue;
    const int64_t rb = load_ptr(a.ptr, r, a.ptr_bytes), re = min(load_ptr(a.ptr, r + 1, a.ptr_bytes), e_total);
    const int64_t m = (re - 1) / a.tile - t + 1;
    const int nb = static_cast<int>((m + kSeqPartials - 1) / kSeqPartials);
    const int base = a.long_base[i];
    if (base + nb > a.max_blocks) continue;
    const int64_t out = a.targets != nullptr ? a.targets[r] : r;
    for (int c = lane * VW; c < a.width; c += 32 * VW) {
      PVec<VW> s, v;
      s.load(a.block_sums + static_cast<int64_t>(base) * a.width + c);
      for (int b = 1; b < nb; ++b) {
        v.load(a.block_sums + static_cast<int64_t>(base + b) * a.width + c);
        s.add(v);
      }
      finish_row<T, VW>(a, s, y + out * a.width + c, re - rb);
    }
  }
}

template <typename T, int CB, int NV, typename IdxT, bool TMA>
cudaError_t launch_stream3(const StreamArgs &a, int valmode, int grid, size_t smem, cudaStream_t st) {
#define CXG_STREAM(VM)                                                                               \
  do {                                                                                               \
    auto k = spmm_stream<T, CB, NV, VM, IdxT, TMA>;                                                  \
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e != cudaSuccess) return e;                                                                  \
    k<<<grid, kSThreads, smem, st>>>(a);                                                             \
  } while (0)
  if (valmode == 0)
    CXG_STREAM(0);
  else if (valmode == 1)
    CXG_STREAM(1);
  else
    CXG_STREAM(2);
#undef CXG_STREAM
  return cudaSuccess;
}

template <typename T, typename IdxT, bool TMA>
cudaError_t launch_stream2(const StreamArgs &a, int cb, int nv, int valmode, int grid, size_t smem,
                           cudaStream_t st) {
  if (cb == 4) return launch_stream3<T, 4, 1, IdxT, TMA>(a, valmode, grid, smem, st);
  if (cb == 8) return launch_stream3<T, 8, 1, IdxT, TMA>(a, valmode, grid, smem, st);
  if (nv == 1) return launch_stream3<T, 16, 1, IdxT, TMA>(a, valmode, grid, smem, st);
  return launch_stream3<T, 16, 2, IdxT, TMA>(a, valmode, grid, smem, st);
}

template <typename T, typename IdxT>
cudaError_t launch_stream1(const StreamArgs &a, int cb, int nv, int valmode, int grid, size_t smem,
                           cudaStream_t st) {
  return a.mode == kModeBulk ? launch_stream2<T, IdxT, true>(a, cb, nv, valmode, grid, smem, st)
                             : launch_stream2<T, IdxT, false>(a, cb, nv, valmode, grid, smem, st);
}

template <typename T, int CB, typename IdxT>
cudaError_t launch_fast3(const StreamArgs &a, int grid, cudaStream_t st) {
  constexpr int RB = 32 * CB;
  // two half-size stages in flight per warp (measured 2-3 % faster than one 8 KiB stage on every graph size)
  const bool two = kStageBytes / 2 / RB >= 4;
  const int rows = two ? 2 * ((kStageBytes / 2) / RB > 32 ? 32 : (kStageBytes / 2) / RB)
                       : (kStageBytes / RB > 32 ? 32 : kStageBytes / RB);
  const bool idxs = two && a.tma_index;
  const size_t smem = static_cast<size_t>(rows) * RB * kSWarps + (idxs ? kSWarps * (2 * kIdxChunkBytes + 16) : 0);
  auto k = idxs ? (a.accumulate ? spmm_stream_fast<T, CB, IdxT, true, 2, true> : spmm_stream_fast<T, CB, IdxT, false, 2, true>)
           : a.accumulate
               ? (two ? spmm_stream_fast<T, CB, IdxT, true, 2, false> : spmm_stream_fast<T, CB, IdxT, true, 1, false>)
               : (two ? spmm_stream_fast<T, CB, IdxT, false, 2, false> : spmm_stream_fast<T, CB, IdxT, false, 1, false>);
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  k<<<grid, kSThreads, smem, st>>>(a);
  return cudaSuccess;
}

template <typename T, typename IdxT>
cudaError_t launch_fast2(const StreamArgs &a, int cb, int grid, cudaStream_t st) {
  if (cb == 4) return launch_fast3<T, 4, IdxT>(a, grid, st);
  if (cb == 8) return launch_fast3<T, 8, IdxT>(a, grid, st);
  return launch_fast3<T, 16, IdxT>(a, grid, st);
}

cudaError_t launch_fast(const StreamArgs &a, int dtype, int cb, int idx_bytes, int grid, cudaStream_t st) {
  if (dtype == CXG_F32)
    return idx_bytes == 8 ? launch_fast2<float, int64_t>(a, cb, grid, st) : launch_fast2<float, int32_t>(a, cb, grid, st);
  return idx_bytes == 8 ? launch_fast2<__nv_bfloat16, int64_t>(a, cb, grid, st)
                        : launch_fast2<__nv_bfloat16, int32_t>(a, cb, grid, st);
}

}  // namespace

bool stream_eligible(const cxg_spmm_desc *d) {
  const int elem = d->dtype == CXG_F32 ? 4 : 2;
  const int64_t row_bytes = static_cast<int64_t>(d->feat) * d->heads * elem;
  if (d->edge_mask != nullptr) return false;
  if (row_bytes % 16 != 0 || row_bytes > 1024) return false;
  if (reinterpret_cast<uintptr_t>(d->x) % 16 != 0 || reinterpret_cast<uintptr_t>(d->y) % 16 != 0) return false;
  if (d->heads > 1) {
    // a lane's chunk must stay inside one head
    int cb = row_bytes > 256 ? 16 : (row_bytes > 128 ? 8 : 4);
    if ((static_cast<int64_t>(d->feat) * elem) % cb != 0 || d->heads > 16) return false;
  }
  return true;
}

int stream_tile_edges(const cxg_spmm_desc *d) {
  if (d->split_edges > 0) return d->split_edges;
  // enough tiles that every resident warp gets several, 512 edges at most
  int64_t warps = static_cast<int64_t>(kNumSM) * kCtasPerSM * kSWarps;
  int64_t t = d->nnz / (warps * 4);
  if (t > 512) t = 512;
  if (t < 64) t = 64;
  return static_cast<int>(t / 32 * 32);
}

int stream_layout(int64_t nnz, int64_t width, int tile, StreamLayout *L) {
  int64_t max_tiles = (nnz + tile - 1) / tile + 1;
  if (max_tiles > INT32_MAX) return CXG_ELIMIT;
  size_t off = 0;
  L->hdr = off;
  off = align_up(off + 64 * sizeof(int32_t), 256);
  L->tile_row = off;
  off = align_up(off + max_tiles * sizeof(int64_t), 256);
  L->tail_row = off;
  off = align_up(off + max_tiles * sizeof(int64_t), 256);
  L->long_tiles = off;
  int64_t max_long = max_tiles / kSeqPartials + 1;
  off = align_up(off + max_long * sizeof(int64_t), 256);
  L->long_base = off;
  off = align_up(off + max_long * sizeof(int32_t), 256);
  // a chain of m > 64 partials has ceil(m / 64) <= m / 64 + 1 blocks; chains are disjoint in tiles
  int64_t max_blocks = max_tiles / kSeqPartials + max_long + 1;
  L->block_owner = off;
  off = align_up(off + max_blocks * sizeof(int32_t), 256);
  L->block_sums = off;
  off = align_up(off + static_cast<size_t>(max_blocks) * width * sizeof(float), 256);
  L->partials = off;
  off = align_up(off + static_cast<size_t>(max_tiles) * 2 * width * sizeof(float), 256);
  L->total = off;
  L->max_tiles = max_tiles;
  L->max_long = static_cast<int>(max_long);
  L->max_blocks = static_cast<int>(max_blocks);
  return CXG_OK;
}

int stream_launch(const cxg_spmm_desc *d, void *workspace, size_t workspace_bytes, cudaStream_t st) {
  const int elem = d->dtype == CXG_F32 ? 4 : 2;
  StreamArgs a;
  a.ptr = d->ptr, a.idx = d->idx, a.x = d->x, a.y = d->y;
  a.edge_val = d->edge_val, a.edge_rel = d->edge_rel, a.targets = d->targets;
  a.n_dst = d->n_dst, a.nnz = d->nnz, a.rel_stride = d->rel_stride;
  a.wait_cycles = wait_limit_cycles();
  a.test_stall = (d->flags & CXG_SPMM_TEST_STALL) ? 1 : 0;
  a.tma_index = 0;
  a.feat = d->feat, a.heads = d->heads, a.width = d->feat * d->heads;
  a.ptr_bytes = d->ptr_bytes, a.reduce = d->reduce;
  a.accumulate = (d->flags & CXG_SPMM_ACCUMULATE) ? 1 : 0;
  a.tile = stream_tile_edges(d);
  const int row_bytes = a.width * elem;
  StreamLayout L;
  int rc = stream_layout(d->nnz, a.width, a.tile, &L);
  if (rc != CXG_OK) return set_error(rc, "cxg_spmm_csr: graph too large for 32-bit tile ids");
  if (workspace == nullptr || workspace_bytes < L.total)
    return set_error(CXG_EWORKSPACE, "cxg_spmm_csr: workspace %zu bytes, need %zu", workspace_bytes, L.total);
  char *ws = reinterpret_cast<char *>(workspace);
  a.hdr = reinterpret_cast<int32_t *>(ws + L.hdr);
  a.tile_row = reinterpret_cast<int64_t *>(ws + L.tile_row);
  a.tail_row = reinterpret_cast<int64_t *>(ws + L.tail_row);
  a.long_tiles = reinterpret_cast<int64_t *>(ws + L.long_tiles);
  a.long_base = reinterpret_cast<int32_t *>(ws + L.long_base);
  a.block_owner = reinterpret_cast<int32_t *>(ws + L.block_owner);
  a.block_sums = reinterpret_cast<float *>(ws + L.block_sums);
  a.max_blocks = L.max_blocks;
  a.partials = reinterpret_cast<float *>(ws + L.partials);
  a.max_tiles = L.max_tiles;
  a.max_long = L.max_long;

  int B = kStageBytes / row_bytes;
  if (B > 32) B = 32;
  if (B < 1) B = 1;
  a.stage_edges = B;
  a.stage_bytes = B * row_bytes;
  const int cpr = row_bytes / 16;
  a.cpr_shift = -1;
  for (int sh = 0; sh < 8; ++sh)
    if ((1 << sh) == cpr) a.cpr_shift = sh;
  a.mode = (d->flags & CXG_SPMM_BULK_ROWS) ? kModeBulk : kModeCpAsync;
  const int cb = row_bytes > 256 ? 16 : (row_bytes > 128 ? 8 : 4);
  const int nv = row_bytes > 512 ? 2 : 1;
  const int valmode = d->edge_val == nullptr ? 0 : (d->heads == 1 ? 1 : 2);
  const int vals = valmode == 0 ? 0 : (valmode == 1 ? B : B * d->heads);
  a.slot_offset = static_cast<int>(align_up(64 + static_cast<size_t>(kStages) * vals * sizeof(float), 128));
  a.warp_smem = static_cast<int>(align_up(a.slot_offset + static_cast<size_t>(kStages) * a.stage_bytes, 128));
  const size_t smem = static_cast<size_t>(a.warp_smem) * kSWarps;

  unsigned pb = static_cast<unsigned>((L.max_tiles + 255) / 256);
  spmm_stream_plan<<<pb, 256, 0, st>>>(a);
  // CXG_SPMM_SHARE_SMS: four persistent CTAs per SM instead of six, so that a kernel of another stream (a
  // collective's copy kernel) finds registers and shared memory on every SM while this one runs
  int grid = kNumSM * ((d->flags & CXG_SPMM_SHARE_SMS) ? 4 : kCtasPerSM);
  cudaError_t e;
  // the lean kernel covers full-warp rows without per-edge extras; ids are kept as 32-bit there (a feature matrix
  // of 2^32 rows of 128 bytes would not fit the device)
  const bool fast = row_bytes == 32 * cb && valmode == 0 && a.mode == kModeCpAsync && d->edge_rel == nullptr &&
                    d->targets == nullptr && !(d->flags & CXG_SPMM_GENERIC_WALK);
  if (fast) {
    if (!(d->flags & CXG_SPMM_SHARE_SMS)) {
      grid = kNumSM * CXG_FAST_CTAS;
    }
    // the bulk copies of the id ring need 16-byte aligned sources: tiles are multiples of 32 ids, so the base decides
    a.tma_index = (d->flags & CXG_SPMM_TMA_INDEX) && reinterpret_cast<uintptr_t>(d->idx) % 16 == 0 && a.tile % 32 == 0;
    e = launch_fast(a, d->dtype, cb, d->idx_bytes, grid, st);
  } else if (d->dtype == CXG_F32)
    e = d->idx_bytes == 8 ? launch_stream1<float, int64_t>(a, cb, nv, valmode, grid, smem, st)
                          : launch_stream1<float, int32_t>(a, cb, nv, valmode, grid, smem, st);
  else
    e = d->idx_bytes == 8 ? launch_stream1<__nv_bfloat16, int64_t>(a, cb, nv, valmode, grid, smem, st)
                          : launch_stream1<__nv_bfloat16, int32_t>(a, cb, nv, valmode, grid, smem, st);
  if (e != cudaSuccess) return set_error(CXG_ECUDA, "cxg_spmm_csr: %s", cudaGetErrorString(e));
  const bool v4 = a.width % 4 == 0;
  const int fg = kNumSM * 8;
  if (d->dtype == CXG_F32) {
    if (v4) {
      spmm_stream_fix<float, 4><<<fg, 256, 0, st>>>(a);
      spmm_stream_fix_long_blocks<4><<<fg, 256, 0, st>>>(a);
      spmm_stream_fix_long_rows<float, 4><<<kNumSM, 256, 0, st>>>(a);
    } else {
      spmm_stream_fix<float, 1><<<fg, 256, 0, st>>>(a);
      spmm_stream_fix_long_blocks<1><<<fg, 256, 0, st>>>(a);
      spmm_stream_fix_long_rows<float, 1><<<kNumSM, 256, 0, st>>>(a);
    }
  } else {
    if (v4) {
      spmm_stream_fix<__nv_bfloat16, 4><<<fg, 256, 0, st>>>(a);
      spmm_stream_fix_long_blocks<4><<<fg, 256, 0, st>>>(a);
      spmm_stream_fix_long_rows<__nv_bfloat16, 4><<<kNumSM, 256, 0, st>>>(a);
    } else {
      spmm_stream_fix<__nv_bfloat16, 1><<<fg, 256, 0, st>>>(a);
      spmm_stream_fix_long_blocks<1><<<fg, 256, 0, st>>>(a);
      spmm_stream_fix_long_rows<__nv_bfloat16, 1><<<kNumSM, 256, 0, st>>>(a);
    }
  }
  count_launches(5);
  return check_launch("cxg_spmm_csr (streaming)");
}

}  // namespace cxg
