// Fused GAT aggregation for sm_100a: attention score, LeakyReLU, edge softmax and the weighted
// neighbour sum in ONE walk over the edges, forward and backward.
//
// The reference runs this as five kernels with three [E, H] round trips through memory
// (cxgnncomp/graph_conv.py:458-496: two score reductions, edge_softmax_fwd with its mask,
// src/cpp/src/edge_softmax.cu:3-42, then gen_fwd_sum_edge_value_multi_head,
// src/cpp/src/aggr_kernel.cu:155-186; backward: aggr_kernel.cu:443-491 and edge_softmax.cu:44-95).
// Here per-edge values never reach memory:
//
//   forward   y[r,h,:] = sum_e p[e,h] x[s(e),h,:],  p = softmax over the edges of row r of
//             t[e,h] = leaky(a_dst[r,h] + a_src[s(e),h]).  The walk is the edge-tiled one of the
//             streaming SpMM (tiles of consecutive edges, one warp per tile, feature rows staged
//             with 16-byte cp.async); per (row, head) it keeps a running maximum m and a running
//             sum s and rescales the fp32 accumulator when the maximum grows (online softmax):
//                 m' = max(m, t);  acc = acc * exp(m - m') + exp(t - m') * x;  s likewise.
//             Outputs y, row_max = m and row_sum = s per (row, head): [N, H] each instead of [E, H].
//             A row that crosses tile borders leaves (acc, m, s) partials per tile; a second kernel
//             merges them in tile order with the same rescaling. No atomics: results are the same on
//             every run.
//   backward  on the TRANSPOSED graph (row = source s, entries = destinations r), with
//             D[r,h] = <dy[r,h,:], y[r,h,:]> precomputed per row (the softmax-gradient row sum
//             sum_e p dp equals it, so no second pass over the edges is needed):
//                 p  = exp(leaky(a_dst[r] + a_src[s]) - row_max[r]) / row_sum[r]      (recomputed)
//                 dp = <dy[r,h,:], x[s,h,:]>                                          (per-head SDDMM)
//                 dt = p (dp - D[r,h]) * (t > 0 ? 1 : slope)
//                 dx[s,h,:] += p dy[r,h,:];   d a_src[s,h] += dt      (registers, fixed order)
//                 d a_dst[r,h] += dt: with the forward position of every transposed edge at hand (t_eid of
//                 the transpose) dt is stored at that position of a [nnz, H] scratch array and every
//                 destination then adds its edges' values in a fixed order (same bits on every run); without
//                 it, one atomic add per edge and head (order not fixed, as the reference's grad_src atomics).
//
// Shapes covered: fp32 features, heads a power of two <= 16, a feature row (heads * c floats) of exactly
// 128, 256 or 512 bytes (every lane owns 4, 8 or 16 bytes of it, inside one head). Everything else stays on
// the separate kernels (cxg_gat_scores, cxg_edge_softmax_forward, cxg_spmm_csr).
#include "common.cuh"

namespace cxg {
namespace {

constexpr int kGWarps = 4;
constexpr int kGThreads = kGWarps * 32;
constexpr int kGCtasPerSM = 5;
constexpr int kGStageBytes = 8192;
constexpr int kGFar = 1 << 30;
constexpr float kNegBig = -1e30f;  // "no edge yet": exp(kNegBig - t) is 0 for every finite t
constexpr int kFixSeq = 32;        // chains of more partials are joined by a whole CTA
constexpr int kLongRowEdges = 256;  // ordered d a_dst: destinations with more edges are summed piecewise by CTAs
                                    // (a single warp on a longer row is the tail of the kernel)

struct GatArgs {
  const void *ptr;       // graph that is walked: CSR (forward) or transposed CSR (backward)
  const void *idx;
  const float *gathered; // rows fetched per edge: x [n_src, H, C] (forward), dy [n_dst, H, C] (backward)
  const float *g_small;  // small per-node record fetched per edge: a_src [n_src, H] (forward),
                         // stats [n_dst, H, 4] = {a_dst, row_max, 1 / row_sum, D} (backward)
  const float *r_small;  // per walked row: a_dst [n_dst, H] (forward), a_src [n_src, H] (backward)
  const float *r_feat;   // backward: x [n_src, H, C]
  float *out;            // y [n_dst, H, C] (forward), dx [n_src, H, C] (backward)
  float *row_max;        // forward [n_dst, H]
  float *row_sum;        // forward [n_dst, H]
  float *d_r_small;      // backward: d a_src [n_src, H]
  float *d_g_small;      // backward: d a_dst [n_dst, H], added into atomically (when d_edge is NULL)
  const void *eid;       // backward, ordered mode: forward edge of every transposed edge (width of idx)
  float *d_edge;         // backward, ordered mode: [nnz, H] score gradient of every edge at its forward position
  int64_t n_rows, nnz, max_tiles;
  int heads, hshift, c, ptr_bytes, idx_bytes, tile;
  float slope;
  int32_t *hdr;
  int64_t *tile_row, *tail_row;
  int64_t *long_tiles;  // first tile of every chain of more than kFixSeq partials
  int max_long;
  float *part_acc;  // [tile][2][width]
  float *part_ms;   // [tile][2][heads][2]: forward (m, s); backward (d a_src partial, unused)
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
template <int EL>
__device__ __forceinline__ void lds_row(float *f, uint32_t addr) {
  if (EL == 1) {
    f[0] = lds_f32(addr);
  } else if (EL == 2) {
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(f[0]), "=f"(f[EL > 1 ? 1 : 0]) : "r"(addr));
  } else {
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(f[0]), "=f"(f[EL > 1 ? 1 : 0]), "=f"(f[EL > 2 ? 2 : 0]), "=f"(f[EL > 3 ? 3 : 0])
                 : "r"(addr));
  }
}
template <int EL>
__device__ __forceinline__ void stg_row(float *p, const float *f) {
  if (EL == 1)
    *p = f[0];
  else if (EL == 2)
    *reinterpret_cast<float2 *>(p) = make_float2(f[0], f[EL > 1 ? 1 : 0]);
  else
    *reinterpret_cast<float4 *>(p) = make_float4(f[0], f[EL > 1 ? 1 : 0], f[EL > 2 ? 2 : 0], f[EL > 3 ? 3 : 0]);
}
template <int EL>
__device__ __forceinline__ void ldg_row(float *f, const float *p) {
  if (EL == 1) {
    f[0] = __ldg(p);
  } else if (EL == 2) {
    const float2 v = __ldg(reinterpret_cast<const float2 *>(p));
    f[0] = v.x, f[EL > 1 ? 1 : 0] = v.y;
  } else {
    const float4 v = __ldg(reinterpret_cast<const float4 *>(p));
    f[0] = v.x, f[EL > 1 ? 1 : 0] = v.y, f[EL > 2 ? 2 : 0] = v.z, f[EL > 3 ? 3 : 0] = v.w;
  }
}
__device__ __forceinline__ float leaky(float t, float slope) { return fmaxf(t, t * slope); }

// acc = acc * sc + w * f over EL floats; pairs go through the packed f32x2 pipe (each half rounded like the
// scalar operation).
template <int EL>
__device__ __forceinline__ void scale_fma(float *acc, const float *f, float sc, float w) {
  if (EL == 1) {
    acc[0] = fmaf(w, f[0], acc[0] * sc);
  } else {
    unsigned long long s2, w2;
    asm("mov.b64 %0, {%1,%1};" : "=l"(s2) : "f"(sc));
    asm("mov.b64 %0, {%1,%1};" : "=l"(w2) : "f"(w));
#pragma unroll
    for (int i = 0; i < EL; i += 2) {
      unsigned long long a2, f2;
      asm("mov.b64 %0, {%1,%2};" : "=l"(a2) : "f"(acc[i]), "f"(acc[(i + 1) % EL]));
      asm("mov.b64 %0, {%1,%2};" : "=l"(f2) : "f"(f[i]), "f"(f[(i + 1) % EL]));
      asm("mul.rn.f32x2 %0, %0, %1;" : "+l"(a2) : "l"(s2));
      asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(a2) : "l"(w2), "l"(f2));
      asm("mov.b64 {%0,%1}, %2;" : "=f"(acc[i]), "=f"(acc[(i + 1) % EL]) : "l"(a2));
    }
  }
}
__device__ __forceinline__ void red_add_f32(float *addr, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ int64_t edge_total(const GatArgs &a) {
  const int64_t e = load_ptr(a.ptr, a.n_rows, a.ptr_bytes);
  return e > a.nnz ? a.nnz : e;
}

__global__ void gat_plan(GatArgs a) {
  const int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (t == 0) {
    a.hdr[0] = 0;  // number of long chains
    a.hdr[1] = 0;  // number of long destinations (ordered d a_dst)
  }
  if (t >= a.max_tiles) return;
  a.tail_row[t] = -1;
  const int64_t e_total = edge_total(a);
  const int64_t pos = t * a.tile;
  if (pos >= e_total) return;
  int64_t lo = 0, hi = a.n_rows;  // ptr[lo] <= pos < ptr[hi]
  while (hi - lo > 1) {
    const int64_t mid = (lo + hi) >> 1;
    if (load_ptr(a.ptr, mid, a.ptr_bytes) <= pos)
      lo = mid;
    else
      hi = mid;
  }
  a.tile_row[t] = lo;
}

// The walk shared by both directions. CB = bytes of a feature row per lane (row = 32 * CB bytes).
// BWD = false: forward (online softmax). BWD = true: backward on the transposed graph.
template <int CB, typename IdxT, bool BWD>
__global__ void __launch_bounds__(kGThreads, kGCtasPerSM) gat_walk(GatArgs a) {
  constexpr int EL = CB / 4;
  constexpr int RB = 32 * CB;
  constexpr int B = kGStageBytes / RB > 32 ? 32 : kGStageBytes / RB;
  constexpr int CPR = RB / 16, RPI = 32 / CPR, NCOPY = B * CPR / 32;
  constexpr int WIDTH = RB / 4;
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int H = a.heads;
  const int small_bytes = BWD ? H * 16 : H * 4;  // per-edge record
  const int warp_smem = B * RB + B * small_bytes;
  const uint32_t sl = smem_u32(smem + static_cast<size_t>(warp) * warp_smem);
  const uint32_t sv = sl + B * RB;
  const uint32_t my = sl + lane * CB;
  const int lph = (a.c * 4) / CB;  // lanes per head
  const int h = lane / lph;        // this lane's head
  const bool head_lead = (lane % lph) == 0;
  const IdxT *idx = reinterpret_cast<const IdxT *>(a.idx);
  const uint8_t *xg = reinterpret_cast<const uint8_t *>(a.gathered);
  const int64_t e_total = edge_total(a);
  const int64_t n_tiles = (e_total + a.tile - 1) / a.tile;
  const int64_t gwarp = static_cast<int64_t>(blockIdx.x) * kGWarps + warp;
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * kGWarps;
  const int jrow = lane / CPR;
  const uint8_t *xlane = xg + (lane % CPR) * 16;
  const uint32_t cdst = sl + lane * 16;
  const float slope = a.slope;

  // a row of the walked graph without entries: zeros (and "no edge" statistics in the forward direction)
  auto empty_row = [&](int64_t r) {
    float z[EL];
#pragma unroll
    for (int i = 0; i < EL; ++i) z[i] = 0.f;
    stg_row<EL>(a.out + r * WIDTH + lane * EL, z);
    if (head_lead) {
      if (BWD) {
        a.d_r_small[r * H + h] = 0.f;
      } else {
        a.row_max[r * H + h] = kNegBig;
        a.row_sum[r * H + h] = 0.f;
      }
    }
  };

  if (e_total == 0) {
    for (int64_t r = gwarp; r < a.n_rows; r += nwarps) empty_row(r);
    return;
  }

  for (int64_t t = gwarp; t < n_tiles; t += nwarps) {
    const int64_t tb = t * a.tile;
    const int tile_len = static_cast<int>(min(static_cast<int64_t>(a.tile), e_total - tb));
    const int n_stage = (tile_len + B - 1) / B;
    int64_t row = a.tile_row[t];
    if (t == 0)
      for (int64_t r = 0; r < row; ++r) empty_row(r);
    int64_t pbase = row;
    auto load_ends = [&]() -> int {
      const int64_t r = pbase + lane;
      if (r >= a.n_rows) return kGFar;
      const int64_t v = load_ptr(a.ptr, r + 1, a.ptr_bytes) - tb;
      return v > kGFar ? kGFar : static_cast<int>(v);
    };
    int pc = load_ends();
    int rrel = 0;
    int rend = __shfl_sync(0xffffffffu, pc, 0);
    const int64_t rs64 = load_ptr(a.ptr, row, a.ptr_bytes) - tb;
    int rstart = rs64 < -kGFar ? -kGFar : static_cast<int>(rs64);
    const IdxT *idx_t = idx + tb;

    auto load_nid = [&](int k) -> uint32_t {
      const int pos = k * B + lane;
      return (lane < B && pos < tile_len) ? static_cast<uint32_t>(__ldg(idx_t + pos)) : 0u;
    };
    auto fill = [&](int k, uint32_t nid) {
      const int cnt = min(B, tile_len - k * B);
#pragma unroll
      for (int c = 0; c < NCOPY; ++c) {
        const uint32_t nj = __shfl_sync(0xffffffffu, nid, (c * RPI + jrow) & 31);
        if (c * RPI + jrow < cnt) cp_async16(cdst + c * 512, xlane + static_cast<uint64_t>(nj) * RB);
      }
      // the small record of every edge of the stage
      for (int q0 = 0; q0 < B * H; q0 += 32) {
        const int q = q0 + lane;
        const int e = q >> a.hshift;
        const uint32_t nj = __shfl_sync(0xffffffffu, nid, e & 31);
        if (e < cnt) {
          if (BWD)
            cp_async16(sv + q * 16, a.g_small + (static_cast<uint64_t>(nj) * H + (q & (H - 1))) * 4);
          else
            cp_async4(sv + q * 4, a.g_small + static_cast<uint64_t>(nj) * H + (q & (H - 1)));
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // per-row state
    float acc[EL];
    float m = kNegBig, s = 0.f;  // forward: running max and sum; backward: s = d a_src accumulator
    float rsm = 0.f;             // a_dst[row, h] (forward) / a_src[row, h] (backward)
    float xr[EL];                // backward: x[row, h, this lane's columns]
    auto begin_row = [&](int64_t r) {
#pragma unroll
      for (int i = 0; i < EL; ++i) acc[i] = 0.f;
      m = kNegBig, s = 0.f;
      if (r < a.n_rows) {
        rsm = __ldg(a.r_small + r * H + h);
        if (BWD) ldg_row<EL>(xr, a.r_feat + r * WIDTH + lane * EL);
      }
    };
    begin_row(row);
    uint32_t nid_cur = load_nid(0);
    fill(0, nid_cur);
    // ordered d a_dst: the forward position of every transposed edge, fetched like the ids
    const IdxT *eid_t = reinterpret_cast<const IdxT *>(a.eid) + tb;
    const bool ordered = BWD && a.d_edge != nullptr;
    auto load_eid = [&](int k) -> uint32_t {
      const int pos = k * B + lane;
      return (ordered && lane < B && pos < tile_len) ? static_cast<uint32_t>(__ldg(eid_t + pos)) : 0u;
    };
    uint32_t eid_cur = load_eid(0);

    for (int k = 0; k < n_stage; ++k) {
      const uint32_t nid_next = load_nid(k + 1);
      const uint32_t eid_next = load_eid(k + 1);
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncwarp();
      const int sbase = k * B;
      const int send = min(sbase + B, tile_len);
      int pos = sbase;
      uint32_t p = my;
      uint32_t pv = sv + h * (BWD ? 16 : 4);
      while (pos < send) {
        const int stop = min(send, rend);
        for (; pos < stop; ++pos) {
          float f[EL];
          lds_row<EL>(f, p);
          if (!BWD) {
            const float tt = leaky(lds_f32(pv) + rsm, slope);
            const float mn = fmaxf(m, tt);
            const float sc = __expf(m - mn), w = __expf(tt - mn);
            s = fmaf(s, sc, w);
            m = mn;
            scale_fma<EL>(acc, f, sc, w);
          } else {
            float st[4];
            lds_row<4>(st, pv);  // {a_dst, row_max, 1 / row_sum, D} of the destination, this lane's head
            const float t0 = st[0] + rsm;
            const float w = __expf(leaky(t0, slope) - st[1]) * st[2];
            float dp = 0.f;
#pragma unroll
            for (int i = 0; i < EL; ++i) dp = fmaf(f[i], xr[i], dp);
            for (int o = lph >> 1; o > 0; o >>= 1) dp += __shfl_xor_sync(0xffffffffu, dp, o);
            const float dt = w * (dp - st[3]) * (t0 > 0.f ? 1.f : slope);
            s += dt;
#pragma unroll
            for (int i = 0; i < EL; ++i) acc[i] = fmaf(w, f[i], acc[i]);
            if (ordered) {  // left at the edge's forward position; the destinations add theirs up afterwards
              const uint32_t fe = __shfl_sync(0xffffffffu, eid_cur, pos - sbase);
              if (head_lead) a.d_edge[static_cast<uint64_t>(fe) * H + h] = dt;
            } else {
              const uint32_t dst_node = __shfl_sync(0xffffffffu, nid_cur, pos - sbase);
              if (head_lead) red_add_f32(a.d_g_small + static_cast<uint64_t>(dst_node) * H + h, dt);
            }
          }
          p += RB;
          pv += small_bytes;
        }
        if (pos == rend) {
          if (rstart < 0) {
            stg_row<EL>(a.part_acc + (t * 2) * WIDTH + lane * EL, acc);
            if (head_lead) {
              a.part_ms[((t * 2) * H + h) * 2] = m;
              a.part_ms[((t * 2) * H + h) * 2 + 1] = s;
            }
          } else {
            if (!BWD) {
              const float inv = 1.f / s;
              float o[EL];
#pragma unroll
              for (int i = 0; i < EL; ++i) o[i] = acc[i] * inv;
              stg_row<EL>(a.out + row * WIDTH + lane * EL, o);
              if (head_lead) {
                a.row_max[row * H + h] = m;
                a.row_sum[row * H + h] = s;
              }
            } else {
              stg_row<EL>(a.out + row * WIDTH + lane * EL, acc);
              if (head_lead) a.d_r_small[row * H + h] = s;
            }
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
            empty_row(row);
          }
          begin_row(row);
        }
      }
      __syncwarp();
      if (k + 1 < n_stage) fill(k + 1, nid_next);
      nid_cur = nid_next;
      eid_cur = eid_next;
    }
    int64_t tail = -1;
    if (row < a.n_rows && rstart < tile_len && rend > tile_len) {
      const int which = rstart < 0 ? 0 : 1;
      stg_row<EL>(a.part_acc + (t * 2 + which) * WIDTH + lane * EL, acc);
      if (head_lead) {
        a.part_ms[((t * 2 + which) * H + h) * 2] = m;
        a.part_ms[((t * 2 + which) * H + h) * 2 + 1] = s;
      }
      if (which) tail = row;
    }
    if (lane == 0) a.tail_row[t] = tail;
  }
}

// One partial of a chain: element 0 is the tail partial of tile t, element k > 0 the head partial of tile t + k.
template <int EL, int WIDTH>
__device__ __forceinline__ void load_partial(const GatArgs &a, int64_t t, int64_t k, int lane, int h, float *f, float &m,
                                             float &s) {
  const int64_t slot = k == 0 ? t * 2 + 1 : (t + k) * 2;
  ldg_row<EL>(f, a.part_acc + slot * WIDTH + lane * EL);
  m = a.part_ms[(slot * a.heads + h) * 2];
  s = a.part_ms[(slot * a.heads + h) * 2 + 1];
}

// (acc, m, s) <- (acc, m, s) joined with (f, mu, su). Forward: online-softmax merge; backward: plain sums.
template <int EL, bool BWD>
__device__ __forceinline__ void join(float *acc, float &m, float &s, const float *f, float mu, float su) {
  if (BWD) {
#pragma unroll
    for (int i = 0; i < EL; ++i) acc[i] += f[i];
    s += su;
  } else {
    const float mn = fmaxf(m, mu);
    const float ca = __expf(m - mn), cb = __expf(mu - mn);
    scale_fma<EL>(acc, f, ca, cb);
    s = fmaf(s, ca, su * cb);
    m = mn;
  }
}

template <int EL, int WIDTH, bool BWD>
__device__ __forceinline__ void finish_chain(const GatArgs &a, int64_t r, int lane, int h, bool head_lead, float *acc,
                                             float m, float s) {
  if (BWD) {
    stg_row<EL>(a.out + r * WIDTH + lane * EL, acc);
    if (head_lead) a.d_r_small[r * a.heads + h] = s;
  } else {
    const float inv = 1.f / s;
#pragma unroll
    for (int i = 0; i < EL; ++i) acc[i] *= inv;
    stg_row<EL>(a.out + r * WIDTH + lane * EL, acc);
    if (head_lead) {
      a.row_max[r * a.heads + h] = m;
      a.row_sum[r * a.heads + h] = s;
    }
  }
}

// Joins the partials of rows that cross tile borders, in tile order: one warp per chain of up to kFixSeq
// partials; longer chains are listed for gat_fix_long.
template <int CB, bool BWD>
__global__ void __launch_bounds__(256) gat_fix(GatArgs a) {
  constexpr int EL = CB / 4;
  constexpr int WIDTH = 32 * CB / 4;
  const int lane = threadIdx.x & 31;
  const int lph = (a.c * 4) / CB;
  const int h = lane / lph;
  const bool head_lead = (lane % lph) == 0;
  const int64_t e_total = edge_total(a);
  const int64_t n_tiles = (e_total + a.tile - 1) / a.tile;
  const int64_t gwarp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t t = gwarp; t < n_tiles; t += nwarps) {
    const int64_t r = a.tail_row[t];
    if (r < 0 || r >= a.n_rows) continue;
    const int64_t re = min(load_ptr(a.ptr, r + 1, a.ptr_bytes), e_total);
    const int64_t n_part = (re - 1) / a.tile - t + 1;
    if (n_part > kFixSeq) {
      if (lane == 0) {
        const int slot = atomicAdd(a.hdr, 1);
        if (slot < a.max_long) a.long_tiles[slot] = t;
      }
      continue;
    }
    float acc[EL], m, s;
    load_partial<EL, WIDTH>(a, t, 0, lane, h, acc, m, s);
    for (int64_t k = 1; k < n_part; ++k) {
      float f[EL], mu, su;
      load_partial<EL, WIDTH>(a, t, k, lane, h, f, mu, su);
      join<EL, BWD>(acc, m, s, f, mu, su);
    }
    finish_chain<EL, WIDTH, BWD>(a, r, lane, h, head_lead, acc, m, s);
  }
}

// Long chains: the n partials are dealt to the 8 warps of a CTA in contiguous blocks [n w / 8, n (w + 1) / 8); each
// warp joins its block in order, then warp 0 joins the 8 block results in block order.
template <int CB, bool BWD>
__global__ void __launch_bounds__(256) gat_fix_long(GatArgs a) {
  constexpr int EL = CB / 4;
  constexpr int WIDTH = 32 * CB / 4;
  __shared__ float sh_acc[8][WIDTH];
  __shared__ float sh_ms[8][32][2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int lph = (a.c * 4) / CB;
  const int h = lane / lph;
  const bool head_lead = (lane % lph) == 0;
  const int64_t e_total = edge_total(a);
  const int n_long = min(a.hdr[0], a.max_long);
  for (int i = blockIdx.x; i < n_long; i += gridDim.x) {
    const int64_t t = a.long_tiles[i];
    const int64_t r = a.tail_row[t];
    if (r < 0 || r >= a.n_rows) continue;  // uniform over the CTA
    const int64_t re = min(load_ptr(a.ptr, r + 1, a.ptr_bytes), e_total);
    const int64_t n_part = (re - 1) / a.tile - t + 1;
    const int64_t kb = n_part * warp / 8, ke = n_part * (warp + 1) / 8;  // n_part > 32: no block is empty
    float acc[EL], m, s;
    load_partial<EL, WIDTH>(a, t, kb, lane, h, acc, m, s);
#pragma unroll 4
    for (int64_t k = kb + 1; k < ke; ++k) {
      float f[EL], mu, su;
      load_partial<EL, WIDTH>(a, t, k, lane, h, f, mu, su);
      join<EL, BWD>(acc, m, s, f, mu, su);
    }
#pragma unroll
    for (int j = 0; j < EL; ++j) sh_acc[warp][lane * EL + j] = acc[j];
    sh_ms[warp][lane][0] = m;
    sh_ms[warp][lane][1] = s;
    __syncthreads();
    if (warp == 0) {
      for (int w = 1; w < 8; ++w) {
        float f[EL];
#pragma unroll
        for (int j = 0; j < EL; ++j) f[j] = sh_acc[w][lane * EL + j];
        join<EL, BWD>(acc, m, s, f, sh_ms[w][lane][0], sh_ms[w][lane][1]);
      }
      finish_chain<EL, WIDTH, BWD>(a, r, lane, h, head_lead, acc, m, s);
    }
    __syncthreads();
  }
}

// Backward set-up, one warp per destination: stats[r, h] = {a_dst, row_max, 1 / row_sum, <dy[r,h,:], y[r,h,:]>}
// and d a_dst[r, h] = 0 (the walk adds into it).
template <int CB>
__global__ void __launch_bounds__(256) gat_bwd_prepare(const float *dy, const float *y, const float *a_dst,
                                                       const float *row_max, const float *row_sum, float *stats,
                                                       float *d_a_dst, int64_t n_dst, int heads, int c) {
  constexpr int EL = CB / 4;
  constexpr int WIDTH = 32 * CB / 4;
  const int lane = threadIdx.x & 31;
  const int lph = (c * 4) / CB;
  const int h = lane / lph;
  const int64_t gwarp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t r = gwarp; r < n_dst; r += nwarps) {
    float g[EL], v[EL];
    ldg_row<EL>(g, dy + r * WIDTH + lane * EL);
    ldg_row<EL>(v, y + r * WIDTH + lane * EL);
    float d = 0.f;
#pragma unroll
    for (int i = 0; i < EL; ++i) d = fmaf(g[i], v[i], d);
    for (int o = lph >> 1; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
    if ((lane % lph) == 0) {
      const float sum = row_sum[r * heads + h];
      *reinterpret_cast<float4 *>(stats + (r * heads + h) * 4) =
          make_float4(a_dst[r * heads + h], row_max[r * heads + h], sum > 0.f ? 1.f / sum : 0.f, d);
      d_a_dst[r * heads + h] = 0.f;
    }
  }
}

// Ordered d a_dst. The backward walk has left the score gradient of every edge at the edge's forward position
// (d_edge [nnz, H]); a destination's gradient is the sum over its edges, added in an order that depends on the
// graph only: lane (slot, head) of a warp takes every (32 / H)-th edge of the row (four running sums, joined in
// a fixed order), then the slots are joined by a butterfly. Destinations with more than kLongRowEdges edges are
// listed for the two kernels below.
__device__ __forceinline__ float strided_sum(const float *v, int64_t lo, int64_t hi, int64_t step) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int64_t e = lo;
  for (; e + 3 * step < hi; e += 4 * step) {
    s0 += __ldg(v + e);
    s1 += __ldg(v + e + step);
    s2 += __ldg(v + e + 2 * step);
    s3 += __ldg(v + e + 3 * step);
  }
  for (; e < hi; e += step) s0 += __ldg(v + e);
  return (s0 + s1) + (s2 + s3);
}

__global__ void __launch_bounds__(256) gat_dst_sum_rows(const void *ptr, int ptr_bytes, const float *d_edge, float *d_a_dst,
                                                        int64_t n_dst, int64_t nnz, int heads, int hshift, int32_t *hdr,
                                                        int64_t *long_rows, int max_long) {
  constexpr int kRows = 4;  // destinations per warp and round: their loads are in flight together
  const int lane = threadIdx.x & 31;
  const int head = lane & (heads - 1), slot = lane >> hshift, nslot = 32 >> hshift;
  const int64_t gwarp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t r0 = gwarp * kRows; r0 < n_dst; r0 += nwarps * kRows) {
    // ptr[r0 .. r0 + kRows] through the first lanes
    int64_t pe = 0;
    if (lane <= kRows && r0 + lane <= n_dst) pe = min(load_ptr(ptr, r0 + lane, ptr_bytes), nnz);
    int64_t e[kRows + 1];
#pragma unroll
    for (int j = 0; j <= kRows; ++j) e[j] = __shfl_sync(0xffffffffu, pe, j);
    // rows of at most 4 * nslot edges: all their values requested before any is used; a lane's (up to) four values
    // are added as (v0 + v1) + (v2 + v3), which is the order strided_sum gives the same values
    float v[kRows][4];
#pragma unroll
    for (int j = 0; j < kRows; ++j) {
      const bool row_on = r0 + j < n_dst && e[j + 1] - e[j] <= 4 * nslot;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int64_t ed = e[j] + slot + k * nslot;
        v[j][k] = (row_on && ed < e[j + 1]) ? __ldg(d_edge + ed * heads + head) : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < kRows; ++j) {
      const int64_t r = r0 + j;
      if (r >= n_dst) break;
      const int64_t e0 = e[j], e1 = e[j + 1];
      if (e1 - e0 > kLongRowEdges) {
        if (lane == 0) {
          const int s = atomicAdd(hdr + 1, 1);  // the list's order does not enter any sum
          if (s < max_long) long_rows[s] = r;
        }
        continue;
      }
      float acc;
      if (e1 - e0 <= 4 * nslot)
        acc = (v[j][0] + v[j][1]) + (v[j][2] + v[j][3]);
      else  // value (e, head) sits at d_edge[e * heads + head]: this lane walks e = e0 + slot, e0 + slot + nslot, ...
        acc = strided_sum(d_edge + head, (e0 + slot) * heads, e1 * heads, 32);
      for (int o = heads; o < 32; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane < heads) d_a_dst[r * heads + head] = acc;
    }
  }
}

// Long destinations, first level: the edge array is cut into pieces of kPieceEdges consecutive edges; every piece of
// a listed row is summed by one CTA (thread (slot, head) takes every (256 / H)-th edge, then a fixed tree in shared
// memory) into piece_sums. A piece holds at most one listed row's first edges and at most one listed row's later
// edges, hence two slots per piece. The CTAs share a row's pieces round-robin; the rows' edge ranges are read 128
// rows at a time into shared memory.
constexpr int kPieceEdges = 1024;
__global__ void __launch_bounds__(256) gat_dst_sum_pieces(const void *ptr, int ptr_bytes, const float *d_edge,
                                                          float *piece_sums, int64_t nnz, int heads, int hshift,
                                                          const int32_t *hdr, const int64_t *long_rows, int max_long) {
  __shared__ float red[256];
  __shared__ int64_t range[2][128];
  const int tid = threadIdx.x;
  const int head = tid & (heads - 1), slot = tid >> hshift;
  const int n_long = min(hdr[1], max_long);
  const int G = gridDim.x;
  for (int i0 = 0; i0 < n_long; i0 += 128) {
    {
      const int i = i0 + (tid & 127);
      if (i < n_long) range[tid >> 7][tid & 127] = min(load_ptr(ptr, long_rows[i] + (tid >> 7), ptr_bytes), nnz);
    }
    __syncthreads();
    const int cnt = min(128, n_long - i0);
    for (int ii = 0; ii < cnt; ++ii) {
      const int i = i0 + ii;
      const int64_t e0 = range[0][ii], e1 = range[1][ii];
      const int64_t p0 = e0 / kPieceEdges, p1 = (e1 - 1) / kPieceEdges;
      const int first = (static_cast<int>(blockIdx.x) + G - (i % G)) % G;
      for (int64_t p = p0 + first; p <= p1; p += G) {
        const int64_t lo = max(e0, p * kPieceEdges), hi = min(e1, (p + 1) * kPieceEdges);
        red[tid] = strided_sum(d_edge + head, (lo + slot) * heads, hi * heads, 256);
        __syncthreads();
        for (int o = 128; o >= heads; o >>= 1) {
          if (tid < o) red[tid] += red[tid + o];
          __syncthreads();
        }
        if (tid < heads) piece_sums[(2 * p + (p == p0 ? 1 : 0)) * heads + tid] = red[tid];
        __syncthreads();
      }
    }
    __syncthreads();
  }
}

// Second level: one warp per listed destination adds the sums of its pieces, lane (slot, head) every (32 / H)-th
// piece in ascending order, then the butterfly.
__global__ void __launch_bounds__(256) gat_dst_sum_long(const void *ptr, int ptr_bytes, const float *piece_sums,
                                                        float *d_a_dst, int64_t nnz, int heads, int hshift,
                                                        const int32_t *hdr, const int64_t *long_rows, int max_long) {
  const int lane = threadIdx.x & 31;
  const int head = lane & (heads - 1), slot = lane >> hshift, nslot = 32 >> hshift;
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
  const int n_long = min(hdr[1], max_long);
  for (int i = gwarp; i < n_long; i += nwarps) {
    const int64_t r = long_rows[i];
    const int64_t e0 = min(load_ptr(ptr, r, ptr_bytes), nnz), e1 = min(load_ptr(ptr, r + 1, ptr_bytes), nnz);
    const int64_t p0 = e0 / kPieceEdges, p1 = (e1 - 1) / kPieceEdges;
    float acc = 0.f;
    for (int64_t p = p0 + slot; p <= p1; p += nslot) acc += piece_sums[(2 * p + (p == p0 ? 1 : 0)) * heads + head];
    for (int o = heads; o < 32; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane < heads) d_a_dst[r * heads + head] = acc;
  }
}

struct GatLayout {
  size_t hdr, tile_row, tail_row, long_tiles, part_acc, part_ms, stats, long_rows, piece_sums, d_edge, total;
  int64_t max_tiles;
  int max_long;
};

int gat_tile_edges(int64_t nnz) {
  int64_t t = nnz / (static_cast<int64_t>(kNumSM) * kGCtasPerSM * kGWarps * 4);
  if (t > 512) t = 512;
  if (t < 64) t = 64;
  return static_cast<int>(t / 32 * 32);
}

void gat_layout(int64_t n_stats_rows, int64_t nnz, int heads, int c, GatLayout *L) {
  const int64_t width = static_cast<int64_t>(heads) * c;
  L->max_tiles = (nnz + 63) / 64 + 1;  // 64 = smallest tile
  size_t off = 0;
  L->hdr = off;
  off = align_up(off + 256, 256);
  L->tile_row = off;
  off = align_up(off + L->max_tiles * sizeof(int64_t), 256);
  L->tail_row = off;
  off = align_up(off + L->max_tiles * sizeof(int64_t), 256);
  L->max_long = static_cast<int>(L->max_tiles / kFixSeq + 1);
  L->long_tiles = off;
  off = align_up(off + static_cast<size_t>(L->max_long) * sizeof(int64_t), 256);
  L->part_acc = off;
  off = align_up(off + static_cast<size_t>(L->max_tiles) * 2 * width * sizeof(float), 256);
  L->part_ms = off;
  off = align_up(off + static_cast<size_t>(L->max_tiles) * 2 * heads * 2 * sizeof(float), 256);
  L->stats = off;
  off = align_up(off + static_cast<size_t>(n_stats_rows) * heads * 4 * sizeof(float), 256);
  // ordered d a_dst of the backward: destinations of more than kLongRowEdges edges, and one value per edge and head
  L->long_rows = off;
  off = align_up(off + static_cast<size_t>(nnz / kLongRowEdges + 1) * sizeof(int64_t), 256);
  L->piece_sums = off;
  off = align_up(off + static_cast<size_t>(nnz / kPieceEdges + 1) * 2 * heads * sizeof(float), 256);
  L->d_edge = off;
  off = align_up(off + static_cast<size_t>(nnz) * heads * sizeof(float), 256);
  L->total = off;
}

int check_shape(const char *who, int heads, int c) {
  const int row_bytes = heads * c * 4;
  if (heads < 1 || heads > 16 || (heads & (heads - 1)) != 0 || c < 1)
    return set_error(CXG_EUNSUPPORTED, "%s: heads = %d must be a power of two <= 16", who, heads);
  if (row_bytes != 128 && row_bytes != 256 && row_bytes != 512)
    return set_error(CXG_EUNSUPPORTED, "%s: a feature row of heads * c * 4 = %d bytes; 128, 256 or 512 are covered", who,
                     row_bytes);
  const int cb = row_bytes / 32;
  if ((c * 4) % cb != 0)
    return set_error(CXG_EUNSUPPORTED, "%s: c = %d leaves a lane's %d bytes across two heads", who, c, cb);
  return CXG_OK;
}

void fill_args(GatArgs &a, const GatLayout &L, void *workspace, int64_t nnz, int heads, int c, float slope) {
  char *ws = reinterpret_cast<char *>(workspace);
  a.hdr = reinterpret_cast<int32_t *>(ws + L.hdr);
  a.tile_row = reinterpret_cast<int64_t *>(ws + L.tile_row);
  a.tail_row = reinterpret_cast<int64_t *>(ws + L.tail_row);
  a.long_tiles = reinterpret_cast<int64_t *>(ws + L.long_tiles);
  a.max_long = L.max_long;
  a.part_acc = reinterpret_cast<float *>(ws + L.part_acc);
  a.part_ms = reinterpret_cast<float *>(ws + L.part_ms);
  a.max_tiles = L.max_tiles;
  a.nnz = nnz;
  a.heads = heads;
  a.c = c;
  a.hshift = 0;
  while ((1 << a.hshift) < heads) ++a.hshift;
  a.slope = slope;
  a.tile = gat_tile_edges(nnz);
}

template <int CB, bool BWD>
cudaError_t launch_walk(const GatArgs &a, cudaStream_t st) {
  constexpr int RB = 32 * CB;
  constexpr int B = kGStageBytes / RB > 32 ? 32 : kGStageBytes / RB;
  const size_t smem = static_cast<size_t>(kGWarps) * (B * RB + B * a.heads * (BWD ? 16 : 4));
  const unsigned pb = static_cast<unsigned>((a.max_tiles + 255) / 256);
  gat_plan<<<pb, 256, 0, st>>>(a);
  cudaError_t e;
  if (a.idx_bytes == 8) {
    auto k = gat_walk<CB, int64_t, BWD>;
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    k<<<kNumSM * kGCtasPerSM, kGThreads, smem, st>>>(a);
  } else {
    auto k = gat_walk<CB, int32_t, BWD>;
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    k<<<kNumSM * kGCtasPerSM, kGThreads, smem, st>>>(a);
  }
  gat_fix<CB, BWD><<<kNumSM * 4, 256, 0, st>>>(a);
  gat_fix_long<CB, BWD><<<kNumSM, 256, 0, st>>>(a);
  count_launches(4);
  return cudaSuccess;
}

}  // namespace
}  // namespace cxg

using namespace cxg;

extern "C" int cxg_gat_fused_workspace_size(int64_t n_dst, int64_t nnz, int heads, int c, size_t *bytes) {
  CXG_REQUIRE(bytes != nullptr, CXG_ENULL, "cxg_gat_fused_workspace_size: bytes is NULL");
  CXG_REQUIRE(n_dst >= 0 && nnz >= 0 && heads > 0 && c > 0, CXG_EINVAL, "cxg_gat_fused_workspace_size: bad sizes");
  GatLayout L;
  gat_layout(n_dst, nnz, heads, c, &L);
  *bytes = L.total;
  return CXG_OK;
}

extern "C" int cxg_gat_fused_forward(const void *ptr, const void *idx, int ptr_bytes, int idx_bytes, const float *x,
                                     const float *a_src, const float *a_dst, float *y, float *row_max, float *row_sum,
                                     int64_t n_dst, int64_t nnz, int heads, int c, float slope, void *workspace,
                                     size_t workspace_bytes, void *stream) {
  CXG_REQUIRE(n_dst >= 0 && nnz >= 0, CXG_EINVAL, "cxg_gat_fused_forward: negative size");
  CXG_REQUIRE((ptr_bytes == 4 || ptr_bytes == 8) && (idx_bytes == 4 || idx_bytes == 8), CXG_EINVAL,
              "cxg_gat_fused_forward: index widths %d/%d", ptr_bytes, idx_bytes);
  int rc = check_shape("cxg_gat_fused_forward", heads, c);
  if (rc != CXG_OK) return rc;
  if (n_dst == 0) return CXG_OK;
  CXG_REQUIRE(ptr && a_dst && y && row_max && row_sum, CXG_ENULL, "cxg_gat_fused_forward: NULL argument");
  CXG_REQUIRE(nnz == 0 || (idx && x && a_src), CXG_ENULL, "cxg_gat_fused_forward: idx, x or a_src is NULL");
  CXG_REQUIRE(reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0, CXG_EINVAL,
              "cxg_gat_fused_forward: x and y must be 16-byte aligned");
  GatLayout L;
  gat_layout(n_dst, nnz, heads, c, &L);
  CXG_REQUIRE(workspace != nullptr && workspace_bytes >= L.total, CXG_EWORKSPACE,
              "cxg_gat_fused_forward: workspace %zu bytes, need %zu", workspace_bytes, L.total);
  CXG_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0, CXG_EINVAL, "cxg_gat_fused_forward: workspace alignment");
  GatArgs a = {};
  fill_args(a, L, workspace, nnz, heads, c, slope);
  a.ptr = ptr, a.idx = idx, a.ptr_bytes = ptr_bytes, a.idx_bytes = idx_bytes;
  a.gathered = x, a.g_small = a_src, a.r_small = a_dst;
  a.out = y, a.row_max = row_max, a.row_sum = row_sum;
  a.n_rows = n_dst;
  cudaStream_t st = as_stream(stream);
  const int cb = heads * c * 4 / 32;
  cudaError_t e = cb == 4 ? launch_walk<4, false>(a, st) : (cb == 8 ? launch_walk<8, false>(a, st) : launch_walk<16, false>(a, st));
  if (e != cudaSuccess) return set_error(CXG_ECUDA, "cxg_gat_fused_forward: %s", cudaGetErrorString(e));
  return check_launch("cxg_gat_fused_forward");
}

extern "C" int cxg_gat_fused_backward(const void *t_ptr, const void *t_idx, int ptr_bytes, int idx_bytes, const float *dy,
                                      const float *y, const float *x, const float *a_src, const float *a_dst,
                                      const float *row_max, const float *row_sum, float *dx, float *d_a_src,
                                      float *d_a_dst, int64_t n_src, int64_t n_dst, int64_t nnz, int heads, int c,
                                      float slope, const void *t_eid, const void *fwd_ptr, int fwd_ptr_bytes,
                                      void *workspace, size_t workspace_bytes, void *stream) {
  CXG_REQUIRE(n_src >= 0 && n_dst >= 0 && nnz >= 0, CXG_EINVAL, "cxg_gat_fused_backward: negative size");
  CXG_REQUIRE((ptr_bytes == 4 || ptr_bytes == 8) && (idx_bytes == 4 || idx_bytes == 8), CXG_EINVAL,
              "cxg_gat_fused_backward: index widths %d/%d", ptr_bytes, idx_bytes);
  int rc = check_shape("cxg_gat_fused_backward", heads, c);
  if (rc != CXG_OK) return rc;
  if (n_src == 0) return CXG_OK;
  CXG_REQUIRE(t_ptr && x && a_src && dx && d_a_src && d_a_dst, CXG_ENULL, "cxg_gat_fused_backward: NULL argument");
  CXG_REQUIRE(n_dst == 0 || (dy && y && a_dst && row_max && row_sum), CXG_ENULL, "cxg_gat_fused_backward: NULL argument");
  CXG_REQUIRE(nnz == 0 || t_idx, CXG_ENULL, "cxg_gat_fused_backward: t_idx is NULL");
  CXG_REQUIRE((t_eid == nullptr) == (fwd_ptr == nullptr), CXG_EINVAL,
              "cxg_gat_fused_backward: t_eid and fwd_ptr select the ordered d_a_dst together");
  CXG_REQUIRE(fwd_ptr == nullptr || fwd_ptr_bytes == 4 || fwd_ptr_bytes == 8, CXG_EINVAL,
              "cxg_gat_fused_backward: fwd_ptr_bytes %d", fwd_ptr_bytes);
  CXG_REQUIRE(reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(dy) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(y) % 16 == 0 && reinterpret_cast<uintptr_t>(dx) % 16 == 0,
              CXG_EINVAL, "cxg_gat_fused_backward: feature matrices must be 16-byte aligned");
  GatLayout L;
  gat_layout(n_dst, nnz, heads, c, &L);
  CXG_REQUIRE(workspace != nullptr && workspace_bytes >= L.total, CXG_EWORKSPACE,
              "cxg_gat_fused_backward: workspace %zu bytes, need %zu", workspace_bytes, L.total);
  CXG_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 16 == 0, CXG_EINVAL, "cxg_gat_fused_backward: workspace alignment");
  GatArgs a = {};
  fill_args(a, L, workspace, nnz, heads, c, slope);
  float *stats = reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + L.stats);
  a.ptr = t_ptr, a.idx = t_idx, a.ptr_bytes = ptr_bytes, a.idx_bytes = idx_bytes;
  a.gathered = dy, a.g_small = stats, a.r_small = a_src, a.r_feat = x;
  a.out = dx, a.d_r_small = d_a_src, a.d_g_small = d_a_dst;
  const bool ordered = t_eid != nullptr && nnz > 0 && n_dst > 0;
  a.eid = ordered ? t_eid : nullptr;
  a.d_edge = ordered ? reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + L.d_edge) : nullptr;
  a.n_rows = n_src;
  cudaStream_t st = as_stream(stream);
  const int cb = heads * c * 4 / 32;
  if (n_dst > 0) {
    const unsigned pg = static_cast<unsigned>(n_dst / 8 + 1 < kNumSM * 8 ? n_dst / 8 + 1 : kNumSM * 8);
    if (cb == 4)
      gat_bwd_prepare<4><<<pg, 256, 0, st>>>(dy, y, a_dst, row_max, row_sum, stats, d_a_dst, n_dst, heads, c);
    else if (cb == 8)
      gat_bwd_prepare<8><<<pg, 256, 0, st>>>(dy, y, a_dst, row_max, row_sum, stats, d_a_dst, n_dst, heads, c);
    else
      gat_bwd_prepare<16><<<pg, 256, 0, st>>>(dy, y, a_dst, row_max, row_sum, stats, d_a_dst, n_dst, heads, c);
    count_launches(1);
  }
  cudaError_t e = cb == 4 ? launch_walk<4, true>(a, st) : (cb == 8 ? launch_walk<8, true>(a, st) : launch_walk<16, true>(a, st));
  if (e != cudaSuccess) return set_error(CXG_ECUDA, "cxg_gat_fused_backward: %s", cudaGetErrorString(e));
  if (ordered) {
    int64_t *long_rows = reinterpret_cast<int64_t *>(reinterpret_cast<char *>(workspace) + L.long_rows);
    const int max_long = static_cast<int>(nnz / kLongRowEdges + 1);
    // one warp per destination, all of them resident at once while they fit (a row costs two dependent loads)
    const unsigned pg = static_cast<unsigned>(n_dst / 8 + 1 < kNumSM * 64 ? n_dst / 8 + 1 : kNumSM * 64);
    gat_dst_sum_rows<<<pg, 256, 0, st>>>(fwd_ptr, fwd_ptr_bytes, a.d_edge, d_a_dst, n_dst, nnz, heads, a.hshift, a.hdr,
                                         long_rows, max_long);
    float *piece_sums = reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + L.piece_sums);
    gat_dst_sum_pieces<<<kNumSM * 2, 256, 0, st>>>(fwd_ptr, fwd_ptr_bytes, a.d_edge, piece_sums, nnz, heads, a.hshift,
                                                   a.hdr, long_rows, max_long);
    gat_dst_sum_long<<<kNumSM, 256, 0, st>>>(fwd_ptr, fwd_ptr_bytes, piece_sums, d_a_dst, nnz, heads, a.hshift, a.hdr,
                                             long_rows, max_long);
    count_launches(3);
  }
  return check_launch("cxg_gat_fused_backward");
}
