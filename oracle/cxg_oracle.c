/*
 * cxg_oracle.c — CPU restatement of the arithmetic of CxGNN-Compute's aggregation
 * kernels. TEST INFRASTRUCTURE ONLY: it is the checker the CUDA library is compared
 * against (tests, the smoke check and the CPU-baseline leg of the benchmark); nothing
 * in the shipped package may call it.
 *
 * Every function names the reference source it follows. The reference has no CPU
 * implementation and cannot be built or imported without its GPU toolchain, so the
 * restatement is pinned against the reference's own pure-torch formulations
 * (tests/golden/make_golden.py runs those on CPU and stores their outputs).
 *
 * Plain C99, no dependencies beyond libm:  gcc -O2 -shared -fPIC -ffp-contract=off
 * (-ffp-contract=off so that "a += b * c" never silently becomes an fma; fmaf() is
 * called where the GPU kernels contract).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ---- bf16 helpers (round to nearest even, like __float2bfloat16_rn) --------------- */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

/*
 * CSR SpMM forward, one fp32 accumulator per (row, head, column), edges in CSR order.
 * Follows gen_fwd_sum / gen_fwd_mean / gen_fwd_sum_edge_value{,_multi_head}
 * (src/cpp/src/aggr_kernel.cu:3-53,88-116,155-186): `rs += vin[...]` or
 * `rs += vin[...] * val` (contracted to an fma by nvcc) over j = begin..end, then the
 * store, divided by the edge count for mean. Deviations, on purpose:
 *   - mean divides exactly (the reference is built with --use_fast_math, whose division
 *     is approximate) and writes 0 for empty rows (the reference leaves the zero of its
 *     freshly zeroed output);
 *   - edge_mask / edge_rel / targets / accumulate restate selective_aggr_fwd_kernel
 *     (aggr_kernel.cu:493-521), aggr_rel_fwd (src/cpp/src/rel_spmm.cu:8-35) and target_aggr
 *     (aggr_kernel.cu:557-581), which add their row sum into the existing output.
 * `bf16` selects 16-bit storage for x and y (fp32 accumulation, one rounding at the end).
 */
ORC_API void orc_spmm_csr(const int64_t *ptr, const int64_t *idx, const void *x, void *y,
                          const float *edge_val, const uint8_t *edge_mask, const int32_t *edge_rel,
                          int64_t rel_stride, const int64_t *targets, int64_t n_dst, int feat,
                          int heads, int mean, int accumulate, int bf16) {
  const int width = feat * heads;
  const float *xf = (const float *)x;
  const uint16_t *xh = (const uint16_t *)x;
  float *yf = (float *)y;
  uint16_t *yh = (uint16_t *)y;
  float *acc = (float *)malloc(sizeof(float) * (size_t)width);
  for (int64_t r = 0; r < n_dst; ++r) {
    int64_t b = ptr[r], e = ptr[r + 1];
    for (int c = 0; c < width; ++c) acc[c] = 0.f;
    for (int64_t j = b; j < e; ++j) {
      if (edge_mask && !edge_mask[j]) continue;
      int64_t s = idx[j];
      if (edge_rel) s += (int64_t)edge_rel[j] * rel_stride;
      for (int c = 0; c < width; ++c) {
        float v = bf16 ? bf16_to_f32(xh[s * width + c]) : xf[s * width + c];
        if (edge_val)
          acc[c] = fmaf(v, edge_val[j * heads + c / feat], acc[c]);
        else
          acc[c] += v;
      }
    }
    int64_t out = targets ? targets[r] : r;
    for (int c = 0; c < width; ++c) {
      float v = acc[c];
      if (mean) v = (e > b) ? v / (float)(e - b) : 0.f;
      if (accumulate) v += bf16 ? bf16_to_f32(yh[out * width + c]) : yf[out * width + c];
      if (bf16)
        yh[out * width + c] = f32_to_bf16(v);
      else
        yf[out * width + c] = v;
    }
  }
  free(acc);
}

/*
 * The same SpMM in the summation order of the sm_100a streaming kernel, so that its
 * output can be checked bit for bit. This restates the CUDA library's order, not the
 * reference's: the edge array is cut into tiles of `tile` edges; a row inside one tile
 * is summed sequentially (identical to orc_spmm_csr); a row that crosses tile borders
 * is summed per tile (each partial starting from 0), and its m partials are then added
 * in tile order: sequentially when m <= 64, otherwise in blocks of 64 consecutive
 * partials that are each added in order and then joined in block order.
 */
ORC_API void orc_spmm_csr_tiled(const int64_t *ptr, const int64_t *idx, const void *x, void *y,
                                const float *edge_val, const int32_t *edge_rel, int64_t rel_stride,
                                const int64_t *targets, int64_t n_dst, int feat, int heads, int mean,
                                int accumulate, int bf16, int64_t tile) {
  const int width = feat * heads;
  const float *xf = (const float *)x;
  const uint16_t *xh = (const uint16_t *)x;
  float *yf = (float *)y;
  uint16_t *yh = (uint16_t *)y;
  float *acc = (float *)malloc(sizeof(float) * (size_t)width);
  float *tot = (float *)malloc(sizeof(float) * (size_t)width);
  for (int64_t r = 0; r < n_dst; ++r) {
    int64_t b = ptr[r], e = ptr[r + 1];
    for (int c = 0; c < width; ++c) tot[c] = 0.f;
    if (e > b) {
      int64_t t0 = b / tile, t1 = (e - 1) / tile, m = t1 - t0 + 1;
      float *parts = (float *)malloc(sizeof(float) * (size_t)width * (size_t)m);
      for (int64_t t = t0; t <= t1; ++t) {
        int64_t sb = t * tile > b ? t * tile : b, se = (t + 1) * tile < e ? (t + 1) * tile : e;
        for (int c = 0; c < width; ++c) acc[c] = 0.f;
        for (int64_t j = sb; j < se; ++j) {
          int64_t s = idx[j];
          if (edge_rel) s += (int64_t)edge_rel[j] * rel_stride;
          for (int c = 0; c < width; ++c) {
            float v = bf16 ? bf16_to_f32(xh[s * width + c]) : xf[s * width + c];
            if (edge_val)
              acc[c] = fmaf(v, edge_val[j * heads + c / feat], acc[c]);
            else
              acc[c] += v;
          }
        }
        memcpy(parts + (t - t0) * width, acc, sizeof(float) * (size_t)width);
      }
      if (m <= 64) {
        memcpy(tot, parts, sizeof(float) * (size_t)width);
        for (int64_t k = 1; k < m; ++k)
          for (int c = 0; c < width; ++c) tot[c] += parts[k * width + c];
      } else {
        for (int64_t kb = 0; kb < m; kb += 64) {
          int64_t ke = kb + 64 < m ? kb + 64 : m;
          memcpy(acc, parts + kb * width, sizeof(float) * (size_t)width);
          for (int64_t k = kb + 1; k < ke; ++k)
            for (int c = 0; c < width; ++c) acc[c] += parts[k * width + c];
          for (int c = 0; c < width; ++c) tot[c] = (kb == 0) ? acc[c] : tot[c] + acc[c];
        }
      }
      free(parts);
    }
    int64_t out = targets ? targets[r] : r;
    for (int c = 0; c < width; ++c) {
      float v = tot[c];
      if (mean) v = (e > b) ? v / (float)(e - b) : 0.f;
      if (accumulate) v += bf16 ? bf16_to_f32(yh[out * width + c]) : yf[out * width + c];
      if (bf16)
        yh[out * width + c] = f32_to_bf16(v);
      else
        yf[out * width + c] = v;
    }
  }
  free(acc);
  free(tot);
}

/* Same sum in double precision: the yardstick for rows that the GPU splits. */
ORC_API void orc_spmm_csr_f64(const int64_t *ptr, const int64_t *idx, const void *x, double *y,
                              const float *edge_val, int64_t n_dst, int feat, int heads, int mean,
                              int bf16) {
  const int width = feat * heads;
  const float *xf = (const float *)x;
  const uint16_t *xh = (const uint16_t *)x;
  for (int64_t r = 0; r < n_dst; ++r) {
    int64_t b = ptr[r], e = ptr[r + 1];
    double *out = y + r * width;
    for (int c = 0; c < width; ++c) out[c] = 0.0;
    for (int64_t j = b; j < e; ++j) {
      int64_t s = idx[j];
      for (int c = 0; c < width; ++c) {
        double v = bf16 ? (double)bf16_to_f32(xh[s * width + c]) : (double)xf[s * width + c];
        out[c] += edge_val ? v * (double)edge_val[j * heads + c / feat] : v;
      }
    }
    if (mean)
      for (int c = 0; c < width; ++c) out[c] = (e > b) ? out[c] / (double)(e - b) : 0.0;
  }
}

/*
 * SpMM backward in double precision. Follows gen_bwd_sum / gen_bwd_mean /
 * gen_bwd_sum_edge_value{,_multi_head}{,_edge_grad} (aggr_kernel.cu:188-491):
 *   dx[idx[e]] += val[e] * dy[r] (/ deg for mean);   dval[e,h] = sum_c dy[r,h,c] * x[idx[e],h,c].
 * The reference adds with atomicAdd in no fixed order, so only a tolerance applies.
 * dx must be zero-filled by the caller; dx / dval may be NULL.
 */
ORC_API void orc_spmm_csr_bwd_f64(const int64_t *ptr, const int64_t *idx, const float *dy,
                                  const float *x, const float *edge_val, const uint8_t *edge_mask,
                                  const int64_t *targets, double *dx, double *dval, int64_t n_dst,
                                  int feat, int heads, int mean) {
  const int width = feat * heads;
  for (int64_t r = 0; r < n_dst; ++r) {
    int64_t b = ptr[r], e = ptr[r + 1];
    int64_t gr = targets ? targets[r] : r;
    double inv = (mean && e > b) ? 1.0 / (double)(e - b) : 1.0;
    for (int64_t j = b; j < e; ++j) {
      if (edge_mask && !edge_mask[j]) continue;
      int64_t s = idx[j];
      for (int h = 0; h < heads; ++h) {
        double v = edge_val ? (double)edge_val[j * heads + h] : 1.0;
        double dot = 0.0;
        for (int c = 0; c < feat; ++c) {
          double g = (double)dy[gr * width + h * feat + c] * inv;
          if (dx) dx[s * width + h * feat + c] += g * v;
          if (dval) dot += g * (double)x[s * width + h * feat + c];
        }
        if (dval) dval[j * heads + h] = dot;
      }
    }
  }
}

/* Lane 0's value after the reference's `for (i = 16; i > 0; i >>= 1) v += shfl_down(v, i)`. */
static float warp_tree_sum(float *lane) {
  for (int i = 16; i > 0; i >>= 1)
    for (int l = 0; l < i; ++l) lane[l] += lane[l + i];
  return lane[0];
}

/*
 * Edge softmax forward, following edge_softmax_fwd (src/cpp/src/edge_softmax.cu:3-42)
 * pass by pass for each (dst, head): t = att_dst[d,h] + att_src[idx[e],h];
 * t = max(t, t * slope); mask = t > 0; m = max over the row (start value -100000);
 * p = exp(t - m); the row sum is taken as the reference's warp does it (lane l adds
 * edges l, l+32, ... in order, then the shuffle-down tree); out = p / sum.
 * Deviation: expf() of libm instead of the GPU's fast __expf.
 */
ORC_API void orc_edge_softmax_fwd(const int64_t *ptr, const int64_t *idx, const float *att_dst,
                                  const float *att_src, float *out, uint8_t *mask, int64_t n_dst,
                                  int heads, float slope) {
  for (int64_t d = 0; d < n_dst; ++d) {
    int64_t b = ptr[d], e = ptr[d + 1];
    for (int h = 0; h < heads; ++h) {
      float dst = att_dst[d * heads + h];
      float m = -100000.f;
      for (int64_t i = b; i < e; ++i) {
        float t = dst + att_src[idx[i] * heads + h];
        t = fmaxf(t, t * slope);
        out[i * heads + h] = t;
        mask[i * heads + h] = t > 0.f;
        m = fmaxf(m, t);
      }
      float lane[32];
      for (int l = 0; l < 32; ++l) lane[l] = 0.f;
      for (int64_t i = b; i < e; ++i) {
        float p = expf(out[i * heads + h] - m);
        out[i * heads + h] = p;
      }
      for (int l = 0; l < 32; ++l)
        for (int64_t i = b + l; i < e; i += 32) lane[l] += out[i * heads + h];
      float s = warp_tree_sum(lane);
      for (int64_t i = b; i < e; ++i) out[i * heads + h] /= s;
    }
  }
}

/*
 * Edge softmax backward, following edge_softmax_bwd (edge_softmax.cu:44-95):
 * s = sum_e out*g; tmp = out*(g - s), times slope where the forward mask is false;
 * grad_src[idx[e],h] += tmp; grad_dst[d,h] = sum tmp, written only when the row has
 * both a positive and a non-positive pre-activation (otherwise the sum is 0 up to
 * rounding and the reference leaves the zero-filled output). Sums in double.
 */
ORC_API void orc_edge_softmax_bwd(const int64_t *ptr, const int64_t *idx, const float *grad,
                                  const uint8_t *mask, const float *out, double *grad_dst,
                                  double *grad_src, int64_t n_dst, int heads, float slope) {
  for (int64_t d = 0; d < n_dst; ++d) {
    int64_t b = ptr[d], e = ptr[d + 1];
    for (int h = 0; h < heads; ++h) {
      double s = 0.0;
      for (int64_t i = b; i < e; ++i) s += (double)out[i * heads + h] * (double)grad[i * heads + h];
      double dg = 0.0;
      int pos = 0, neg = 0;
      for (int64_t i = b; i < e; ++i) {
        double tmp = (double)out[i * heads + h] * ((double)grad[i * heads + h] - s);
        if (!mask[i * heads + h]) {
          tmp *= (double)slope;
          neg = 1;
        } else {
          pos = 1;
        }
        dg += tmp;
        grad_src[idx[i] * heads + h] += tmp;
      }
      if (pos && neg) grad_dst[d * heads + h] = dg;
    }
  }
}

/*
 * SDDMM, following sddmm_multihead (src/cpp/src/sddmm_kernel.cu:3-25):
 * out[e,h] = sum_i src_feat[src[e],h,i] * dst_feat[dst[e], (per_head ? h : 0), i], lane l
 * adding i = l, l+32, ... and the shuffle-down tree joining the lanes. per_head = 0 is the
 * reference's layout (dst_feat has no head axis); per_head = 1 is the head-wise product
 * that the multi-head SpMM backward needs.
 */
ORC_API void orc_sddmm(const int64_t *src, const int64_t *dst, const float *src_feat,
                       const float *dst_feat, float *out, int64_t n_edge, int feat, int heads,
                       int per_head) {
  for (int64_t e = 0; e < n_edge; ++e)
    for (int h = 0; h < heads; ++h) {
      float lane[32];
      const float *a = src_feat + (src[e] * heads + h) * feat;
      const float *b = dst_feat + (per_head ? (dst[e] * heads + h) : dst[e]) * (int64_t)feat;
      for (int l = 0; l < 32; ++l) {
        float r = 0.f;
        for (int i = l; i < feat; i += 32) r = fmaf(a[i], b[i], r);
        lane[l] = r;
      }
      out[e * heads + h] = warp_tree_sum(lane);
    }
}

/*
 * Relation padding, following pad_rel / pad_rel_idx (src/cpp/src/stitch_kernel.cu:3-38):
 * pad slot t in [0, num_rel*(thres-1)) belongs to relation t / (thres-1); it becomes a
 * real member of that relation when (t % (thres-1)) < thres - count % thres and
 * count % thres != 0, else it gets the dummy relation num_rel. idx (optional) gets -1.
 */
ORC_API void orc_pad_rel(int64_t *rel, int64_t *idx, const int64_t *count, int thres, int num_rel,
                         int64_t base) {
  for (int t = 0; t < num_rel * (thres - 1); ++t) {
    int which = t / (thres - 1);
    int mod = (int)(count[which] % thres);
    int64_t pos = base + t;
    if ((t % (thres - 1)) < (thres - mod) && mod != 0)
      rel[pos] = which;
    else
      rel[pos] = num_rel;
    if (idx) idx[pos] = -1;
  }
}

/*
 * Per-relation sub-graphs, following rel_schedule (src/cpp/src/schedule.cu:5-63). For
 * relation `rel_iter`: rows that own at least one edge of the relation, their edges in
 * CSR order and the row ids. Outputs must hold nnz / n_dst+1 / n_dst entries; returns the
 * number of kept rows, and n_in_layer[l] = kept rows among the first num_node_in_layer[l].
 */
ORC_API int64_t orc_rel_schedule_one(const int64_t *ptr, const int64_t *idx, const int32_t *rel,
                                     int64_t n_dst, int rel_iter, const int64_t *num_node_in_layer,
                                     int num_layer, int64_t *sub_ptr, int64_t *sub_idx,
                                     int64_t *sub_target, int64_t *n_in_layer) {
  int64_t n_target = 0, n_idx = 0;
  int layer = 0;
  sub_ptr[0] = 0;
  for (int64_t i = 0; i < n_dst; ++i) {
    int64_t cnt = 0;
    for (int64_t j = ptr[i]; j < ptr[i + 1]; ++j)
      if (rel[j] == rel_iter) {
        ++cnt;
        sub_idx[n_idx++] = idx[j];
      }
    if (cnt > 0) {
      sub_target[n_target] = i;
      sub_ptr[n_target + 1] = sub_ptr[n_target] + cnt;
      ++n_target;
    }
    if (layer < num_layer && i == num_node_in_layer[layer] - 1) n_in_layer[layer++] = n_target;
  }
  return n_target;
}

/*
 * Typed linear, exact: out[m,:] = a[src(m),:] @ w[rel[m]]  with double accumulation.
 * The reference computes this with Triton's tl.dot on fp32 inputs (TF32 products, fp32
 * accumulate; cxgnncomp/codegen/triton_typed_matmul.py:363-430) or, per row, with
 * typed_linear_kernel{,_s2e} (src/cpp/src/rel_spmm.cu:231-315). src may be NULL (identity).
 * Rows whose rel is outside [0, num_rel) are skipped (padding).
 */
ORC_API void orc_typed_linear_f64(const float *a, const float *w, const int64_t *src,
                                  const int64_t *rel, double *out, int64_t m, int k, int n,
                                  int num_rel) {
  for (int64_t i = 0; i < m; ++i) {
    int64_t r = rel[i];
    if (r < 0 || r >= num_rel) continue;
    const float *row = a + (src ? src[i] : i) * k;
    const float *wr = w + r * (int64_t)k * n;
    double *o = out + i * n;
    for (int j = 0; j < n; ++j) o[j] = 0.0;
    for (int kk = 0; kk < k; ++kk) {
      double av = (double)row[kk];
      for (int j = 0; j < n; ++j) o[j] += av * (double)wr[kk * n + j];
    }
  }
}

/*
 * Generalised SpMM of the dgSPARSE surface, following weightedCacheCoarsenSPMMKernel and init()
 * (src/cpp/src/dgsparse.cu:324-378, src/cpp/include/dgsparse.h:14-131): per row and column one
 * accumulator that starts at 0 (sum, mean), (float)INT_MIN (max) or (float)INT_MAX (min) when the row
 * has edges and at 0 when it has none; edges in CSR order; reduce(acc, compute(val, x)) with
 * compute add: val + x, sub: x - val, mul: val * x, div: x / val; max/min written as the reference's
 * macros (a < b ? b : a, a < b ? a : b); mean divides by the edge count. val == NULL: operand x.
 * acc + val * x is one fused multiply-add, as nvcc contracts it. rop: 0 sum 1 max 2 min 3 mean;
 * cop: 0 add 1 sub 2 mul 3 div.
 */
ORC_API void orc_gspmm(const int64_t *ptr, const int64_t *idx, const float *val, const float *x,
                       float *y, int64_t n_dst, int feat, int rop, int cop) {
  for (int64_t r = 0; r < n_dst; ++r) {
    const int64_t lo = ptr[r], hi = ptr[r + 1];
    for (int c = 0; c < feat; ++c) {
      float acc = 0.f;
      if (hi > lo && rop == 1) acc = (float)INT32_MIN;
      if (hi > lo && rop == 2) acc = (float)INT32_MAX;
      for (int64_t e = lo; e < hi; ++e) {
        const float xv = x[idx[e] * feat + c];
        float t = xv;
        if (val != NULL) {
          const float v = val[e];
          if ((rop == 0 || rop == 3) && cop == 2) {
            acc = fmaf(v, xv, acc);
            continue;
          }
          t = cop == 0 ? v + xv : cop == 1 ? xv - v : cop == 2 ? v * xv : xv / v;
        }
        if (rop == 1)
          acc = acc < t ? t : acc;
        else if (rop == 2)
          acc = acc < t ? acc : t;
        else
          acc = acc + t;
      }
      if (rop == 3 && hi > lo) acc = acc / (float)(hi - lo);
      y[r * feat + c] = acc;
    }
  }
}

/*
 * topo_sort (src/cpp/src/schedule.cu:72-124): Kahn's algorithm over out-edges ptr/idx with the given
 * in-degrees; when the queue runs dry before every node is out, every node left with degree 1 is
 * released and, if some node has degree > 1, the lowest-numbered node of the smallest such degree is
 * released too (which is how the reference steps through cycles). Returns the number of nodes
 * written to out.
 */
ORC_API int64_t orc_topo_sort(const int64_t *ptr, const int64_t *idx, const int64_t *degree,
                              int64_t n, int64_t *out) {
  int64_t *deg = (int64_t *)malloc(sizeof(int64_t) * (size_t)(n > 0 ? n : 1));
  int64_t *queue = (int64_t *)malloc(sizeof(int64_t) * (size_t)(n > 0 ? n : 1) * 2);
  int64_t qh = 0, qt = 0, cnt = 0;
  memcpy(deg, degree, sizeof(int64_t) * (size_t)n);
  /* a node enters the queue at most twice (once by reaching 0, once released), so 2n slots do */
  for (int64_t i = 0; i < n; ++i)
    if (deg[i] == 0) queue[qt++] = i;
  while (cnt < n) {
    while (qh < qt && cnt < n) {
      const int64_t cur = queue[qh++];
      out[cnt++] = cur;
      for (int64_t e = ptr[cur]; e < ptr[cur + 1]; ++e) {
        const int64_t nx = idx[e];
        if (--deg[nx] == 0 && qt < 2 * n) queue[qt++] = nx;
      }
    }
    if (cnt >= n) break;
    int64_t min_deg = n, pick = -1;
    for (int64_t i = 0; i < n; ++i) {
      if (deg[i] < min_deg && deg[i] > 1) {
        min_deg = deg[i];
        pick = i;
      } else if (deg[i] == 1) {
        deg[i] = 0;
        if (qt < 2 * n) queue[qt++] = i;
      }
    }
    if (pick != -1) {
      if (qt < 2 * n) queue[qt++] = pick;
      deg[pick] = 0;
    } else if (qh == qt) {
      break;
    }
  }
  free(deg);
  free(queue);
  return cnt;
}

/*
 * Neighbour sampling restated from the library's definition (the reference takes this step from its
 * external loader, cxgnncomp/data_preparation.py:214-215): per frontier node v of in-degree d, all
 * neighbours when d <= fanout, else Floyd's subset algorithm over positions 0 .. d-1 with draw number k
 * taken from splitmix64(splitmix64(seed ^ v * 0xD1B54A32D192ED03) + k) by multiply-shift, positions
 * sorted ascending. out_ptr = exclusive prefix sum of min(d, fanout).
 */
static uint64_t orc_splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

ORC_API void orc_sample_neighbors(const int64_t *gptr, const int64_t *gidx, const int64_t *frontier,
                                  int64_t n_front, int fanout, const int64_t *out_ptr, int64_t *out,
                                  uint64_t seed) {
  for (int64_t i = 0; i < n_front; ++i) {
    const int64_t v = frontier[i], lo = gptr[v], deg = gptr[v + 1] - lo;
    int64_t *o = out + out_ptr[i];
    if (deg <= fanout) {
      for (int64_t j = 0; j < deg; ++j) o[j] = gidx[lo + j];
      continue;
    }
    int64_t pick[64];
    int k = 0;
    const uint64_t base = orc_splitmix64(seed ^ ((uint64_t)v * 0xD1B54A32D192ED03ull));
    for (int64_t j = deg - fanout; j < deg; ++j) {
      const uint64_t h = orc_splitmix64(base + (uint64_t)k);
      int64_t t = (int64_t)(((h >> 32) * (uint64_t)(j + 1)) >> 32);
      int seen = 0;
      for (int q = 0; q < k; ++q) seen |= pick[q] == t;
      if (seen) t = j;
      int q = k;
      for (; q > 0 && pick[q - 1] > t; --q) pick[q] = pick[q - 1];
      pick[q] = t;
      ++k;
    }
    for (int q = 0; q < fanout; ++q) o[q] = gidx[lo + pick[q]];
  }
}
