/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the torkit3d neighbour-search / sampling operators.
 *
 * This header is included twice by tk3d_oracle.c, once with T = float (suffix _f32) and once with
 * T = double (suffix _f64).  It must be compiled with -ffp-contract=off so that every multiply and
 * add is rounded on its own, which is the arithmetic the reference source spells out.
 *
 * Every function names the reference lines it restates (paths are relative to the torkit3d
 * project root).  Nothing here is used by the product library; only the tests, the smoke check and
 * the CPU-baseline leg of the benchmark call it.
 */

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUFFIX)

/* Squared distance, accumulated x, y, z from zero with each operation rounded:
 * torkit3d/csrc/cuda/chamfer_distance_kernel.cu:65-71 (same loop in knn_distance_kernel.cu:70-77,
 * ball_query_kernel.cu:70-77, sample_farthest_points_kernel.cu:49-57). */
static inline T FN(sqdist)(const T *a, const T *b) {
  T dx = a[0] - b[0];
  T dy = a[1] - b[1];
  T dz = a[2] - b[2];
  T d = dx * dx;
  d = d + dy * dy;
  d = d + dz * dz;
  return d;
}

/* One direction of the chamfer forward: for every point of `a` the nearest point of `b`.
 * Ascending scan with a strict "<" so the lowest index wins a tie; the running minimum starts at
 * +inf (1e40 overflows to inf in fp32) and the index at -1:
 * torkit3d/csrc/cuda/chamfer_distance_kernel.cu:42-43, 60-78, 82-87. */
static void FN(nn_dir)(const T *a, const T *b, int64_t bs, int64_t na, int64_t nb, T *dist, int64_t *idx) {
  for (int64_t s = 0; s < bs; ++s) {
    for (int64_t i = 0; i < na; ++i) {
      const T *p = a + (s * na + i) * 3;
      const T *q = b + s * nb * 3;
      T best = (T)INFINITY;
      int64_t arg = -1;
      for (int64_t j = 0; j < nb; ++j) {
        T d = FN(sqdist)(q + j * 3, p);
        if (d < best) {
          best = d;
          arg = j;
        }
      }
      dist[s * na + i] = best;
      idx[s * na + i] = arg;
    }
  }
}

/* torkit3d/csrc/cuda/chamfer_distance_kernel.cu:91-151 (both directions). */
void FN(orc_chamfer_fwd)(const T *xyz1, const T *xyz2, int64_t bs, int64_t n1, int64_t n2, T *dist1,
                         int64_t *idx1, T *dist2, int64_t *idx2) {
  FN(nn_dir)(xyz1, xyz2, bs, n1, n2, dist1, idx1);
  FN(nn_dir)(xyz2, xyz1, bs, n2, n1, dist2, idx2);
}

/* One backward pass: torkit3d/csrc/cuda/chamfer_distance_kernel.cu:170-196.
 * g = 2*grad_dist; own row += g*(p - q); matched row -= the same.  Sequential accumulation. */
static void FN(chamfer_bwd_dir)(T *grad_a, T *grad_b, const T *gdist, const int64_t *index, const T *a,
                                const T *b, int64_t bs, int64_t na, int64_t nb) {
  for (int64_t s = 0; s < bs; ++s) {
    for (int64_t i = 0; i < na; ++i) {
      int64_t lin = s * na + i;
      int64_t j = index[lin];
      if (j < 0 || j >= nb) continue; /* empty partner cloud: nothing to propagate */
      const T *p = a + lin * 3;
      const T *q = b + (s * nb + j) * 3;
      T g = gdist[lin] * (T)2;
      for (int d = 0; d < 3; ++d) {
        T gv = g * (p[d] - q[d]);
        grad_a[lin * 3 + d] += gv;
        grad_b[(s * nb + j) * 3 + d] += -gv;
      }
    }
  }
}

/* torkit3d/csrc/cuda/chamfer_distance_kernel.cu:200-274: zero-initialised grads, two passes. */
void FN(orc_chamfer_bwd)(const T *g1, const T *g2, const T *xyz1, const T *xyz2, const int64_t *idx1,
                         const int64_t *idx2, int64_t bs, int64_t n1, int64_t n2, T *grad1, T *grad2) {
  memset(grad1, 0, sizeof(T) * (size_t)(bs * n1 * 3));
  memset(grad2, 0, sizeof(T) * (size_t)(bs * n2 * 3));
  FN(chamfer_bwd_dir)(grad1, grad2, g1, idx1, xyz1, xyz2, bs, n1, n2);
  FN(chamfer_bwd_dir)(grad2, grad1, g2, idx2, xyz2, xyz1, bs, n2, n1);
}

/* Brute-force KNN.  The reference keeps the K smallest keys with a strict "<" against the current
 * maximum while scanning in ascending index order (torkit3d/csrc/cuda/knn_distance_kernel.cu:65-82
 * with the bounded set of torkit3d/csrc/include/mink.cuh:61-89), so the retained SET is the K
 * smallest under (distance, index) order.  Its slot order is an artefact; this restatement emits
 * each row sorted ascending by (distance, index).  Distances are squared.  A NaN distance (a NaN
 * coordinate) orders after every number, so keys with NaN coordinates are returned only when fewer
 * than K keys have a numeric distance; the reference leaves that case to chance (a NaN in its set
 * is never displaced, ibid. mink.cuh:70-84, because every comparison with it is false). */
static int FN(knn_before)(T d, T e) { return d < e || (e != e && d == d); }

void FN(orc_knn)(const T *query, const T *key, int64_t bs, int64_t n1, int64_t n2, int64_t k, T *dist,
                 int64_t *idx) {
  for (int64_t s = 0; s < bs; ++s) {
    for (int64_t i = 0; i < n1; ++i) {
      const T *p = query + (s * n1 + i) * 3;
      const T *q = key + s * n2 * 3;
      T *od = dist + (s * n1 + i) * k;
      int64_t *oi = idx + (s * n1 + i) * k;
      int64_t cnt = 0;
      for (int64_t j = 0; j < n2; ++j) {
        T d = FN(sqdist)(q + j * 3, p);
        if (cnt == k && !FN(knn_before)(d, od[k - 1])) continue;
        int64_t pos = (cnt < k) ? cnt : k - 1;
        /* stable: an equal distance with a higher index stays behind */
        while (pos > 0 && FN(knn_before)(d, od[pos - 1])) {
          od[pos] = od[pos - 1];
          oi[pos] = oi[pos - 1];
          --pos;
        }
        od[pos] = d;
        oi[pos] = j;
        if (cnt < k) ++cnt;
      }
    }
  }
}

/* KNN in a C-dimensional feature space: the operator torkit3d/ops/native.py:4-30 defines as
 * torch.cdist + torch.topk (called on [B, C, N] features by models/classification/dgcnn.py:58-61).
 * cdist goes through a matrix product whose rounding is not specified, so this restatement fixes
 * the arithmetic instead: acc = fma(d_c, d_c, acc) over the channels in order, d_c = key_c - query_c
 * (fmaf is correctly rounded whatever -ffp-contract says).  Rows are the k smallest under
 * (squared distance, index), sorted ascending.  `cf` != 0: tensors are [B, C, N], else [B, N, C]. */
void FN(orc_feature_knn)(const T *query, const T *key, int64_t bs, int64_t c, int64_t n1, int64_t n2, int64_t k,
                         int cf, T *dist, int64_t *idx) {
  for (int64_t s = 0; s < bs; ++s) {
    const T *qb = query + s * c * n1, *kb = key + s * c * n2;
    for (int64_t i = 0; i < n1; ++i) {
      T *od = dist + (s * n1 + i) * k;
      int64_t *oi = idx + (s * n1 + i) * k;
      int64_t cnt = 0;
      for (int64_t j = 0; j < n2; ++j) {
        T d = 0;
        for (int64_t ch = 0; ch < c; ++ch) {
          const T qv = cf ? qb[ch * n1 + i] : qb[i * c + ch];
          const T kv = cf ? kb[ch * n2 + j] : kb[j * c + ch];
          const T df = kv - qv;
#if defined(ORC_T_IS_FLOAT)
          d = fmaf(df, df, d);
#else
          d = fma(df, df, d);
#endif
        }
        if (cnt == k && !(d < od[k - 1])) continue;
        int64_t pos = (cnt < k) ? cnt : k - 1;
        while (pos > 0 && d < od[pos - 1]) { /* stable: an equal distance with a higher index stays behind */
          od[pos] = od[pos - 1];
          oi[pos] = oi[pos - 1];
          --pos;
        }
        od[pos] = d;
        oi[pos] = j;
        if (cnt < k) ++cnt;
      }
    }
  }
}

/* Farthest point sampling from index 0; min-distance update then arg-max, lowest index among exact
 * maxima (numpy argmax rule of tests/ops/test_sample_farthest_points.py:24-36; the kernel is
 * torkit3d/csrc/cuda/sample_farthest_points_kernel.cu:28-103, which differs only when two distinct
 * points tie exactly for the maximum). */
void FN(orc_fps)(const T *points, int64_t bs, int64_t n, int64_t s, int64_t *index) {
  for (int64_t b = 0; b < bs; ++b) {
    const T *p = points + b * n * 3;
    T *md = (T *)malloc(sizeof(T) * (size_t)n);
    int64_t cur = 0;
    index[b * s] = 0;
    for (int64_t i = 0; i < n; ++i) md[i] = (T)INFINITY;
    for (int64_t it = 1; it < s; ++it) {
      T best = (T)-1;
      int64_t arg = 0;
      for (int64_t j = 0; j < n; ++j) {
        T d = FN(sqdist)(p + j * 3, p + cur * 3);
        if (d < md[j]) md[j] = d;
        if (md[j] > best) {
          best = md[j];
          arg = j;
        }
      }
      cur = arg;
      index[b * s + it] = cur;
    }
    free(md);
  }
}

/* Ball query: first k key indices, ascending, with d < r*r (strict); the radius arrives as a C
 * float and is squared in T; short rows are padded with their first hit, empty rows stay -1:
 * torkit3d/csrc/cuda/ball_query_kernel.cu:26, 66-101, 108, 123. */
void FN(orc_ball_query)(const T *query, const T *key, int64_t bs, int64_t n1, int64_t n2, float radius,
                        int64_t k, int64_t *index) {
  const T r = (T)radius;
  const T r2 = r * r;
  for (int64_t s = 0; s < bs; ++s) {
    for (int64_t i = 0; i < n1; ++i) {
      const T *p = query + (s * n1 + i) * 3;
      const T *q = key + s * n2 * 3;
      int64_t *o = index + (s * n1 + i) * k;
      int64_t cnt = 0;
      for (int64_t j = 0; j < n2 && cnt < k; ++j) {
        T d = FN(sqdist)(q + j * 3, p);
        if (d < r2) o[cnt++] = j;
      }
      int64_t pad = cnt > 0 ? o[0] : -1;
      for (int64_t c = cnt; c < k; ++c) o[c] = pad;
    }
  }
}

/* out[b,c,n2,k] = in[b,c,index[b,n2,k]]: torkit3d/csrc/cuda/group_points_kernel.cu:26-29. */
void FN(orc_group_fwd)(const T *in, const int64_t *index, int64_t b, int64_t c, int64_t n1, int64_t n2,
                       int64_t k, T *out) {
  for (int64_t s = 0; s < b; ++s)
    for (int64_t ch = 0; ch < c; ++ch)
      for (int64_t e = 0; e < n2 * k; ++e) out[(s * c + ch) * n2 * k + e] = in[(s * c + ch) * n1 + index[s * n2 * k + e]];
}

/* grad_in[b,c,index[b,n2,k]] += grad_out[b,c,n2,k]: torkit3d/csrc/cuda/group_points_kernel.cu:57-63. */
void FN(orc_group_bwd)(const T *gout, const int64_t *index, int64_t b, int64_t c, int64_t n1, int64_t n2,
                       int64_t k, T *gin) {
  memset(gin, 0, sizeof(T) * (size_t)(b * c * n1));
  for (int64_t s = 0; s < b; ++s)
    for (int64_t ch = 0; ch < c; ++ch)
      for (int64_t e = 0; e < n2 * k; ++e) gin[(s * c + ch) * n1 + index[s * n2 * k + e]] += gout[(s * c + ch) * n2 * k + e];
}

/* out[b,c,n2] = sum_i in[b,c,index[b,n2,i]] * weight[b,n2,i], accumulated i = 0..k-1 from zero:
 * torkit3d/csrc/cuda/interpolate_kernel.cu:31-45. */
void FN(orc_interp_fwd)(const T *in, const int64_t *index, const T *weight, int64_t b, int64_t c, int64_t n1,
                        int64_t n2, int64_t k, T *out) {
  for (int64_t s = 0; s < b; ++s)
    for (int64_t ch = 0; ch < c; ++ch)
      for (int64_t j = 0; j < n2; ++j) {
        T acc = (T)0;
        for (int64_t i = 0; i < k; ++i)
          acc += in[(s * c + ch) * n1 + index[(s * n2 + j) * k + i]] * weight[(s * n2 + j) * k + i];
        out[(s * c + ch) * n2 + j] = acc;
      }
}

/* grad_in[b,c,index[b,n2,i]] += grad_out[b,c,n2] * weight[b,n2,i]:
 * torkit3d/csrc/cuda/interpolate_kernel.cu:129-143. */
void FN(orc_interp_bwd)(const T *gout, const int64_t *index, const T *weight, int64_t b, int64_t c, int64_t n1,
                        int64_t n2, int64_t k, T *gin) {
  memset(gin, 0, sizeof(T) * (size_t)(b * c * n1));
  for (int64_t s = 0; s < b; ++s)
    for (int64_t ch = 0; ch < c; ++ch)
      for (int64_t j = 0; j < n2; ++j)
        for (int64_t i = 0; i < k; ++i)
          gin[(s * c + ch) * n1 + index[(s * n2 + j) * k + i]] += gout[(s * c + ch) * n2 + j] * weight[(s * n2 + j) * k + i];
}

/* Inverse-(squared-)distance weights of the three nearest neighbours:
 * inv = 1 / max(d, 1e-10); w = inv / sum(inv)  -- torkit3d/layers/pointnet2.py:128-130
 * (the sum over the last axis is taken in index order). */
void FN(orc_three_nn_weight)(const T *dist, int64_t rows, int64_t k, T *weight) {
  for (int64_t r = 0; r < rows; ++r) {
    T inv[8];
    T sum = (T)0;
    for (int64_t i = 0; i < k && i < 8; ++i) {
      T d = dist[r * k + i];
      if (d < (T)1e-10) d = (T)1e-10;
      inv[i] = (T)1 / d;
      sum += inv[i];
    }
    for (int64_t i = 0; i < k && i < 8; ++i) weight[r * k + i] = inv[i] / sum;
  }
}

#undef FN
#undef CAT
#undef CAT_
