/*
 * CPU oracle for the sparse-kernel hot path of bobbyyyan/scorch.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a checker: the test-suite, the smoke check and the
 * CPU-baseline leg of the benchmark may link it; the product path (the CUDA library) never
 * does and has no CPU fallback.
 *
 * Every function restates, in plain C, the algorithm of one reference kernel; the reference
 * location it follows is cited above it (paths are relative to the reference project root).
 * Index arrays are int32 and values are 1-D, dense operands row-major, exactly as the
 * reference hands them to its kernels (src/scorch/storage.py:46-51, src/scorch/stensor.py:448).
 *
 * Parity status: PINNED.  tests/test_oracle_pinning.py checks these functions against
 *   (1) the known-answer SpGEMM vectors of the reference's own test-suite
 *       (tests/test_scorch/test_kernels.py:473-615),
 *   (2) golden vectors produced by importing the reference's Python package in the build
 *       container (tests/golden/, generator script committed beside them),
 *   (3) the reference's compiled scorch_ops extension (oracle/_ref) where that binary exists.
 *
 * The "_acc64" functions are not restatements: they are the float64-accumulating form of the
 * same sums used as the tolerance oracle (rtol 1e-4 / atol 1e-5 is checked against them).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define SO_API __attribute__((visibility("default")))

SO_API int so_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------------------------------
 * CSR x dense SpMM, fp32, k-tiled workspace form.
 * Follows spmm_csr_float_v2, csrc/spmm.h:2007-2089: output zero-filled; rows without stored
 * entries are skipped and stay zero (:2051); for each k-tile of width roundup16(tile) the row's
 * entries are accumulated in order into a zeroed tile which is then copied out (:2055-2074).
 * The reference hands rows to threads through an atomic counter; row ownership is disjoint, so
 * a dynamic OpenMP loop gives the same result.
 * ------------------------------------------------------------------------------------------ */
SO_API void so_spmm_csr_f32_v2(int m, int k, const int32_t* pos, const int32_t* crd,
                               const float* val, const float* B, float* C, int tile) {
  const int kt = (tile + 15) & ~15;
  memset(C, 0, sizeof(float) * (size_t)m * (size_t)k);
#pragma omp parallel
  {
    float* ws = (float*)aligned_alloc(64, ((size_t)kt * sizeof(float) + 63) & ~(size_t)63);
#pragma omp for schedule(dynamic, 64)
    for (int i = 0; i < m; i++) {
      const int b = pos[i], e = pos[i + 1];
      if (b == e) continue;
      float* crow = C + (size_t)i * (size_t)k;
      for (int k0 = 0; k0 < k; k0 += kt) {
        const int kw = (k - k0 < kt) ? (k - k0) : kt;
        for (int c = 0; c < kw; c++) ws[c] = 0.0f;
        for (int p = b; p < e; p++) {
          const float a = val[p];
          const float* brow = B + (size_t)crd[p] * (size_t)k + k0;
          for (int c = 0; c < kw; c++) ws[c] += a * brow[c];
        }
        memcpy(crow + k0, ws, sizeof(float) * (size_t)kw);
      }
    }
    free(ws);
  }
}

/* ------------------------------------------------------------------------------------------
 * CSR x dense SpMM, typed, direct accumulation into a zeroed output.
 * Follows spmm_csr_typed<T>, csrc/spmm.h:91-150 (bound as prebuilt_spmm_csr_{f32,f64,i32,i64},
 * csrc/ops.cpp:91-103).  Integer types wrap like the reference's C++ arithmetic (computed in
 * the unsigned type to keep the wrap well-defined in C).
 * ------------------------------------------------------------------------------------------ */
#define SO_DEFINE_SPMM_TYPED(NAME, T, ACC)                                                  \
  SO_API void NAME(int m, int k, const int32_t* pos, const int32_t* crd, const T* val,      \
                   const T* B, T* C) {                                                       \
    memset(C, 0, sizeof(T) * (size_t)m * (size_t)k);                                         \
    _Pragma("omp parallel for schedule(dynamic, 16)") for (int i = 0; i < m; i++) {         \
      T* crow = C + (size_t)i * (size_t)k;                                                   \
      for (int p = pos[i]; p < pos[i + 1]; p++) {                                            \
        const T a = val[p];                                                                  \
        const T* brow = B + (size_t)crd[p] * (size_t)k;                                      \
        for (int c = 0; c < k; c++) crow[c] = (T)((ACC)crow[c] + (ACC)a * (ACC)brow[c]);     \
      }                                                                                      \
    }                                                                                        \
  }
SO_DEFINE_SPMM_TYPED(so_spmm_csr_f32, float, float)
SO_DEFINE_SPMM_TYPED(so_spmm_csr_f64, double, double)
SO_DEFINE_SPMM_TYPED(so_spmm_csr_i32, int32_t, uint32_t)
SO_DEFINE_SPMM_TYPED(so_spmm_csr_i64, int64_t, uint64_t)

/* ------------------------------------------------------------------------------------------
 * Fused SpMM + bias (+ ReLU), fp32.
 * Follows spmm_csr_bias_act<float, relu>, csrc/spmm.h:28-89: EVERY row (also rows without
 * stored entries) starts from the bias vector (:56-58), then accumulates, then clamps (:74-79).
 * ------------------------------------------------------------------------------------------ */
SO_API void so_spmm_csr_bias_act_f32(int m, int k, const int32_t* pos, const int32_t* crd,
                                     const float* val, const float* B, const float* bias,
                                     int relu, float* C) {
#pragma omp parallel for schedule(dynamic, 16)
  for (int i = 0; i < m; i++) {
    float* crow = C + (size_t)i * (size_t)k;
    for (int c = 0; c < k; c++) crow[c] = bias[c];
    for (int p = pos[i]; p < pos[i + 1]; p++) {
      const float a = val[p];
      const float* brow = B + (size_t)crd[p] * (size_t)k;
      for (int c = 0; c < k; c++) crow[c] += a * brow[c];
    }
    if (relu)
      for (int c = 0; c < k; c++) crow[c] = crow[c] > 0.0f ? crow[c] : 0.0f;
  }
}

/* ------------------------------------------------------------------------------------------
 * CSR SpMV, typed.  Follows spmv_csr<T>, csrc/kernels.h:12-49: one sequential accumulator per
 * row, every y[i] written (also zeros).  The compiler-emitted twin (src/scorch/ops.py:48-136)
 * leaves zeros from a memset instead; the results are the same.
 * ------------------------------------------------------------------------------------------ */
#define SO_DEFINE_SPMV(NAME, T, ACC)                                                        \
  SO_API void NAME(int m, const int32_t* pos, const int32_t* crd, const T* val, const T* x, \
                   T* y) {                                                                   \
    _Pragma("omp parallel for schedule(static)") for (int i = 0; i < m; i++) {              \
      ACC acc = 0;                                                                           \
      for (int p = pos[i]; p < pos[i + 1]; p++) acc += (ACC)val[p] * (ACC)x[crd[p]];         \
      y[i] = (T)acc;                                                                         \
    }                                                                                        \
  }
SO_DEFINE_SPMV(so_spmv_csr_f32, float, float)
SO_DEFINE_SPMV(so_spmv_csr_f64, double, double)
SO_DEFINE_SPMV(so_spmv_csr_i32, int32_t, uint32_t)
SO_DEFINE_SPMV(so_spmv_csr_i64, int64_t, uint64_t)

/* ------------------------------------------------------------------------------------------
 * SDDMM with a COO mask: D[p] = S_val[p] * dot(A[row[p],:], B[col[p],:]).
 * Follows sddmm_coo_float_prebuilt, csrc/kernels.h:508-570 (the mask value multiplies after the
 * dot, :558).  Output order = input entry order.
 * ------------------------------------------------------------------------------------------ */
SO_API void so_sddmm_coo_f32(int64_t nnz, int kdim, const int32_t* row, const int32_t* col,
                             const float* sval, const float* A, const float* B, float* D) {
#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t p = 0; p < nnz; p++) {
    const float* a = A + (size_t)row[p] * (size_t)kdim;
    const float* b = B + (size_t)col[p] * (size_t)kdim;
    float dot = 0.0f;
    for (int c = 0; c < kdim; c++) dot += a[c] * b[c];
    D[p] = sval[p] * dot;
  }
}

/* ------------------------------------------------------------------------------------------
 * SDDMM with a CSR mask, as the reference's compiler emits it for "ij,ik,jk->ij" (generator:
 * src/scorch/ops.py:638-664, src/scorch/compiler/iter_lattice.py:1011-1098,
 * src/scorch/compiler/cin_lowerer.py:2286-2326): rows in order, entries in order, a scalar
 * accumulator over k, multiplied by the mask value afterwards, and FRESH int32 (row, col)
 * coordinate arrays written next to the values (output format "o,o").
 * ------------------------------------------------------------------------------------------ */
SO_API void so_sddmm_csr_f32(int m, int kdim, const int32_t* pos, const int32_t* crd,
                             const float* mval, const float* Q, const float* K,
                             int32_t* out_row, int32_t* out_col, float* out_val) {
#pragma omp parallel for schedule(dynamic, 16)
  for (int i = 0; i < m; i++) {
    const float* q = Q + (size_t)i * (size_t)kdim;
    for (int p = pos[i]; p < pos[i + 1]; p++) {
      const int j = crd[p];
      const float* kk = K + (size_t)j * (size_t)kdim;
      float acc = 0.0f;
      for (int c = 0; c < kdim; c++) acc += q[c] * kk[c];
      acc *= mval[p];
      out_val[p] = acc;
      if (out_row) out_row[p] = i;
      if (out_col) out_col[p] = j;
    }
  }
}

/* ------------------------------------------------------------------------------------------
 * Row softmax over the stored entries of a CSR matrix.
 * Follows _sparse_softmax_csr_vectorized, bench/bench_sparse_transformer.py:277-297 (caller-side
 * torch code in the reference): per row, exp(v - max) / sum; rows without entries untouched.
 * ------------------------------------------------------------------------------------------ */
SO_API void so_csr_row_softmax_f32(int m, const int32_t* pos, const float* val, float* out) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int i = 0; i < m; i++) {
    const int b = pos[i], e = pos[i + 1];
    if (b == e) continue;
    float mx = val[b];
    for (int p = b + 1; p < e; p++) mx = val[p] > mx ? val[p] : mx;
    float s = 0.0f;
    for (int p = b; p < e; p++) {
      out[p] = expf(val[p] - mx);
      s += out[p];
    }
    for (int p = b; p < e; p++) out[p] = out[p] / s;
  }
}

/* ------------------------------------------------------------------------------------------
 * CSR x CSR SpGEMM (Gustavson), two phases.
 * Follows spmspm_csr<T>, csrc/kernels.h:51-202.
 *   symbolic (:69-111): per row, count the distinct columns reached through (A entry, B entry)
 *     pairs with a per-thread marker array, then a serial prefix sum into int32 row pointers;
 *   numeric (:117-184): accumulate products in visit order into a dense per-thread accumulator,
 *     emit the row, then sort the row's columns ascending.
 * The structure is the symbolic union: an entry whose products cancel to 0.0 is kept.
 * The reference collects a row through a linked list and then sorts it; the sorted row does not
 * depend on the collection order, so this restatement keeps a plain touched-list.
 * Returns the total number of stored entries as int64 (the reference stores it in an int).
 * ------------------------------------------------------------------------------------------ */
SO_API int64_t so_spgemm_symbolic(int m, int n, const int32_t* Apos, const int32_t* Acrd,
                                  const int32_t* Bpos, const int32_t* Bcrd, int32_t* Cpos) {
  int32_t* cnt = (int32_t*)calloc((size_t)m + 1, sizeof(int32_t));
#pragma omp parallel
  {
    uint8_t* mark = (uint8_t*)calloc((size_t)n + 1, 1);
    int32_t* touched = (int32_t*)malloc(sizeof(int32_t) * ((size_t)n + 1));
#pragma omp for schedule(dynamic, 64)
    for (int i = 0; i < m; i++) {
      int len = 0;
      for (int pa = Apos[i]; pa < Apos[i + 1]; pa++) {
        const int j = Acrd[pa];
        for (int pb = Bpos[j]; pb < Bpos[j + 1]; pb++) {
          const int c = Bcrd[pb];
          if (!mark[c]) { mark[c] = 1; touched[len++] = c; }
        }
      }
      cnt[i] = len;
      for (int t = 0; t < len; t++) mark[touched[t]] = 0;
    }
    free(mark);
    free(touched);
  }
  int64_t total = 0;
  Cpos[0] = 0;
  for (int i = 0; i < m; i++) {
    total += cnt[i];
    Cpos[i + 1] = (int32_t)total;
  }
  free(cnt);
  return total;
}

static int so_cmp_i32(const void* a, const void* b) {
  const int32_t x = *(const int32_t*)a, y = *(const int32_t*)b;
  return (x > y) - (x < y);
}

#define SO_DEFINE_SPGEMM_NUMERIC(NAME, T, ACC)                                               \
  SO_API void NAME(int m, int n, const int32_t* Apos, const int32_t* Acrd, const T* Aval,    \
                   const int32_t* Bpos, const int32_t* Bcrd, const T* Bval,                   \
                   const int32_t* Cpos, int32_t* Ccrd, T* Cval) {                             \
    _Pragma("omp parallel") {                                                                 \
      uint8_t* mark = (uint8_t*)calloc((size_t)n + 1, 1);                                     \
      T* sums = (T*)calloc((size_t)n + 1, sizeof(T));                                         \
      _Pragma("omp for schedule(dynamic, 64)") for (int i = 0; i < m; i++) {                  \
        int32_t* ccrd = Ccrd + Cpos[i];                                                       \
        T* cval = Cval + Cpos[i];                                                             \
        int len = 0;                                                                          \
        for (int pa = Apos[i]; pa < Apos[i + 1]; pa++) {                                      \
          const int j = Acrd[pa];                                                             \
          const T v = Aval[pa];                                                               \
          for (int pb = Bpos[j]; pb < Bpos[j + 1]; pb++) {                                    \
            const int c = Bcrd[pb];                                                           \
            sums[c] = (T)((ACC)sums[c] + (ACC)v * (ACC)Bval[pb]);                             \
            if (!mark[c]) { mark[c] = 1; ccrd[len++] = c; }                                   \
          }                                                                                   \
        }                                                                                     \
        qsort(ccrd, (size_t)len, sizeof(int32_t), so_cmp_i32);                                \
        for (int t = 0; t < len; t++) {                                                       \
          const int c = ccrd[t];                                                              \
          cval[t] = sums[c];                                                                  \
          sums[c] = 0;                                                                        \
          mark[c] = 0;                                                                        \
        }                                                                                     \
      }                                                                                       \
      free(mark);                                                                             \
      free(sums);                                                                             \
    }                                                                                         \
  }
SO_DEFINE_SPGEMM_NUMERIC(so_spgemm_numeric_f32, float, float)
SO_DEFINE_SPGEMM_NUMERIC(so_spgemm_numeric_f64, double, double)
SO_DEFINE_SPGEMM_NUMERIC(so_spgemm_numeric_i32, int32_t, uint32_t)
SO_DEFINE_SPGEMM_NUMERIC(so_spgemm_numeric_i64, int64_t, uint64_t)

/* ==========================================================================================
 * float64-accumulating tolerance oracles (fp32 inputs, fp64 sums and outputs).
 * ========================================================================================== */
SO_API void so_spmm_csr_acc64(int m, int k, const int32_t* pos, const int32_t* crd,
                              const float* val, const float* B, const float* bias, int relu,
                              double* C) {
#pragma omp parallel for schedule(dynamic, 16)
  for (int i = 0; i < m; i++) {
    double* crow = C + (size_t)i * (size_t)k;
    for (int c = 0; c < k; c++) crow[c] = bias ? (double)bias[c] : 0.0;
    for (int p = pos[i]; p < pos[i + 1]; p++) {
      const double a = (double)val[p];
      const float* brow = B + (size_t)crd[p] * (size_t)k;
      for (int c = 0; c < k; c++) crow[c] += a * (double)brow[c];
    }
    if (relu)
      for (int c = 0; c < k; c++) crow[c] = crow[c] > 0.0 ? crow[c] : 0.0;
  }
}

SO_API void so_spmv_csr_acc64(int m, const int32_t* pos, const int32_t* crd, const float* val,
                              const float* x, double* y) {
#pragma omp parallel for schedule(dynamic, 256)
  for (int i = 0; i < m; i++) {
    double acc = 0.0;
    for (int p = pos[i]; p < pos[i + 1]; p++) acc += (double)val[p] * (double)x[crd[p]];
    y[i] = acc;
  }
}

SO_API void so_sddmm_csr_acc64(int m, int kdim, const int32_t* pos, const int32_t* crd,
                               const float* mval, const float* Q, const float* K, double* out) {
#pragma omp parallel for schedule(dynamic, 16)
  for (int i = 0; i < m; i++) {
    const float* q = Q + (size_t)i * (size_t)kdim;
    for (int p = pos[i]; p < pos[i + 1]; p++) {
      const float* kk = K + (size_t)crd[p] * (size_t)kdim;
      double acc = 0.0;
      for (int c = 0; c < kdim; c++) acc += (double)q[c] * (double)kk[c];
      out[p] = acc * (double)(mval ? mval[p] : 1.0f);
    }
  }
}

SO_API void so_csr_row_softmax_acc64(int m, const int32_t* pos, const double* val, double* out) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int i = 0; i < m; i++) {
    const int b = pos[i], e = pos[i + 1];
    if (b == e) continue;
    double mx = val[b];
    for (int p = b + 1; p < e; p++) mx = val[p] > mx ? val[p] : mx;
    double s = 0.0;
    for (int p = b; p < e; p++) { out[p] = exp(val[p] - mx); s += out[p]; }
    for (int p = b; p < e; p++) out[p] /= s;
  }
}

SO_API void so_spgemm_numeric_acc64(int m, int n, const int32_t* Apos, const int32_t* Acrd,
                                    const float* Aval, const int32_t* Bpos, const int32_t* Bcrd,
                                    const float* Bval, const int32_t* Cpos, const int32_t* Ccrd,
                                    double* Cval) {
  /* Values for an already known (sorted) structure Cpos/Ccrd. */
#pragma omp parallel
  {
    double* sums = (double*)calloc((size_t)n + 1, sizeof(double));
#pragma omp for schedule(dynamic, 64)
    for (int i = 0; i < m; i++) {
      for (int pa = Apos[i]; pa < Apos[i + 1]; pa++) {
        const int j = Acrd[pa];
        const double v = (double)Aval[pa];
        for (int pb = Bpos[j]; pb < Bpos[j + 1]; pb++) sums[Bcrd[pb]] += v * (double)Bval[pb];
      }
      for (int t = Cpos[i]; t < Cpos[i + 1]; t++) {
        Cval[t] = sums[Ccrd[t]];
        sums[Ccrd[t]] = 0.0;
      }
    }
    free(sums);
  }
}
