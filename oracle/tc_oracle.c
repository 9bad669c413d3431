/*
 * TEST INFRASTRUCTURE -- CPU restatement of the reference's loop-nest
 * contraction.  Only tests, the smoke check and the bench's CPU-baseline leg
 * may call this; the product library never does.
 *
 * The reference checks every generated kernel against a hand-written loop nest,
 * one per expression: post_Correctness in
 *   cogent/drivers/tccg/code_main_tccg_02.c:109-133        (3-D output, 1 sum index)
 *   cogent/drivers/tccg/code_main_tccg_29.c:110-138        (4-D output, 2 sum indices)
 *   cogent/drivers/tccg/code_main_tccg_40.c:113-137        (6-D output)
 *   cogent/drivers/tccg-float/code_main_tccg_40.c:113-137  (fp32: accumulates in float)
 * All of them have the same shape, restated here for any rank:
 *   - loops over the OUTPUT indices in written order, first index outermost;
 *   - inside, loops over the contraction indices in sum(...) order, first outermost;
 *   - the innermost statement is  C[r] += A[ra] * B[rb]  (or -=), accumulated
 *     directly in the tensor's own type, one product at a time;
 *   - r, ra, rb are column-major address polynomials (first index fastest).
 * Differences: 64-bit offsets instead of int (the reference overflows beyond
 * 2^31 elements), '=' supported (C[r] is zeroed before the sum), and an
 * optional OpenMP split of the OUTERMOST output loop, which leaves every
 * element's summation order -- and so every bit of the result -- unchanged.
 *
 * Parity status: pinned.  oracle/build_oracle.py compiles the reference's own
 * 57 driver files into oracle/_ref/ and tests/test_oracle.py checks this
 * restatement against each of them bit for bit (and against the committed
 * golden vectors made from them when the reference tree is absent).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define TC_ORACLE_MAX_RANK 16

typedef struct {
  int n_out, n_sum, n_a, n_b;
  int64_t out_ext[TC_ORACLE_MAX_RANK], sum_ext[TC_ORACLE_MAX_RANK];
  int64_t out_sc[TC_ORACLE_MAX_RANK];                  /* stride of output index i in C */
  int64_t out_sa[TC_ORACLE_MAX_RANK], out_sb[TC_ORACLE_MAX_RANK]; /* ... in A / B (0 if absent) */
  int64_t sum_sa[TC_ORACLE_MAX_RANK], sum_sb[TC_ORACLE_MAX_RANK];
} nest_t;

/* a_idx / b_idx: for each written index of A / B its id: 0..n_out-1 = output
 * index, n_out.. = contraction index.  Strides are compact column-major unless
 * given explicitly (str_* may be NULL). */
static int build_nest(nest_t* t, int n_out, const int64_t* out_ext, int n_sum, const int64_t* sum_ext, int n_a,
                      const int32_t* a_idx, int n_b, const int32_t* b_idx, const int64_t* str_c,
                      const int64_t* str_a, const int64_t* str_b) {
  int i;
  int64_t acc;
  if (n_out < 0 || n_sum < 0 || n_out > TC_ORACLE_MAX_RANK || n_sum > TC_ORACLE_MAX_RANK ||
      n_a > TC_ORACLE_MAX_RANK || n_b > TC_ORACLE_MAX_RANK)
    return 1;
  memset(t, 0, sizeof(*t));
  t->n_out = n_out; t->n_sum = n_sum; t->n_a = n_a; t->n_b = n_b;
  for (i = 0; i < n_out; ++i) t->out_ext[i] = out_ext[i];
  for (i = 0; i < n_sum; ++i) t->sum_ext[i] = sum_ext[i];
  acc = 1;
  for (i = 0; i < n_out; ++i) { t->out_sc[i] = str_c ? str_c[i] : acc; acc *= out_ext[i]; }
  acc = 1;
  for (i = 0; i < n_a; ++i) {
    const int id = a_idx[i];
    const int64_t s = str_a ? str_a[i] : acc;
    if (id < 0 || id >= n_out + n_sum) return 1;
    if (id < n_out) { t->out_sa[id] = s; acc *= out_ext[id]; }
    else { t->sum_sa[id - n_out] = s; acc *= sum_ext[id - n_out]; }
  }
  acc = 1;
  for (i = 0; i < n_b; ++i) {
    const int id = b_idx[i];
    const int64_t s = str_b ? str_b[i] : acc;
    if (id < 0 || id >= n_out + n_sum) return 1;
    if (id < n_out) { t->out_sb[id] = s; acc *= out_ext[id]; }
    else { t->sum_sb[id - n_out] = s; acc *= sum_ext[id - n_out]; }
  }
  return 0;
}

/* Offsets of the flattened contraction loops in their nested order
 * (first sum index outermost => last sum index fastest). */
static int build_ktable(const nest_t* t, int64_t* ktot, int64_t** ka, int64_t** kb) {
  int64_t n = 1, k;
  int i;
  for (i = 0; i < t->n_sum; ++i) n *= t->sum_ext[i];
  *ka = (int64_t*)malloc(sizeof(int64_t) * (size_t)(n > 0 ? n : 1));
  *kb = (int64_t*)malloc(sizeof(int64_t) * (size_t)(n > 0 ? n : 1));
  if (!*ka || !*kb) return 1;
  for (k = 0; k < n; ++k) {
    int64_t r = k, oa = 0, ob = 0;
    for (i = t->n_sum - 1; i >= 0; --i) {
      const int64_t c = r % t->sum_ext[i];
      r /= t->sum_ext[i];
      oa += c * t->sum_sa[i];
      ob += c * t->sum_sb[i];
    }
    (*ka)[k] = oa;
    (*kb)[k] = ob;
  }
  *ktot = n;
  return 0;
}

#define DEFINE_NEST(NAME, T)                                                                          \
  static void NAME(const nest_t* t, int op, T* C, const T* A, const T* B, int64_t ktot,                \
                   const int64_t* ka, const int64_t* kb, int64_t first_lo, int64_t first_hi) {         \
    /* odometer over output indices 1..n_out-1 (last fastest), index 0 in [first_lo, first_hi) */     \
    int64_t idx[TC_ORACLE_MAX_RANK];                                                                  \
    int64_t i0;                                                                                       \
    const int n = t->n_out;                                                                           \
    for (i0 = first_lo; i0 < first_hi; ++i0) {                                                        \
      int d;                                                                                          \
      int done = 0;                                                                                   \
      for (d = 0; d < n; ++d) idx[d] = 0;                                                             \
      if (n > 0) idx[0] = i0;                                                                         \
      while (!done) {                                                                                 \
        int64_t r = 0, ra = 0, rb = 0, k;                                                             \
        for (d = 0; d < n; ++d) {                                                                     \
          r += idx[d] * t->out_sc[d];                                                                 \
          ra += idx[d] * t->out_sa[d];                                                                \
          rb += idx[d] * t->out_sb[d];                                                                \
        }                                                                                             \
        if (op == 0) C[r] = (T)0;                                                                     \
        if (op < 0) {                                                                                 \
          for (k = 0; k < ktot; ++k) C[r] -= A[ra + ka[k]] * B[rb + kb[k]];                           \
        } else {                                                                                      \
          for (k = 0; k < ktot; ++k) C[r] += A[ra + ka[k]] * B[rb + kb[k]];                           \
        }                                                                                             \
        /* advance: last index fastest, index 0 fixed */                                              \
        d = n - 1;                                                                                    \
        while (d >= 1) {                                                                              \
          if (++idx[d] < t->out_ext[d]) break;                                                        \
          idx[d] = 0;                                                                                 \
          --d;                                                                                        \
        }                                                                                             \
        if (d < 1) done = 1;                                                                          \
      }                                                                                               \
    }                                                                                                 \
  }

DEFINE_NEST(nest_f64, double)
DEFINE_NEST(nest_f32, float)

/* dtype: 0 = fp64, 1 = fp32.  op: +1 '+=', -1 '-=', 0 '='.
 * threads <= 1: the serial nest exactly as the reference runs it.
 * Returns 0 on success. */
int tc_oracle_contract(int dtype, int n_out, const int64_t* out_ext, int n_sum, const int64_t* sum_ext, int n_a,
                       const int32_t* a_idx, int n_b, const int32_t* b_idx, const int64_t* str_c,
                       const int64_t* str_a, const int64_t* str_b, int op, void* C, const void* A, const void* B,
                       int threads) {
  nest_t t;
  int64_t ktot = 0, *ka = NULL, *kb = NULL;
  int64_t first = 1;
  int i;
  if (build_nest(&t, n_out, out_ext, n_sum, sum_ext, n_a, a_idx, n_b, b_idx, str_c, str_a, str_b)) return 1;
  for (i = 0; i < n_out; ++i) if (out_ext[i] <= 0) return 1;
  for (i = 0; i < n_sum; ++i) if (sum_ext[i] <= 0) return 1;
  if (build_ktable(&t, &ktot, &ka, &kb)) { free(ka); free(kb); return 1; }
  if (n_out > 0) first = out_ext[0];
  if (threads <= 1 || first <= 1) {
    if (dtype == 0) nest_f64(&t, op, (double*)C, (const double*)A, (const double*)B, ktot, ka, kb, 0, first);
    else nest_f32(&t, op, (float*)C, (const float*)A, (const float*)B, ktot, ka, kb, 0, first);
  } else {
    int64_t i0;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
#endif
    for (i0 = 0; i0 < first; ++i0) {
      if (dtype == 0) nest_f64(&t, op, (double*)C, (const double*)A, (const double*)B, ktot, ka, kb, i0, i0 + 1);
      else nest_f32(&t, op, (float*)C, (const float*)A, (const float*)B, ktot, ka, kb, i0, i0 + 1);
    }
  }
  free(ka);
  free(kb);
  return 0;
}

/* Seeded inputs: element i of tensor `tensor_id` for `seed`, uniform[-1,1).
 * Same counter-based generator as the device fill of the library, restated. */
static uint64_t splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

void tc_oracle_fill(int dtype, void* dst, int64_t count, uint64_t seed, int tensor_id, int64_t first_index) {
  const uint64_t key = (seed * 0x9E3779B97F4A7C15ull) ^ ((uint64_t)tensor_id << 60);
  int64_t i;
  for (i = 0; i < count; ++i) {
    const uint64_t x = splitmix64(key ^ (uint64_t)(first_index + i));
    if (dtype == 0) ((double*)dst)[i] = (double)(x >> 11) * (1.0 / 9007199254740992.0) * 2.0 - 1.0;
    else ((float*)dst)[i] = (float)(x >> 40) * (1.0f / 16777216.0f) * 2.0f - 1.0f;
  }
}

int tc_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
