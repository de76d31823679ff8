/* CPU restatement of the weight update inside INQAffine / INQConvolution (incremental network
 * quantization: at given iterations half of the still learnable weights are fixed to powers of two).
 * TEST INFRASTRUCTURE ONLY (see oracle.py). Follows src/nbla/function/generic/inq_affine.cpp:82-203
 * step by step; the affine itself is oracle_contract.c's. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

/* floor(log2 a) + (log2 a - floor(log2 a) >= log2 1.5) with the logarithm and the difference in float. The
 * reference writes the threshold in two ways: for the largest magnitude (inq_affine.cpp:152-154) it is the
 * double std::log2(1.5), for the weights (:173-177) a float variable initialised with 0.58496250072115619.
 * They differ exactly at a = 1.5 * 2^e, where the float difference equals the float threshold. */
int oracle_inq_exponent_of_max(float a) {
  const float b = log2f(a);
  return (int)(floorf(b) + ((b - floorf(b)) >= log2(1.5)));
}
int oracle_inq_exponent(float a) {
  const float b = log2f(a);
  const float d = 0.58496250072115619;
  return (int)(floorf(b) + ((b - floorf(b)) >= d));
}

typedef struct {
  float mag;
  int64_t index;
} inq_item;

static int by_magnitude_desc(const void *pa, const void *pb) {
  const inq_item *a = (const inq_item *)pa, *b = (const inq_item *)pb;
  if (a->mag > b->mag)
    return -1;
  if (a->mag < b->mag)
    return 1;
  /* equal magnitudes: the reference's std::sort leaves their order unspecified; lower index first here */
  return a->index < b->index ? -1 : (a->index > b->index ? 1 : 0);
}

/* One forward pass's weight update. trigger: 0 = not an INQ iteration, 1 = fix half of the learnable
 * weights by largest magnitude, 2 = last INQ iteration (fix all), 3 = random selection with the Bernoulli
 * draws given in `draws` (one per still learnable weight, in index order). */
void oracle_inq_update(float *w, int32_t *ind, float *old_w, int32_t *old_ind, int64_t n, int num_bits, int trigger,
                       const int32_t *draws) {
  /* A (:101-105): fixed weights keep the value they were fixed to */
  for (int64_t i = 0; i < n; ++i)
    if (old_ind[i] == 1)
      w[i] = old_w[i];
  /* B (:108-148) */
  if (trigger == 2) {
    for (int64_t i = 0; i < n; ++i)
      ind[i] = 1;
  } else if (trigger == 1) {
    inq_item *items = (inq_item *)malloc(sizeof(inq_item) * (size_t)(n > 0 ? n : 1));
    for (int64_t i = 0; i < n; ++i) {
      items[i].mag = fabsf(w[i]);
      items[i].index = i;
    }
    qsort(items, (size_t)n, sizeof(inq_item), by_magnitude_desc);
    int64_t learnable = 0, fixed = 0;
    for (int64_t i = 0; i < n; ++i)
      learnable += ind[i] == 0;
    for (int64_t i = 0; i < n; ++i) {
      if (ind[items[i].index] == 0) {
        ind[items[i].index] = 1;
        ++fixed;
      }
      if (fixed >= learnable / 2)
        break;
    }
    free(items);
  } else if (trigger == 3) {
    int64_t k = 0;
    for (int64_t i = 0; i < n; ++i)
      if (ind[i] == 0)
        ind[i] = draws[k++];
  }
  /* C (:150-186): fixed weights become powers of two (or zero) */
  float max_absval = 0.0f;
  for (int64_t i = 0; i < n; ++i)
    if (fabsf(w[i]) > max_absval)
      max_absval = fabsf(w[i]);
  if (max_absval == 0.0f)
    max_absval = 1.0f;
  const int n1 = oracle_inq_exponent_of_max(max_absval);
  const int n2 = n1 + 1 - (int)pow(2, num_bits - 2);
  const float pruning_threshold = (float)pow(2, n2 - 1);
  for (int64_t i = 0; i < n; ++i) {
    if (ind[i] != 1)
      continue;
    if (fabsf(w[i]) < pruning_threshold) {
      w[i] = 0.0f;
    } else {
      const float s = (w[i] < 0.0) ? -1.0f : 1.0f;
      int e = oracle_inq_exponent(fabsf(w[i]));
      if (e > n1)
        e = n1;
      if (e < n2)
        e = n2;
      w[i] = ldexpf(s, e);
    }
  }
  /* F (:200-203) */
  for (int64_t i = 0; i < n; ++i) {
    old_w[i] = w[i];
    old_ind[i] = ind[i];
  }
}
