/* CPU oracle for the raised-contraction path.  TEST INFRASTRUCTURE ONLY: it is
 * the checker for the CUDA library and the timed CPU baseline, never a product
 * code path.  Build with -O2 -fno-fast-math -ffp-contract=off so results do
 * not depend on the host's FMA selection.
 *
 * The kernels follow the reference's PolyBench/C loop nests (see
 * pb_oracle_impl.h for the file:line of each).  The input generator is this
 * project's own counter-based uniform generator; the CUDA library implements
 * the identical integer recurrence so host and device agree bit for bit
 * without shipping multi-GB inputs. */
#include <stdint.h>
#include <stddef.h>

static inline uint64_t splitmix64(uint64_t z)
{
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

/* Element (array_id, r, c) of a logical rows x cols array:
 *   h = splitmix64(seed ^ (array_id << 56));  x = splitmix64(h + r*cols + c)
 *   fp64: u = (x >> 11) * 2^-53 ;  fp32: u = (x >> 40) * 2^-24
 *   value = lo + (hi - lo) * u   (one multiply, one add, no contraction) */
void pbo_fill_f64(double *dst, int64_t row0, int64_t rows, int64_t cols,
                  int64_t ld, uint64_t seed, uint32_t array_id, double lo,
                  double hi)
{
  const uint64_t h = splitmix64(seed ^ ((uint64_t)array_id << 56));
  const double span = hi - lo;
  for (int64_t r = 0; r < rows; r++)
    for (int64_t c = 0; c < cols; c++) {
      const uint64_t x = splitmix64(h + (uint64_t)((row0 + r) * cols + c));
      const double u = (double)(x >> 11) * 0x1.0p-53;
      dst[r * ld + c] = lo + span * u;
    }
}

void pbo_fill_f32(float *dst, int64_t row0, int64_t rows, int64_t cols,
                  int64_t ld, uint64_t seed, uint32_t array_id, float lo,
                  float hi)
{
  const uint64_t h = splitmix64(seed ^ ((uint64_t)array_id << 56));
  const float span = hi - lo;
  for (int64_t r = 0; r < rows; r++)
    for (int64_t c = 0; c < cols; c++) {
      const uint64_t x = splitmix64(h + (uint64_t)((row0 + r) * cols + c));
      const float u = (float)(x >> 40) * 0x1.0p-24f;
      dst[r * ld + c] = lo + span * u;
    }
}

#define T double
#define SUF _f64
#include "pb_oracle_impl.h"
#undef T
#undef SUF

#define T float
#define SUF _f32
#include "pb_oracle_impl.h"
#undef T
#undef SUF
