/* Exhaustive host check of the row-scale computation of the quantisation kernels: for every float a from
 * 1e-30 to FLT_MAX, q0 = RN(a * r), q = fma(fma(-q0, 127, a), r, q0) with r = RN(1/127) equals the IEEE
 * quotient a / 127.  Prints the number of differing inputs (expected 0).  Build: gcc -O2 -mfma -ffp-contract=off. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

int main(void) {
  const float r = 1.0f / 127.0f;
  uint32_t lo, hi, rb;
  const float flo = 1e-30f, fhi = 3.4028234e38f;
  memcpy(&lo, &flo, 4);
  memcpy(&hi, &fhi, 4);
  memcpy(&rb, &r, 4);
  long bad = 0;
  for (uint64_t uu = lo; uu <= hi; ++uu) {
    const uint32_t u = (uint32_t)uu;
    float a;
    memcpy(&a, &u, 4);
    const float q0 = a * r;
    const float q = fmaf(fmaf(-q0, 127.0f, a), r, q0);
    if (q != a / 127.0f) ++bad;
  }
  printf("%08x %ld %u\n", rb, bad, hi - lo + 1);
  return 0;
}
