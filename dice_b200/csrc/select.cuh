// Top-2 selection shared by the two router kernels.
#pragma once
#include <math.h>

// Top-2 of l[0..n_experts): larger first, lower index first among equals;
// softmax scores of the two in fp32.
template <int EP>
__device__ __forceinline__ void select_top2(const float (&l)[EP], int n_experts, int renorm, int& i0,
                                            int& i1, float& p0, float& p1) {
  float best0 = -INFINITY;
  i0 = 0;
#pragma unroll
  for (int e = 0; e < EP; ++e)
    if (e < n_experts && l[e] > best0) { best0 = l[e]; i0 = e; }
  float best1 = -INFINITY;
  i1 = (i0 == 0) ? 1 : 0;
#pragma unroll
  for (int e = 0; e < EP; ++e)
    if (e < n_experts && e != i0 && l[e] > best1) { best1 = l[e]; i1 = e; }
  float sum = 0.f;
#pragma unroll
  for (int e = 0; e < EP; ++e)
    if (e < n_experts) sum += expf(l[e] - best0);
  p0 = 1.0f / sum;
  p1 = expf(best1 - best0) / sum;
  if (renorm) {
    const float d = p0 + p1 + 1e-20f;
    p0 /= d;
    p1 /= d;
  }
}

