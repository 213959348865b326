// A softmax sink: one more score in a row's denominator that has no key and no value -- the fixed score 0, or a learned
// number per query head (`val` [heads] float32, in natural units, not multiplied by the scores' factor).  With the row's
// sums formed relative to a maximum m the sink's term is e^(sink - m); kernels whose scores are in base 2 (already
// multiplied by log2 e) use the second form.  Where a row's keys are cut into ranges the term is added once, in the merge.
#pragma once

__device__ __forceinline__ float sink_term(const float* __restrict__ val, int h, float m) {
    return expf((val ? val[h] : 0.f) - m);
}

__device__ __forceinline__ float sink_term2(const float* __restrict__ val, int h, float m2) {
    return exp2f((val ? val[h] * 1.4426950408889634f : 0.f) - m2);
}
