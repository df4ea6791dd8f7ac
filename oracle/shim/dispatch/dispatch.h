// Stand-in for Apple's <dispatch/dispatch.h>: the reference's two GCD
// dispatch_apply(^block) loops are rewritten by build_ref.sh into calls of
// shim_parallel_for with a lambda (g++ has no blocks extension).
#pragma once
#include <cstddef>
template <class F> static inline void shim_parallel_for(size_t n, F f) {
#pragma omp parallel for schedule(dynamic)
  for (long i = 0; i < (long)n; ++i) f((size_t)i);
}
