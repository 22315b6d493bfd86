// Column-sum entry point for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference; it exists only in this library.
//
// Who needs it: code that runs where cudaMalloc (and anything that may call it, such as a
// framework's caching allocator growing its pool) is not permitted or not safe - for example a
// host callback enqueued on a stream, a thread that only holds a stream handle from another
// runtime and owns no allocator, or a latency-critical loop that must never take the allocator's
// lock.  `oa_col_sum` needs the caller to pass a scratch buffer for its per-block partial sums;
// such callers have nowhere to get one.  `oa_col_sum_static` keeps that scratch inside the library
// instead, in a fixed `static __device__` array, so the call allocates nothing: no cudaMalloc,
// no cudaFree, no allocating library routine.
//
// Contract
//   out[c] = sum_r x[r, c]  (+ out[c] when accumulate != 0), x row-major [rows, cols], fp32 or bf16,
//   same math and same fixed reduction order as `oa_col_sum`.
//   The caller still passes input and output pointers and the stream.
//   Limit: ceil(rows / 256) * cols must not exceed OA_COL_SUM_STATIC_MAX_FLOATS (1 Mi floats = 4 MiB);
//   a larger problem is refused with OA_ERR_TOO_LARGE and nothing is launched.
//   The 4 MiB array is part of the library image: every GPU that loads the library holds it until
//   the process exits.
//   The first call on each device looks up the array's device address (cudaGetSymbolAddress) with that
//   device current; make that first call outside any stream capture.
//   All calls share the one array, and it keeps whatever the previous call left in it.  Nothing in it has
//   to start at zero: each call overwrites every partial it later reads.  Two calls that overlap on the
//   GPU (different streams, or different threads without ordering) race on the array: order them.
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { OA_COL_SUM_STATIC_MAX_FLOATS = 1 << 20 };

// dtype / out_dtype: 0 = fp32, 1 = bf16.  Returns 0 when launched, OA_ERR_TOO_LARGE (6) beyond the limit,
// OA_ERR_DRIVER (3) if the array's address cannot be resolved, OA_ERR_ARG / OA_ERR_UNSUPPORTED for bad input.
int oa_col_sum_static(int dtype, const void* x, void* out, int out_dtype, long long rows, int cols, int accumulate,
                      void* stream);
// The limit above, for callers that want to check before calling.
size_t oa_col_sum_static_max_floats(void);

#ifdef __cplusplus
}
#endif
