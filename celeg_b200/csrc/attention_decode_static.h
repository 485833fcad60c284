/* Declaration of the one entry point of libceleg_b200 that allocates nothing.
 *
 * It has no counterpart in celsowm/celeg. It exists for hosts that cannot call cudaMalloc at the
 * moment they need decode attention: a process that gave all free device memory to its own pool,
 * or a loop that cannot afford the device-wide synchronisation an allocation brings. The scratch
 * memory of the split-key decode kernel is a fixed 8 MiB array inside the library (held by every
 * GPU that loads it, until exit); inputs and outputs are still the caller's.
 *
 * Rules for callers:
 *   - sizes whose scratch exceeds celeg_attention_decode_static_capacity() are refused with an
 *     error (celeg_last_error() says how many bytes were needed);
 *   - the first call on a device finds the array's device address; make it before any stream
 *     capture starts;
 *   - all calls share the array: calls that may run at the same time on one GPU race on it.
 *
 * Arguments are those of celeg_attention_decode without the three scratch pointers:
 *   q [tokens, q_row_stride] bf16, out [tokens, q_heads*head_dim] bf16, k_cache/v_cache one
 *   layer's pages [pages, kv_heads, page_tokens, head_dim] bf16 with page_stride elements between
 *   pages, positions/token_span int32 [tokens], block_table int32 [spans, table_stride],
 *   window 0 = none, chunk keys per split, max_splits >= ceil(longest context / chunk),
 *   error_flag int32 [1] on the device. Returns 0, or a negative code with a message. A token whose
 *   keys need more than max_splits chunks gets no output and error_flag receives 3.
 */
#pragma once

#include <cuda_runtime.h>

#if defined(__GNUC__)
#define CELEG_B200_PUBLIC __attribute__((visibility("default")))
#else
#define CELEG_B200_PUBLIC
#endif

#ifdef __cplusplus
extern "C" {
#endif

CELEG_B200_PUBLIC long long celeg_attention_decode_static_capacity(void);

CELEG_B200_PUBLIC int celeg_attention_decode_static(const void* q, int q_row_stride, void* out, const void* k_cache,
                                  const void* v_cache, long long page_stride, const int* positions,
                                  const int* token_span, const int* block_table, int table_stride, int tokens,
                                  int q_heads, int kv_heads, int head_dim, int page_tokens, int window,
                                  float scale, int chunk, int max_splits, int* error_flag, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
