/*
 * Test hooks of the B200 HSTU library: exported by libhstu_b200.so for its own test-suite, not part of the operator
 * interface (which is include/hstu_b200.h).  No counterpart in the reference API.
 */
#ifndef HSTU_B200_TESTING_H_
#define HSTU_B200_TESTING_H_

#include "hstu_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Testing hooks: the device mask predicate and K-tile classifier evaluated on the host (same source, compiled
 * for the host).  hstu_debug_mask_host fills out[len_q * len_k] with 0/1 visibility; hstu_debug_tiles_host returns
 * how many K tiles of width bn the q-tile rows [r0, r0+rows) visits and which of them need no per-element
 * predicate.  No counterpart in the reference API; its kernel-side equivalent is
 * ascendc/attention/hstu_v1/hstu_forward_v1/op_kernel/atlas950/hstu_dense_causal_mask.h:63-260. */
HSTU_API int hstu_debug_mask_host(int32_t len_q, int32_t len_k, int32_t num_context, int32_t num_target,
                         int32_t target_group_size, int32_t mask_type, uint8_t* out);
HSTU_API int hstu_debug_tiles_host(int32_t len_q, int32_t len_k, int32_t num_context, int32_t num_target,
                          int32_t target_group_size, int32_t mask_type, int32_t r0, int32_t rows, int32_t bn,
                          uint64_t* full_bits);

#ifdef __cplusplus
}
#endif
#endif /* HSTU_B200_TESTING_H_ */
