/*
 * paged_attention_b200_test_aids.h -- C ABI of libpaged_attention_b200_test_aids.so.
 *
 * Test and measurement aids of the B200 paged-attention library.  They are not part of the
 * product: they allocate a few bytes of device memory and block, which the product library
 * (include/paged_attention_b200.h) never does.  None has a counterpart in the reference.
 */
#ifndef PAGED_ATTENTION_B200_TEST_AIDS_H_
#define PAGED_ATTENTION_B200_TEST_AIDS_H_

#include <stdint.h>

#include "paged_attention_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Self-test of the failure path: launches one CTA that waits, through the product's own
 * bounded-wait helper (pa::mbar_wait_bounded), on a barrier nothing ever completes, with the
 * given limit (1..500000 us).  Returns PA_OK if the wait gave up within the limit and the
 * kernel left through its normal exit; *status_word (optional) then receives the device
 * status word that exit recorded (PA_ERR_TIMEOUT = 4), read and cleared by the same code
 * pa_device_status() applies to the product's kernels.  Allocates 4 bytes of device memory and
 * synchronises the device. */
PA_API int pa_aid_selftest_wait_timeout(uint32_t limit_us, int32_t *status_word);

/* Times `iters` launches of a kernel that only reads, with CUDA events on `stream`, and stores
 * the read rate in GB/s.  One launch reads `bytes` at `buf` and then, if `buf2` is not NULL,
 * `bytes2` at `buf2` (both 16-byte aligned) -- e.g. the K pool and the V pool, so that the
 * figure is for the same byte count in one launch as the attention kernel reads.  method 0:
 * 16-byte loads with a grid stride, folded into a checksum; method 1: 16 KB bulk copies into a
 * shared-memory ring (the copy engine the attention kernels use), data never looked at, whole
 * 16 KB chunks only.  Blocks until done; allocates 4 bytes of device memory.  With buffers
 * much larger than L2 this is the HBM read rate a kernel that does nothing but read reaches
 * at that size. */
PA_API int pa_aid_measure_read_bandwidth(const void *buf, uint64_t bytes, const void *buf2, uint64_t bytes2,
                                         uint32_t method, uint32_t iters, void *stream, float *gb_per_s);

/* One of the product's four launchers (launch_kernels_loop and its siblings). */
typedef int (*pa_aid_launch_fn)(const pa_params *p, void *stream, float *us_out);

/* Times `calls` asynchronous calls of `launch`, issued back to back from C on `stream` between
 * two CUDA events, call i with params[i % num_params] (e.g. one argument block per rotated
 * KV-cache copy), and stores the mean microseconds per call.  This is the rate a C or C++ host
 * of the library sees; a Python loop over the same calls adds its own microseconds per call,
 * which matters for batches that take ten.  Blocks until done; allocates nothing on the device. */
PA_API int pa_aid_time_launches(pa_aid_launch_fn launch, const pa_params *params, uint32_t num_params,
                                uint32_t calls, void *stream, float *us_per_call);

/* Message of the last non-PA_OK return of this library on the calling thread. */
PA_API const char *pa_aid_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* PAGED_ATTENTION_B200_TEST_AIDS_H_ */
