/* Allocation-free entry point (this function has no counterpart in the reference project).
 *
 * Who needs it: code that drives this library from a place where device memory cannot be
 * allocated or freed. Examples are a host callback that runs between the nodes of a captured
 * stream, a real-time serving thread that must not take the CUDA allocator's locks or trigger an
 * implicit device synchronisation, and a process that was given a fixed memory budget at start-up
 * and may not grow it. cudaMalloc / cudaFree synchronise the device and can fail late; such
 * callers need a call whose only device-side effects are kernel launches on their stream.
 *
 * What it does: the same stable two-way row partition as FB_OpPartition (rows whose bin of one
 * feature group is <= threshold go to the front, order preserved on both sides), but all of its
 * scratch memory (go-left bit words, per-chunk counters, the small descriptor records) lives in
 * one fixed array inside the library image instead of in freshly allocated buffers. The caller
 * still owns and passes every input and output buffer.
 *
 * Limits and rules:
 *  - at most FB_NO_ALLOC_MAX_ROWS rows per call; larger calls are refused with an error;
 *  - the scratch array (about 0.6 MB) is part of the library: every GPU that loads the library
 *    holds it until the process exits;
 *  - the first call on each device looks up the array's device address (no allocation, but a
 *    runtime query): make that first call outside of any stream capture. Host threads that race
 *    on that first call each do the lookup and store the same address, which is harmless;
 *  - the feature group must lie inside a row (0 <= group < row_stride) and the buffers must be
 *    non-null device pointers; a call with count == 0 is valid and reports 0 rows on the left;
 *  - all calls share the one array and it keeps whatever the previous call left in it, so two
 *    calls that overlap on the same GPU (different streams or threads) corrupt each other: issue
 *    them one after another;
 *  - no cudaMalloc, cudaFree or allocating library routine is called on this path.
 */
#ifndef FB_NO_ALLOC_H_
#define FB_NO_ALLOC_H_
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FB_NO_ALLOC_MAX_ROWS (1 << 22)

/* rows: device, uint8 [n x row_stride]; idx: device int32 [count] row ids; out_idx: device int32
 * [count]; left_count_device: device int32 [1] receiving the number of rows that went left.
 * stream: a cudaStream_t passed as a pointer-sized value (0 = default stream).
 * Returns 0 on success, -1 on error (message from FB_NoAllocLastError). */
int FB_OpPartitionNoAlloc(const uint8_t* rows, int row_stride, const int* idx, int count, int group, int threshold, int default_left,
                          int missing_type, int default_bin, int num_bin, int* out_idx, int* left_count_device, void* stream);
const char* FB_NoAllocLastError();

#ifdef __cplusplus
}
#endif
#endif /* FB_NO_ALLOC_H_ */
