/* Allocation-free entry point of the kernel library.
 *
 * This entry point has no counterpart in the reference project; it exists for embedders of this library.
 *
 * Who needs it: code that drives the kernels from a place where it must not (or cannot) obtain device memory
 * at call time.  Typical cases are a serving loop whose memory pool is owned by another runtime and sized to
 * the last byte at start-up (a late cudaMalloc there can fail, and it serialises the whole device while it
 * runs), latency-critical decode threads that are forbidden to make any call that may block on the driver's
 * allocator lock, and hosts written in other languages that only pass in buffers they already own.  Such
 * callers can still hand over their inputs and outputs, but they have nowhere to get the split-KV scratch
 * (partial outputs and log-sum-exp values) that flash-decoding needs.
 *
 * omni_mla_decode_noalloc() is the split-KV MLA decode attention with that scratch taken from a fixed array
 * that lives inside the library image (file-scope `static __device__`, 256-byte aligned).  The array costs
 * OMNI_MLA_NOALLOC_SCRATCH_BYTES of device memory on every GPU that loads the library, from load to exit.
 *
 * Contract
 *   - Arguments are those of omni_mla_decode() without the two scratch pointers.
 *   - Limits: Bq * num_splits * H * 512 * 4 bytes of partial outputs must fit OMNI_MLA_NOALLOC_OPART_BYTES
 *     (16 MiB, i.e. Bq * num_splits * H <= 8192) and Bq * num_splits * H log-sum-exp values must fit
 *     OMNI_MLA_NOALLOC_LSE_FLOATS.  Larger problems are refused with OMNI_NOALLOC_TOO_LARGE (-100) and a
 *     message on stderr; nothing is launched.  The limit applies to num_splits > 1 only: a call with one
 *     split writes `out` directly, uses no scratch and may be of any size.
 *   - The call makes no cudaMalloc / cudaFree and uses no allocating library routine.
 *   - The first call on each device looks up the device address of the array (cudaGetSymbolAddress, return
 *     code checked) and remembers it.  Make that first call before starting any stream capture, and do not
 *     let two threads make their first call on the same device at the same moment (the look-up is not
 *     locked; later calls are free to come from any thread).
 *   - All calls share the one array and it keeps whatever the previous call left in it.  The kernels write
 *     every partial result they later read, so nothing has to be cleared between calls; but two calls whose
 *     kernels overlap on the GPU (different streams, or the same stream from two threads without ordering)
 *     race on the array and must be serialised by the caller.
 *   - Returns 0 on success, a negative argument error, or a positive CUDA error code.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OMNI_MLA_NOALLOC_OPART_BYTES (16u << 20)
#define OMNI_MLA_NOALLOC_LSE_FLOATS 16384u
#define OMNI_MLA_NOALLOC_SCRATCH_BYTES (OMNI_MLA_NOALLOC_OPART_BYTES + OMNI_MLA_NOALLOC_LSE_FLOATS * 4u)
#define OMNI_NOALLOC_TOO_LARGE (-100)

int omni_mla_decode_noalloc(const void* q, const void* cache, int cache_ld, long long num_slots,
                            const int* block_table, int bt_ld, const int* seq_lens, const int* q_to_seq, int Bq, int H,
                            int block_size, float scale, int num_splits, void* out, void* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
