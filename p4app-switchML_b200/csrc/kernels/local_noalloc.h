/* switchml_local_allreduce_noalloc: the single-worker aggregation round trip for callers
 * that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference library.
 *
 * Who needs it. Some hosts call into this library from places where asking CUDA for
 * memory is off the table: a serving process that handed every free byte of HBM to its
 * own pool at start-up (cudaMalloc would simply fail there, or steal from that pool's
 * budget), a latency-critical loop that cannot afford the device-wide synchronisation an
 * allocation or a free may imply, or a callback that runs while another component holds
 * allocator locks. All other entry points of the library allocate staging memory
 * (cudaMalloc or the virtual-memory API); this one calls no cudaMalloc, no cudaFree and
 * no allocating library routine, torch's included.
 *
 * What it does. It runs the streaming aggregation kernel (the one behind
 * sml_emu_allreduce and the cuda backend) for ONE worker on the current device:
 *   mode 1 (quantised): block max -> exponent -> int32 fixed point -> sum over the single
 *                       worker -> back to float, i.e. exactly what one rank contributes
 *                       and receives, bit for bit as the multi-rank path computes it;
 *   mode 0 (sum):       the same pipeline without conversion (a staged copy).
 * The staging slots, flags and counters that the kernel needs live in a file-scope
 * `static __device__` array of SWITCHML_NOALLOC_SCRATCH_BYTES (1 MiB), which every GPU that
 * loads the library keeps until the process exits. The caller passes only input and output.
 *
 * Rules.
 *  - numel may be at most SWITCHML_NOALLOC_MAX_NUMEL; block_numel a power of two in
 *    [32, 1024]; elem_type 0 float32, 1 int32 (mode 0 only), 2 bfloat16. Anything else is
 *    refused with a negative code (switchml_noalloc_strerror explains it) and nothing runs.
 *  - The first call on each device looks up the device address of the scratch array
 *    (cudaGetSymbolAddress, with that device current) and caches it. Make that first call
 *    before any stream capture begins on that device.
 *  - All calls on a device share the one scratch array, and it still holds what the last
 *    call left there. The entry point itself clears, on `stream`, the flags and counters
 *    that have to start at zero. Two calls whose work overlaps on the GPU (different
 *    streams without ordering between them) race on the scratch and give wrong results:
 *    order them on one stream or with events. Host threads may call at the same time: each
 *    call's clears and its kernel reach the stream as one unit.
 *  - The kernel's own verdict (0 = fine, otherwise a Status code of allreduce_kernels.h in the
 *    low four bits, e.g. 1 when one of its bounded waits gave up) stays in the scratch; the
 *    return code of the call only covers the launch. switchml_noalloc_last_status waits for
 *    `stream` and reads it back. It describes the call that ran last on this device.
 *  - The work is enqueued on `stream` (a cudaStream_t, NULL = default stream); the result
 *    is in `out` when the stream gets there. `in` and `out` may be the same buffer.
 */
#ifndef SWITCHML_LOCAL_NOALLOC_H_
#define SWITCHML_LOCAL_NOALLOC_H_

#ifdef __cplusplus
extern "C" {
#endif

#define SWITCHML_NOALLOC_SCRATCH_BYTES (1u << 20)
#define SWITCHML_NOALLOC_MAX_NUMEL (1ull << 26)

#define SWITCHML_NOALLOC_OK 0
#define SWITCHML_NOALLOC_BAD_ARGUMENT (-1)
#define SWITCHML_NOALLOC_TOO_LARGE (-2)
#define SWITCHML_NOALLOC_CUDA_ERROR (-3)

int switchml_local_allreduce_noalloc(const void* in, void* out, unsigned long long numel,
                                     int elem_type, int mode, int block_numel, void* stream);

/* Wait for `stream`, then store the status word that the last call on the current device left
 * in the scratch (0 = the kernel completed normally). Allocates nothing either. */
int switchml_noalloc_last_status(void* stream, int* status);

/* Static text for a return code of the functions above. */
const char* switchml_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif /* SWITCHML_LOCAL_NOALLOC_H_ */
