/* sga_compact_mask_noalloc -- mask compaction for callers that cannot allocate.
 *
 * This entry point has no counterpart in the reference framework; it is an
 * addition of this library.
 *
 * Who it is for. sga_compact_mask() needs a work array of one int per 4096
 * mask bytes and expects the caller to supply it. Some callers have no way to
 * get one: a host program that embeds this library without PyTorch and has
 * handed all of the device's memory to its own arena, so a cudaMalloc would
 * fail or break its budget; a latency-critical loop that must not hit the
 * device-wide synchronisation cudaMalloc / cudaFree imply; a plug-in that is
 * only ever given input and output buffers. For them the work array lives
 * inside the library, as a file-scope device array. Nothing is allocated:
 * no cudaMalloc, no cudaFree, no allocating library call, on any call.
 *
 * Limit. The built-in work array holds SGA_COMPACT_NOALLOC_MAX_BLOCKS ints
 * (256 KiB), which covers masks of up to SGA_COMPACT_NOALLOC_MAX_ELEMS bytes
 * (268,435,456). A larger mask is refused with
 * SGA_COMPACT_NOALLOC_E_TOO_LARGE and a message on stderr; nothing is
 * launched in that case. Every GPU that loads the library holds those 256 KiB
 * until the process exits.
 *
 * Set-up. The first call on each device resolves the device address of the
 * work array (cudaGetSymbolAddress, with that device current) and remembers
 * it. Make that first call during initialisation, before any stream capture
 * is begun on the device.
 *
 * Sharing. All calls on a device use the same work array, and it keeps
 * whatever the previous call left in it. The kernels overwrite every entry
 * they later read, so no clearing is needed between calls. Two calls whose
 * kernels can overlap on the GPU (different streams without an ordering
 * between them, or different host threads) race on the array and produce
 * garbage: keep calls on one device ordered.
 *
 * Semantics are those of sga_compact_mask(): idx_out receives the ascending
 * positions of the non-zero bytes of mask[0..n), *total_out their number;
 * positions beyond cap are dropped and SGA_ERR_CAPACITY (16) is OR-ed into
 * *err. mask bytes must be 0 or 1. Returns 0 on success. With n <= 0 the call
 * returns 0 at once and writes nothing, *total_out included.
 *
 * Alignment. The kernels read the mask 16 bytes at a time, so mask must start
 * on a 16-byte boundary (a pointer from cudaMalloc does; an odd offset into a
 * larger buffer may not). A misaligned mask is refused with
 * SGA_COMPACT_NOALLOC_E_ALIGN before anything is launched.
 */
#ifndef SGA_COMPACT_NOALLOC_H
#define SGA_COMPACT_NOALLOC_H

#include <stdint.h>

#define SGA_COMPACT_NOALLOC_MAX_BLOCKS 65536
#define SGA_COMPACT_NOALLOC_MAX_ELEMS (65536LL * 4096LL)

#define SGA_COMPACT_NOALLOC_E_TOO_LARGE (-8) /* n exceeds SGA_COMPACT_NOALLOC_MAX_ELEMS */
#define SGA_COMPACT_NOALLOC_E_SETUP (-9)     /* the work array's device address could not be resolved */
#define SGA_COMPACT_NOALLOC_E_LAUNCH (-4)    /* a kernel launch failed */
#define SGA_COMPACT_NOALLOC_E_ALIGN (-10)    /* mask does not start on a 16-byte boundary */

#ifdef __cplusplus
extern "C" {
#endif

int sga_compact_mask_noalloc(const uint8_t* mask, long long n, int* idx_out, long long cap, long long* total_out,
                             int* err, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* SGA_COMPACT_NOALLOC_H */
