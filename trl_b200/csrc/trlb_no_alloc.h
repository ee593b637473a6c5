// Allocation-free variant of the split-KV paged decode attention.
//
// This entry point has no counterpart in the reference (huggingface/trl ships no native code and
// reaches attention only through libraries that allocate their own workspaces).
//
// Who needs it: code that must not call cudaMalloc or any allocating routine while it launches
// work.  Typical cases are a serving loop whose memory budget was fixed at start-up and has no
// allocator attached (every byte already belongs to weights or the KV cache), a caller that runs
// inside a region where allocation would synchronise the device or fail (for example between
// other frameworks' captured work), and plain C callers that link this library without PyTorch
// and therefore have no caching allocator to hand a workspace from.
//
// The ordinary entry point, trlb_paged_decode_attn, takes two caller-provided scratch buffers for
// the per-split partial results.  This variant keeps that scratch inside the library instead, in a
// fixed array in device memory (about 4.1 MB) that every GPU that loads the library holds until
// the process exits.  The caller passes inputs and outputs only.
//
// Limits and rules
//   * B * Hq * splits must not exceed TRLB_NOALLOC_MAX_PARTS (8192) and head_dim must be 128;
//     larger requests are rejected with TRLB_NOALLOC_ERR_TOO_LARGE and a message on stderr,
//     nothing is launched.
//   * The first call on each device looks up the device address of the scratch array (one
//     cudaGetSymbolAddress with that device current).  Make that first call before starting any
//     stream capture on that device.
//   * All calls share the one array, which keeps whatever the previous call left in it.  The
//     kernels overwrite every partial they later read, so nothing has to start at zero; but two
//     calls that overlap on the GPU (different streams, no ordering between them) race on the
//     array.  Order them on one stream or with events.
//   * Host threads: the looked-up addresses are cached per device ordinal without a lock.  Two host
//     threads that make the first call on one device at the same moment both look the addresses up
//     and store the same values, which is harmless, but it is cleaner to make the first call from
//     one thread (during set-up) before others use the device.  The cache does not survive
//     cudaDeviceReset: do not reset a device between calls.
//   * An error left behind by earlier work on the device (a sticky error) is returned by this call's
//     launch check like by any other CUDA call; it does not come from this entry point.
//   * No cudaMalloc, cudaFree or allocating library routine is called on any path.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRLB_NOALLOC_MAX_PARTS 8192
#define TRLB_NOALLOC_ERR_TOO_LARGE (-70)
#define TRLB_NOALLOC_ERR_BAD_SHAPE (-71)
#define TRLB_NOALLOC_ERR_SYMBOL (-72)

// q [B,Hq,128] bf16; kc/vc paged caches [blocks, block_size, Hk, 128] bf16; seq_lens[slot] = tokens in
// the cache before the current one (the kernel attends over seq_lens + 1); slot_ids may be NULL (slot = row);
// block_table [slots, max_blocks] int32; out [B,Hq,128] bf16.  Returns 0, a TRLB_NOALLOC_ERR_* code, or a
// cudaError_t from the launch.
int trlb_paged_decode_attn_noalloc(const void* q, const void* kc, const void* vc, const int* seq_lens,
                                   const int* slot_ids, const int* block_table, int max_blocks, int block_size, int B,
                                   int Hq, int Hk, int D, float scale, int splits, void* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
