/* Decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the MicroInfer reference; it is an
 * addition of this library.
 *
 * Who it is for. The regular entry point, sakv_decode_attention, needs two scratch
 * buffers for the partial results of its key splits, and its callers get them from
 * an allocator (the Python side asks torch's). Some callers have no allocator to
 * ask: a host program that handed all of the GPU's memory to its own pool at
 * start-up and gives this library nothing but the input and output buffers; a
 * plain C, C++ or FFI caller that links this shared library without torch; code on
 * a path where cudaMalloc is not acceptable because it synchronises the whole
 * device. For them the scratch lives inside the library instead: a file-scope
 * device array of SAKV_DECODE_STATIC_SCRATCH_FLOATS floats (8 MiB), which every GPU
 * that loads the library holds from load until the process exits.
 *
 * What it does. Exactly what sakv_decode_attention does, with the same arguments
 * except that the two scratch pointers are gone. It calls no cudaMalloc, cudaFree
 * or any routine that allocates.
 *
 * Limits and rules.
 *  - sequences * heads * splits * (head_dim + 2) must not exceed
 *    SAKV_DECODE_STATIC_SCRATCH_FLOATS; a larger problem is refused with
 *    cudaErrorInvalidValue (1) and, if `why` is given, a sentence that says so.
 *    Nothing is launched then.
 *  - The first call on each device looks up the array's device address (with that
 *    device current) and remembers it. Make that first call outside any stream
 *    capture.
 *  - All calls share the one array, and it keeps what the last call left. Nothing
 *    in it has to start at zero: every element that the folding kernel reads was
 *    written by the split kernel of the same call.
 *  - Two calls that overlap on the GPU (different streams, or different host
 *    threads) race on the array. Keep calls on one stream, or order them.
 */
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define SAKV_DECODE_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

/* Returns 0 when the kernels were launched on `stream`, else a cudaError_t value.
 * `k_map`, `v_map`: 128-byte TMA descriptors made by sakv_decode_attention_map.
 * `why`/`why_len`: optional buffer for a message when the call is refused. */
int sakv_decode_attention_static_scratch(const void* k_map, const void* v_map, const void* q,
                                         long long q_stride, const int32_t* seq_lens,
                                         const int32_t* block_table, int max_blocks, void* out,
                                         int sequences, int heads, int kv_heads, int head_dim,
                                         int splits, float scale, int window, char* why,
                                         int why_len, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
