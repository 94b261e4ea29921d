// An allocation-free way into the split-KV decode attention kernel.
//
// This entry point has no counterpart in ghyathmoussa/rLLM; it exists for hosts
// that must not allocate device memory when they call us: a C or C++ program
// that links this library without PyTorch's caching allocator, a process that
// has already handed every free byte of the GPU to its own pool (so a
// cudaMalloc here would fail or fragment it), or a latency-critical loop in
// which cudaMalloc's implicit device synchronisation is not acceptable.
//
// The ordinary entry point, rllm_attention_decode_bf16, takes its scratch
// (the per-chunk partial results and the merge counters) from the caller.  This
// one keeps that scratch inside the library, in a fixed array in device memory
// (RLLM_DECODE_STATIC_FLOATS floats and RLLM_DECODE_STATIC_COUNTERS ints, about
// 16 MiB, held by every GPU that loads the library until the process ends), and
// calls no cudaMalloc, cudaFree or allocating library routine.
//
// Rules for the caller:
//  * Sizes: num_seqs * nq * ceil(max_seq_len / 128) * (d + 2) (half of what
//    rllm_attention_decode_workspace reports; where that whole amount fits too, this
//    entry point cuts short sequences into chunks of 64 keys exactly as the ordinary
//    one does, else it keeps to chunks of 128 and its results may differ from the
//    ordinary one's in the last bit) must not exceed RLLM_DECODE_STATIC_FLOATS and num_seqs * nkv must not exceed
//    RLLM_DECODE_STATIC_COUNTERS; otherwise the call returns
//    RLLM_E_STATIC_TOO_LARGE (-3) and launches nothing.
//  * The first call on a device looks up the array's device address (once per
//    device, with that device current).  With CUDA's lazy module loading that
//    first call is also the moment at which the driver loads this library's
//    device code and reserves the array, so it may take longer and may
//    synchronise; later calls do neither.  Make that first call before any
//    stream capture begins on that device.  Two host threads may make their
//    first call at the same time.
//  * All calls share the one array, and it keeps what the last call left in it.
//    The counters are cleared on the caller's stream at the start of every call;
//    the partial results need no clearing (every slot is written before it is
//    read).  Two calls that overlap on the GPU (different streams without an
//    ordering between them) race on the array: order them.
//  * Inputs, outputs and their meaning are exactly those of
//    rllm_attention_decode_bf16, and so is its ordering rule: with write_kv the
//    kernel reads seq_lens, the block table and older cache rows before it
//    waits for the kernel ahead of it in the stream, so those must be complete
//    by the time that kernel starts (here the memset of the counters stands
//    between, which is enough); every seq_lens[s] is at least 1.
#pragma once
#include <cuda_runtime.h>

#define RLLM_DECODE_STATIC_FLOATS (4 * 1024 * 1024)
#define RLLM_DECODE_STATIC_COUNTERS (16 * 1024)
#define RLLM_E_STATIC_TOO_LARGE (-3)

#ifdef __cplusplus
extern "C" {
#endif
int rllm_attention_decode_bf16_static(void* qkv, int q_stride, void* out, void* kcache, void* vcache,
                                      const int* block_table, int max_blocks, const int* seq_lens,
                                      int num_seqs, int max_seq_len, int nq, int nkv, int d, int page_size,
                                      int num_pages, int window, float scale, const double* inv_freq,
                                      int rotary_dim, int write_kv, int* err, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
