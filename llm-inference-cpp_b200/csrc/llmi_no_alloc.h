/* Entry point of libllmi_b200 for callers that cannot allocate device memory.
 *
 * This has no counterpart in the reference engine (fernandojcardenas/llm-inference-cpp runs on the CPU
 * and allocates its temporaries with std::vector in every call, src/model/transformer.cpp:223-233).
 *
 * Who needs it.  Every other launcher of this library takes its scratch memory from the caller, who gets
 * it from an allocator (here: PyTorch's).  Some callers have no allocator to ask, or must not ask one
 * where the call happens: code that runs inside someone else's stream capture or latency-critical loop,
 * where cudaMalloc would synchronise the device or is simply forbidden; a host program written in C that
 * links this library alone, without a framework's caching allocator behind it; a plug-in whose host
 * application hands it input and output buffers and nothing else.  For them the split decode attention —
 * the one kernel of the decode step whose scratch grows with the batch — exists in a second form that
 * brings its scratch along.
 *
 * What it is.  llmi_attention_decode_static computes exactly what llmi_attention_decode computes (same
 * kernel, same arguments for inputs and outputs; see attention_decode.cu), but the per-split partial
 * results, the tickets and the error word live in one file-scope `static __device__` array of the
 * library instead of in caller memory.  The function calls no cudaMalloc, no cudaFree and no allocating
 * library routine; it launches on `stream` and returns.
 *
 * Limits.  The array has a fixed size, held by every GPU that loads the library until the process ends:
 * 4 MiB of partial results (1,048,576 floats), 16,384 tickets (64 KiB) and the error word.  A call needs
 *     n_seqs * n_heads * ceil(max_pages / pages_per_split) * (head_dim + 2)   floats and
 *     n_seqs * n_kv_heads                                                      tickets;
 * one that needs more is refused with LLMI_ERR_STATIC_SCRATCH (-7) and launches nothing.  (Example: 64
 * sequences, 32 heads of 64, 4,096 positions in splits of 16 pages need 540,672 floats.)
 *
 * First call.  The first call on a device asks the runtime for the array's device address
 * (cudaGetSymbolAddress, with that device current) and keeps it.  Make that first call outside of any
 * stream capture; later calls on the same device do not repeat it.
 *
 * Sharing.  All calls on a device share the one array, and it keeps what the last call left.  Each call
 * clears what has to start at zero (its tickets and the error word, with cudaMemsetAsync on `stream`)
 * and overwrites the partials before reading them.  Two calls that overlap on the GPU — different
 * streams, or the same call from two threads — race on the array and give wrong results: run them one
 * after the other.
 *
 * error_out (optional, device pointer to one int, caller-owned): receives 0, or the code of a bounded wait
 * inside the kernel that gave up (then `out` is invalid).  It is written by a copy queued on `stream` after
 * the kernel, like `out` itself: read it only after the stream (or an event recorded behind the call) has
 * been synchronised.  Pass NULL to ignore it.
 *
 * Several GPUs.  Each device that calls has its own copy of the array, its own resolved address and its own
 * launch set-up; make each device's first call with that device current.
 *
 * Returns 0, or a negative LLMI_ERR_* code (common.cuh): -2 bad size, -4 misaligned pointer or pitch,
 * -5 no kernel for this head size and group, -6 the runtime refused cudaGetDevice/cudaGetSymbolAddress,
 * -7 more scratch needed than the array holds, -3 the launch failed.
 */
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int llmi_attention_decode_static(const void* q, long ldq, void* out, long ldo, const void* k_cache,
                                 const void* v_cache, const int32_t* seq_pages, int pages_stride,
                                 const int32_t* seq_kv_len, const int32_t* seq_q_start, int n_seqs, int n_heads,
                                 int n_kv_heads, int head_dim, float scale, int window, int max_pages,
                                 int pages_per_split, int* error_out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
